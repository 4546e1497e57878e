/*
 * Vendor-BLAS comparison column: cublasSgemm behind the same kind of thin wrapper the reference
 * keeps around rocblas_sgemm (rocblas_wrapper/include/rocblas_wrapper/gemm.hpp:18-68,
 * rocblas_wrapper/src/gemm.cpp:6-64).  It exists so that benchmarks can print a cuBLAS number next
 * to this library's; it is never a fallback for the library's own kernels.
 * Math mode is pinned to CUBLAS_PEDANTIC_MATH: true FP32 multiply-add, no TF32 tensor cores.
 */
#ifndef B200_CUBLAS_WRAPPER_H
#define B200_CUBLAS_WRAPPER_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Creates the process-wide cuBLAS handle; 1 on success (also when already initialised).
 * Replaces rocblas_wrapper::init_rocblas (rocblas_wrapper/src/gemm.cpp:6-16). */
int b200_cublas_init(void);

/* Destroys the handle; safe to call repeatedly.
 * Replaces rocblas_wrapper::cleanup_rocblas (rocblas_wrapper/src/gemm.cpp:18-25). */
void b200_cublas_cleanup(void);

/* Column-major C (ldc = M) = op(A) * op(B), alpha = 1, beta = 0, with lda = transpose_a ? K : M and
 * ldb = transpose_b ? N : K: a row-major input is passed as the transpose of a column-major one.
 * Replaces rocblas_wrapper::gemm<TRANSPOSE_A, TRANSPOSE_B> (rocblas_wrapper/src/gemm.cpp:27-64).
 * Returns 0, -1 when not initialised, or the cublasStatus_t value. */
int b200_cublas_gemm(int transpose_a, int transpose_b, float* C, const float* A, const float* B, size_t M, size_t N,
                     size_t K, void* cuda_stream);

/* All eight layout permutations (0 = row-major, 1 = col-major), so that every layout of this
 * library has a vendor number beside it: a row-major C is computed as C^T = B^T * A^T. */
int b200_cublas_gemm_layout(int layout_c, int layout_a, int layout_b, float* C, const float* A, const float* B,
                            size_t M, size_t N, size_t K, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif
