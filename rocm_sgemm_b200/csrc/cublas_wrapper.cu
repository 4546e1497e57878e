// cuBLAS comparison wrapper; see include/b200_cublas_wrapper.h for the reference counterparts.
#include "../../include/b200_cublas_wrapper.h"

#include <cublas_v2.h>
#include <cuda_runtime.h>
#include <mutex>

namespace
{
cublasHandle_t g_handle = nullptr;
std::mutex     g_mutex;
} // namespace

extern "C" {

int b200_cublas_init(void)
{
    std::lock_guard<std::mutex> lock(g_mutex);
    if(g_handle)
        return 1;
    if(cublasCreate(&g_handle) != CUBLAS_STATUS_SUCCESS)
    {
        g_handle = nullptr;
        return 0;
    }
    // strict FP32: no TF32 tensor-core path, no reduced-precision accumulation
    cublasSetMathMode(g_handle, CUBLAS_PEDANTIC_MATH);
    return 1;
}

void b200_cublas_cleanup(void)
{
    std::lock_guard<std::mutex> lock(g_mutex);
    if(g_handle)
    {
        cublasDestroy(g_handle);
        g_handle = nullptr;
    }
}

int b200_cublas_gemm(int transpose_a, int transpose_b, float* C, const float* A, const float* B, size_t M, size_t N,
                     size_t K, void* cuda_stream)
{
    if(!g_handle)
        return -1;
    cublasStatus_t st = cublasSetStream(g_handle, static_cast<cudaStream_t>(cuda_stream));
    if(st != CUBLAS_STATUS_SUCCESS)
        return (int)st;
    const float alpha = 1.0f, beta = 0.0f;
    st = cublasSgemm(g_handle, transpose_a ? CUBLAS_OP_T : CUBLAS_OP_N, transpose_b ? CUBLAS_OP_T : CUBLAS_OP_N,
                     (int)M, (int)N, (int)K, &alpha, A, (int)(transpose_a ? K : M), B, (int)(transpose_b ? N : K),
                     &beta, C, (int)M);
    return (int)st;
}

int b200_cublas_gemm_layout(int layout_c, int layout_a, int layout_b, float* C, const float* A, const float* B,
                            size_t M, size_t N, size_t K, void* cuda_stream)
{
    if(layout_c == 1)
        // column-major C: a row-major operand is the transpose of a column-major one
        return b200_cublas_gemm(layout_a == 0, layout_b == 0, C, A, B, M, N, K, cuda_stream);
    // row-major C (MxN) is column-major C^T (NxM) = B^T (NxK) * A^T (KxM).
    // B^T in column-major terms: row-major B (KxN) already is column-major NxK (no transpose);
    // column-major B (KxN) needs one.  Same for A^T.
    return b200_cublas_gemm(layout_b == 1, layout_a == 1, C, B, A, N, M, K, cuda_stream);
}
}
