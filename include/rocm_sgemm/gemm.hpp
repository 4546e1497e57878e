// Drop-in C++ surface of the reference operator on top of the C ABI (include/b200_sgemm.h).
//
// Source-compatible with rocm_sgemm/include/rocm_sgemm/gemm.hpp:51-121 apart from the stream type
// (cudaStream_t& instead of hipStream_t&):
//
//     rocm_sgemm::gemm<layout_C, layout_A, layout_B>(C, A, B, M, N, K, stream);
//
// with template arguments in the order C, A, B, non-const element pointers, size_t dimensions, and
// the enum rocm_sgemm::m_layout {row_major, col_major} of kernel/common.hpp:36-40.  As in the
// reference the call is asynchronous on `stream` and performs no error check of the kernel's
// execution; the only exception is std::runtime_error when no kernel can be launched
// (kernel_launcher.hpp:89-94) or the arguments are invalid.  get_gemm_params has the reference's
// signature (generated header, rocm_sgemm/config/generate_config.py:282-303) but is a run-time
// function: the tuned table lives inside the library, not in a generated constexpr header.
#ifndef ROCM_SGEMM_GEMM_HPP
#define ROCM_SGEMM_GEMM_HPP

#include "../b200_sgemm.h"

#include <cstddef>
#include <cuda_runtime_api.h>
#include <stdexcept>
#include <string>

namespace rocm_sgemm
{

enum class m_layout
{
    row_major, ///< elements of a row are consecutive in memory
    col_major  ///< elements of a column are consecutive in memory
};

/// Tile parameters chosen for a problem: the reference's nine fields, then the CUDA-side additions.
struct gemm_params
{
    int block_size;
    int block_m;
    int block_n;
    int block_k;
    int warp_tile_m_count;
    int warp_tile_n_count;
    int thread_tile_m;
    int thread_tile_n;
    int threads_n;
    int stages;
    int fma_mode;
    int raster;
    int min_blocks;
    int pipeline;
    int split_k;
    int pretranspose;
};

inline gemm_params get_gemm_params(size_t m, size_t n, size_t k, m_layout layout_c, m_layout layout_a,
                                   m_layout layout_b)
{
    b200_sgemm_params p{};
    const int status = b200_sgemm_select_config(static_cast<int>(layout_c), static_cast<int>(layout_a),
                                                static_cast<int>(layout_b), m, n, k, &p, nullptr);
    if(status != B200_SGEMM_OK)
        throw std::runtime_error(std::string("rocm_sgemm::get_gemm_params: ") + b200_sgemm_status_string(status));
    return gemm_params{p.block_size, p.block_m,       p.block_n,       p.block_k,   p.warp_tile_m_count,
                       p.warp_tile_n_count, p.thread_tile_m, p.thread_tile_n, p.threads_n, p.stages,
                       p.fma_mode,   p.raster,        p.min_blocks,    p.pipeline,  p.split_k,
                       p.pretranspose};
}

/// Number of kernel variants built into the library (the reference's constant KERNEL_VARIANTS).
inline size_t kernel_variants()
{
    return static_cast<size_t>(b200_sgemm_num_variants());
}

/**
 * @brief GPU matrix multiplication C = A * B (FP32, alpha = 1, beta = 0, C overwritten).
 *
 * @param C      output, M x N, device memory, layout_C
 * @param A      input,  M x K, device memory, layout_A
 * @param B      input,  K x N, device memory, layout_B
 * @param stream CUDA stream the work is queued on
 */
template<m_layout layout_C, m_layout layout_A, m_layout layout_B, class T>
void gemm(T* C, T* A, T* B, size_t M, size_t N, size_t K, cudaStream_t& stream);

// The library provides float, like the reference's INSTANTIATE_GEMM_FOR_TYPE(float)
// (rocm_sgemm/src/gemm.cpp:44-111): one inline specialisation per layout permutation.
#define ROCM_SGEMM_DEFINE_GEMM(LC, LA, LB)                                                                     \
    template<>                                                                                                 \
    inline void gemm<m_layout::LC, m_layout::LA, m_layout::LB, float>(float* C, float* A, float* B, size_t M,  \
                                                                      size_t N, size_t K, cudaStream_t& stream) \
    {                                                                                                          \
        const int status = b200_sgemm(static_cast<int>(m_layout::LC), static_cast<int>(m_layout::LA),          \
                                      static_cast<int>(m_layout::LB), C, A, B, M, N, K, stream);               \
        if(status != B200_SGEMM_OK)                                                                            \
            throw std::runtime_error(std::string("rocm_sgemm::gemm: ") + b200_sgemm_status_string(status));    \
    }

ROCM_SGEMM_DEFINE_GEMM(row_major, row_major, row_major)
ROCM_SGEMM_DEFINE_GEMM(row_major, row_major, col_major)
ROCM_SGEMM_DEFINE_GEMM(row_major, col_major, row_major)
ROCM_SGEMM_DEFINE_GEMM(row_major, col_major, col_major)
ROCM_SGEMM_DEFINE_GEMM(col_major, row_major, row_major)
ROCM_SGEMM_DEFINE_GEMM(col_major, row_major, col_major)
ROCM_SGEMM_DEFINE_GEMM(col_major, col_major, row_major)
ROCM_SGEMM_DEFINE_GEMM(col_major, col_major, col_major)
#undef ROCM_SGEMM_DEFINE_GEMM

// The signature of the reference's vendor wrapper, rocblas_wrapper::gemm<TRANSPOSE_A, TRANSPOSE_B>(C, A, B, M, N, K,
// stream) (rocblas_wrapper/include/rocblas_wrapper/gemm.hpp:55-68; column-major C, lda = TA ? K : M,
// ldb = TB ? N : K, ldc = M), served by this library's own kernels instead of the vendor BLAS.
namespace blas
{
template<bool TRANSPOSE_A, bool TRANSPOSE_B>
inline void gemm(float* C, float* A, float* B, size_t M, size_t N, size_t K, cudaStream_t& stream)
{
    const int status = b200_sgemm_blas(TRANSPOSE_A, TRANSPOSE_B, M, N, K, 1.0f, A, TRANSPOSE_A ? K : M, B,
                                       TRANSPOSE_B ? N : K, 0.0f, C, M, stream);
    if(status != B200_SGEMM_OK)
        throw std::runtime_error(std::string("rocm_sgemm::blas::gemm: ") + b200_sgemm_status_string(status));
}
} // namespace blas

} // namespace rocm_sgemm

#endif // ROCM_SGEMM_GEMM_HPP
