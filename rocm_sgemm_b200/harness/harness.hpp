// Shared pieces of the C++ harnesses gemm_test and gemm_bench: a host matrix with a layout-aware
// indexer, error checking, an event timer, input generators and the host GEMM used for verification.
// Counterparts in the reference: common/matrix.hpp:24-145 (matrix<T,Layout>), common/hip_utils.hpp:11-56
// (HIP_CHECK, gpu_timer), test/test.hpp:11-45 (init_matrix, sgemm_cpu), benchmark/bench.hpp:15-29
// (pattern init).  Self-contained: no GoogleTest, no Google Benchmark.
#pragma once
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <random>
#include <stdexcept>
#include <vector>

namespace harness
{

enum class layout
{
    row_major = 0,
    col_major = 1
};

// Host-side M x N matrix stored packed in the given layout (run-time layout, unlike the reference's
// compile-time one, so that one code path serves all eight permutations).
class host_matrix
{
public:
    host_matrix(size_t rows, size_t cols, layout l) : rows_(rows), cols_(cols), layout_(l), data_(rows * cols)
    {
        if(rows == 0 || cols == 0)
            throw std::invalid_argument("matrix dimensions must be positive");
    }
    float& operator()(size_t i, size_t j) { return data_[index(i, j)]; }
    float  operator()(size_t i, size_t j) const { return data_[index(i, j)]; }
    float*       data() { return data_.data(); }
    const float* data() const { return data_.data(); }
    size_t       rows() const { return rows_; }
    size_t       cols() const { return cols_; }
    size_t       size() const { return data_.size(); }
    size_t       bytes() const { return data_.size() * sizeof(float); }
    layout       order() const { return layout_; }

private:
    size_t index(size_t i, size_t j) const { return layout_ == layout::row_major ? i * cols_ + j : j * rows_ + i; }
    size_t             rows_, cols_;
    layout             layout_;
    std::vector<float> data_;
};

#define CUDA_CHECK(call)                                                                                  \
    do                                                                                                    \
    {                                                                                                     \
        cudaError_t status_ = (call);                                                                     \
        if(status_ != cudaSuccess)                                                                        \
        {                                                                                                 \
            std::fprintf(stderr, "CUDA error: %s failed with %d: %s\n", #call, (int)status_,              \
                         cudaGetErrorString(status_));                                                    \
            std::exit(EXIT_FAILURE);                                                                      \
        }                                                                                                 \
    } while(0)

// event pair on a stream; stop() returns milliseconds
class gpu_timer
{
public:
    gpu_timer()
    {
        CUDA_CHECK(cudaEventCreate(&start_));
        CUDA_CHECK(cudaEventCreate(&stop_));
    }
    ~gpu_timer()
    {
        cudaEventDestroy(start_);
        cudaEventDestroy(stop_);
    }
    void  start(cudaStream_t s) { CUDA_CHECK(cudaEventRecord(start_, s)); }
    float stop(cudaStream_t s)
    {
        CUDA_CHECK(cudaEventRecord(stop_, s));
        CUDA_CHECK(cudaEventSynchronize(stop_));
        float ms = 0.f;
        CUDA_CHECK(cudaEventElapsedTime(&ms, start_, stop_));
        return ms;
    }

private:
    cudaEvent_t start_, stop_;
};

// U(-1,1) from a caller-owned generator, filled in logical (row, col) order whatever the layout
inline void fill_uniform(host_matrix& m, std::mt19937& gen)
{
    std::uniform_real_distribution<float> dis(-1.0f, 1.0f);
    for(size_t i = 0; i < m.rows(); ++i)
        for(size_t j = 0; j < m.cols(); ++j)
            m(i, j) = dis(gen);
}
// the reference test's initialisation: a fresh mt19937(1) per matrix
inline void fill_like_reference_test(host_matrix& m)
{
    std::mt19937 gen(1);
    fill_uniform(m, gen);
}
// the reference benchmark's cyclic five-value pattern
inline void fill_pattern(host_matrix& m)
{
    static const float v[5] = {1.025f, 1.05f, 1.075f, 1.1f, 1.0f};
    size_t             l    = 0;
    for(size_t i = 0; i < m.rows(); ++i)
        for(size_t j = 0; j < m.cols(); ++j)
            m(i, j) = v[(l++) % 5];
}
inline void fill_identity(host_matrix& m)
{
    for(size_t i = 0; i < m.rows(); ++i)
        for(size_t j = 0; j < m.cols(); ++j)
            m(i, j) = i == j ? 1.0f : 0.0f;
}

// host verification GEMM: float accumulator, k ascending; rows [r0, r1) of C only, split over the
// host threads when built with OpenMP.  Returns nothing; C rows outside the band are left alone.
inline void host_sgemm(host_matrix& C, const host_matrix& A, const host_matrix& B, size_t r0, size_t r1)
{
    const long long K = (long long)A.cols(), N = (long long)C.cols();
#pragma omp parallel for schedule(static)
    for(long long i = (long long)r0; i < (long long)r1; ++i)
        for(long long j = 0; j < N; ++j)
        {
            float acc = 0.0f;
            for(long long k = 0; k < K; ++k)
                acc += A(i, k) * B(k, j);
            C(i, j) = acc;
        }
}

inline const char* layout_letter(layout l)
{
    return l == layout::row_major ? "r" : "c";
}

} // namespace harness
