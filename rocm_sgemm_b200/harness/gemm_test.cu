// gemm_test: the reference's GPU test suite on the drop-in header.
//
// Follows test/gemm/test.cpp:36-96,113-176 of the reference: for each of the eight layout permutations
// and each of its 13 shapes, inputs from mt19937(1) re-seeded per matrix, one rocm_sgemm::gemm call,
// comparison of every element against the host GEMM with absolute tolerance 1e-4.  Added on top: the
// identity-multiply check (C must equal A bit for bit) and two ragged shapes, which the reference's
// unguarded loads could not pass.  A third group, CublasTest, holds the vendor wrapper to the same bar, as the
// reference's test/rocblas/test.cpp:31-186 does for its rocBLAS wrapper (13 shapes, 1e-4 against the host GEMM;
// here for all eight layouts, the reference covers the four with a column-major C).  Built a second time with
// -DHARNESS_VENDOR_ONLY as `cublas_test`, which runs that group alone (the reference's test_rocblas target,
// test/CMakeLists.txt:11).  Exit code 0 only if everything passed.
#include "harness.hpp"

#include <b200_cublas_wrapper.h>
#include <rocm_sgemm/gemm.hpp>

#include <cmath>
#include <cstring>

using namespace harness;
using rocm_sgemm::m_layout;

namespace
{
using gemm_fn = void (*)(float*, float*, float*, size_t, size_t, size_t, cudaStream_t&);

template<m_layout LC, m_layout LA, m_layout LB>
void call(float* C, float* A, float* B, size_t M, size_t N, size_t K, cudaStream_t& s)
{
    rocm_sgemm::gemm<LC, LA, LB>(C, A, B, M, N, K, s);
}

// index = A*4 + B*2 + C, the reference's layout numbering (kernel_launcher.hpp:53-79)
gemm_fn table[8] = {
    call<m_layout::row_major, m_layout::row_major, m_layout::row_major>,
    call<m_layout::col_major, m_layout::row_major, m_layout::row_major>,
    call<m_layout::row_major, m_layout::row_major, m_layout::col_major>,
    call<m_layout::col_major, m_layout::row_major, m_layout::col_major>,
    call<m_layout::row_major, m_layout::col_major, m_layout::row_major>,
    call<m_layout::col_major, m_layout::col_major, m_layout::row_major>,
    call<m_layout::row_major, m_layout::col_major, m_layout::col_major>,
    call<m_layout::col_major, m_layout::col_major, m_layout::col_major>,
};

struct device_buffers
{
    float *A = nullptr, *B = nullptr, *C = nullptr;
    device_buffers(size_t a, size_t b, size_t c)
    {
        CUDA_CHECK(cudaMalloc(&A, a));
        CUDA_CHECK(cudaMalloc(&B, b));
        CUDA_CHECK(cudaMalloc(&C, c));
    }
    ~device_buffers()
    {
        cudaFree(A);
        cudaFree(B);
        cudaFree(C);
    }
};

bool verify_gemm(int la, int lb, int lc, size_t M, size_t N, size_t K, cudaStream_t stream, bool identity)
{
    host_matrix hA(M, K, (layout)la), hB(K, N, (layout)lb), hC(M, N, (layout)lc), hRef(M, N, (layout)lc);
    fill_like_reference_test(hA);
    if(identity)
        fill_identity(hB);
    else
        fill_like_reference_test(hB);
    device_buffers d(hA.bytes(), hB.bytes(), hC.bytes());
    CUDA_CHECK(cudaMemcpy(d.A, hA.data(), hA.bytes(), cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemcpy(d.B, hB.data(), hB.bytes(), cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemset(d.C, 0xff, hC.bytes()));
    table[la * 4 + lb * 2 + lc](d.C, d.A, d.B, M, N, K, stream);
    CUDA_CHECK(cudaPeekAtLastError());
    CUDA_CHECK(cudaDeviceSynchronize());
    CUDA_CHECK(cudaMemcpy(hC.data(), d.C, hC.bytes(), cudaMemcpyDeviceToHost));
    if(identity)
    {
        for(size_t i = 0; i < M; ++i)
            for(size_t j = 0; j < N; ++j)
            {
                const float got = hC(i, j), want = hA(i, j);
                if(std::memcmp(&got, &want, sizeof(float)) != 0)
                {
                    std::printf("    identity mismatch at (%zu,%zu): %.9g vs %.9g\n", i, j, got, want);
                    return false;
                }
            }
        return true;
    }
    host_sgemm(hRef, hA, hB, 0, M);
    constexpr float tolerance = 1e-4f;
    for(size_t i = 0; i < M; ++i)
        for(size_t j = 0; j < N; ++j)
            if(!(std::fabs(hC(i, j) - hRef(i, j)) <= tolerance))
            {
                std::printf("    mismatch at (%zu,%zu): %.9g vs %.9g\n", i, j, hC(i, j), hRef(i, j));
                return false;
            }
    return true;
}
// The vendor-wrapper signature served by this library (rocm_sgemm::blas::gemm<TA, TB>): column-major C, the
// transpose flags select how A and B are stored; what the reference's test/rocblas/test.cpp checks for its wrapper.
template<bool TA, bool TB>
bool verify_blas(size_t M, size_t N, size_t K, cudaStream_t stream)
{
    // op(A) = A^T means A is stored K x M column-major, i.e. the M x K operand is row-major
    const layout la = TA ? layout::row_major : layout::col_major, lb = TB ? layout::row_major : layout::col_major;
    host_matrix hA(M, K, la), hB(K, N, lb), hC(M, N, layout::col_major), hRef(M, N, layout::col_major);
    fill_like_reference_test(hA);
    fill_like_reference_test(hB);
    device_buffers d(hA.bytes(), hB.bytes(), hC.bytes());
    CUDA_CHECK(cudaMemcpy(d.A, hA.data(), hA.bytes(), cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemcpy(d.B, hB.data(), hB.bytes(), cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemset(d.C, 0xff, hC.bytes()));
    rocm_sgemm::blas::gemm<TA, TB>(d.C, d.A, d.B, M, N, K, stream);
    CUDA_CHECK(cudaPeekAtLastError());
    CUDA_CHECK(cudaDeviceSynchronize());
    CUDA_CHECK(cudaMemcpy(hC.data(), d.C, hC.bytes(), cudaMemcpyDeviceToHost));
    host_sgemm(hRef, hA, hB, 0, M);
    for(size_t i = 0; i < M; ++i)
        for(size_t j = 0; j < N; ++j)
            if(!(std::fabs(hC(i, j) - hRef(i, j)) <= 1e-4f))
            {
                std::printf("    mismatch at (%zu,%zu): %.9g vs %.9g\n", i, j, hC(i, j), hRef(i, j));
                return false;
            }
    return true;
}

// The vendor wrapper behind the comparison column: cublasSgemm in strict FP32 for layout (la, lb, lc).
bool verify_cublas(int la, int lb, int lc, size_t M, size_t N, size_t K, cudaStream_t stream)
{
    host_matrix hA(M, K, (layout)la), hB(K, N, (layout)lb), hC(M, N, (layout)lc), hRef(M, N, (layout)lc);
    fill_like_reference_test(hA);
    fill_like_reference_test(hB);
    device_buffers d(hA.bytes(), hB.bytes(), hC.bytes());
    CUDA_CHECK(cudaMemcpy(d.A, hA.data(), hA.bytes(), cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemcpy(d.B, hB.data(), hB.bytes(), cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemset(d.C, 0xff, hC.bytes()));
    if(b200_cublas_gemm_layout(lc, la, lb, d.C, d.A, d.B, M, N, K, stream) != 0)
    {
        std::printf("    cublasSgemm returned an error\n");
        return false;
    }
    CUDA_CHECK(cudaDeviceSynchronize());
    CUDA_CHECK(cudaMemcpy(hC.data(), d.C, hC.bytes(), cudaMemcpyDeviceToHost));
    host_sgemm(hRef, hA, hB, 0, M);
    for(size_t i = 0; i < M; ++i)
        for(size_t j = 0; j < N; ++j)
            if(!(std::fabs(hC(i, j) - hRef(i, j)) <= 1e-4f))
            {
                std::printf("    mismatch at (%zu,%zu): %.9g vs %.9g\n", i, j, hC(i, j), hRef(i, j));
                return false;
            }
    return true;
}
} // namespace

int main()
{
    const size_t shapes[][3] = {{128, 128, 128}, {128, 256, 128}, {128, 128, 256}, {256, 128, 128}, {256, 256, 256},
                                {320, 320, 320}, {320, 512, 512}, {512, 320, 320}, {512, 512, 320}, {512, 320, 512},
                                {512, 512, 512}, {1024, 256, 256}, {256, 1024, 256}, {130, 70, 33}, {257, 255, 100}};
    cudaStream_t stream;
    CUDA_CHECK(cudaStreamCreate(&stream));
    int run = 0, failed = 0;
#ifndef HARNESS_VENDOR_ONLY
    for(int la = 0; la < 2; ++la)
        for(int lb = 0; lb < 2; ++lb)
            for(int lc = 0; lc < 2; ++lc)
            {
                for(const auto& s : shapes)
                {
                    const bool ok = verify_gemm(la, lb, lc, s[0], s[1], s[2], stream, false);
                    ++run;
                    failed += !ok;
                    std::printf("[%s] GEMMTest/%s%s%s.Size%zux%zux%zu\n", ok ? "  OK  " : "FAILED", layout_letter((layout)la),
                                layout_letter((layout)lb), layout_letter((layout)lc), s[0], s[1], s[2]);
                }
                const bool ok = verify_gemm(la, lb, lc, 512, 512, 512, stream, true);
                ++run;
                failed += !ok;
                std::printf("[%s] GEMMTest/%s%s%s.IdentityBitExact512\n", ok ? "  OK  " : "FAILED", layout_letter((layout)la),
                            layout_letter((layout)lb), layout_letter((layout)lc));
            }
    const size_t blas_shapes[][3] = {{128, 128, 128}, {320, 512, 512}, {130, 70, 33}, {1024, 256, 256}};
    for(const auto& s : blas_shapes)
    {
        const bool ok[4] = {verify_blas<false, false>(s[0], s[1], s[2], stream), verify_blas<true, false>(s[0], s[1], s[2], stream),
                            verify_blas<false, true>(s[0], s[1], s[2], stream), verify_blas<true, true>(s[0], s[1], s[2], stream)};
        const char* names[4] = {"NN", "TN", "NT", "TT"};
        for(int i = 0; i < 4; ++i)
        {
            ++run;
            failed += !ok[i];
            std::printf("[%s] BlasWrapperTest/%s.Size%zux%zux%zu\n", ok[i] ? "  OK  " : "FAILED", names[i], s[0], s[1], s[2]);
        }
    }
#endif
    if(!b200_cublas_init())
    {
        std::printf("[FAILED] CublasTest: cuBLAS initialisation failed\n");
        ++run;
        ++failed;
    }
    else
    {
        for(int la = 0; la < 2; ++la)
            for(int lb = 0; lb < 2; ++lb)
                for(int lc = 0; lc < 2; ++lc)
                    for(int i = 0; i < 13; ++i) // the reference suite's 13 shapes
                    {
                        const auto& s  = shapes[i];
                        const bool  ok = verify_cublas(la, lb, lc, s[0], s[1], s[2], stream);
                        ++run;
                        failed += !ok;
                        std::printf("[%s] CublasTest/%s%s%s.Size%zux%zux%zu\n", ok ? "  OK  " : "FAILED",
                                    layout_letter((layout)la), layout_letter((layout)lb), layout_letter((layout)lc), s[0],
                                    s[1], s[2]);
                    }
        b200_cublas_cleanup();
    }
    CUDA_CHECK(cudaStreamDestroy(stream));
    std::printf("%d tests, %d failed\n", run, failed);
    return failed == 0 ? 0 : 1;
}
