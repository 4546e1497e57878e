// tuner: times ONE kernel configuration on ONE problem and prints the result for tune.py to parse.
//
// The counterpart of the reference's one-trial executable (rocm_sgemm/config/tuner.cpp:183-512): there,
// each trial JIT-compiles one kernel_gemm instantiation with hipRTC and times it with events under
// Google Benchmark's manual-time loop; the Python driver starts one process per trial so that a bad
// configuration cannot take the search down.  Here the candidate kernels are compiled by nvcc into a
// candidate build of the library (tune.py does that, a batch at a time, through
// rocm_sgemm_b200/build.py) and this program loads that build, finds the variant whose parameters match
// the command line and times it through b200_sgemm_trial: the drop-in entry's own path (arena scratch,
// pre-transposition, split-K or the balanced schedules) with the candidate standing in for the table entry, so
// that every property of an entry is searched through the code that will use it.  (The reference's tuner launches
// its JIT-compiled kernel directly, tuner.cpp:419-429; its table entries have no property beyond the kernel.)
//
//   tuner <library.so> M N K  <14 variant parameters>  split_k pretranspose  layout_A layout_B layout_C  [iters] [warmup]
//
// Inputs are the reference benchmark's cyclic five-value pattern (tuner.cpp:105-120).  Output, one line:
//   manual_time <mean ms> ms min <min ms> ms tflops <avg TFLOP/s>
// Exit code 2 = the variant is not in the library / no kernel for the layout, 3 = CUDA error.
#include "../../include/b200_sgemm.h"

#include <cuda_runtime.h>
#include <dlfcn.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#define CHECK(call)                                                                       \
    do                                                                                    \
    {                                                                                     \
        cudaError_t e_ = (call);                                                          \
        if(e_ != cudaSuccess)                                                             \
        {                                                                                 \
            std::fprintf(stderr, "CUDA error %d (%s) in %s\n", (int)e_, cudaGetErrorString(e_), #call); \
            return 3;                                                                     \
        }                                                                                 \
    } while(0)

namespace
{
void fill_pattern(std::vector<float>& v)
{
    static const float p[5] = {1.025f, 1.05f, 1.075f, 1.1f, 1.0f};
    for(size_t i = 0; i < v.size(); ++i)
        v[i] = p[i % 5];
}
template<class F>
F sym(void* lib, const char* name)
{
    void* p = dlsym(lib, name);
    if(!p)
    {
        std::fprintf(stderr, "symbol %s missing from the library\n", name);
        std::exit(2);
    }
    return reinterpret_cast<F>(p);
}
} // namespace

int main(int argc, char** argv)
{
    if(argc < 24)
    {
        std::fprintf(stderr, "usage: %s <library.so> M N K <14 variant parameters> split_k pretranspose layout_A layout_B "
                             "layout_C [iters] [warmup]\n", argv[0]);
        return 1;
    }
    void* lib = dlopen(argv[1], RTLD_NOW | RTLD_LOCAL);
    if(!lib)
    {
        std::fprintf(stderr, "cannot load %s: %s\n", argv[1], dlerror());
        return 2;
    }
    const size_t M = std::strtoull(argv[2], nullptr, 10), N = std::strtoull(argv[3], nullptr, 10),
                 K = std::strtoull(argv[4], nullptr, 10);
    int want[14];
    for(int i = 0; i < 14; ++i)
        want[i] = std::atoi(argv[5 + i]);
    const int split_k = std::atoi(argv[19]), pretranspose = std::atoi(argv[20]);
    const int la = std::atoi(argv[21]), lb = std::atoi(argv[22]), lc = std::atoi(argv[23]);
    const int iters = argc > 24 ? std::atoi(argv[24]) : 20, warmup = argc > 25 ? std::atoi(argv[25]) : 3;

    auto num_variants = sym<int (*)(void)>(lib, "b200_sgemm_num_variants");
    auto get_variant  = sym<int (*)(int, b200_sgemm_params*)>(lib, "b200_sgemm_get_variant");
    auto has_kernel   = sym<int (*)(int, int, int)>(lib, "b200_sgemm_has_kernel");
    auto gemm_trial   = sym<int (*)(int, int, int, float*, const float*, const float*, size_t, size_t, size_t, int, int, int,
                                    void*)>(lib, "b200_sgemm_trial");
    auto status_str   = sym<const char* (*)(int)>(lib, "b200_sgemm_status_string");

    int variant = -1;
    for(int v = 0; v < num_variants() && variant < 0; ++v)
    {
        b200_sgemm_params p;
        get_variant(v, &p);
        const int have[14] = {p.block_size, p.block_m, p.block_n, p.block_k, p.warp_tile_m_count, p.warp_tile_n_count,
                              p.thread_tile_m, p.thread_tile_n, p.threads_n, p.stages, p.fma_mode, p.raster,
                              p.min_blocks, p.pipeline};
        if(std::equal(have, have + 14, want))
            variant = v;
    }
    if(variant < 0 || !has_kernel(variant, la * 4 + lb * 2 + lc, 0))
    {
        std::fprintf(stderr, "variant not built for this layout\n");
        return 2;
    }

    std::vector<float> hA(M * K), hB(K * N);
    fill_pattern(hA);
    fill_pattern(hB);
    float *dA, *dB, *dC;
    CHECK(cudaMalloc(&dA, hA.size() * sizeof(float)));
    CHECK(cudaMalloc(&dB, hB.size() * sizeof(float)));
    CHECK(cudaMalloc(&dC, M * N * sizeof(float)));
    CHECK(cudaMemcpy(dA, hA.data(), hA.size() * sizeof(float), cudaMemcpyHostToDevice));
    CHECK(cudaMemcpy(dB, hB.data(), hB.size() * sizeof(float), cudaMemcpyHostToDevice));
    cudaStream_t stream;
    CHECK(cudaStreamCreate(&stream));
    cudaEvent_t e0, e1;
    CHECK(cudaEventCreate(&e0));
    CHECK(cudaEventCreate(&e1));

    double total = 0, best = 1e30;
    for(int i = 0; i < warmup + iters; ++i)
    {
        CHECK(cudaEventRecord(e0, stream));
        // the path of the drop-in entry with this candidate as the table entry: arena scratch, pre-transposition,
        // split-K or the balanced schedules
        const int st = gemm_trial(lc, la, lb, dC, dA, dB, M, N, K, variant, split_k, pretranspose, stream);
        if(st != 0)
        {
            std::fprintf(stderr, "b200_sgemm_trial: %s\n", status_str(st));
            return st > 0 ? 3 : 2;
        }
        CHECK(cudaEventRecord(e1, stream));
        CHECK(cudaEventSynchronize(e1));
        float ms = 0.f;
        CHECK(cudaEventElapsedTime(&ms, e0, e1));
        if(i >= warmup)
        {
            total += ms;
            best = std::min(best, (double)ms);
        }
    }
    CHECK(cudaDeviceSynchronize());
    const double mean = total / iters;
    std::printf("manual_time %.6f ms min %.6f ms tflops %.3f\n", mean, best, 2.0 * M * N * K / (mean * 1e-3) * 1e-12);
    return 0;
}
