// gemm_bench: the reference's benchmark on the drop-in header, with the vendor column beside it.
//
// Follows benchmark/gemm/bench.cpp:31-114 (per-launch event timing on the call's stream, FLOPs =
// 2*M*N*K, avg TFLOPS = mean of per-launch TFLOPS, min / max milliseconds, bytes = 4*(MK+KN+MN)) and
// :125-228 (--shapes "M,N,K:M,N,K" or "M:..." for cubes, --batch_count).  In the slot of the
// reference's rocBLAS benchmark (benchmark/rocblas/bench.cpp) the same table row carries cublasSgemm in
// strict FP32 mode for the same layout.  Extra switches: --layouts rrr,crc,... (default all eight),
// --iters / --warmup (fixed launch counts instead of Google Benchmark's adaptive count), --identity (B =
// identity and a bit-exact check of C == A: the identity-multiply methodology), --cpu ROWS (time the
// host verification GEMM on ROWS rows and print its GFLOP/s and thread count), --json (one JSON object
// per row on stdout), --vendor-only (time cublasSgemm alone: the rows of the reference's
// benchmark/rocblas/bench.cpp:43-123; the default of the `cublas_bench` build, -DHARNESS_VENDOR_ONLY).
#include "harness.hpp"

#include <b200_cublas_wrapper.h>
#include <rocm_sgemm/gemm.hpp>

#include <algorithm>
#include <chrono>
#include <cstring>
#include <limits>
#include <sstream>
#include <string>
#include <tuple>
#ifdef _OPENMP
#include <omp.h>
#endif

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
// index = A*4 + B*2 + C
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

struct options
{
    std::vector<std::tuple<size_t, size_t, size_t>> shapes{{1024, 1024, 1024}, {2048, 2048, 2048}, {4096, 4096, 4096},
                                                           {8192, 8192, 8192}};
    std::vector<int> layouts{7, 3, 5, 1, 6, 2, 4, 0}; // the reference's registration order: ccc rcc crc rrc ccr rcr crr rrr
    int    batch_count = 1;
    int    iters = 100, warmup = 10;
    bool   identity = false, json = false, vendor = true, tf32x3 = false;
#ifdef HARNESS_VENDOR_ONLY
    bool   vendor_only = true;
#else
    bool   vendor_only = false;
#endif
    size_t cpu_rows = 0;
};

std::vector<std::tuple<size_t, size_t, size_t>> parse_shapes(const std::string& text)
{
    std::vector<std::tuple<size_t, size_t, size_t>> out;
    std::stringstream                               ss(text);
    std::string                                     tok;
    while(std::getline(ss, tok, ':'))
    {
        std::vector<size_t> dims;
        std::stringstream   ds(tok);
        std::string         d;
        while(std::getline(ds, d, ','))
            if(!d.empty())
                dims.push_back(std::stoul(d));
        if(dims.size() == 1)
            out.emplace_back(dims[0], dims[0], dims[0]);
        else if(dims.size() == 3)
            out.emplace_back(dims[0], dims[1], dims[2]);
        else
            std::fprintf(stderr, "Warning: invalid shape '%s' (expected 'M' or 'M,N,K')\n", tok.c_str());
    }
    return out;
}

std::vector<int> parse_layouts(const std::string& text)
{
    std::vector<int>  out;
    std::stringstream ss(text);
    std::string       tok;
    while(std::getline(ss, tok, ','))
    {
        if(tok.size() != 3)
            continue;
        int idx = 0;
        for(char ch : tok)
            idx = idx * 2 + (ch == 'c' ? 1 : 0);
        out.push_back(idx);
    }
    return out;
}

void usage(const char* prog)
{
    std::printf("Usage: %s [options]\n"
                "  --shapes <list>     colon-separated shapes, 'M,N,K' or 'M' (default 1024:2048:4096:8192)\n"
                "  --layouts <list>    comma-separated A,B,C layouts such as rrr,crc (default: all eight)\n"
                "  --batch_count <n>   n independent products per timed call (b200_sgemm_strided_batched; the reference only\n"
                "                      replicates its buffers, benchmark/gemm/bench.cpp:49-64)\n"
                "  --iters <n>         timed launches per row (default 100)   --warmup <n> (default 10)\n"
                "  --identity          B = identity, verify C == A bit for bit\n"
                "  --cpu <rows>        also time the host GEMM on <rows> rows of C\n"
                "  --no-vendor         skip the cuBLAS column      --json   machine-readable rows\n"
                "  --vendor-only       time cublasSgemm alone (what cublas_bench does by default)\n"
                "  --tf32x3            also time the optional 3xTF32 tensor-core entry (its own column)\n",
                prog);
}

struct stats
{
    double avg_tflops = 0, min_ms = 0, max_ms = 0, avg_ms = 0;
};

template<class F>
stats time_launches(F&& launch, cudaStream_t stream, double flops, int warmup, int iters)
{
    for(int i = 0; i < warmup; ++i)
        launch();
    CUDA_CHECK(cudaStreamSynchronize(stream));
    gpu_timer timer;
    stats     s;
    s.min_ms     = std::numeric_limits<double>::max();
    double total = 0;
    for(int i = 0; i < iters; ++i)
    {
        timer.start(stream);
        launch();
        CUDA_CHECK(cudaPeekAtLastError());
        const double ms = timer.stop(stream);
        s.min_ms        = std::min(s.min_ms, ms);
        s.max_ms        = std::max(s.max_ms, ms);
        total += ms;
        s.avg_tflops += flops / (ms * 1e-3) * 1e-12;
    }
    s.avg_tflops /= iters;
    s.avg_ms = total / iters;
    return s;
}
} // namespace

int main(int argc, char** argv)
{
    options opt;
    for(int i = 1; i < argc; ++i)
    {
        const std::string a = argv[i];
        auto              next = [&]() -> const char* { return i + 1 < argc ? argv[++i] : ""; };
        if(a == "--shapes") opt.shapes = parse_shapes(next());
        else if(a == "--layouts") opt.layouts = parse_layouts(next());
        else if(a == "--batch_count") opt.batch_count = std::stoi(next());
        else if(a == "--iters") opt.iters = std::stoi(next());
        else if(a == "--warmup") opt.warmup = std::stoi(next());
        else if(a == "--identity") opt.identity = true;
        else if(a == "--cpu") opt.cpu_rows = std::stoul(next());
        else if(a == "--json") opt.json = true;
        else if(a == "--no-vendor") opt.vendor = false;
        else if(a == "--vendor-only") opt.vendor_only = true;
        else if(a == "--tf32x3") opt.tf32x3 = true;
        else if(a == "--help") { usage(argv[0]); return 0; }
        else std::fprintf(stderr, "ignoring unknown argument %s\n", a.c_str());
    }

    int            device = 0;
    cudaDeviceProp prop;
    CUDA_CHECK(cudaGetDevice(&device));
    CUDA_CHECK(cudaGetDeviceProperties(&prop, device));
    int clock_khz = 0;
    CUDA_CHECK(cudaDeviceGetAttribute(&clock_khz, cudaDevAttrClockRate, device));
    // FP32 non-tensor peak: SMs x 128 lanes x 2 flops x clock
    const double peak_tflops = prop.multiProcessorCount * 128.0 * 2.0 * clock_khz * 1e3 * 1e-12;
    if(opt.vendor_only)
        opt.vendor = true;
    if(opt.vendor && !b200_cublas_init())
    {
        std::fprintf(stderr, "cuBLAS initialisation failed; vendor column disabled\n");
        if(opt.vendor_only)
            return 1;
        opt.vendor = false;
    }
    if(!opt.json)
    {
        std::printf("device: %s, %d SMs, %.0f MHz, FP32 peak %.2f TFLOP/s\n", prop.name, prop.multiProcessorCount,
                    clock_khz * 1e-3, peak_tflops);
        std::printf("%-44s %10s %10s %10s %11s %8s %12s %9s%s\n", "benchmark", "avg_ms", "min_ms", "max_ms", "avg_tflops",
                    "%peak", "cublas_tflops", "vs_cublas", opt.tf32x3 ? " tf32x3_tflops" : "");
    }

    cudaStream_t stream;
    CUDA_CHECK(cudaStreamCreate(&stream));
    int failures = 0;
    for(const auto& shape : opt.shapes)
    {
        const size_t M = std::get<0>(shape), N = std::get<1>(shape), K = std::get<2>(shape);
        for(int idx : opt.layouts)
        {
            const int   la = (idx >> 2) & 1, lb = (idx >> 1) & 1, lc = idx & 1;
            host_matrix hA(M, K, (layout)la), hB(K, N, (layout)lb), hC(M, N, (layout)lc);
            if(opt.identity)
            {
                std::mt19937 gen(1);
                fill_uniform(hA, gen);
                fill_identity(hB);
            }
            else
            {
                fill_pattern(hA);
                fill_pattern(hB);
            }
            const size_t bc = (size_t)opt.batch_count;
            float *      dA, *dB, *dC;
            CUDA_CHECK(cudaMalloc(&dA, hA.bytes() * bc));
            CUDA_CHECK(cudaMalloc(&dB, hB.bytes() * bc));
            CUDA_CHECK(cudaMalloc(&dC, hC.bytes() * bc));
            for(size_t b = 0; b < bc; ++b)
            {
                CUDA_CHECK(cudaMemcpy(dA + b * hA.size(), hA.data(), hA.bytes(), cudaMemcpyHostToDevice));
                CUDA_CHECK(cudaMemcpy(dB + b * hB.size(), hB.data(), hB.bytes(), cudaMemcpyHostToDevice));
            }
            const double flops = 2.0 * M * N * K * bc;
            const stats  ours  = time_launches(
                [&] {
                    if(opt.vendor_only)
                    {
                        for(size_t b = 0; b < bc; ++b)
                            b200_cublas_gemm_layout(lc, la, lb, dC + b * M * N, dA + b * M * K, dB + b * K * N, M, N, K, stream);
                    }
                    else if(bc == 1)
                        table[idx](dC, dA, dB, M, N, K, stream);
                    else if(b200_sgemm_strided_batched(lc, la, lb, dC, dA, dB, M, N, K, M * N, M * K, K * N, bc, stream)
                            != B200_SGEMM_OK)
                        throw std::runtime_error("b200_sgemm_strided_batched failed");
                },
                stream, flops, opt.warmup, opt.iters);
            bool exact = true;
            if(opt.identity)
            {
                CUDA_CHECK(cudaMemcpy(hC.data(), dC, hC.bytes(), cudaMemcpyDeviceToHost));
                for(size_t i = 0; i < M && exact; ++i)
                    for(size_t j = 0; j < N; ++j)
                    {
                        const float g = hC(i, j), w = hA(i, j);
                        if(std::memcmp(&g, &w, sizeof(float)) != 0)
                        {
                            exact = false;
                            break;
                        }
                    }
                failures += !exact;
            }
            stats vendor;
            if(opt.vendor_only)
                vendor = ours;
            else if(opt.vendor)
                vendor = time_launches(
                    [&] {
                        for(size_t b = 0; b < bc; ++b)
                            b200_cublas_gemm_layout(lc, la, lb, dC + b * M * N, dA + b * M * K, dB + b * K * N, M, N, K, stream);
                    },
                    stream, flops, opt.warmup, opt.iters);
            stats tensor; // the optional 3xTF32 tensor-core entry: its own column, not the graded arithmetic
            if(opt.tf32x3 && !opt.vendor_only)
                tensor = time_launches(
                    [&] {
                        for(size_t b = 0; b < bc; ++b)
                            b200_sgemm_3xtf32(lc, la, lb, dC + b * M * N, dA + b * M * K, dB + b * K * N, M, N, K, stream);
                    },
                    stream, flops, opt.warmup, opt.iters);
            char name[96];
            std::snprintf(name, sizeof name, "{A:%s,B:%s,C:%s,m:%zu,n:%zu,k:%zu}", layout_letter((layout)la),
                          layout_letter((layout)lb), layout_letter((layout)lc), M, N, K);
            const double bytes_per_s = (double)(M * K + K * N + M * N) * sizeof(float) / (ours.avg_ms * 1e-3);
            if(opt.json)
                std::printf("{\"name\":\"%s\",\"M\":%zu,\"N\":%zu,\"K\":%zu,\"layout\":\"%s%s%s\",\"avg_ms\":%.5f,"
                            "\"min_ms\":%.5f,\"max_ms\":%.5f,\"avg_tflops\":%.3f,\"min_time_tflops\":%.3f,"
                            "\"pct_fp32_peak\":%.2f,\"bytes_per_second\":%.4g,\"cublas_avg_tflops\":%.3f,"
                            "\"cublas_min_ms\":%.5f,\"tf32x3_avg_tflops\":%.3f,\"identity_exact\":%s}\n",
                            name, M, N, K, layout_letter((layout)la), layout_letter((layout)lb), layout_letter((layout)lc),
                            ours.avg_ms, ours.min_ms, ours.max_ms, ours.avg_tflops, flops / (ours.min_ms * 1e-3) * 1e-12,
                            100.0 * ours.avg_tflops / peak_tflops, bytes_per_s, vendor.avg_tflops, vendor.min_ms,
                            tensor.avg_tflops, opt.identity ? (exact ? "true" : "false") : "null");
            else
            {
                std::printf("%-44s %10.4f %10.4f %10.4f %11.2f %7.1f%% %12.2f %8.3fx", name, ours.avg_ms, ours.min_ms,
                            ours.max_ms, ours.avg_tflops, 100.0 * ours.avg_tflops / peak_tflops, vendor.avg_tflops,
                            vendor.avg_tflops > 0 ? ours.avg_tflops / vendor.avg_tflops : 0.0);
                if(opt.tf32x3)
                    std::printf(" %13.2f", tensor.avg_tflops);
                std::printf("%s\n", opt.identity ? (exact ? "  C==A" : "  C!=A (FAILED)") : "");
            }
            std::fflush(stdout);
            CUDA_CHECK(cudaFree(dA));
            CUDA_CHECK(cudaFree(dB));
            CUDA_CHECK(cudaFree(dC));

            if(opt.cpu_rows > 0 && idx == opt.layouts.front())
            {
                // the host verification GEMM on a band of rows of the same problem
                const size_t rows = std::min(opt.cpu_rows, M);
                host_matrix  hRef(M, N, (layout)lc);
                const auto   t0 = std::chrono::steady_clock::now();
                host_sgemm(hRef, hA, hB, 0, rows);
                const double sec = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
                int          threads = 1;
#ifdef _OPENMP
                threads = omp_get_max_threads();
#endif
                std::printf("  host GEMM: %zu rows of %zux%zux%zu in %.3f s on %d thread(s): %.2f GFLOP/s "
                            "(full problem ~%.1f s, sampled)\n",
                            rows, M, N, K, sec, threads, 2.0 * rows * N * K / sec * 1e-9, sec * M / rows);
            }
        }
    }
    if(opt.vendor)
        b200_cublas_cleanup();
    CUDA_CHECK(cudaStreamDestroy(stream));
    return failures == 0 ? 0 : 1;
}
