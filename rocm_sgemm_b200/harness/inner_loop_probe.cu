// inner_loop_probe: how fast can one SM run the SGEMM register-tile update (128-bit shared-memory fragment
// reads + packed fma.rn.f32x2) when nothing else is in the way: no global loads, no barriers, no
// pipeline.  The numbers bound what the real kernels can reach and decided their FMA order, pairing
// direction and thread-tile shape; profiles/inner_loop_probes.md records a run.
//   inner_loop_probe [name filter]
#include <cstdio>
#include <cstdlib>
#include <cstdint>
#include <cstring>
#include <cuda_runtime.h>

__device__ __forceinline__ uint64_t pack2(float lo, float hi) { uint64_t r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r; }
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ void fma2(uint64_t& acc, uint64_t a, uint64_t b) { asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b)); }

// ORDER: 0 i-major, 1 j-major, 2 zigzag(i-major, j alternating direction)
// PAIR:  0 pairs along n (dup a), 1 pairs along m (dup b)
// NOLDS: 1 = fragments loaded once outside the loop (pure register FMA rate)
template<int TMT, int TNT, int ORDER, int PAIR, int NOLDS, int BK, int LN, int MAP, int THREADS>
__global__ void __launch_bounds__(THREADS) probe(float* out, int ntiles)
{
    constexpr int WM = TMT / 4, WN = TNT / 4;
    constexpr int LM = 32 / LN;
    constexpr int SUB_M = 4 * LM, SUB_N = 4 * LN;
    constexpr int WARP_M = WM * SUB_M, WARP_N = WN * SUB_N;
    constexpr int BM = (THREADS / 128) * WARP_M, BN = 4 * WARP_N;
    extern __shared__ __align__(128) float smem[];
    float* As = smem;
    float* Bs = smem + BK * BM;
    for (int i = threadIdx.x; i < BK * (BM + BN); i += THREADS) smem[i] = 1.0f + 1e-6f * i;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int lane_m = MAP == 0 ? lane / LN : lane % LM;
    const int lane_n = MAP == 0 ? lane % LN : lane / LM;
    const int tm0 = (warp / 4) * WARP_M + lane_m * 4;
    const int tn0 = (warp % 4) * WARP_N + lane_n * 4;

    constexpr int NA = PAIR == 0 ? TMT : TMT / 2;   // acc2 rows
    constexpr int NB = PAIR == 0 ? TNT / 2 : TNT;   // acc2 cols
    uint64_t acc2[NA][NB];
#pragma unroll
    for (int i = 0; i < NA; ++i)
#pragma unroll
        for (int j = 0; j < NB; ++j) acc2[i][j] = 0ull;

    float a[2][TMT], b[2][TNT];
    auto load = [&](int buf, int kk) {
#pragma unroll
        for (int im = 0; im < WM; ++im) {
            float4 v = *reinterpret_cast<const float4*>(As + kk * BM + tm0 + im * SUB_M);
            a[buf][im * 4 + 0] = v.x; a[buf][im * 4 + 1] = v.y; a[buf][im * 4 + 2] = v.z; a[buf][im * 4 + 3] = v.w;
        }
#pragma unroll
        for (int in = 0; in < WN; ++in) {
            float4 v = *reinterpret_cast<const float4*>(Bs + kk * BN + tn0 + in * SUB_N);
            b[buf][in * 4 + 0] = v.x; b[buf][in * 4 + 1] = v.y; b[buf][in * 4 + 2] = v.z; b[buf][in * 4 + 3] = v.w;
        }
    };
    auto step = [&](int buf) {
        uint64_t pa[NA], pb[NB];
        if constexpr (PAIR == 0) {
#pragma unroll
            for (int i = 0; i < NA; ++i) pa[i] = pack2(a[buf][i], a[buf][i]);
#pragma unroll
            for (int j = 0; j < NB; ++j) pb[j] = pack2(b[buf][2 * j], b[buf][2 * j + 1]);
        } else {
#pragma unroll
            for (int i = 0; i < NA; ++i) pa[i] = pack2(a[buf][2 * i], a[buf][2 * i + 1]);
#pragma unroll
            for (int j = 0; j < NB; ++j) pb[j] = pack2(b[buf][j], b[buf][j]);
        }
        if constexpr (ORDER == 0) {
#pragma unroll
            for (int i = 0; i < NA; ++i)
#pragma unroll
                for (int j = 0; j < NB; ++j) fma2(acc2[i][j], pa[i], pb[j]);
        } else if constexpr (ORDER == 1) {
#pragma unroll
            for (int j = 0; j < NB; ++j)
#pragma unroll
                for (int i = 0; i < NA; ++i) fma2(acc2[i][j], pa[i], pb[j]);
        } else {
#pragma unroll
            for (int i = 0; i < NA; ++i)
#pragma unroll
                for (int jj = 0; jj < NB; ++jj) { const int j = (i & 1) ? NB - 1 - jj : jj; fma2(acc2[i][j], pa[i], pb[j]); }
        }
    };

    if constexpr (NOLDS) { load(0, 0); load(1, 1); }
    for (int t = 0; t < ntiles; ++t) {
        if constexpr (!NOLDS) {
            asm volatile("" ::: "memory");
            load(0, 0);
        }
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            if constexpr (!NOLDS) { if (kk + 1 < BK) load((kk + 1) & 1, kk + 1); }
            step(kk & 1);
        }
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NA; ++i)
#pragma unroll
        for (int j = 0; j < NB; ++j) { float lo, hi; unpack2(acc2[i][j], lo, hi); s += lo + hi; }
    if (s == 12345.678f) out[threadIdx.x] = s;
}

template<int TMT, int TNT, int ORDER, int PAIR, int NOLDS, int LN = 8, int MAP = 0, int THREADS = 256, int CTAS = 1>
void run(const char* name, const char* filter, float* out)
{
    if (!strstr(name, filter)) return;
    constexpr int BK = 16;
    int dev = 0; cudaDeviceProp prop; cudaGetDeviceProperties(&prop, dev);
    const int ntiles = 4096;
    constexpr int BM = (THREADS / 128) * (TMT / 4) * 4 * (32 / LN), BN = 4 * (TNT / 4) * 4 * LN;
    size_t smem = (size_t)BK * (BM + BN) * 4;
    auto k = probe<TMT, TNT, ORDER, PAIR, NOLDS, BK, LN, MAP, THREADS>;
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncAttributes attr; cudaFuncGetAttributes(&attr, k);
    int grid = prop.multiProcessorCount * CTAS;
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    k<<<grid, THREADS, smem>>>(out, 64);
    float best = 1e30f;
    for (int r = 0; r < 3; ++r) {
        cudaEventRecord(e0); k<<<grid, THREADS, smem>>>(out, ntiles); cudaEventRecord(e1); cudaEventSynchronize(e1);
        float ms; cudaEventElapsedTime(&ms, e0, e1); if (ms < best) best = ms;
    }
    cudaError_t err = cudaGetLastError();
    double flops = 2.0 * TMT * TNT * BK * (double)ntiles * THREADS * grid;
    printf("%-34s regs=%3d  %.3f ms  %.2f TFLOP/s  %s\n", name, attr.numRegs, best, flops / best / 1e9,
           err == cudaSuccess ? "" : cudaGetErrorString(err));
}

int main(int argc, char** argv)
{
    float* out;
    cudaMalloc(&out, 4096);
    const char* f = argc > 1 ? argv[1] : "";
    //  rows, cols per thread | order | pair dir | no LDS | lanes along n | lane map | threads | CTAs per SM
    run<8, 8, 0, 0, 0, 8, 0, 256, 1>("8x8 dup-outer order, pairs along n", f, out);
    run<8, 8, 1, 0, 0, 8, 0, 256, 1>("8x8 pair-outer order, pairs along n", f, out);
    run<8, 8, 0, 1, 0, 8, 0, 256, 1>("8x8 pair-outer order, pairs along m", f, out);
    run<8, 8, 1, 1, 0, 8, 0, 256, 1>("8x8 dup-outer order, pairs along m", f, out);
    run<8, 8, 0, 0, 1, 8, 0, 256, 1>("8x8 dup-outer order, registers only", f, out);
    run<8, 8, 1, 0, 1, 8, 0, 256, 1>("8x8 pair-outer order, registers only", f, out);
    run<8, 8, 1, 0, 0, 4, 0, 256, 1>("8x8 pair-outer, 8x4 lanes", f, out);
    run<8, 8, 1, 0, 0, 16, 0, 256, 1>("8x8 pair-outer, 2x16 lanes", f, out);
    run<8, 8, 1, 0, 0, 8, 0, 128, 2>("8x8 pair-outer, 128 thr x2 CTAs", f, out);
    run<8, 8, 1, 0, 0, 8, 0, 384, 1>("8x8 pair-outer, 384 thr (3 warps/scheduler)", f, out);
    run<8, 8, 1, 0, 0, 8, 0, 512, 1>("8x8 pair-outer, 512 thr (4 warps/scheduler)", f, out);
    run<8, 8, 1, 1, 0, 8, 0, 512, 1>("8x8 pairs along m, 512 thr", f, out);
    run<16, 8, 1, 0, 0, 8, 0, 256, 1>("16x8 pair-outer, 256 thr", f, out);
    run<16, 8, 1, 0, 0, 8, 0, 128, 1>("16x8 pair-outer, 128 thr x1 CTA", f, out);
    run<16, 8, 1, 0, 0, 8, 0, 128, 2>("16x8 pair-outer, 128 thr x2 CTAs", f, out);
    run<8, 16, 1, 0, 0, 8, 0, 256, 1>("8x16 pair-outer, 256 thr", f, out);
    return 0;
}
