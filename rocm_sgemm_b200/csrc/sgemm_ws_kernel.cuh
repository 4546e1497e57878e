// Warp-specialised, persistent FP32 GEMM kernel for sm_100a (pipeline = 1 variants).
//
// Same arithmetic and the same [k][m] / [k][n] shared-memory tiles as sgemm_kernel.cuh, but the roles
// the reference's kernel gives to halves of one thread block (the lower half stages B, the upper half
// stages A, everybody computes: rocm_sgemm/include/rocm_sgemm/kernel/kernel.hpp:147-199,272-293) are
// split between dedicated warps that never meet at a block-wide barrier:
//
//   * CONSUMER warps (block_size/32 of them) only read fragments from shared memory and issue packed
//     FP32 FMAs.  They wait on a per-stage "full" mbarrier and release the stage through an "empty"
//     mbarrier, so a warp that is ahead is never held back by the others.
//   * PRODUCER warps (one warpgroup) fill the ring.  An operand whose non-K dimension is contiguous in
//     global memory (A col-major, B row-major) is fetched by ONE thread with a TMA tile copy
//     (cp.async.bulk.tensor.2d, out-of-bounds elements zero-filled by the hardware) that signals the
//     stage's mbarrier by byte count; a K-contiguous operand (A row-major, B col-major) is fetched with
//     128-bit loads and transposed into the tile with conflict-free swizzled stores by the producer
//     threads, off the consumers' critical path.  Operands that do not meet TMA's alignment rules fall
//     back to guarded loads in the same warps.
//   * the CTA is persistent: it walks work units (tile, K-slice) blockIdx.x, +gridDim.x, ... and the
//     producers run ahead into the next unit while the consumers store C.
//
// Every wait on an mbarrier is bounded: after SPIN_LIMIT failed polls the thread records an error in
// *status, raises the CTA's abort flag and leaves; nobody waits forever on a peer that bailed out.
#pragma once
#include "sgemm_kernel.cuh"
#include <cuda.h>

namespace sgemm_b200
{

constexpr int      WS_PRODUCER_THREADS = 128;
constexpr uint32_t WS_SPIN_LIMIT       = 1u << 20;

// status word values written by the kernel (0 = ok)
constexpr int WS_ERR_FULL_TIMEOUT  = 1; // a consumer gave up waiting for a stage to fill
constexpr int WS_ERR_EMPTY_TIMEOUT = 2; // a producer gave up waiting for a stage to drain

struct WsArgs
{
    GemmArgs g;
    int      total_units;  // tiles * splits
    int      tma_a, tma_b; // 1: the operand is fetched by TMA through the tensor map below
    int*     status;       // device status word
};

// ---- mbarrier / TMA helpers ------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return ok != 0;
}
// bounded wait: false when the phase did not complete within WS_SPIN_LIMIT polls
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity)
{
    for(uint32_t i = 0; i < WS_SPIN_LIMIT; ++i)
        if(mbar_try_wait(bar, parity))
            return true;
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}

template<class Cfg>
struct WsLayout
{
    static constexpr int    STAGE_FLOATS = (Cfg::BM + Cfg::BN) * Cfg::BK;
    static constexpr size_t TILE_BYTES   = size_t(Cfg::STAGES) * STAGE_FLOATS * sizeof(float);
    // after the tiles: full[STAGES], empty[STAGES] (8 bytes each), abort flag
    static constexpr size_t SMEM_BYTES = TILE_BYTES + size_t(2 * Cfg::STAGES) * 8 + 16;
    static constexpr int    THREADS    = Cfg::BLOCK_SIZE + WS_PRODUCER_THREADS;
};

template<class Cfg, int LA, int LB, int LC, bool ALIGNED>
__global__ void __launch_bounds__(WsLayout<Cfg>::THREADS, 1)
    sgemm_ws_kernel(const __grid_constant__ WsArgs w, const __grid_constant__ CUtensorMap map_a,
                    const __grid_constant__ CUtensorMap map_b)
{
    constexpr int  BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, STAGES = Cfg::STAGES;
    constexpr int  TM = Cfg::TM, TN = Cfg::TN, TMT = Cfg::TMT, TNT = Cfg::TNT;
    constexpr int  MODE     = Cfg::FMA_MODE;
    constexpr bool A_KMAJOR = (LA == LAYOUT_ROW);
    constexpr bool B_KMAJOR = (LB == LAYOUT_COL);
    constexpr int  CONSUMER_WARPS = Cfg::BLOCK_SIZE / 32;
    using SwzA                    = Swizzle<BM, BK>;
    using SwzB                    = Swizzle<BN, BK>;
    using L                       = WsLayout<Cfg>;
    static_assert(MODE != FMA_SCALAR || true, "");

    extern __shared__ __align__(128) float smem[];
    const GemmArgs& p = w.g;

    const uint32_t bar_base = smem_u32(smem) + (uint32_t)L::TILE_BYTES;
    auto           full_bar  = [&](int s) -> uint32_t { return bar_base + 8u * s; };
    auto           empty_bar = [&](int s) -> uint32_t { return bar_base + 8u * (STAGES + s); };
    volatile int*  abort_flag = reinterpret_cast<volatile int*>(reinterpret_cast<char*>(smem) + L::TILE_BYTES
                                                               + 2 * STAGES * 8);
    auto tile_a = [&](int s) -> float* { return smem + s * L::STAGE_FLOATS; };
    auto tile_b = [&](int s) -> float* { return smem + s * L::STAGE_FLOATS + BM * BK; };

    const int tid = threadIdx.x;
    if(tid == 0)
    {
        for(int s = 0; s < STAGES; ++s)
        {
            mbar_init(full_bar(s), WS_PRODUCER_THREADS + 1);
            mbar_init(empty_bar(s), CONSUMER_WARPS);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads(); // the only block-wide barrier: everything below is role-local

    const int tiles = p.grid_m * p.grid_n;

    if(tid >= Cfg::BLOCK_SIZE)
    {
        // =========================== PRODUCERS ==========================================================
        const int      ptid     = tid - Cfg::BLOCK_SIZE;
        const uint32_t tx_bytes = (w.tma_a ? BM * BK * 4u : 0u) + (w.tma_b ? BN * BK * 4u : 0u);
        OperandStager<WS_PRODUCER_THREADS, BM, BK, A_KMAJOR, ALIGNED> stage_a;
        OperandStager<WS_PRODUCER_THREADS, BN, BK, B_KMAJOR, ALIGNED> stage_b;
        uint32_t it = 0; // k-tiles issued by this CTA so far (ring position)
        for(int unit = blockIdx.x; unit < w.total_units; unit += gridDim.x)
        {
            const int split   = unit / tiles;
            const int tile_id = unit - split * tiles;
            int       tile_m, tile_n;
            map_tile<Cfg::RASTER>(tile_id, p.grid_m, p.grid_n, tile_m, tile_n);
            const int m0 = tile_m * BM, n0 = tile_n * BN;
            const int k_begin = split * p.k_per_split;
            const int k_end   = min(p.K, k_begin + p.k_per_split);
            const int ntiles  = (k_end - k_begin + BK - 1) / BK;
            for(int t = 0; t < ntiles; ++t, ++it)
            {
                const int      s      = it % STAGES;
                const uint32_t parity = ((it / STAGES) & 1u) ^ 1u; // first lap passes immediately
                if(*abort_flag || !mbar_wait(empty_bar(s), parity))
                {
                    if(!*abort_flag)
                    {
                        *abort_flag = 1;
                        atomicCAS(w.status, 0, WS_ERR_EMPTY_TIMEOUT);
                    }
                    __nanosleep(200000); // let copies already in flight land before the CTA retires
                    return;
                }
                const int k0 = k_begin + t * BK;
                if(ptid == 0)
                {
                    if(tx_bytes)
                    {
                        mbar_arrive_expect_tx(full_bar(s), tx_bytes);
                        // tile origin: x is a multiple of 32 elements, so the 16-byte start rule of TMA holds
                        if(w.tma_a)
                            tma_load_2d(smem_u32(tile_a(s)), &map_a, m0, k0, full_bar(s));
                        if(w.tma_b)
                            tma_load_2d(smem_u32(tile_b(s)), &map_b, n0, k0, full_bar(s));
                    }
                    else
                    {
                        mbar_arrive(full_bar(s));
                    }
                }
                if(!w.tma_a)
                    stage_a.fetch(p.A, p.lda, p.M, m0, k0, k_end, p.vec_a, tile_a(s), ptid);
                if(!w.tma_b)
                    stage_b.fetch(p.B, p.ldb, p.N, n0, k0, k_end, p.vec_b, tile_b(s), ptid);
                if(!w.tma_a)
                    stage_a.commit(tile_a(s), ptid);
                if(!w.tma_b)
                    stage_b.commit(tile_b(s), ptid);
                if((!A_KMAJOR && !w.tma_a) || (!B_KMAJOR && !w.tma_b))
                {
                    cp_async_commit();
                    cp_async_wait<0>(); // fallback path of an unaligned M/N-contiguous operand
                }
                mbar_arrive(full_bar(s)); // release: this thread's stores to the stage are done
            }
        }
        return;
    }

    // =============================== CONSUMERS ==========================================================
    const int warp_id  = tid >> 5;
    const int lane     = tid & 31;
    const int warp_row = warp_id / Cfg::WARPS_N;
    const int warp_col = warp_id % Cfg::WARPS_N;
    const int lane_m   = lane / Cfg::THREADS_N;
    const int lane_n   = lane % Cfg::THREADS_N;
    const int tm0      = warp_row * Cfg::WARP_M + lane_m * TM;
    const int tn0      = warp_col * Cfg::WARP_N + lane_n * TN;

    float a_frag[2][TMT];
    float b_frag[2][TNT];

    auto load_frags = [&](int buf, const float* as, const float* bs, int kk) {
        const int xa = A_KMAJOR ? SwzA::of_chunk(kk >> 2) : 0;
        const int xb = B_KMAJOR ? SwzB::of_chunk(kk >> 2) : 0;
#pragma unroll
        for(int im = 0; im < Cfg::WM_CNT; ++im)
        {
            const float* src = as + kk * BM + ((tm0 + im * Cfg::SUB_M) ^ xa);
#pragma unroll
            for(int v = 0; v < TM / 4; ++v)
            {
                const float4 q = *reinterpret_cast<const float4*>(src + 4 * v);
                float*       d = &a_frag[buf][im * TM + 4 * v];
                d[0] = q.x; d[1] = q.y; d[2] = q.z; d[3] = q.w;
            }
        }
#pragma unroll
        for(int in = 0; in < Cfg::WN_CNT; ++in)
        {
            const float* src = bs + kk * BN + ((tn0 + in * Cfg::SUB_N) ^ xb);
#pragma unroll
            for(int v = 0; v < TN / 4; ++v)
            {
                const float4 q = *reinterpret_cast<const float4*>(src + 4 * v);
                float*       d = &b_frag[buf][in * TN + 4 * v];
                d[0] = q.x; d[1] = q.y; d[2] = q.z; d[3] = q.w;
            }
        }
    };

    uint32_t it = 0;
    for(int unit = blockIdx.x; unit < w.total_units; unit += gridDim.x)
    {
        const int split   = unit / tiles;
        const int tile_id = unit - split * tiles;
        int       tile_m, tile_n;
        map_tile<Cfg::RASTER>(tile_id, p.grid_m, p.grid_n, tile_m, tile_n);
        const int m0 = tile_m * BM, n0 = tile_n * BN;
        const int k_begin = split * p.k_per_split;
        const int k_end   = min(p.K, k_begin + p.k_per_split);
        const int ntiles  = (k_end - k_begin + BK - 1) / BK;

        float    acc[MODE == FMA_SCALAR ? TMT : 1][MODE == FMA_SCALAR ? TNT : 1];
        uint64_t acc2[MODE == FMA_SCALAR ? 1 : TMT][MODE == FMA_SCALAR ? 1 : TNT / 2];
        if constexpr(MODE == FMA_SCALAR)
        {
#pragma unroll
            for(int i = 0; i < TMT; ++i)
#pragma unroll
                for(int j = 0; j < TNT; ++j)
                    acc[i][j] = 0.f;
        }
        else
        {
#pragma unroll
            for(int i = 0; i < TMT; ++i)
#pragma unroll
                for(int j = 0; j < TNT / 2; ++j)
                    acc2[i][j] = 0ull;
        }

        auto fma_step = [&](int buf) {
            if constexpr(MODE == FMA_SCALAR)
            {
#pragma unroll
                for(int i = 0; i < TMT; ++i)
#pragma unroll
                    for(int j = 0; j < TNT; ++j)
                        acc[i][j] = fmaf(a_frag[buf][i], b_frag[buf][j], acc[i][j]);
            }
            else if constexpr(MODE == FMA_X2_DUP)
            {
                uint64_t b2[TNT / 2];
#pragma unroll
                for(int j = 0; j < TNT / 2; ++j)
                    b2[j] = pack2(b_frag[buf][2 * j], b_frag[buf][2 * j + 1]);
#pragma unroll
                for(int i = 0; i < TMT; ++i)
                {
                    const uint64_t a2 = pack2(a_frag[buf][i], a_frag[buf][i]);
#pragma unroll
                    for(int j = 0; j < TNT / 2; ++j)
                        fma2(acc2[i][j], a2, b2[j]);
                }
            }
            else
            {
                uint64_t bn[TNT / 2], bx[TNT / 2];
#pragma unroll
                for(int j = 0; j < TNT / 2; ++j)
                {
                    bn[j] = pack2(b_frag[buf][2 * j], b_frag[buf][2 * j + 1]);
                    bx[j] = pack2(b_frag[buf][2 * j + 1], b_frag[buf][2 * j]);
                }
#pragma unroll
                for(int ip = 0; ip < TMT / 2; ++ip)
                {
                    const uint64_t a2 = pack2(a_frag[buf][2 * ip], a_frag[buf][2 * ip + 1]);
#pragma unroll
                    for(int j = 0; j < TNT / 2; ++j)
                    {
                        fma2(acc2[2 * ip][j], a2, bn[j]);
                        fma2(acc2[2 * ip + 1][j], a2, bx[j]);
                    }
                }
            }
        };

        bool ok = true;
        // first stage of this unit
        {
            const int s = it % STAGES;
            ok          = !*abort_flag && mbar_wait(full_bar(s), (it / STAGES) & 1u);
            if(ok)
                load_frags(0, tile_a(s), tile_b(s), 0);
        }
        for(int t = 0; ok && t < ntiles; ++t, ++it)
        {
            const int    s  = it % STAGES;
            const float* as = tile_a(s);
            const float* bs = tile_b(s);
#pragma unroll
            for(int kk = 0; kk < BK; ++kk)
            {
                if(kk + 1 < BK)
                {
                    load_frags((kk + 1) & 1, as, bs, kk + 1);
                }
                else if(t + 1 < ntiles)
                {
                    // fragment 0 of the next stage is fetched under the last FMAs of this one
                    const int s2 = (it + 1) % STAGES;
                    ok           = !*abort_flag && mbar_wait(full_bar(s2), ((it + 1) / STAGES) & 1u);
                    if(ok)
                        load_frags(BK & 1, tile_a(s2), tile_b(s2), 0);
                }
                fma_step(kk & 1);
            }
            __syncwarp();
            if(lane == 0)
                mbar_arrive(empty_bar(s)); // this warp is done reading stage s
        }
        if(!ok)
        {
            if(!*abort_flag)
            {
                *abort_flag = 1;
                atomicCAS(w.status, 0, WS_ERR_FULL_TIMEOUT);
            }
            return;
        }

        // ---- epilogue ---------------------------------------------------------------------------------
        float c[TMT][TNT];
        if constexpr(MODE == FMA_SCALAR)
        {
#pragma unroll
            for(int i = 0; i < TMT; ++i)
#pragma unroll
                for(int j = 0; j < TNT; ++j)
                    c[i][j] = acc[i][j];
        }
        else if constexpr(MODE == FMA_X2_DUP)
        {
#pragma unroll
            for(int i = 0; i < TMT; ++i)
#pragma unroll
                for(int j = 0; j < TNT / 2; ++j)
                    unpack2(acc2[i][j], c[i][2 * j], c[i][2 * j + 1]);
        }
        else
        {
#pragma unroll
            for(int ip = 0; ip < TMT / 2; ++ip)
#pragma unroll
                for(int j = 0; j < TNT / 2; ++j)
                {
                    unpack2(acc2[2 * ip][j], c[2 * ip][2 * j], c[2 * ip + 1][2 * j + 1]);
                    unpack2(acc2[2 * ip + 1][j], c[2 * ip][2 * j + 1], c[2 * ip + 1][2 * j]);
                }
        }
        store_tile<Cfg, LC, ALIGNED>(c, p, p.C + (long long)split * p.split_stride, m0 + tm0, n0 + tn0);
    }
}

} // namespace sgemm_b200
