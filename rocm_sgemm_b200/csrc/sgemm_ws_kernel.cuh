// Warp-specialised, persistent FP32 GEMM kernel for sm_100a (pipeline = 1 variants).
//
// Same arithmetic as sgemm_kernel.cuh, but the roles the reference's kernel gives to halves of one
// thread block (the lower half stages B, the upper half stages A, everybody computes:
// rocm_sgemm/include/rocm_sgemm/kernel/kernel.hpp:147-199,272-293) are split between dedicated warps
// that never meet at a block-wide barrier:
//
//   * CONSUMER warps (block_size/32 of them) only read fragments from shared memory and issue packed
//     FP32 FMAs.  They wait on a per-stage "full" mbarrier and release the stage through an "empty"
//     mbarrier, so a warp that is ahead is never held back by the others.
//   * PRODUCER warps fill the ring.  Wherever alignment allows, ONE thread issues TMA tile copies
//     (cp.async.bulk.tensor.2d; out-of-bounds elements are zero-filled by the hardware) that signal the
//     stage's mbarrier by byte count, and the other producer threads have nothing to do.
//   * the CTA is persistent: it walks work units (tile, K-slice) blockIdx.x, +gridDim.x, ... and the
//     producers run ahead into the next unit while the consumers store C.
//
// How each operand reaches the FMAs (the "plan", chosen at compile time from the layouts):
//   XTILE             the operand's M / N extent is contiguous in memory (A col-major, B row-major): the
//                     tile is [k][x], one 128-bit shared-memory read yields four consecutive rows /
//                     columns for one k.  Filled by TMA, or by guarded cp.async when unaligned.
//   KTILE             the operand is K-contiguous (A row-major, B col-major) and block_k is 32: the tile
//                     keeps memory order, [x][32 k], with TMA's 128-byte swizzle so that the reads are
//                     bank-conflict free; one 128-bit read yields four consecutive k of one row, used over
//                     four k-steps.  No transposition anywhere.  Filled by TMA, or by guarded cp.async
//                     into the same swizzled layout.
//   XTILE_TRANSPOSED  K-contiguous operand that has to look like XTILE: producer threads fetch 4x4 blocks
//                     with 128-bit loads, transpose them in registers and store them swizzled.  Used for B
//                     when A and B are both K-contiguous, and for any block_k other than 32.
// A packed FMA needs one operand as a natural pair of neighbours and the other duplicated into both
// halves.  With pairs along n, B must be an XTILE (neighbouring columns share a 64-bit register) and A
// may be anything; with pairs along m (used when B is a KTILE) A must be an XTILE.  Either way every C
// element is one k-ascending FMA chain, bit-identical to the other kernels.
//
// Every wait on an mbarrier is bounded: after WS_SPIN_LIMIT failed polls the thread records an error in
// *status, raises the CTA's abort flag and leaves; nobody waits forever on a peer that bailed out.
#pragma once
#include "sgemm_kernel.cuh"
#include <cuda.h>

namespace sgemm_b200
{

// producer warps per CTA: one warpgroup beside 8 or more consumer warps, two warps beside fewer
__host__ __device__ constexpr int ws_producer_threads(int consumer_threads)
{
    return consumer_threads >= 256 ? 128 : 64;
}
constexpr uint32_t WS_SPIN_LIMIT = 1u << 20;

// status word values written by the kernel (0 = ok)
constexpr int WS_ERR_FULL_TIMEOUT  = 1; // a consumer gave up waiting for a stage to fill
constexpr int WS_ERR_EMPTY_TIMEOUT = 2; // a producer gave up waiting for a stage to drain
constexpr int WS_ERR_SMEM_ALIGNMENT = 3; // dynamic shared memory did not start on a 1024-byte boundary

enum : int
{
    PLAN_XTILE            = 0,
    PLAN_XTILE_TRANSPOSED = 1,
    PLAN_KTILE            = 2
};

// plan of operand A / B for a layout pair and block_k (also evaluated by the host to build tensor maps)
// `pipeline` is the variant's pipeline field: 1 = K-contiguous operands are transposed by the producer
// warps, 2 = they stay K-major (KTILE) wherever block_k and the pairing rule allow it.
__host__ __device__ constexpr int ws_plan_a(int la, int /*lb*/, int bk, int pipeline)
{
    return la == LAYOUT_COL ? PLAN_XTILE : ((pipeline == 2 && bk == 32) ? PLAN_KTILE : PLAN_XTILE_TRANSPOSED);
}
__host__ __device__ constexpr int ws_plan_b(int la, int lb, int bk, int pipeline)
{
    if(lb == LAYOUT_ROW)
        return PLAN_XTILE;
    // B is K-contiguous: keep it as a KTILE only when A can supply the natural pairs
    return (pipeline == 2 && bk == 32 && ws_plan_a(la, lb, bk, pipeline) == PLAN_XTILE) ? PLAN_KTILE
                                                                                        : PLAN_XTILE_TRANSPOSED;
}

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
// tile copy global -> shared; (c0, c1) are element coordinates, c0 along the contiguous dimension
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar)
                 : "memory");
}

// ---- guarded fill of a KTILE when TMA cannot be used: same [x][32] layout, same 128-byte swizzle -------
template<int THREADS, int BX>
struct KTileStager
{
    static constexpr int ITEMS = BX * 8; // 16-byte chunks
    static constexpr int ITERS = (ITEMS + THREADS - 1) / THREADS;
    __device__ __forceinline__ static void fetch(const float* __restrict__ g, long long ld, int X, int x0, int k0,
                                                 int k_end, int vec_ok, float* tile, int tid)
    {
#pragma unroll
        for(int it = 0; it < ITERS; ++it)
        {
            const int q = tid + it * THREADS;
            if(ITEMS % THREADS == 0 || q < ITEMS)
            {
                const int      r = q >> 3, c = q & 7;
                const uint32_t dst = smem_u32(tile + r * 32 + ((c ^ (r & 7)) << 2));
                const int      gx = x0 + r, gk = k0 + 4 * c;
                const float*   src = g + (long long)gx * ld + gk;
                const bool     row = gx < X;
                if(vec_ok && (!row || gk + 3 < k_end || gk >= k_end))
                {
                    const bool in = row && gk < k_end;
                    cp_async_16(dst, in ? src : g, in ? 16 : 0);
                }
                else
                {
#pragma unroll
                    for(int j = 0; j < 4; ++j)
                    {
                        const bool in = row && gk + j < k_end;
                        cp_async_4(dst + 4 * j, in ? src + j : g, in ? 4 : 0);
                    }
                }
            }
        }
    }
};

template<class Cfg>
struct WsLayout
{
    static constexpr int    STAGE_FLOATS = (Cfg::BM + Cfg::BN) * Cfg::BK;
    static constexpr size_t TILE_BYTES   = size_t(Cfg::STAGES) * STAGE_FLOATS * sizeof(float);
    // after the tiles: full[STAGES], empty[STAGES] (8 bytes each), abort flag
    static constexpr size_t SMEM_BYTES = TILE_BYTES + size_t(2 * Cfg::STAGES) * 8 + 16;
    static constexpr int    PRODUCERS  = ws_producer_threads(Cfg::BLOCK_SIZE);
    static constexpr int    THREADS    = Cfg::BLOCK_SIZE + PRODUCERS;
};

__device__ __forceinline__ float f4_get(const float4& v, int i)
{
    return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w;
}

template<class Cfg, int LA, int LB, int LC, bool ALIGNED>
__global__ void __launch_bounds__(WsLayout<Cfg>::THREADS, Cfg::MIN_BLOCKS)
    sgemm_ws_kernel(const __grid_constant__ WsArgs w, const __grid_constant__ CUtensorMap map_a,
                    const __grid_constant__ CUtensorMap map_b)
{
    constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, STAGES = Cfg::STAGES;
    constexpr int TM = Cfg::TM, TN = Cfg::TN, TMT = Cfg::TMT, TNT = Cfg::TNT;
    constexpr int MODE   = Cfg::FMA_MODE;
    constexpr int PLAN_A = ws_plan_a(LA, LB, BK, Cfg::PIPELINE);
    constexpr int PLAN_B = ws_plan_b(LA, LB, BK, Cfg::PIPELINE);
    // pairs along m only when B stays K-major in shared memory (then A is an XTILE by construction)
    constexpr bool PAIR_M = (PLAN_B == PLAN_KTILE);
    constexpr int  CONSUMER_WARPS = Cfg::BLOCK_SIZE / 32;
    using SwzA = Swizzle<BM, BK>;
    using SwzB = Swizzle<BN, BK>;
    using L    = WsLayout<Cfg>;
    static_assert(MODE == FMA_SCALAR || MODE == FMA_X2_DUP, "warp-specialised kernel: fma_mode 0 or 1");
    static_assert(TM % 4 == 0 && TN % 4 == 0, "warp-specialised kernel reads 128-bit fragments");
    static_assert(!(PLAN_A == PLAN_KTILE && PLAN_B == PLAN_KTILE), "one operand must supply natural pairs");

    extern __shared__ __align__(1024) float smem[];
    const GemmArgs& p = w.g;

    const uint32_t bar_base = smem_u32(smem) + (uint32_t)L::TILE_BYTES;
    auto           full_bar  = [&](int s) -> uint32_t { return bar_base + 8u * s; };
    auto           empty_bar = [&](int s) -> uint32_t { return bar_base + 8u * (STAGES + s); };
    volatile int*  abort_flag = reinterpret_cast<volatile int*>(reinterpret_cast<char*>(smem) + L::TILE_BYTES
                                                               + 2 * STAGES * 8);
    auto tile_a = [&](int s) -> float* { return smem + s * L::STAGE_FLOATS; };
    auto tile_b = [&](int s) -> float* { return smem + s * L::STAGE_FLOATS + BM * BK; };

    const int tid = threadIdx.x;
    if((PLAN_A == PLAN_KTILE || PLAN_B == PLAN_KTILE) && (smem_u32(smem) & 1023u) != 0)
    {
        // the swizzled K-major tiles must start on a 1024-byte boundary; refuse to compute otherwise
        if(tid == 0)
            atomicCAS(w.status, 0, WS_ERR_SMEM_ALIGNMENT);
        return;
    }
    if(tid == 0)
    {
        for(int s = 0; s < STAGES; ++s)
        {
            mbar_init(full_bar(s), L::PRODUCERS + 1);
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
        OperandStager<L::PRODUCERS, BM, BK, PLAN_A == PLAN_XTILE_TRANSPOSED, ALIGNED> stage_a;
        OperandStager<L::PRODUCERS, BN, BK, PLAN_B == PLAN_XTILE_TRANSPOSED, ALIGNED> stage_b;
        // work left to the producer threads themselves (everything TMA does not cover)
        const bool manual_a = !w.tma_a, manual_b = !w.tma_b;
        uint32_t   it       = 0; // k-tiles issued by this CTA so far (ring position)
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
                        // the coordinate along the contiguous dimension is a multiple of 32 elements
                        // (tile origins and K slices are), so TMA's 16-byte start rule holds
                        if(w.tma_a)
                        {
                            if constexpr(PLAN_A == PLAN_KTILE)
                                tma_load_2d(smem_u32(tile_a(s)), &map_a, k0, m0, full_bar(s));
                            else
                                tma_load_2d(smem_u32(tile_a(s)), &map_a, m0, k0, full_bar(s));
                        }
                        if(w.tma_b)
                        {
                            if constexpr(PLAN_B == PLAN_KTILE)
                                tma_load_2d(smem_u32(tile_b(s)), &map_b, k0, n0, full_bar(s));
                            else
                                tma_load_2d(smem_u32(tile_b(s)), &map_b, n0, k0, full_bar(s));
                        }
                    }
                    else
                    {
                        mbar_arrive(full_bar(s));
                    }
                }
                if(manual_a)
                {
                    if constexpr(PLAN_A == PLAN_KTILE)
                        KTileStager<L::PRODUCERS, BM>::fetch(p.A, p.lda, p.M, m0, k0, k_end, p.vec_a, tile_a(s), ptid);
                    else
                        stage_a.fetch(p.A, p.lda, p.M, m0, k0, k_end, p.vec_a, tile_a(s), ptid);
                }
                if(manual_b)
                {
                    if constexpr(PLAN_B == PLAN_KTILE)
                        KTileStager<L::PRODUCERS, BN>::fetch(p.B, p.ldb, p.N, n0, k0, k_end, p.vec_b, tile_b(s), ptid);
                    else
                        stage_b.fetch(p.B, p.ldb, p.N, n0, k0, k_end, p.vec_b, tile_b(s), ptid);
                }
                if constexpr(PLAN_A == PLAN_XTILE_TRANSPOSED)
                    stage_a.commit(tile_a(s), ptid);
                if constexpr(PLAN_B == PLAN_XTILE_TRANSPOSED)
                    stage_b.commit(tile_b(s), ptid);
                if((manual_a && PLAN_A != PLAN_XTILE_TRANSPOSED) || (manual_b && PLAN_B != PLAN_XTILE_TRANSPOSED))
                {
                    cp_async_commit();
                    cp_async_wait<0>(); // guarded-copy fallback of an operand TMA could not take
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

    // XTILE fragments: one k-step, double buffered.  KTILE fragments: four k-steps per row, double buffered.
    float  a_frag[2][PLAN_A == PLAN_KTILE ? 1 : TMT];
    float  b_frag[2][PLAN_B == PLAN_KTILE ? 1 : TNT];
    float4 a_kq[2][PLAN_A == PLAN_KTILE ? TMT : 1];
    float4 b_kq[2][PLAN_B == PLAN_KTILE ? TNT : 1];

    // [k][x] tile: fragment of k-step kk (x ^ swizzle when the tile was transposed by the producers)
    auto load_x = [&](float* dst, const float* tile, int kk, int x_first, int BX, int SUB, int CNT, int T,
                      int xor_val) {
#pragma unroll
        for(int im = 0; im < CNT; ++im)
#pragma unroll
            for(int v = 0; v < T / 4; ++v)
            {
                const float4 q4 = *reinterpret_cast<const float4*>(tile + kk * BX + ((x_first + im * SUB) ^ xor_val) + 4 * v);
                float*       d  = dst + im * T + 4 * v;
                d[0] = q4.x; d[1] = q4.y; d[2] = q4.z; d[3] = q4.w;
            }
    };
    // [x][32] tile with the 128-byte swizzle: 16-byte chunk c of row r sits at chunk c ^ (r & 7).
    // For this thread r = x_first + d with d a compile-time offset and x_first a multiple of 4, so
    // r & 7 = (d & 7) ^ (x_first & 4): the runtime part flips bit 2 of the chunk index only and is folded
    // into two base pointers (plus / minus 16 * (x_first & 4) bytes); everything else is an immediate.
    auto load_k_row = [&](float4* dst, const char* base_plus, const char* base_minus, int quad, int i, int SUB,
                          int T) {
        const int d = (i / T) * SUB + (i % T);
        const int c = quad ^ (d & 7);
        const char* b = (c & 4) ? base_minus : base_plus;
        dst[i]        = *reinterpret_cast<const float4*>(b + d * 128 + c * 16);
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

        constexpr int ACC_R = MODE == FMA_SCALAR ? 1 : (PAIR_M ? TMT / 2 : TMT);
        constexpr int ACC_C = MODE == FMA_SCALAR ? 1 : (PAIR_M ? TNT : TNT / 2);
        float         acc[MODE == FMA_SCALAR ? TMT : 1][MODE == FMA_SCALAR ? TNT : 1];
        uint64_t      acc2[ACC_R][ACC_C];
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
            for(int i = 0; i < ACC_R; ++i)
#pragma unroll
                for(int j = 0; j < ACC_C; ++j)
                    acc2[i][j] = 0ull;
        }

        // per-stage fragment sources
        auto a_bases = [&](int s, const char*& plus, const char*& minus) {
            const char* row0 = reinterpret_cast<const char*>(tile_a(s)) + tm0 * 128;
            plus             = row0 + 16 * (tm0 & 4);
            minus            = row0 - 16 * (tm0 & 4);
        };
        auto b_bases = [&](int s, const char*& plus, const char*& minus) {
            const char* row0 = reinterpret_cast<const char*>(tile_b(s)) + tn0 * 128;
            plus             = row0 + 16 * (tn0 & 4);
            minus            = row0 - 16 * (tn0 & 4);
        };
        // fragments for k-step kk of stage s (XTILE) / rows [r0, r1) of quad `quad` (KTILE)
        auto prefetch = [&](int s, int kk_next, int quad_next, int part) {
            if constexpr(PLAN_A == PLAN_KTILE)
            {
                const char *pp, *pm;
                a_bases(s, pp, pm);
                constexpr int PER = TMT / 4;
#pragma unroll
                for(int r = 0; r < PER; ++r)
                    load_k_row(a_kq[quad_next & 1], pp, pm, quad_next, part * PER + r, Cfg::SUB_M, TM);
            }
            else
            {
                const int xa = PLAN_A == PLAN_XTILE_TRANSPOSED ? SwzA::of_chunk(kk_next >> 2) : 0;
                load_x(a_frag[kk_next & 1], tile_a(s), kk_next, tm0, BM, Cfg::SUB_M, Cfg::WM_CNT, TM, xa);
            }
            if constexpr(PLAN_B == PLAN_KTILE)
            {
                const char *pp, *pm;
                b_bases(s, pp, pm);
                constexpr int PER = TNT / 4;
#pragma unroll
                for(int r = 0; r < PER; ++r)
                    load_k_row(b_kq[quad_next & 1], pp, pm, quad_next, part * PER + r, Cfg::SUB_N, TN);
            }
            else
            {
                const int xb = PLAN_B == PLAN_XTILE_TRANSPOSED ? SwzB::of_chunk(kk_next >> 2) : 0;
                load_x(b_frag[kk_next & 1], tile_b(s), kk_next, tn0, BN, Cfg::SUB_N, Cfg::WN_CNT, TN, xb);
            }
        };

        auto fma_step = [&](int kk) {
            const int buf = kk & 1, quad = kk >> 2, kq = kk & 3;
            auto      a_val = [&](int i) -> float {
                if constexpr(PLAN_A == PLAN_KTILE)
                    return f4_get(a_kq[quad & 1][i], kq);
                else
                    return a_frag[buf][i];
            };
            auto b_val = [&](int j) -> float {
                if constexpr(PLAN_B == PLAN_KTILE)
                    return f4_get(b_kq[quad & 1][j], kq);
                else
                    return b_frag[buf][j];
            };
            if constexpr(MODE == FMA_SCALAR)
            {
#pragma unroll
                for(int i = 0; i < TMT; ++i)
#pragma unroll
                    for(int j = 0; j < TNT; ++j)
                        acc[i][j] = fmaf(a_val(i), b_val(j), acc[i][j]);
            }
            else if constexpr(!PAIR_M)
            {
                // pairs along n: b supplies the natural pair, a is duplicated.  Pair-major order (the
                // natural pair stays, the duplicated operand changes) measured fastest on B200.
                uint64_t a2[TMT];
#pragma unroll
                for(int i = 0; i < TMT; ++i)
                    a2[i] = pack2(a_val(i), a_val(i));
                {
#pragma unroll
                    for(int j = 0; j < TNT / 2; ++j)
                    {
                        const uint64_t b2 = pack2(b_val(2 * j), b_val(2 * j + 1));
#pragma unroll
                        for(int i = 0; i < TMT; ++i)
                            fma2(acc2[i][j], a2[i], b2);
                    }
                }
            }
            else
            {
                // pairs along m: a supplies the natural pair, b is duplicated
                uint64_t b2[TNT];
#pragma unroll
                for(int j = 0; j < TNT; ++j)
                    b2[j] = pack2(b_val(j), b_val(j));
                {
#pragma unroll
                    for(int i = 0; i < TMT / 2; ++i)
                    {
                        const uint64_t a2 = pack2(a_val(2 * i), a_val(2 * i + 1));
#pragma unroll
                        for(int j = 0; j < TNT; ++j)
                            fma2(acc2[i][j], a2, b2[j]);
                    }
                }
            }
        };

        bool ok = true;
        // first stage of this unit: k-step 0 (XTILE) and the whole first quad (KTILE)
        {
            const int s = it % STAGES;
            ok          = !*abort_flag && mbar_wait(full_bar(s), (it / STAGES) & 1u);
            if(ok)
            {
                // k-step 0 of the XTILE operands, all four row groups of quad 0 of a KTILE operand
                // (prefetch() reloads the XTILE fragment on every pass; that only happens here)
#pragma unroll
                for(int part = 0; part < 4; ++part)
                    if(part == 0 || PLAN_A == PLAN_KTILE || PLAN_B == PLAN_KTILE)
                        prefetch(s, 0, 0, part);
            }
        }
        for(int t = 0; ok && t < ntiles; ++t, ++it)
        {
            const int  s        = it % STAGES;
            const int  s2       = (it + 1) % STAGES;
            const bool has_next = t + 1 < ntiles;
#pragma unroll
            for(int kk = 0; kk < BK; ++kk)
            {
                // with a KTILE operand the first rows of the next stage are fetched four k-steps early
                if(kk == ((PLAN_A == PLAN_KTILE || PLAN_B == PLAN_KTILE) ? BK - 4 : BK - 1) && has_next)
                    // the next stage must have landed before anything of it is prefetched
                    ok = !*abort_flag && mbar_wait(full_bar(s2), ((it + 1) / STAGES) & 1u);
                // next k-step (XTILE) and a quarter of the next quad's rows (KTILE)
                const bool wraps = (kk + 1 == BK);            // XTILE fragment comes from the next stage
                const bool quadw = ((kk >> 2) + 1 == BK / 4); // KTILE rows come from the next stage
                if constexpr(PLAN_A != PLAN_KTILE && PLAN_B != PLAN_KTILE)
                {
                    if(!wraps)
                        prefetch(s, kk + 1, 0, 0);
                    else if(has_next && ok)
                        prefetch(s2, 0, 0, 0);
                }
                else
                {
                    // mixed: the XTILE operand follows kk + 1, the KTILE operand follows the quad
                    const int kn = wraps ? 0 : kk + 1;
                    const int qn = quadw ? 0 : (kk >> 2) + 1;
                    if constexpr(PLAN_A == PLAN_KTILE)
                    {
                        if(!quadw || (has_next && ok))
                        {
                            const char *pp, *pm;
                            a_bases(quadw ? s2 : s, pp, pm);
#pragma unroll
                            for(int r = 0; r < TMT / 4; ++r)
                                load_k_row(a_kq[((kk >> 2) + 1) & 1], pp, pm, qn, (kk & 3) * (TMT / 4) + r, Cfg::SUB_M,
                                           TM);
                        }
                        if(!wraps || (has_next && ok))
                        {
                            const int xb = PLAN_B == PLAN_XTILE_TRANSPOSED ? SwzB::of_chunk(kn >> 2) : 0;
                            load_x(b_frag[(kk + 1) & 1], tile_b(wraps ? s2 : s), kn, tn0, BN, Cfg::SUB_N, Cfg::WN_CNT,
                                   TN, xb);
                        }
                    }
                    else
                    {
                        if(!quadw || (has_next && ok))
                        {
                            const char *pp, *pm;
                            b_bases(quadw ? s2 : s, pp, pm);
#pragma unroll
                            for(int r = 0; r < TNT / 4; ++r)
                                load_k_row(b_kq[((kk >> 2) + 1) & 1], pp, pm, qn, (kk & 3) * (TNT / 4) + r, Cfg::SUB_N,
                                           TN);
                        }
                        if(!wraps || (has_next && ok))
                        {
                            const int xa = PLAN_A == PLAN_XTILE_TRANSPOSED ? SwzA::of_chunk(kn >> 2) : 0;
                            load_x(a_frag[(kk + 1) & 1], tile_a(wraps ? s2 : s), kn, tm0, BM, Cfg::SUB_M, Cfg::WM_CNT,
                                   TM, xa);
                        }
                    }
                }
                fma_step(kk);
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
        else if constexpr(!PAIR_M)
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
            for(int i = 0; i < TMT / 2; ++i)
#pragma unroll
                for(int j = 0; j < TNT; ++j)
                    unpack2(acc2[i][j], c[2 * i][j], c[2 * i + 1][j]);
        }
        store_tile<Cfg, LC, ALIGNED>(c, p, p.C + (long long)split * p.split_stride, m0 + tm0, n0 + tn0);
    }
}

} // namespace sgemm_b200
