// FP32 GEMM kernel family for sm_100a:  C[MxN] = A[MxK] * B[KxN], true FP32 FMA (no tensor cores).
//
// Plays the role of the reference's kernel_gemm (rocm_sgemm/include/rocm_sgemm/kernel/kernel.hpp:66-362)
// together with its staging helpers (kernel/load.hpp:32-173), register fragments
// (kernel/fragment.hpp:37-162) and tile mapper (kernel/mapping.hpp:34-237).  The tiling vocabulary
// is the reference's (block_m/n/k, warp_tile_m/n_count, thread_tile_m/n, threads_n); the
// implementation is written for Blackwell:
//
//   * packed FP32 FMA (PTX fma.rn.f32x2): one instruction performs two IEEE round-to-nearest FMAs,
//     halving the issue slots the accumulation needs so that shared-memory reads, address
//     arithmetic and staging no longer compete with the FMA pipe for the scheduler;
//   * STAGES-deep shared-memory ring.  Operands whose non-K dimension is contiguous in global memory
//     (A col-major, B row-major) are staged with 16-byte cp.async straight into the [k][m] / [k][n]
//     tile, never touching registers.  Operands that are K-contiguous (A row-major, B col-major) are
//     fetched with 128-bit loads and transposed on the way into shared memory with an XOR swizzle
//     that makes both the scalar transposing stores and the 128-bit fragment reads conflict-free
//     (the reference pads by 4 instead: kernel/load.hpp:73-101);
//   * every accumulator is one k-ascending FMA chain starting from zero, so the result of a
//     non-split launch is bit-identical to a sequential fmaf loop, and a split-K launch to the ordered
//     sum of such chains;
//   * loads are predicated / zero-filled, so ragged M, N and K are handled (the reference's loads are
//     unguarded: kernel/load.hpp:57,85,129,157);
//   * 64-bit global offsets (the reference uses int: kernel/kernel.hpp:318,322).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace sgemm_b200
{

constexpr int LAYOUT_ROW = 0;
constexpr int LAYOUT_COL = 1;

enum : int
{
    FMA_SCALAR  = 0, // fma.rn.f32, one accumulator register per C element
    FMA_X2_DUP  = 1, // fma.rn.f32x2, accumulator pairs along n, A value duplicated into both halves
    FMA_X2_DIAG = 2  // fma.rn.f32x2, accumulator pairs on 2x2 diagonals: (a0,a1)*(b0,b1) and (a0,a1)*(b1,b0)
};

enum : int
{
    RASTER_ROW     = 0, // tile id -> (id / grid_n, id % grid_n)
    RASTER_GROUPED = 1, // bands of RASTER_GROUP tile-rows walked column by column (L2 reuse of the B panel)
    RASTER_HILBERT = 2  // Hilbert curve over the padded power-of-two tile grid
};

struct GemmArgs
{
    float*       C;       // result, or split-K partial buffer when splits > 1
    const float* A;
    const float* B;
    int          M, N, K;
    long long    lda, ldb, ldc; // leading dimensions in elements (row-major: row pitch, col-major: column pitch)
    int          grid_m, grid_n;
    int          splits;        // number of K slices
    int          k_per_split;   // slice length, a multiple of block_k
    long long    split_stride;  // elements between consecutive partial results
    int          vec_a, vec_b, vec_c; // 1 when 16-byte vector access is legal for that matrix
};

// ------------------------------------------------------------------------------------------------
// small PTX helpers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src, int src_bytes)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit()
{
    asm volatile("cp.async.commit_group;\n" ::: "memory");
}
template<int N>
__device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint64_t pack2(float lo, float hi)
{
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
// two independent round-to-nearest FP32 FMAs: acc.lo = a.lo*b.lo + acc.lo ; acc.hi = a.hi*b.hi + acc.hi
__device__ __forceinline__ void fma2(uint64_t& acc, uint64_t a, uint64_t b)
{
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}

// ------------------------------------------------------------------------------------------------
// compile-time description of one kernel variant
// ------------------------------------------------------------------------------------------------
template<int BLOCK_SIZE_, int BM_, int BN_, int BK_, int WM_CNT_, int WN_CNT_, int TM_, int TN_, int THREADS_N_,
         int STAGES_, int FMA_MODE_, int RASTER_, int MIN_BLOCKS_, int PIPELINE_ = 0>
struct TileConfig
{
    static constexpr int BLOCK_SIZE = BLOCK_SIZE_, BM = BM_, BN = BN_, BK = BK_;
    static constexpr int WM_CNT = WM_CNT_, WN_CNT = WN_CNT_, TM = TM_, TN = TN_;
    static constexpr int THREADS_N = THREADS_N_, THREADS_M = 32 / THREADS_N_;
    static constexpr int STAGES = STAGES_, FMA_MODE = FMA_MODE_, RASTER = RASTER_, MIN_BLOCKS = MIN_BLOCKS_;
    static constexpr int PIPELINE = PIPELINE_;

    static constexpr int SUB_M  = TM * THREADS_M; // rows covered by one warp sub-tile
    static constexpr int SUB_N  = TN * THREADS_N;
    static constexpr int WARP_M = WM_CNT * SUB_M; // warp tile
    static constexpr int WARP_N = WN_CNT * SUB_N;
    static constexpr int WARPS_M = BM / WARP_M, WARPS_N = BN / WARP_N;
    static constexpr int TMT = WM_CNT * TM; // per-thread rows
    static constexpr int TNT = WN_CNT * TN; // per-thread columns

    static_assert(32 % THREADS_N == 0, "threads_n must divide the warp");
    static_assert(BM % WARP_M == 0 && BN % WARP_N == 0, "warp tile must divide the block tile");
    static_assert(WARPS_M * WARPS_N * 32 == BLOCK_SIZE, "warp grid must match the block size");
    static_assert(TM == 1 || TM == 2 || TM == 4 || TM == 8, "thread_tile_m in {1,2,4,8}");
    static_assert(TN == 1 || TN == 2 || TN == 4 || TN == 8, "thread_tile_n in {1,2,4,8}");
    static_assert(BK % 4 == 0 && BK >= 4, "block_k must be a multiple of 4");
    static_assert(BM % 32 == 0 && BN % 32 == 0, "block_m and block_n must be multiples of 32");
    static_assert(STAGES >= 2, "at least double buffering");
    static_assert(FMA_MODE == FMA_SCALAR || (TN % 2 == 0), "packed FMA needs an even thread_tile_n");
    static_assert(FMA_MODE != FMA_X2_DIAG || (TM % 2 == 0), "diagonal packing needs an even thread_tile_m");

    static constexpr int    STAGE_FLOATS = (BM + BN) * BK;
    static constexpr size_t SMEM_BYTES   = size_t(STAGES) * STAGE_FLOATS * sizeof(float);
};

// ------------------------------------------------------------------------------------------------
// global -> shared staging of one operand tile.
// The operand is seen as X x K where X is its non-K extent (M for A, N for B); the shared tile is
// always [BK][BX] floats.  KMAJOR = the operand is K-contiguous in global memory.
// ------------------------------------------------------------------------------------------------
template<int BX, int BK>
struct Swizzle
{
    static constexpr int L     = BK / 4;                    // 16-byte chunks per operand row
    static constexpr int RPW   = (32 / L) < 1 ? 1 : 32 / L; // operand rows one warp covers per load
    static constexpr int SHIFT = RPW >= 16 ? 4 : RPW >= 8 ? 3 : 2;
    static constexpr int MODN  = 32 >> SHIFT;               // distinct XOR values
    // XOR applied to the x index of every element whose k lies in 16-byte chunk c = k/4
    __device__ __forceinline__ static constexpr int of_chunk(int c)
    {
        return (c % MODN) << SHIFT;
    }
};

// SWIZZLED = false writes the plain [k][x] tile instead (the warp-specialised kernel's consumers then read every
// operand the same way; the transposing stores of this fallback route then conflict, which only it pays for).
template<int BLOCK_SIZE, int BX, int BK, bool KMAJOR, bool ALIGNED, bool SWIZZLED = true>
struct OperandStager
{
    // X-contiguous operand: one 16-byte chunk of a k-row per work item.
    // K-contiguous operand: one 4 (x) by 4 (k) block per work item, fetched as four 128-bit loads (one
    // per operand row), transposed in registers (pure renaming) and written as four 128-bit stores.
    static constexpr int L      = BK / 4; // 16-byte chunks per operand row
    static constexpr int ITEMS  = KMAJOR ? (BX / 4) * L : BX * BK / 4;
    static constexpr int ITERS  = (ITEMS + BLOCK_SIZE - 1) / BLOCK_SIZE;
    static constexpr bool EXACT = (ITEMS % BLOCK_SIZE) == 0;
    using Swz                   = Swizzle<BX, BK>;

    float4 regs[KMAJOR ? ITERS : 1][KMAJOR ? 4 : 1];

    // Issue the global reads of the tile whose origin is (x0, k0); k_end bounds this CTA's K slice.
    // X-contiguous operands go straight to shared memory with cp.async; K-contiguous ones into regs.
    __device__ __forceinline__ void fetch(const float* __restrict__ g, long long ld, int X, int x0, int k0, int k_end,
                                          int vec_ok, float* tile, int tid)
    {
        if constexpr(!KMAJOR)
        {
            constexpr int CPR = BX / 4; // chunks per k-row
#pragma unroll
            for(int it = 0; it < ITERS; ++it)
            {
                const int q = tid + it * BLOCK_SIZE;
                if(EXACT || q < ITEMS)
                {
                    const int      k   = q / CPR;
                    const int      x4  = (q % CPR) * 4;
                    const uint32_t dst = smem_u32(tile + k * BX + x4);
                    const int      gk = k0 + k, gx = x0 + x4;
                    if constexpr(ALIGNED)
                    {
                        cp_async_16(dst, g + (long long)gk * ld + gx, 16);
                    }
                    else
                    {
                        const bool krow = gk < k_end;
                        if(vec_ok && (!krow || gx + 3 < X || gx >= X))
                        {
                            const bool in = krow && gx < X;
                            cp_async_16(dst, in ? g + (long long)gk * ld + gx : g, in ? 16 : 0);
                        }
                        else
                        {
#pragma unroll
                            for(int j = 0; j < 4; ++j)
                            {
                                const bool in = krow && gx + j < X;
                                cp_async_4(dst + 4 * j, in ? g + (long long)gk * ld + gx + j : g, in ? 4 : 0);
                            }
                        }
                    }
                }
            }
        }
        else
        {
            // lanes of a warp: chunk index c fastest, so each load instruction reads whole 16*L-byte row
            // segments (a full 128-byte line per row when BK = 32)
#pragma unroll
            for(int it = 0; it < ITERS; ++it)
            {
                const int q = tid + it * BLOCK_SIZE;
#pragma unroll
                for(int r = 0; r < 4; ++r)
                {
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    if(EXACT || q < ITEMS)
                    {
                        const int    c  = q % L;
                        const int    gx = x0 + 4 * (q / L) + r, gk = k0 + 4 * c;
                        const float* src = g + (long long)gx * ld + gk;
                        if constexpr(ALIGNED)
                        {
                            v = __ldg(reinterpret_cast<const float4*>(src));
                        }
                        else if(gx < X)
                        {
                            if(vec_ok && gk + 3 < k_end)
                            {
                                v = __ldg(reinterpret_cast<const float4*>(src));
                            }
                            else
                            {
                                if(gk + 0 < k_end) v.x = __ldg(src + 0);
                                if(gk + 1 < k_end) v.y = __ldg(src + 1);
                                if(gk + 2 < k_end) v.z = __ldg(src + 2);
                                if(gk + 3 < k_end) v.w = __ldg(src + 3);
                            }
                        }
                    }
                    regs[it][r] = v;
                }
            }
        }
    }

    // Second half of a K-contiguous fetch: the 4x4 block goes out transposed, one 128-bit store per k,
    // into the [k][x ^ swizzle] tile.  The eight lanes of a quarter warp hold different (chunk, x-group)
    // pairs whose swizzled 16-byte slots fall into eight different bank groups: conflict-free.
    __device__ __forceinline__ void commit(float* tile, int tid)
    {
        if constexpr(KMAJOR)
        {
#pragma unroll
            for(int it = 0; it < ITERS; ++it)
            {
                const int q = tid + it * BLOCK_SIZE;
                if(EXACT || q < ITEMS)
                {
                    const int c  = q % L;
                    const int xs = SWIZZLED ? (4 * (q / L)) ^ Swz::of_chunk(c) : 4 * (q / L);
                    float*    d  = tile + (4 * c) * BX + xs;
                    const float4 r0 = regs[it][0], r1 = regs[it][1], r2 = regs[it][2], r3 = regs[it][3];
                    *reinterpret_cast<float4*>(d + 0 * BX) = make_float4(r0.x, r1.x, r2.x, r3.x);
                    *reinterpret_cast<float4*>(d + 1 * BX) = make_float4(r0.y, r1.y, r2.y, r3.y);
                    *reinterpret_cast<float4*>(d + 2 * BX) = make_float4(r0.z, r1.z, r2.z, r3.z);
                    *reinterpret_cast<float4*>(d + 3 * BX) = make_float4(r0.w, r1.w, r2.w, r3.w);
                }
            }
        }
    }
};

// ------------------------------------------------------------------------------------------------
// CTA id -> tile coordinates (the reference's tile_mapper role, kernel/mapping.hpp:211-237)
// ------------------------------------------------------------------------------------------------
// Position d along the Hilbert curve of an s x s square (s a power of two) -> (x, y)
__host__ __device__ inline void hilbert_d2xy(int s, int d, int& x, int& y)
{
    x = 0;
    y = 0;
    int t = d;
    for(int side = 1; side < s; side <<= 1)
    {
        const int rx = 1 & (t >> 1);
        const int ry = 1 & (t ^ rx);
        if(ry == 0)
        {
            if(rx == 1)
            {
                x = side - 1 - x;
                y = side - 1 - y;
            }
            const int tmp = x;
            x             = y;
            y             = tmp;
        }
        x += side * rx;
        y += side * ry;
        t >>= 2;
    }
}

// Hilbert order over an arbitrary grid_m x grid_n tile grid: the grid is cut into the largest
// power-of-two squares that fit along its shorter side (each walked along a Hilbert curve, one after the
// other along the longer side), and the remaining strips are handled the same way, iteratively.  Tiles
// that are close in the order are close in both m and n, which keeps the A and B panels of the tiles in
// flight together small.  (The reference: kernel/mapping.hpp:34-166, Hilbert curve over power-of-two
// sub-squares with remainder strips; this is an independent formulation.)
__host__ __device__ inline void hilbert_map(int id, int grid_m, int grid_n, int& tile_m, int& tile_n)
{
    int om = 0, on = 0, rows = grid_m, cols = grid_n;
    for(int guard = 0; guard < 64; ++guard)
    {
        const int shorter = rows < cols ? rows : cols;
        int       s       = 1;
        while(2 * s <= shorter)
            s *= 2;
        const int ss = s * s;
        if(cols >= rows)
        {
            const int nsq = cols / s, count = nsq * ss;
            if(id < count)
            {
                const int sq = id / ss;
                int       x, y;
                hilbert_d2xy(s, id - sq * ss, x, y);
                tile_m = om + y;
                tile_n = on + sq * s + x;
                return;
            }
            id -= count;
            const int right = s * (cols - nsq * s); // strip to the right of the squares, s rows tall
            if(id < right)
            {
                on += nsq * s;
                cols -= nsq * s;
                rows = s;
            }
            else
            {
                id -= right;
                om += s;
                rows -= s;
            }
        }
        else
        {
            const int nsq = rows / s, count = nsq * ss;
            if(id < count)
            {
                const int sq = id / ss;
                int       x, y;
                hilbert_d2xy(s, id - sq * ss, x, y);
                tile_m = om + sq * s + y;
                tile_n = on + x;
                return;
            }
            id -= count;
            const int below = s * (rows - nsq * s); // strip below the squares, s columns wide
            if(id < below)
            {
                om += nsq * s;
                rows -= nsq * s;
                cols = s;
            }
            else
            {
                id -= below;
                on += s;
                cols -= s;
            }
        }
    }
    tile_m = 0; // not reached for id < grid_m * grid_n
    tile_n = 0;
}

template<int RASTER>
__host__ __device__ __forceinline__ void map_tile(int tile_id, int grid_m, int grid_n, int& tile_m, int& tile_n)
{
    if constexpr(RASTER == RASTER_HILBERT)
    {
        hilbert_map(tile_id, grid_m, grid_n, tile_m, tile_n);
    }
    else if constexpr(RASTER == RASTER_GROUPED)
    {
        constexpr int GROUP    = 8;
        const int     per_band = GROUP * grid_n;
        const int     band     = tile_id / per_band;
        const int     first_m  = band * GROUP;
        const int     rows     = (GROUP < grid_m - first_m) ? GROUP : grid_m - first_m;
        const int     in_band  = tile_id - band * per_band;
        tile_m                 = first_m + in_band % rows;
        tile_n                 = in_band / rows;
    }
    else
    {
        tile_m = tile_id / grid_n;
        tile_n = tile_id % grid_n;
    }
}

// ------------------------------------------------------------------------------------------------
// register tile -> global C.  (m_base, n_base) is the first row / column this thread owns; its
// sub-tiles repeat every SUB_M rows and SUB_N columns.  128-bit stores along C's contiguous dimension
// (the reference stores scalars: kernel/kernel.hpp:299-361); guarded unless ALIGNED.
// ------------------------------------------------------------------------------------------------
// SCALE: instead of the plain store, out = alpha * c (+ beta * out when beta != 0) with every operation rounded
// separately (multiply, multiply, add: no contraction), the arithmetic of the vendor-BLAS convention's entry.
template<class Cfg, int LC, bool ALIGNED, bool SCALE = false>
__device__ __forceinline__ void store_tile(const float (&c)[Cfg::TMT][Cfg::TNT], const GemmArgs& p,
                                           float* __restrict__ out, int m_base, int n_base, float alpha = 1.f,
                                           float beta = 0.f)
{
    constexpr int TM = Cfg::TM, TN = Cfg::TN;
    auto put4 = [&](float* dst, float x, float y, float z, float w) {
        if constexpr(SCALE)
        {
            float4 o = make_float4(__fmul_rn(alpha, x), __fmul_rn(alpha, y), __fmul_rn(alpha, z), __fmul_rn(alpha, w));
            if(beta != 0.f)
            {
                const float4 q = *reinterpret_cast<const float4*>(dst);
                o.x = __fadd_rn(o.x, __fmul_rn(beta, q.x));
                o.y = __fadd_rn(o.y, __fmul_rn(beta, q.y));
                o.z = __fadd_rn(o.z, __fmul_rn(beta, q.z));
                o.w = __fadd_rn(o.w, __fmul_rn(beta, q.w));
            }
            *reinterpret_cast<float4*>(dst) = o;
        }
        else
            *reinterpret_cast<float4*>(dst) = make_float4(x, y, z, w);
    };
    auto put1 = [&](float* dst, float x) {
        if constexpr(SCALE)
        {
            const float o = __fmul_rn(alpha, x);
            *dst          = beta != 0.f ? __fadd_rn(o, __fmul_rn(beta, *dst)) : o;
        }
        else
            *dst = x;
    };
    if constexpr(LC == LAYOUT_ROW)
    {
#pragma unroll
        for(int im = 0; im < Cfg::WM_CNT; ++im)
#pragma unroll
            for(int ii = 0; ii < TM; ++ii)
            {
                const int i = im * TM + ii;
                const int m = m_base + im * Cfg::SUB_M + ii;
#pragma unroll
                for(int in = 0; in < Cfg::WN_CNT; ++in)
                {
                    const int n   = n_base + in * Cfg::SUB_N;
                    float*    dst = out + (long long)m * p.ldc + n;
                    if constexpr(ALIGNED && TN % 4 == 0)
                    {
#pragma unroll
                        for(int v = 0; v < TN / 4; ++v)
                            put4(dst + 4 * v, c[i][in * TN + 4 * v], c[i][in * TN + 4 * v + 1], c[i][in * TN + 4 * v + 2],
                                 c[i][in * TN + 4 * v + 3]);
                    }
                    else if(m < p.M)
                    {
                        if(TN % 4 == 0 && p.vec_c && n + TN <= p.N)
                        {
#pragma unroll
                            for(int v = 0; v < TN / 4; ++v)
                                put4(dst + 4 * v, c[i][in * TN + 4 * v], c[i][in * TN + 4 * v + 1],
                                     c[i][in * TN + 4 * v + 2], c[i][in * TN + 4 * v + 3]);
                        }
                        else
                        {
#pragma unroll
                            for(int jj = 0; jj < TN; ++jj)
                                if(n + jj < p.N)
                                    put1(dst + jj, c[i][in * TN + jj]);
                        }
                    }
                }
            }
    }
    else
    {
#pragma unroll
        for(int in = 0; in < Cfg::WN_CNT; ++in)
#pragma unroll
            for(int jj = 0; jj < TN; ++jj)
            {
                const int j = in * TN + jj;
                const int n = n_base + in * Cfg::SUB_N + jj;
#pragma unroll
                for(int im = 0; im < Cfg::WM_CNT; ++im)
                {
                    const int m   = m_base + im * Cfg::SUB_M;
                    float*    dst = out + (long long)n * p.ldc + m;
                    if constexpr(ALIGNED && TM % 4 == 0)
                    {
#pragma unroll
                        for(int v = 0; v < TM / 4; ++v)
                            put4(dst + 4 * v, c[im * TM + 4 * v][j], c[im * TM + 4 * v + 1][j], c[im * TM + 4 * v + 2][j],
                                 c[im * TM + 4 * v + 3][j]);
                    }
                    else if(n < p.N)
                    {
                        if(TM % 4 == 0 && p.vec_c && m + TM <= p.M)
                        {
#pragma unroll
                            for(int v = 0; v < TM / 4; ++v)
                                put4(dst + 4 * v, c[im * TM + 4 * v][j], c[im * TM + 4 * v + 1][j],
                                     c[im * TM + 4 * v + 2][j], c[im * TM + 4 * v + 3][j]);
                        }
                        else
                        {
#pragma unroll
                            for(int ii = 0; ii < TM; ++ii)
                                if(m + ii < p.M)
                                    put1(dst + ii, c[im * TM + ii][j]);
                        }
                    }
                }
            }
    }
}

// ------------------------------------------------------------------------------------------------
// the kernel
// ------------------------------------------------------------------------------------------------
template<class Cfg, int LA, int LB, int LC, bool ALIGNED>
__global__ void __launch_bounds__(Cfg::BLOCK_SIZE, Cfg::MIN_BLOCKS) sgemm_kernel(const GemmArgs p)
{
    constexpr int  BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, STAGES = Cfg::STAGES;
    constexpr int  TM = Cfg::TM, TN = Cfg::TN, TMT = Cfg::TMT, TNT = Cfg::TNT;
    constexpr int  MODE     = Cfg::FMA_MODE;
    constexpr bool A_KMAJOR = (LA == LAYOUT_ROW); // A(m,k) at m*lda + k
    constexpr bool B_KMAJOR = (LB == LAYOUT_COL); // B(k,n) at n*ldb + k
    using SwzA              = Swizzle<BM, BK>;
    using SwzB              = Swizzle<BN, BK>;

    extern __shared__ __align__(128) float smem[];

    const int tid      = threadIdx.x;
    const int warp_id  = tid >> 5;
    const int lane     = tid & 31;
    const int warp_row = warp_id / Cfg::WARPS_N;
    const int warp_col = warp_id % Cfg::WARPS_N;
    const int lane_m   = lane / Cfg::THREADS_N;
    const int lane_n   = lane % Cfg::THREADS_N;

    // tile and K slice of this CTA
    const int tiles    = p.grid_m * p.grid_n;
    const int split    = blockIdx.x / tiles;
    const int tile_id  = blockIdx.x - split * tiles;
    int       tile_m, tile_n;
    map_tile<Cfg::RASTER>(tile_id, p.grid_m, p.grid_n, tile_m, tile_n);
    const int m0      = tile_m * BM;
    const int n0      = tile_n * BN;
    const int k_begin = split * p.k_per_split;
    const int k_end   = min(p.K, k_begin + p.k_per_split);
    const int ntiles  = (k_end - k_begin + BK - 1) / BK;

    // first row / column this thread owns inside the CTA tile (sub-tile 0)
    const int tm0 = warp_row * Cfg::WARP_M + lane_m * TM;
    const int tn0 = warp_col * Cfg::WARP_N + lane_n * TN;

    OperandStager<Cfg::BLOCK_SIZE, BM, BK, A_KMAJOR, ALIGNED> stage_a;
    OperandStager<Cfg::BLOCK_SIZE, BN, BK, B_KMAJOR, ALIGNED> stage_b;

    auto tile_a = [&](int s) -> float* { return smem + s * Cfg::STAGE_FLOATS; };
    auto tile_b = [&](int s) -> float* { return smem + s * Cfg::STAGE_FLOATS + BM * BK; };

    // ---- accumulators ---------------------------------------------------------------------------
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

    // ---- prologue: tiles 0 .. STAGES-2 ----------------------------------------------------------
#pragma unroll
    for(int s = 0; s < STAGES - 1; ++s)
    {
        if(s < ntiles)
        {
            const int k0 = k_begin + s * BK;
            stage_a.fetch(p.A, p.lda, p.M, m0, k0, k_end, p.vec_a, tile_a(s), tid);
            stage_b.fetch(p.B, p.ldb, p.N, n0, k0, k_end, p.vec_b, tile_b(s), tid);
            stage_a.commit(tile_a(s), tid);
            stage_b.commit(tile_b(s), tid);
        }
        cp_async_commit();
    }

    // register fragments, double buffered over k
    float a_frag[2][TMT];
    float b_frag[2][TNT];

    auto load_frags = [&](int buf, const float* as, const float* bs, int kk) {
        const int xa = A_KMAJOR ? SwzA::of_chunk(kk >> 2) : 0;
        const int xb = B_KMAJOR ? SwzB::of_chunk(kk >> 2) : 0;
#pragma unroll
        for(int im = 0; im < Cfg::WM_CNT; ++im)
        {
            const float* src = as + kk * BM + ((tm0 + im * Cfg::SUB_M) ^ xa);
            if constexpr(TM == 8)
            {
                const float4 v0 = *reinterpret_cast<const float4*>(src);
                // second 16-byte chunk: the swizzle applies to its own index
                const float4 v1 = *reinterpret_cast<const float4*>(as + kk * BM + ((tm0 + im * Cfg::SUB_M + 4) ^ xa));
                float*       d  = &a_frag[buf][im * TM];
                d[0] = v0.x; d[1] = v0.y; d[2] = v0.z; d[3] = v0.w;
                d[4] = v1.x; d[5] = v1.y; d[6] = v1.z; d[7] = v1.w;
            }
            else if constexpr(TM == 4)
            {
                const float4 v = *reinterpret_cast<const float4*>(src);
                float*       d = &a_frag[buf][im * TM];
                d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
            }
            else if constexpr(TM == 2)
            {
                const float2 v = *reinterpret_cast<const float2*>(src);
                a_frag[buf][im * TM + 0] = v.x;
                a_frag[buf][im * TM + 1] = v.y;
            }
            else
            {
                a_frag[buf][im] = *src;
            }
        }
#pragma unroll
        for(int in = 0; in < Cfg::WN_CNT; ++in)
        {
            const float* src = bs + kk * BN + ((tn0 + in * Cfg::SUB_N) ^ xb);
            if constexpr(TN == 8)
            {
                const float4 v0 = *reinterpret_cast<const float4*>(src);
                const float4 v1 = *reinterpret_cast<const float4*>(bs + kk * BN + ((tn0 + in * Cfg::SUB_N + 4) ^ xb));
                float*       d  = &b_frag[buf][in * TN];
                d[0] = v0.x; d[1] = v0.y; d[2] = v0.z; d[3] = v0.w;
                d[4] = v1.x; d[5] = v1.y; d[6] = v1.z; d[7] = v1.w;
            }
            else if constexpr(TN == 4)
            {
                const float4 v = *reinterpret_cast<const float4*>(src);
                float*       d = &b_frag[buf][in * TN];
                d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
            }
            else if constexpr(TN == 2)
            {
                const float2 v = *reinterpret_cast<const float2*>(src);
                b_frag[buf][in * TN + 0] = v.x;
                b_frag[buf][in * TN + 1] = v.y;
            }
            else
            {
                b_frag[buf][in] = *src;
            }
        }
    };

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
            uint64_t a2[TMT];
#pragma unroll
            for(int i = 0; i < TMT; ++i)
                a2[i] = pack2(a_frag[buf][i], a_frag[buf][i]);
            // column-pair major: consecutive packed FMAs keep the natural pair (b) and change the
            // duplicated operand; measured 4 % faster on B200 than the row-major order
#pragma unroll
            for(int j = 0; j < TNT / 2; ++j)
#pragma unroll
                for(int i = 0; i < TMT; ++i)
                    fma2(acc2[i][j], a2[i], b2[j]);
        }
        else
        {
            // acc2[2*ip  ][jp] = (c[2ip][2jp]  , c[2ip+1][2jp+1])
            // acc2[2*ip+1][jp] = (c[2ip][2jp+1], c[2ip+1][2jp]  )
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

    // ---- main loop over K tiles -----------------------------------------------------------------
    for(int t = 0; t < ntiles; ++t)
    {
        cp_async_wait<STAGES - 2>(); // tile t has landed (this thread's copies)
        __syncthreads();             // ... and everybody's; everybody is also done reading tile t-1

        const int  s_cur  = t % STAGES;
        const int  t_next = t + STAGES - 1;
        const int  s_next = t_next % STAGES;
        const bool more   = t_next < ntiles;
        if(more)
        {
            const int k0 = k_begin + t_next * BK;
            stage_a.fetch(p.A, p.lda, p.M, m0, k0, k_end, p.vec_a, tile_a(s_next), tid);
            stage_b.fetch(p.B, p.ldb, p.N, n0, k0, k_end, p.vec_b, tile_b(s_next), tid);
        }

        const float* as = tile_a(s_cur);
        const float* bs = tile_b(s_cur);
        load_frags(0, as, bs, 0);
#pragma unroll
        for(int kk = 0; kk < BK; ++kk)
        {
            if(kk + 1 < BK)
                load_frags((kk + 1) & 1, as, bs, kk + 1);
            fma_step(kk & 1);
        }

        if(more)
        {
            // stage s_next was last read during iteration t-1, which every thread left before the
            // barrier at the top of this iteration
            stage_a.commit(tile_a(s_next), tid);
            stage_b.commit(tile_b(s_next), tid);
        }
        cp_async_commit();
    }
    cp_async_wait<0>();

    // ---- epilogue -------------------------------------------------------------------------------
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

    float* __restrict__ out = p.C + (long long)split * p.split_stride;
    store_tile<Cfg, LC, ALIGNED>(c, p, out, m0 + tm0, n0 + tn0);
}

} // namespace sgemm_b200
