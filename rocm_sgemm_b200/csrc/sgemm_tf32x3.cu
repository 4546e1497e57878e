// b200_sgemm_3xtf32: C = A * B on the 5th-generation tensor cores with FP32 operands split into two TF32
// halves (the "3xTF32" scheme).  A separate, optional entry beside the true-FP32 FMA path: it is NOT
// bit-identical to the reference's arithmetic (rocm_sgemm/include/rocm_sgemm/kernel/kernel.hpp:188-266
// is an FP32 FMA chain) and has no counterpart in the reference; it exists as a comparison column
// showing what the same FP32 problem costs when a relative error of about 2e-6 is acceptable.
//
//   a = a_hi + a_lo,  a_hi = a with its low 13 mantissa bits dropped (what the tensor core reads from the raw
//   word),  a_lo = the exact remainder a - a_hi rounded to nearest TF32
//   A*B ~= A_lo*B_hi + A_hi*B_lo + A_hi*B_hi                          (three tensor-core products)
//
// Kernel: one persistent CTA per SM (16 warps), 128 x 256 tiles, K blocks of 16 floats (= one 64-byte swizzle row),
// a ring of four 48 KB stages [A raw][B raw][A lo][B lo].
//   warp 12        TMA producer: cp.async.bulk.tensor.2d of the raw FP32 A and B tiles (K-major, 64B swizzle)
//   warps 8-11,14-15  converters.  The tensor core ignores the low 13 mantissa bits of an FP32 word it reads as
//                  TF32, so the raw tile is the hi half as it lies; the converters write lo = tf32(x - hi) at the
//                  same offset of a second buffer (elementwise, so the swizzled placement holds for both) and
//                  fence to the async proxy
//   warp 13        one thread issues tcgen05.mma.kind::tf32 (M=128, N=256, K=8), 6 per K block, into one of two
//                  accumulators in tensor memory (all 512 columns); tcgen05.commit releases the stage and, every
//                  T_CHUNK K blocks, publishes the partial sum
//   warps 0-7      accumulate + epilogue: tcgen05.ld the finished partial sum (warp w owns TMEM lanes 32*(w%4)..
//                  = tile rows, and columns 128*(w/4)..), add it to 128 register accumulators per thread, store C
//                  at the end of the tile.  The tensor core adds into its FP32 accumulator with truncation, which
//                  biases long sums (measured: error growing linearly with K, 2.4e-5 at K = 1024); moving the sum
//                  to registers (round-to-nearest adds) every 64 k keeps the error at about 1.7e-6 for every K.
//                  These warps get their registers from a converter warpgroup (setmaxnreg, see T_LAUNCH_REGS).
// Operands must be K-contiguous for this kernel (A row-major, B col-major); the host entry repacks the
// other layouts (and operands whose pitch is not a multiple of 16 bytes) into a scratch arena first.
// Every mbarrier wait is bounded; on a time-out the CTA records a status word, stops and frees its TMEM.
#include "../../include/b200_sgemm.h"
#include "sgemm_ws_kernel.cuh"
#include "transpose.hpp"

#include <cuda.h>
#include <cuda_runtime.h>

#include <map>
#include <mutex>

namespace
{
using namespace sgemm_b200;

constexpr int T_BM           = 128;
constexpr int T_BK           = 16;  // floats: 64 bytes, one swizzle row
constexpr int T_ACCUMULATORS = 256; // warps 0-7
constexpr int T_CONVERTERS   = 192; // warps 8-11 and 14-15
constexpr int T_TMA_WARP     = 12;
constexpr int T_MMA_WARP     = 13;
constexpr int T_THREADS      = 512;
// Register budget.  A launch of 512 threads gets 128 registers per thread (the whole file of 65 536).  The accumulate
// warps keep 128 partial sums per thread, so one converter warpgroup hands registers over (setmaxnreg works on whole
// warpgroups): 256 x 168 (warps 0-7) + 128 x 48 (warps 8-11) + 128 x 128 (warps 12-15, unchanged) = 65 536, exactly
// the launch allocation, so the increase can always be granted.  The host refuses to launch a build whose kernel
// was given fewer than T_LAUNCH_REGS registers.
constexpr int T_LAUNCH_REGS  = 128;
constexpr int T_ACC_REGS     = 168;
constexpr int T_CVT_REGS     = 48;
static_assert(T_ACCUMULATORS * T_ACC_REGS + 128 * T_CVT_REGS + 128 * T_LAUNCH_REGS == T_THREADS * T_LAUNCH_REGS,
              "register budgets must add up to the launch allocation");
constexpr int T_CHUNK        = 4;  // K blocks accumulated inside the tensor core before the sum moves to registers
constexpr int T_ERR_WAIT     = 16; // status bit: a wait in this kernel timed out; bits 8..13 say which one first

__device__ int g_tf32_status;

template<int BN>
struct TLayout
{
    static constexpr int    A_BYTES     = T_BM * T_BK * 4; // 8 KB
    static constexpr int    B_BYTES     = BN * T_BK * 4;   // 16 KB at BN = 256
    static constexpr int    STAGE_BYTES = 2 * (A_BYTES + B_BYTES); // raw (= hi) and lo halves of both tiles
    static constexpr int    STAGES      = (200 * 1024) / STAGE_BYTES;
    static constexpr int    BARRIERS    = 3 * STAGES + 4;
    static constexpr size_t SMEM_BYTES  = size_t(STAGES) * STAGE_BYTES + 1024 /*alignment slack*/
                                         + 256 /*barriers, TMEM address, abort flag*/;
    static constexpr int    TMEM_COLS   = 2 * BN; // two partial accumulators
    static_assert(8 * BARRIERS + 16 <= 256, "barrier area");
    static_assert(TMEM_COLS <= 512, "tensor memory has 512 columns");
};

struct TArgs
{
    float* C;
    int    M, N, K;
    int    ldc;
    int    layout_c;
    int    tiles_m, tiles_n;
    int*   status;
};

// ---- tcgen05 helpers ---------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// 32 lanes x 32 columns of 32-bit accumulators: thread = lane (row), v[j] = column j
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                   "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                   "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile stored as rows of T_BK floats (64 bytes) with the 64-byte
// swizzle: start address (16-byte units), leading byte offset (unused for this layout, 1), stride byte offset =
// 512 bytes between groups of eight rows, descriptor version 1, layout type 4 (SWIZZLE_64B).
__device__ __forceinline__ uint64_t umma_desc_kmajor(uint32_t smem_addr)
{
    static_assert(T_BK * 4 == 64, "descriptor written for 64-byte rows");
    return uint64_t((smem_addr & 0x3FFFFu) >> 4) | (uint64_t(1) << 16) | (uint64_t(512 >> 4) << 32) | (uint64_t(1) << 46)
           | (uint64_t(4) << 61);
}
// Instruction descriptor: FP32 accumulator, TF32 A and B, both K-major, N >> 3, M >> 4.
template<int BN>
__device__ __forceinline__ constexpr uint32_t umma_idesc_tf32()
{
    return (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(BN >> 3) << 17) | (uint32_t(T_BM >> 4) << 24);
}
// lo half of x for a hi half that is x with its low 13 mantissa bits dropped (what the tensor core sees when it reads
// the raw word): x - hi is exact in FP32; it is rounded to nearest TF32 with integer instructions (measured 9 %
// faster for the whole kernel than cvt.rna.tf32.f32, whose issue rate is lower).
__device__ __forceinline__ float lo_half(float x)
{
    const float hi = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
    return __uint_as_float((__float_as_uint(x - hi) + 0x1000u) & 0xFFFFE000u);
}

// Tile order: bands of 16 tile rows, tile columns advancing inside a band, so that the CTAs running at the same
// time share 16 row panels of A and about nine column panels of B (about 100 MB at K = 8192: within the L2).
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn)
{
    constexpr int BAND = 16;
    const int     band = tile / (BAND * tiles_n);
    const int     rows = min(BAND, tiles_m - band * BAND);
    const int     idx  = tile - band * BAND * tiles_n;
    tm = band * BAND + idx % rows;
    tn = idx / rows;
}

template<int BN>
__global__ void __launch_bounds__(T_THREADS, 1)
    sgemm_tf32x3_kernel(const __grid_constant__ TArgs t, const __grid_constant__ CUtensorMap map_a,
                        const __grid_constant__ CUtensorMap map_b)
{
    using L = TLayout<BN>;
    constexpr int STAGES = L::STAGES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr  = (uint32_t)__cvta_generic_to_shared(smem_raw);
    const uint32_t tile_base = (raw_addr + 1023u) & ~1023u;
    uint8_t*       tiles     = smem_raw + (tile_base - raw_addr);
    // stage: [A as TMA wrote it = hi half][B likewise][A lo half][B lo half]; then the barriers
    const uint32_t bar_base = tile_base + STAGES * L::STAGE_BYTES;
    auto raw_full  = [&](int s) { return bar_base + 8u * s; };
    auto cvt_full  = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto empty     = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
    auto acc_full  = [&](int b) { return bar_base + 8u * (3 * STAGES + b); };
    auto acc_empty = [&](int b) { return bar_base + 8u * (3 * STAGES + 2 + b); };
    uint8_t*      misc       = tiles + STAGES * L::STAGE_BYTES + 8 * L::BARRIERS;
    uint32_t*     tmem_slot  = reinterpret_cast<uint32_t*>(misc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(misc + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if(threadIdx.x == 0)
    {
        for(int s = 0; s < STAGES; ++s)
        {
            mbar_init(raw_full(s), 1);
            mbar_init(cvt_full(s), T_CONVERTERS / 32);
            mbar_init(empty(s), 1);
        }
        for(int b = 0; b < 2; ++b)
        {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), T_ACCUMULATORS / 32);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if(warp == T_MMA_WARP)
    {
        tmem_alloc((uint32_t)__cvta_generic_to_shared(tmem_slot), L::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int total_tiles = t.tiles_m * t.tiles_n;
    const int kblocks     = (t.K + T_BK - 1) / T_BK;
    // the first wait of the CTA that gives up records where (bits 8..13) and raises the abort flag for the others
    auto fail = [&](int where) {
        if(atomicExch(const_cast<int*>(abort_flag), 1) == 0)
            atomicOr(t.status, T_ERR_WAIT | (256 << where));
    };

    if(warp == T_TMA_WARP)
    {
        // ---------------- TMA producer ----------------
        if(lane == 0)
        {
            uint32_t it = 0;
            bool     ok = true;
            for(int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x)
            {
                int tm, tn;
                tile_coords(tile, t.tiles_m, t.tiles_n, tm, tn);
                for(int kb = 0; kb < kblocks; ++kb, ++it)
                {
                    const int      s  = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if(!mbar_wait(empty(s), ph ^ 1, abort_flag)) { fail(0); ok = false; break; }
                    const uint32_t st = tile_base + s * L::STAGE_BYTES;
                    mbar_arrive_expect_tx(raw_full(s), L::A_BYTES + L::B_BYTES);
                    tma_load_2d(st, &map_a, kb * T_BK, tm * T_BM, raw_full(s));
                    tma_load_2d(st + L::A_BYTES, &map_b, kb * T_BK, tn * BN, raw_full(s));
                }
            }
        }
    }
    else if(warp >= T_ACCUMULATORS / 32 && warp != T_MMA_WARP)
    {
        // ---------------- converters: lo half of the raw tiles ----------------
        if(warp < T_TMA_WARP) // the whole warpgroup 8-11 gives registers up; warps 14-15 keep theirs
            asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(T_CVT_REGS));
        // The tensor core ignores the low 13 mantissa bits of an FP32 word it reads as TF32, so the raw tile IS the
        // hi half (hi = the word truncated).  The converters add the lo half, lo = tf32(x - hi), elementwise and at
        // the same offset in a second buffer, so the swizzled placement TMA applied holds for both.
        const int ct = warp < T_TMA_WARP ? threadIdx.x - T_ACCUMULATORS : threadIdx.x - T_ACCUMULATORS - 64;
        uint32_t  it = 0;
        bool      ok = true;
        for(int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x)
        {
            for(int kb = 0; kb < kblocks; ++kb, ++it)
            {
                const int      s  = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                if(!mbar_wait(raw_full(s), ph, abort_flag)) { fail(1); ok = false; break; }
                const float4* raw = reinterpret_cast<const float4*>(tiles + s * L::STAGE_BYTES);
                float4*       lo  = reinterpret_cast<float4*>(tiles + s * L::STAGE_BYTES + L::A_BYTES + L::B_BYTES);
                constexpr int NV = (L::A_BYTES + L::B_BYTES) / 16 / T_CONVERTERS; // 16-byte chunks per thread
                static_assert(NV * T_CONVERTERS * 16 == L::A_BYTES + L::B_BYTES && NV % 4 == 0, "converter split");
#pragma unroll
                for(int r = 0; r < NV; r += 4) // four loads in flight at a time: fits the reduced register budget
                {
                    float4 v[4];
#pragma unroll
                    for(int i = 0; i < 4; ++i)
                        v[i] = raw[ct + T_CONVERTERS * (r + i)];
#pragma unroll
                    for(int i = 0; i < 4; ++i)
                        lo[ct + T_CONVERTERS * (r + i)] =
                            make_float4(lo_half(v[i].x), lo_half(v[i].y), lo_half(v[i].z), lo_half(v[i].w));
                }
                fence_async_smem(); // the lo tiles are read by the tensor core (async proxy)
                __syncwarp();
                if(lane == 0) // one arrival per warp
                    mbar_arrive(cvt_full(s));
            }
        }
    }
    else if(warp == T_MMA_WARP)
    {
        // ---------------- MMA issuer ----------------
        if(lane == 0)
        {
            constexpr uint32_t idesc = umma_idesc_tf32<BN>();
            uint32_t           it = 0, ccount = 0;
            bool               ok = true;
            for(int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x)
            {
                for(int kb = 0; kb < kblocks; ++kb, ++it)
                {
                    // a new partial accumulator every T_CHUNK K blocks (drained into registers by the accumulate warps)
                    const bool     first = kb % T_CHUNK == 0;
                    const uint32_t buf = ccount & 1, aph = (ccount >> 1) & 1;
                    if(first)
                    {
                        if(!mbar_wait(acc_empty(buf), aph ^ 1, abort_flag)) { fail(3); ok = false; break; }
                        tc_fence_after();
                    }
                    const uint32_t d  = tmem_base + buf * BN;
                    const int      s  = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if(!mbar_wait(cvt_full(s), ph, abort_flag)) { fail(4); ok = false; break; }
                    tc_fence_after();
                    const uint32_t st   = tile_base + s * L::STAGE_BYTES;
                    const uint32_t a_hi = st, b_hi = st + L::A_BYTES, a_lo = b_hi + L::B_BYTES, b_lo = a_lo + L::A_BYTES;
#pragma unroll
                    for(int kk = 0; kk < T_BK / 8; ++kk)
                    {
                        const uint32_t off = kk * 32; // 8 TF32 = 32 bytes along the swizzled row
                        const uint64_t dah = umma_desc_kmajor(a_hi + off), dal = umma_desc_kmajor(a_lo + off);
                        const uint64_t dbh = umma_desc_kmajor(b_hi + off), dbl = umma_desc_kmajor(b_lo + off);
                        tc_mma_tf32(d, dal, dbh, idesc, !(first && kk == 0));
                        tc_mma_tf32(d, dah, dbl, idesc, 1);
                        tc_mma_tf32(d, dah, dbh, idesc, 1);
                    }
                    tc_commit(empty(s)); // the stage may be refilled once these MMAs have read it
                    if(kb % T_CHUNK == T_CHUNK - 1 || kb == kblocks - 1)
                    {
                        tc_commit(acc_full(buf)); // the partial sum is complete once every MMA above has finished
                        ++ccount;
                    }
                }
            }
        }
    }
    else
    {
        // ---------------- accumulate + epilogue warps ----------------
        // Thread = one row of the tile and one half of its columns (warp w: TMEM lanes 32*(w%4).., columns
        // (w/4)*BN/2..).  The tensor core adds into its FP32 accumulator with truncation, which biases long
        // sums; so the MMA warp starts a fresh TMEM accumulator every T_CHUNK K blocks and these warps add
        // the finished partial sums in registers with round-to-nearest.
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(T_ACC_REGS));
        constexpr int HALF = BN / 2;
        const int     q = warp & 3, h = warp >> 2;
        uint32_t      ccount = 0;
        bool          ok     = true;
        const int     chunks = (kblocks + T_CHUNK - 1) / T_CHUNK;
        for(int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x)
        {
            int tm, tn;
            tile_coords(tile, t.tiles_m, t.tiles_n, tm, tn);
            float acc[HALF];
            for(int ch = 0; ch < chunks; ++ch, ++ccount)
            {
                const uint32_t buf = ccount & 1, aph = (ccount >> 1) & 1;
                if(!mbar_wait(acc_full(buf), aph, abort_flag)) { fail(5); ok = false; break; }
                tc_fence_after();
#pragma unroll
                for(int c = 0; c < HALF / 32; ++c)
                {
                    uint32_t v[32];
                    tmem_ld32(tmem_base + buf * BN + h * HALF + c * 32 + (uint32_t(q * 32) << 16), v);
                    tmem_ld_wait();
                    if(ch == 0)
                    {
#pragma unroll
                        for(int j = 0; j < 32; ++j)
                            acc[c * 32 + j] = __uint_as_float(v[j]);
                    }
                    else
                    {
#pragma unroll
                        for(int j = 0; j < 32; ++j)
                            acc[c * 32 + j] += __uint_as_float(v[j]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if(lane == 0)
                    mbar_arrive(acc_empty(buf));
            }
            if(!ok)
                break;
            const int  row    = tm * T_BM + q * 32 + lane;
            const bool row_ok = row < t.M;
#pragma unroll
            for(int c = 0; c < HALF / 32; ++c)
            {
                const int col0 = tn * BN + h * HALF + c * 32;
                if(t.layout_c == B200_SGEMM_ROW_MAJOR)
                {
                    if(row_ok)
                    {
                        float* dst = t.C + size_t(row) * t.ldc + col0;
                        if(col0 + 32 <= t.N && (t.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(t.C) & 15) == 0)
                        {
#pragma unroll
                            for(int j = 0; j < 32; j += 4)
                                *reinterpret_cast<float4*>(dst + j) =
                                    make_float4(acc[c * 32 + j], acc[c * 32 + j + 1], acc[c * 32 + j + 2], acc[c * 32 + j + 3]);
                        }
                        else
                        {
#pragma unroll
                            for(int j = 0; j < 32; ++j)
                                if(col0 + j < t.N)
                                    dst[j] = acc[c * 32 + j];
                        }
                    }
                }
                else
                {
#pragma unroll
                    for(int j = 0; j < 32; ++j)
                        if(row_ok && col0 + j < t.N)
                            t.C[size_t(col0 + j) * t.ldc + row] = acc[c * 32 + j];
                }
            }
        }
    }

    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if(warp == T_MMA_WARP)
    {
        tc_fence_after();
        tmem_dealloc(tmem_base, L::TMEM_COLS);
    }
}

// ---- repacking of operands that the kernel cannot read in place ------------------------------------------
// A K-contiguous operand whose pitch is not a multiple of 16 bytes (K % 4 != 0) or whose base is misaligned is copied
// into R rows of Kp floats (zero padded from K to Kp).  Operands that are not K-contiguous go through the library's
// transposition (launch_transpose) instead.
// One-dimensional grid (k-blocks fastest): neither extent is bound by the 65535 limit of gridDim.y.
__global__ void __launch_bounds__(256) repack_kernel(float* __restrict__ dst, const float* __restrict__ src, int R, int K,
                                                     int Kp, unsigned k_blocks)
{
    const unsigned rb = blockIdx.x / k_blocks;
    const int      r0 = (int)rb * 32, k0 = (int)(blockIdx.x - rb * k_blocks) * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5; // 32 x 8
    for(int i = ty; i < 32; i += 8)
    {
        const int r = r0 + i, k = k0 + tx;
        if(r < R && k < Kp)
            dst[size_t(r) * Kp + k] = k < K ? src[size_t(r) * K + k] : 0.f;
    }
}

// ---- host side -----------------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encoder()
{
    static EncodeFn fn = [] {
        void*                            p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess
           || q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeFn>(p);
    }();
    return fn;
}

// rows x K operand, K contiguous, pitch ld floats; box = T_BK floats (64 bytes) x box_rows rows, 64-byte swizzle
bool encode_kmajor(CUtensorMap* map, const float* base, size_t rows, size_t K, size_t ld, int box_rows)
{
    EncodeFn fn = encoder();
    if(!fn)
        return false;
    // the encoder is a driver call: the device's context must be current in this host thread
    static thread_local bool context_bound = false;
    if(!context_bound)
    {
        int device = 0;
        if(cudaGetDevice(&device) == cudaSuccess)
            cudaSetDevice(device);
        context_bound = true;
    }
    const cuuint64_t dims[2]    = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(float)};
    const cuuint32_t box[2]     = {(cuuint32_t)T_BK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2]    = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// per device: facts looked up once.  per (device, stream): the repack buffers, so that calls on different
// streams never share one (a second call's repack would overwrite what the first call's kernel still reads).
struct Scratch
{
    int* status = nullptr;
    int  sms = 0;
    bool attr_set[2] = {false, false};
};
struct Repack
{
    float* a = nullptr;
    float* b = nullptr;
    size_t bytes_a = 0, bytes_b = 0;
};
std::mutex                                     g_mutex;
std::map<int, Scratch>                         g_scratch;
std::map<std::pair<int, cudaStream_t>, Repack> g_repack;

cudaError_t grow(float** p, size_t* have, size_t need, cudaStream_t stream)
{
    if(*have >= need)
        return cudaSuccess;
    if(*p)
    {
        // kernels queued on this stream may still read the old block
        cudaError_t e = cudaStreamSynchronize(stream);
        if(e != cudaSuccess)
            return e;
        cudaFree(*p);
    }
    *p    = nullptr;
    *have = 0;
    cudaError_t e = cudaMalloc(p, need);
    if(e == cudaSuccess)
        *have = need;
    return e;
}

cudaError_t launch_repack(float* dst, const float* src, size_t R, size_t K, size_t Kp, cudaStream_t stream)
{
    const unsigned long long kb = (Kp + 31) / 32, rb = (R + 31) / 32;
    if(kb * rb > 0x7fffffffull)
        return cudaErrorInvalidConfiguration;
    repack_kernel<<<(unsigned)(kb * rb), 256, 0, stream>>>(dst, src, (int)R, (int)K, (int)Kp, (unsigned)kb);
    return cudaPeekAtLastError();
}

template<int BN>
int launch(Scratch& s, int which, const TArgs& t, const CUtensorMap& ma, const CUtensorMap& mb, cudaStream_t stream)
{
    auto kernel = sgemm_tf32x3_kernel<BN>;
    if(!s.attr_set[which])
    {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TLayout<BN>::SMEM_BYTES);
        if(e != cudaSuccess)
            return (int)e;
        cudaFuncAttributes fa;
        if((e = cudaFuncGetAttributes(&fa, kernel)) != cudaSuccess)
            return (int)e;
        if(fa.numRegs < T_LAUNCH_REGS) // the register hand-over inside the kernel would not add up
            return B200_SGEMM_NO_KERNEL;
        s.attr_set[which] = true;
    }
    const int tiles = t.tiles_m * t.tiles_n;
    const int grid  = tiles < s.sms ? tiles : s.sms;
    kernel<<<grid, T_THREADS, TLayout<BN>::SMEM_BYTES, stream>>>(t, ma, mb);
    return (int)cudaPeekAtLastError();
}
} // namespace

extern "C" int b200_sgemm_3xtf32(int layout_c, int layout_a, int layout_b, float* C, const float* A, const float* B,
                                 size_t M, size_t N, size_t K, void* cuda_stream)
{
    if(!C || !A || !B || M == 0 || N == 0 || K == 0 || (layout_a | layout_b | layout_c) & ~1)
        return B200_SGEMM_INVALID_ARGUMENT;
    if(M > (1u << 30) || N > (1u << 30) || K > (1u << 30))
        return B200_SGEMM_UNSUPPORTED_SIZE;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    int          device = 0;
    cudaError_t  e      = cudaGetDevice(&device);
    if(e != cudaSuccess)
        return (int)e;
    std::lock_guard<std::mutex> lock(g_mutex);
    Scratch&                    s = g_scratch[device];
    Repack&                     r = g_repack[std::make_pair(device, stream)];
    if(!s.status)
    {
        if((e = cudaDeviceGetAttribute(&s.sms, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess) return (int)e;
        if((e = cudaGetSymbolAddress(reinterpret_cast<void**>(&s.status), g_tf32_status)) != cudaSuccess) return (int)e;
    }
    const size_t Kp       = (K + 3) / 4 * 4;
    const bool   a_direct = layout_a == B200_SGEMM_ROW_MAJOR && K == Kp && (reinterpret_cast<uintptr_t>(A) & 15) == 0;
    const bool   b_direct = layout_b == B200_SGEMM_COL_MAJOR && K == Kp && (reinterpret_cast<uintptr_t>(B) & 15) == 0;
    const float* a_src    = A;
    const float* b_src    = B;
    if(!a_direct)
    {
        if((e = grow(&r.a, &r.bytes_a, M * Kp * sizeof(float), stream)) != cudaSuccess) return (int)e;
        if(layout_a == B200_SGEMM_ROW_MAJOR) // K-contiguous already: copy with the padded pitch
        {
            if((e = launch_repack(r.a, A, M, K, Kp, stream)) != cudaSuccess) return (int)e;
        }
        else // col-major A = K rows of M contiguous floats -> M rows of K (the pad columns are never read)
        {
            if((e = launch_transpose(A, r.a, K, M, M, Kp, stream)) != cudaSuccess) return (int)e;
        }
        a_src = r.a;
    }
    if(!b_direct)
    {
        if((e = grow(&r.b, &r.bytes_b, N * Kp * sizeof(float), stream)) != cudaSuccess) return (int)e;
        if(layout_b == B200_SGEMM_COL_MAJOR)
        {
            if((e = launch_repack(r.b, B, N, K, Kp, stream)) != cudaSuccess) return (int)e;
        }
        else // row-major B = K rows of N contiguous floats -> N rows of K
        {
            if((e = launch_transpose(B, r.b, K, N, N, Kp, stream)) != cudaSuccess) return (int)e;
        }
        b_src = r.b;
    }
    if((e = cudaPeekAtLastError()) != cudaSuccess)
        return (int)e;

    const int bn = 256;
    CUtensorMap ma, mb;
    if(!encode_kmajor(&ma, a_src, M, K, Kp, T_BM) || !encode_kmajor(&mb, b_src, N, K, Kp, bn))
        return B200_SGEMM_NO_KERNEL;
    TArgs t;
    t.C        = C;
    t.M        = (int)M;
    t.N        = (int)N;
    t.K        = (int)K;
    t.layout_c = layout_c;
    t.ldc      = (int)(layout_c == B200_SGEMM_ROW_MAJOR ? N : M);
    t.tiles_m  = (int)((M + T_BM - 1) / T_BM);
    t.tiles_n  = (int)((N + bn - 1) / bn);
    t.status   = s.status;
    return launch<256>(s, 0, t, ma, mb, stream);
}

extern "C" int b200_sgemm_3xtf32_device_status(void)
{
    cudaError_t e = cudaDeviceSynchronize();
    if(e != cudaSuccess)
        return -(int)e;
    int v = 0, zero = 0;
    if((e = cudaMemcpyFromSymbol(&v, g_tf32_status, sizeof(int))) != cudaSuccess)
        return -(int)e;
    if(v != 0)
        cudaMemcpyToSymbol(g_tf32_status, &zero, sizeof(int));
    return v;
}


extern "C" int b200_sgemm_3xtf32_shutdown(void)
{
    std::lock_guard<std::mutex> lock(g_mutex);
    int                         saved = 0;
    cudaGetDevice(&saved);
    for(auto& kv : g_repack)
    {
        cudaSetDevice(kv.first.first);
        cudaFree(kv.second.a);
        cudaFree(kv.second.b);
    }
    g_repack.clear();
    cudaSetDevice(saved);
    return B200_SGEMM_OK;
}
