// b200_sgemm_3xtf32: C = A * B on the 5th-generation tensor cores with FP32 operands split into two TF32
// halves (the "3xTF32" scheme).  A separate, optional entry beside the true-FP32 FMA path: it is NOT
// bit-identical to the reference's arithmetic (rocm_sgemm/include/rocm_sgemm/kernel/kernel.hpp:188-266
// is an FP32 FMA chain) and has no counterpart in the reference; it exists as a comparison column
// showing what the same FP32 problem costs when an error of a few 1e-7 relative is acceptable.
//
//   a = a_hi + a_lo,  a_hi = tf32(a),  a_lo = tf32(a - a_hi)          (both round-to-nearest)
//   A*B ~= A_lo*B_hi + A_hi*B_lo + A_hi*B_hi                          (FP32 accumulation in tensor memory)
//
// Kernel (one persistent CTA per SM, 128 x BN tiles, K blocks of 32 floats = one 128-byte swizzle row):
//   warp 8      TMA producer: cp.async.bulk.tensor.2d of the raw FP32 A and B tiles (K-major, 128B swizzle)
//   warps 4-7   converters: rewrite each tile in place as its hi half and write the lo half next to it
//               (elementwise, so the swizzled placement is preserved), then fence to the async proxy
//   warp 9      one thread issues tcgen05.mma.kind::tf32 (M=128, N=BN, K=8), 12 per K block, accumulating
//               into one of two TMEM accumulators; tcgen05.commit releases the stage / publishes the tile
//   warps 0-3   epilogue: tcgen05.ld the finished accumulator (warp w owns TMEM lanes 32w..32w+31 = tile
//               rows) and store C, while the MMA warp already works on the next tile in the other buffer
// Operands must be K-contiguous for this kernel (A row-major, B col-major); the host entry repacks the
// other layouts (and operands whose pitch is not a multiple of 16 bytes) into a scratch arena first.
// Every mbarrier wait is bounded; on a time-out the CTA records a status word, stops and frees its TMEM.
#include "../../include/b200_sgemm.h"
#include "sgemm_ws_kernel.cuh"

#include <cuda.h>
#include <cuda_runtime.h>

#include <map>
#include <mutex>

namespace
{
using namespace sgemm_b200;

constexpr int T_BM      = 128;
constexpr int T_BK      = 32; // floats: 128 bytes, one swizzle row
constexpr int T_THREADS = 320;
constexpr int T_CHUNK   = 2;  // K blocks accumulated inside the tensor core before the sum moves to registers
constexpr int T_ERR_WAIT = 16; // status bit: some wait in the tensor-core kernel timed out

__device__ int g_tf32_status;

template<int BN>
struct TLayout
{
    static constexpr int    A_BYTES     = T_BM * T_BK * 4; // 16 KB
    static constexpr int    B_BYTES     = BN * T_BK * 4;
    static constexpr int    STAGE_BYTES = 2 * (A_BYTES + B_BYTES); // hi + lo of both
    static constexpr int    STAGES      = (200 * 1024) / STAGE_BYTES;
    static constexpr size_t SMEM_BYTES  = size_t(STAGES) * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
    static constexpr int    TMEM_COLS   = 2 * BN; // two accumulators
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

// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes with the 128-byte swizzle:
// start address (16-byte units), leading byte offset (unused for this layout, 1), stride byte offset =
// 1024 bytes between groups of eight rows, descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc_k128(uint32_t smem_addr)
{
    return uint64_t((smem_addr & 0x3FFFFu) >> 4) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46)
           | (uint64_t(2) << 61);
}
// Instruction descriptor: FP32 accumulator, TF32 A and B, both K-major, N >> 3, M >> 4.
template<int BN>
__device__ __forceinline__ constexpr uint32_t umma_idesc_tf32()
{
    return (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(BN >> 3) << 17) | (uint32_t(T_BM >> 4) << 24);
}
__device__ __forceinline__ float to_tf32(float x)
{
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
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
    const uint32_t bar_base  = tile_base + STAGES * L::STAGE_BYTES;
    // barriers: raw_full[S], cvt_full[S], empty[S], acc_full[2], acc_empty[2]; then the TMEM address and the abort flag
    auto raw_full  = [&](int s) { return bar_base + 8u * s; };
    auto cvt_full  = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto empty     = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
    auto acc_full  = [&](int b) { return bar_base + 8u * (3 * STAGES + b); };
    auto acc_empty = [&](int b) { return bar_base + 8u * (3 * STAGES + 2 + b); };
    uint8_t*      misc       = tiles + STAGES * L::STAGE_BYTES + 8 * (3 * STAGES + 4);
    uint32_t*     tmem_slot  = reinterpret_cast<uint32_t*>(misc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(misc + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if(threadIdx.x == 0)
    {
        for(int s = 0; s < STAGES; ++s)
        {
            mbar_init(raw_full(s), 1);
            mbar_init(cvt_full(s), 128);
            mbar_init(empty(s), 1);
        }
        for(int b = 0; b < 2; ++b)
        {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), 128);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if(warp == 9)
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
    auto fail = [&]() {
        *abort_flag = 1;
        atomicOr(t.status, T_ERR_WAIT);
    };

    if(warp == 8)
    {
        // ---------------- TMA producer ----------------
        if(lane == 0)
        {
            uint32_t it = 0;
            bool     ok = true;
            for(int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x)
            {
                const int tm = tile % t.tiles_m, tn = tile / t.tiles_m;
                for(int kb = 0; kb < kblocks; ++kb, ++it)
                {
                    const int      s  = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if(!mbar_wait(empty(s), ph ^ 1, abort_flag)) { fail(); ok = false; break; }
                    const uint32_t st = tile_base + s * L::STAGE_BYTES;
                    mbar_arrive_expect_tx(raw_full(s), L::A_BYTES + L::B_BYTES);
                    tma_load_2d(st, &map_a, kb * T_BK, tm * T_BM, raw_full(s));
                    tma_load_2d(st + 2 * L::A_BYTES, &map_b, kb * T_BK, tn * BN, raw_full(s));
                }
            }
        }
    }
    else if(warp >= 4 && warp < 8)
    {
        // ---------------- converters: raw FP32 -> hi (in place) and lo ----------------
        const int ct = threadIdx.x - 128;
        uint32_t  it = 0;
        bool      ok = true;
        for(int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x)
        {
            for(int kb = 0; kb < kblocks; ++kb, ++it)
            {
                const int      s  = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                if(!mbar_wait(raw_full(s), ph, abort_flag)) { fail(); ok = false; break; }
                uint8_t* st = tiles + s * L::STAGE_BYTES;
                float4*  a_hi = reinterpret_cast<float4*>(st);
                float4*  a_lo = reinterpret_cast<float4*>(st + L::A_BYTES);
                float4*  b_hi = reinterpret_cast<float4*>(st + 2 * L::A_BYTES);
                float4*  b_lo = reinterpret_cast<float4*>(st + 2 * L::A_BYTES + L::B_BYTES);
                auto split = [](float4* hi, float4* lo, int i) {
                    const float4 v = hi[i];
                    float4       h, l;
                    h.x = to_tf32(v.x); h.y = to_tf32(v.y); h.z = to_tf32(v.z); h.w = to_tf32(v.w);
                    l.x = to_tf32(v.x - h.x); l.y = to_tf32(v.y - h.y); l.z = to_tf32(v.z - h.z); l.w = to_tf32(v.w - h.w);
                    hi[i] = h;
                    lo[i] = l;
                };
#pragma unroll
                for(int i = 0; i < L::A_BYTES / 16 / 128; ++i)
                    split(a_hi, a_lo, ct + 128 * i);
#pragma unroll
                for(int i = 0; i < L::B_BYTES / 16 / 128; ++i)
                    split(b_hi, b_lo, ct + 128 * i);
                fence_async_smem();
                mbar_arrive(cvt_full(s));
            }
        }
    }
    else if(warp == 9)
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
                    // a new partial accumulator every T_CHUNK K blocks (drained into registers by the epilogue warps)
                    const bool     first = kb % T_CHUNK == 0;
                    const uint32_t buf = ccount & 1, aph = (ccount >> 1) & 1;
                    if(first)
                    {
                        if(!mbar_wait(acc_empty(buf), aph ^ 1, abort_flag)) { fail(); ok = false; break; }
                        tc_fence_after();
                    }
                    const uint32_t d  = tmem_base + buf * BN;
                    const int      s  = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if(!mbar_wait(cvt_full(s), ph, abort_flag)) { fail(); ok = false; break; }
                    tc_fence_after();
                    const uint32_t st   = tile_base + s * L::STAGE_BYTES;
                    const uint32_t a_hi = st, a_lo = st + L::A_BYTES, b_hi = st + 2 * L::A_BYTES,
                                   b_lo = st + 2 * L::A_BYTES + L::B_BYTES;
#pragma unroll
                    for(int kk = 0; kk < T_BK / 8; ++kk)
                    {
                        const uint32_t off = kk * 32; // 8 TF32 = 32 bytes along the swizzled row
                        const uint64_t dah = umma_desc_k128(a_hi + off), dal = umma_desc_k128(a_lo + off);
                        const uint64_t dbh = umma_desc_k128(b_hi + off), dbl = umma_desc_k128(b_lo + off);
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
        // ---------------- accumulate + epilogue warps 0-3 ----------------
        // Thread = one row of the tile.  The tensor core adds into its FP32 accumulator with truncation, which
        // biases long sums; so the MMA warp starts a fresh TMEM accumulator every T_CHUNK K blocks and these
        // warps add the finished partial sums in registers with round-to-nearest.
        uint32_t ccount = 0;
        bool     ok     = true;
        const int chunks = (kblocks + T_CHUNK - 1) / T_CHUNK;
        for(int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x)
        {
            const int tm = tile % t.tiles_m, tn = tile / t.tiles_m;
            float     acc[BN];
            for(int ch = 0; ch < chunks; ++ch, ++ccount)
            {
                const uint32_t buf = ccount & 1, aph = (ccount >> 1) & 1;
                if(!mbar_wait(acc_full(buf), aph, abort_flag)) { fail(); ok = false; break; }
                tc_fence_after();
#pragma unroll
                for(int c = 0; c < BN / 32; ++c)
                {
                    uint32_t v[32];
                    tmem_ld32(tmem_base + buf * BN + c * 32 + (uint32_t(warp * 32) << 16), v);
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
                mbar_arrive(acc_empty(buf));
            }
            if(!ok)
                break;
            const int  row    = tm * T_BM + warp * 32 + lane;
            const bool row_ok = row < t.M;
#pragma unroll
            for(int c = 0; c < BN / 32; ++c)
            {
                const int col0 = tn * BN + c * 32;
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
    if(warp == 9)
    {
        tc_fence_after();
        tmem_dealloc(tmem_base, L::TMEM_COLS);
    }
}

// ---- repacking of operands that the kernel cannot read in place ------------------------------------------
// dst is R rows of Kp floats (K-contiguous, zero padded from K to Kp).  src is the packed R x K operand,
// either K-contiguous (src[r*K + k]) or R-contiguous (src[k*R + r]).
__global__ void __launch_bounds__(256) repack_kernel(float* __restrict__ dst, const float* __restrict__ src, int R, int K,
                                                     int Kp, int src_k_contiguous)
{
    __shared__ float tile[32][33];
    const int r0 = blockIdx.y * 32, k0 = blockIdx.x * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5; // 32 x 8
    if(src_k_contiguous)
    {
        for(int i = ty; i < 32; i += 8)
        {
            const int r = r0 + i, k = k0 + tx;
            if(r < R && k < Kp)
                dst[size_t(r) * Kp + k] = k < K ? src[size_t(r) * K + k] : 0.f;
        }
        return;
    }
    for(int i = ty; i < 32; i += 8)
    {
        const int k = k0 + i, r = r0 + tx;
        tile[i][tx] = (k < K && r < R) ? src[size_t(k) * R + r] : 0.f;
    }
    __syncthreads();
    for(int i = ty; i < 32; i += 8)
    {
        const int r = r0 + i, k = k0 + tx;
        if(r < R && k < Kp)
            dst[size_t(r) * Kp + k] = tile[tx][i];
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

// rows x K operand, K contiguous, pitch ld floats; box = 32 floats x box_rows rows, 128-byte swizzle
bool encode_kmajor(CUtensorMap* map, const float* base, size_t rows, size_t K, size_t ld, int box_rows)
{
    EncodeFn fn = encoder();
    if(!fn)
        return false;
    const cuuint64_t dims[2]    = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(float)};
    const cuuint32_t box[2]     = {(cuuint32_t)T_BK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2]    = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct Scratch
{
    float* a = nullptr;
    float* b = nullptr;
    size_t bytes_a = 0, bytes_b = 0;
    int*   status = nullptr;
    int    sms = 0;
    bool   attr_set[2] = {false, false};
};
std::mutex             g_mutex;
std::map<int, Scratch> g_scratch;

cudaError_t grow(float** p, size_t* have, size_t need)
{
    if(*have >= need)
        return cudaSuccess;
    if(*p)
        cudaFree(*p);
    *p    = nullptr;
    *have = 0;
    cudaError_t e = cudaMalloc(p, need);
    if(e == cudaSuccess)
        *have = need;
    return e;
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
        if((e = grow(&s.a, &s.bytes_a, M * Kp * sizeof(float))) != cudaSuccess) return (int)e;
        dim3 grid((unsigned)((Kp + 31) / 32), (unsigned)((M + 31) / 32));
        repack_kernel<<<grid, 256, 0, stream>>>(s.a, A, (int)M, (int)K, (int)Kp, layout_a == B200_SGEMM_ROW_MAJOR);
        a_src = s.a;
    }
    if(!b_direct)
    {
        if((e = grow(&s.b, &s.bytes_b, N * Kp * sizeof(float))) != cudaSuccess) return (int)e;
        dim3 grid((unsigned)((Kp + 31) / 32), (unsigned)((N + 31) / 32));
        repack_kernel<<<grid, 256, 0, stream>>>(s.b, B, (int)N, (int)K, (int)Kp, layout_b == B200_SGEMM_COL_MAJOR);
        b_src = s.b;
    }
    if((e = cudaPeekAtLastError()) != cudaSuccess)
        return (int)e;

    const int bn = 128;
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
    return launch<128>(s, 0, t, ma, mb, stream);
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
    for(auto& kv : g_scratch)
    {
        cudaSetDevice(kv.first);
        cudaFree(kv.second.a);
        cudaFree(kv.second.b);
    }
    g_scratch.clear();
    cudaSetDevice(saved);
    return B200_SGEMM_OK;
}
