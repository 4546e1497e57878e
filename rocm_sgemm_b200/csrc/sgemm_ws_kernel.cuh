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
//   * PRODUCER warps fill the ring.  An operand whose M / N extent is contiguous in global memory
//     (A col-major, B row-major) is fetched by ONE thread with a TMA tile copy (cp.async.bulk.tensor.2d;
//     out-of-bounds elements are zero-filled by the hardware) that signals the stage's mbarrier by byte
//     count.  A K-contiguous operand (A row-major, B col-major) also arrives by TMA, as a [rows][32 k] box
//     with the 128-byte swizzle in a small staging ring; the other producer warps move it from there into the
//     stage's plain [k][x] tile as 4 x 4 blocks (four 128-bit reads, transposition in registers, four 128-bit
//     writes, both sides conflict-free thanks to the row order the tensor map gives the slot).  The consumers
//     read every operand the same way, no thread ever waits on global memory and ragged K edges are the
//     hardware's zero fill.  Operands that do not meet TMA's alignment
//     rules (or K tiles other than 32) take the older route through registers: 128-bit global loads /
//     guarded cp.async issued by all four producer warps.
//     When the host has rebound a K-contiguous operand to scratch memory that is to hold it as [K][X] (WsArgs::coop_*),
//     both operands take the TMA route from the start and the three producer warps it leaves idle fill that scratch:
//     every block of block_x rows x block_k columns is transposed once, by whichever warp of the grid it falls to, K tile
//     by K tile, and published through a flag word that the copy-issuing thread acquires before it fetches a stage.
//   * the CTA is persistent and the producers run ahead into the next piece of work while the consumers store C.
//     Two schedules (WsArgs::sched):
//       0  work units (tile, K slice) dealt round-robin: blockIdx.x, +gridDim.x, ...
//       1  the tiles' K tiles, laid end to end in tile order, are cut into gridDim.x equal contiguous ranges, one
//          per CTA, so every CTA does the same amount of work whatever the tile count (no partly filled last wave).
//          A range starts inside one tile and ends inside another.  The CTA computes the HEAD of its last tile first
//          (k from 0) and parks the accumulators in global memory; it finishes with the TAIL of its first tile, whose
//          accumulators it takes over from the neighbour that computed that tile's head at the very start of the
//          kernel.  Every C element is therefore still ONE k-ascending FMA chain (bit-identical to schedule 0
//          without split-K); the chain merely changes hands once.  Needs ranges of at least one whole tile
//          (tiles >= CTAs), so that no tile is shared by more than two CTAs.
//       2  the same equal ranges when there are FEWER tiles than CTAs (small or skinny problems): a tile is then shared
//          by several CTAs, each of which runs its K range as a chain of its own starting from zero.  All but the last
//          range of a tile are parked; the CTA that owns the last range waits for them and adds them to its own chain
//          in ascending K order, so the result is the deterministic ordered sum of chains - the arithmetic of
//          split-K with tile-dependent cut points, which ws_stream_cuts() reports to the host.
//
// Packed FMA: the B fragment supplies natural pairs of neighbouring columns (64-bit halves of the
// 128-bit shared-memory read), the A value is duplicated into both halves.  The FMA order keeps the pair
// fixed and cycles the duplicated operand (measured 4 % faster on B200 than the opposite order).  Every C
// element is one k-ascending FMA chain, bit-identical to the other kernels and to the CPU oracle.
//
// Every wait on an mbarrier is bounded (one second of wall-clock time): then the thread records an error in
// *status, raises the CTA's abort flag and leaves; nobody waits forever on a peer that bailed out.
#pragma once
#include "sgemm_kernel.cuh"
#include <cuda.h>

namespace sgemm_b200
{

// Producer threads per CTA: one warpgroup beside 8 or more consumer warps, two warps beside fewer - and two warps
// beside consumers whose thread tile holds more than 64 accumulators.  Those need about 190 registers; with
// 256 + 64 threads per CTA the launch bound itself allows 204, so the compiler allocates them directly.  (Handing
// registers over from a producer warpgroup with setmaxnreg also works, but the code the compiler made for the
// enlarged budget moved values between registers about ten times per k-step - counted with the profiler's
// per-opcode instruction counters - and ran at 80 % of the FMA rate where the same loop alone reaches 93 %.  The
// launch bound cannot be raised by dropping warps either: with nine to twelve warps per CTA an SM sub-partition
// holds three of them and the compiler's bound is 168 whatever the thread count; only eight warps allow 255, and
// a build without producer warps - one consumer thread issuing the TMA copies between its FMAs - measured 3 %
// slower with the 8 x 8 tile and 60.9 TFLOP/s with the 16 x 8 tile at 8192^3.)
__host__ __device__ constexpr int ws_producer_threads(int consumer_threads, int accumulators_per_thread)
{
    return (consumer_threads >= 256 && accumulators_per_thread <= 64) ? 128 : 64;
}
constexpr int      WS_MAX_EXTRA     = 7; // peers of an 8-GPU node
#ifdef WS_SELFTEST_LIMITS
// the self-test's private copy of the kernel (sgemm_selftest.cu) gives up after a millisecond
constexpr uint32_t WS_SPIN_LIMIT    = 1u << 10;
constexpr uint64_t WS_WAIT_LIMIT_NS = 1000ull * 1000ull;
#else
constexpr uint32_t WS_SPIN_LIMIT    = 1u << 22;
constexpr uint64_t WS_WAIT_LIMIT_NS = 1000ull * 1000ull * 1000ull; // one second per wait
#endif

// status word values written by the kernel (0 = ok)
constexpr int WS_ERR_FULL_TIMEOUT  = 1; // a consumer gave up waiting for a stage to fill
constexpr int WS_ERR_EMPTY_TIMEOUT = 2; // a producer gave up waiting for a stage to drain
constexpr int WS_ERR_PEER_TIMEOUT  = 3; // a consumer gave up waiting for the neighbour CTA's parked accumulators
constexpr int WS_ERR_COOP_TIMEOUT  = 4; // the copy-issuing thread gave up waiting for a block of a transposed operand

struct WsArgs
{
    GemmArgs g;
    int      total_units;  // tiles * splits
    int      tma_a, tma_b; // 1: the operand is fetched by TMA straight into the stage through the tensor map below
    int      stg_a, stg_b; // 1: K-contiguous operand fetched by TMA into the staging ring and transposed from there
    int*     status;       // device status word
    // Further destinations of the result (same leading dimension as C): the tile is stored to each of them as well.
    // Used to write this GPU's block of C straight into the other GPUs' copies of C through peer mappings, which
    // folds the all-gather that follows a column-sharded product into the epilogue.  Only without split-K.
    int      n_extra;
    float*   extra_c[WS_MAX_EXTRA];
    // schedules 1 and 2 (see the head of this file)
    int       sched;
    int       k_tiles;  // K tiles per tile: ceil(K / block_k)
    int       rr_tiles; // schedule 1: this many leading tiles (a multiple of gridDim.x) are dealt round-robin as whole
                        // tiles first - neighbouring CTAs then work on neighbouring tiles, which the L2 likes -
                        // and only the rest (between one and two waves) is cut into equal ranges
    float*    handover; // gridDim.x slots of block_m x block_n floats: slot c holds what CTA c parked
    unsigned* flags;    // one word per (CTA, consumer warp): == epoch once that warp's part of slot c is complete
    unsigned  epoch;    // differs from launch to launch, so the words never need clearing
    // schedules 1 and 2: the units cut into ranges, (tiles - rr_tiles) * k_tiles = range_q * gridDim.x + range_r
    long long range_q;
    unsigned  range_r;
    // Batch of equal problems at fixed element strides (batch 1: one problem).  The tile sequence of all schedules is
    // then batch x (grid_m x grid_n) long: tile id = matrix * tiles_per_matrix + tile.  The tensor maps carry the
    // batch as one more dimension; bstep_a / bstep_b are 0 for an operand that all problems share.
    int       batch;
    int       bstep_a, bstep_b;
    long long stride_a, stride_b, stride_c;
    // In-kernel transposition of K-contiguous operands ("cooperative": every block is transposed once, by whichever
    // CTA it falls to, for all CTAs that will read it).  coop_src_x != nullptr: g.A / g.B points at scratch memory that
    // is to hold the operand as [K][X]; the producer warps that the TMA route leaves idle transpose it there from
    // coop_src_x ([X rows][K], pitch coop_ld_x) in blocks of block_x rows x block_k columns, K tile by K tile, and
    // publish each block through one word of coop_flags (== epoch: in place).  The thread that issues the TMA copies
    // waits for the words of the two blocks a stage needs.  Block of A: word kt * XT + tile_m; block of B: word
    // kt * XT + XA + tile_n, where XA = grid_m if A is transposed here (else 0) and XT = XA + (grid_n if B is).
    const float* coop_src_a;
    const float* coop_src_b;
    long long    coop_ld_a, coop_ld_b;
    unsigned*    coop_flags;
    // Every transposing warp adds one to *coop_done when its last block is published; the word is never cleared (the
    // launches that use it are ordered by their stream): coop_done_target is what it reads once all warps of THIS
    // launch have finished, i.e. the total over all launches so far, modulo 2^32.
    unsigned*    coop_done;
    unsigned     coop_done_target;
    // The epilogue stores alpha * (A B) + beta * C (three separately rounded operations, C read only when beta != 0).
    // alpha = 1, beta = 0 everywhere except in the vendor-BLAS convention's entry, which uses other values only without
    // K slices and without further destinations.
    float alpha, beta;
    // Self-test only (0 everywhere else): the thread that issues the TMA copies leaves out the very last K tile of its
    // last piece - no copy, no arrival - so the consumers' wait for that stage runs into its limit.
    int       test_omit_last_fill;
};

// One contiguous piece of work of a CTA: K range [k_begin, k_end) of one tile.
struct WsPiece
{
    int tile_id;
    int k_begin, k_end;
    int split;  // schedule 0: index of the K slice (selects the partial-sum matrix)
    int recv;   // schedule 1, >= 0: start from the accumulators parked in this slot instead of zero
    int send;   // >= 0: park the accumulators in this slot instead of storing C
    int reduce; // schedule 2, >= 0: before storing C add the parked accumulators of slots reduce .. blockIdx.x-1
};

// First unit (K tile of the tile sequence) of CTA c when `units` units are cut into `ctas` equal ranges.
__host__ __device__ inline long long ws_range_begin(long long units, int ctas, int c)
{
    return units * c / ctas;
}

// The same value from units = q * ctas + r (q, r from the host): q * c + floor(r * c / ctas).  r * c stays below
// ctas^2, so the device divides 32-bit numbers instead of 64-bit ones (the schedule is set up before the first copy
// can be issued: its arithmetic is on the critical path of a short kernel).
__device__ __forceinline__ long long ws_range_begin_qr(long long q, unsigned r, unsigned ctas, unsigned c)
{
    return q * (long long)c + (long long)(ctas < 65536u ? (r * c) / ctas : (unsigned)(((unsigned long long)r * c) / ctas));
}
// floor and remainder of u / kts, with 32-bit division when u fits
__device__ __forceinline__ void ws_divmod(long long u, int kts, int& quo, int& rem)
{
    if(u <= 0x7fffffffLL)
    {
        const unsigned uu = (unsigned)u;
        quo = (int)(uu / (unsigned)kts);
        rem = (int)(uu - (unsigned)quo * (unsigned)kts);
    }
    else
    {
        const long long x = u / kts;
        quo = (int)x;
        rem = (int)(u - x * kts);
    }
}

// The list of pieces of this CTA, identical for its producer and consumer threads.
struct WsSchedule
{
    int n;
    int sched, tiles, stride, first; // schedule 0
    // schedules 1 and 2: the range is [tail of a tile][whole tiles][head of a tile]; the head (or a piece from the
    // middle of a tile) is parked and comes first, the tail continues / gathers and comes last
    int park_tile, park_a, park_b; // parked piece: K tiles [park_a, park_b) of park_tile, park_tile < 0: none
    int last_tile, last_a;         // tail piece: K tiles [last_a, kts) of last_tile, last_tile < 0: none
    int last_first;                // schedule 2: the CTA that owns the first piece of last_tile
    int whole0, nwhole, kts;
    int n_rr, tile0; // schedule 1: whole tiles dealt round-robin before the range, first tile of the ranges
    int bk, K, k_per_split;

    __device__ __forceinline__ void init(const WsArgs& w, int tiles_, int BK)
    {
        sched = w.sched;
        tiles = tiles_;
        bk    = BK;
        K     = w.g.K;
        k_per_split = w.g.k_per_split;
        if(sched == 0)
        {
            first  = blockIdx.x;
            stride = gridDim.x;
            n      = first < w.total_units ? (w.total_units - first + stride - 1) / stride : 0;
            return;
        }
        kts   = w.k_tiles;
        tile0 = sched == 1 ? w.rr_tiles : 0;
        n_rr  = tile0 / (int)gridDim.x;
        const long long u0 = ws_range_begin_qr(w.range_q, w.range_r, gridDim.x, blockIdx.x);
        const long long u1 = ws_range_begin_qr(w.range_q, w.range_r, gridDim.x, blockIdx.x + 1);
        park_tile = last_tile = -1;
        park_a = park_b = last_a = last_first = 0;
        whole0 = nwhole = 0;
        if(u1 > u0)
        {
            int x, a, y, b;
            ws_divmod(u0, kts, x, a);     // first segment: tile x from K tile a
            ws_divmod(u1 - 1, kts, y, b); // last segment: tile y up to K tile b (exclusive)
            b += 1;
            if(x == y)
            {
                if(a == 0 && b == kts) { whole0 = x; nwhole = 1; }
                else if(b == kts) { last_tile = x; last_a = a; }
                else { park_tile = x; park_a = a; park_b = b; }
            }
            else
            {
                whole0 = a == 0 ? x : x + 1;
                nwhole = (b == kts ? y + 1 : y) - whole0;
                if(a > 0) { last_tile = x; last_a = a; }
                if(b < kts) { park_tile = y; park_a = 0; park_b = b; }
            }
            if(last_tile >= 0 && sched == 2)
            {
                // the owner of the first K tile of last_tile: walk down from the neighbour
                int c = blockIdx.x - 1;
                while(c > 0 && ws_range_begin_qr(w.range_q, w.range_r, gridDim.x, c) > (long long)last_tile * kts)
                    --c;
                last_first = c;
            }
        }
        n = n_rr + (park_tile >= 0 ? 1 : 0) + nwhole + (last_tile >= 0 ? 1 : 0);
    }
    __device__ __forceinline__ WsPiece piece(int i) const
    {
        WsPiece p;
        p.recv = p.send = p.reduce = -1;
        p.split = 0;
        if(sched == 0)
        {
            const int unit = first + i * stride;
            p.split        = unit / tiles;
            p.tile_id      = unit - p.split * tiles;
            p.k_begin      = p.split * k_per_split;
            p.k_end        = min(K, p.k_begin + k_per_split);
            return p;
        }
        if(i < n_rr)
        {
            p.tile_id = (int)blockIdx.x + i * (int)gridDim.x;
            p.k_begin = 0;
            p.k_end   = K;
            return p;
        }
        i -= n_rr;
        const int h = park_tile >= 0 ? 1 : 0;
        if(h && i == 0)
        {
            p.tile_id = tile0 + park_tile; // first of the range: the piece somebody else waits for
            p.k_begin = park_a * bk;
            p.k_end   = park_b * bk; // < K: a parked piece never reaches the last K tile
            p.send    = blockIdx.x;
        }
        else if(i - h < nwhole)
        {
            p.tile_id = tile0 + whole0 + (i - h);
            p.k_begin = 0;
            p.k_end   = K;
        }
        else
        {
            p.tile_id = tile0 + last_tile; // last of all: the tail of the first tile of the range
            p.k_begin = last_a * bk;
            p.k_end   = K;
            if(sched == 1)
                p.recv = blockIdx.x - 1; // continue the neighbour's chain
            else
                p.reduce = last_first;   // own chain, then the ordered sum of the earlier pieces
        }
        return p;
    }
};

// Host-side view of schedule 2: the K cut points of the tile at position `pos` of the tile order, in K tiles:
// writes the cut points strictly inside (0, kts) in ascending order and returns how many there are.
inline int ws_stream_cuts(long long tiles, int kts, int ctas, long long pos, int* cuts, int capacity)
{
    const long long units = tiles * kts;
    int             n     = 0;
    // CTAs whose range begins inside this tile
    long long c = (pos * kts * ctas) / units; // a CTA at or before the first candidate
    while(c > 0 && ws_range_begin(units, ctas, (int)c) > pos * kts)
        --c;
    for(; c <= ctas; ++c)
    {
        const long long u = ws_range_begin(units, ctas, (int)c);
        if(u >= (pos + 1) * kts)
            break;
        if(u > pos * kts)
        {
            if(n < capacity)
                cuts[n] = (int)(u - pos * kts);
            ++n;
        }
    }
    return n;
}

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
__device__ __forceinline__ uint64_t global_timer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Same poll, but the hardware may park the thread for up to `hint_ns` nanoseconds while the phase is incomplete
// (instead of returning at once), so that a thread that waits long executes few instructions.
__device__ __forceinline__ bool mbar_try_wait_parked(uint32_t bar, uint32_t parity, uint32_t hint_ns)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity), "r"(hint_ns)
                 : "memory");
    return ok != 0;
}
// Bounded wait.  The common case (the phase already completed) is one poll; otherwise poll for at most
// WS_WAIT_LIMIT_NS of wall-clock time and at most WS_SPIN_LIMIT polls, looking at the CTA's abort flag
// now and then.  false = gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag)
{
    if(mbar_try_wait(bar, parity))
        return true;
    const uint64_t t0 = global_timer_ns();
    for(uint32_t i = 0; i < WS_SPIN_LIMIT; ++i)
    {
        if(mbar_try_wait(bar, parity))
            return true;
        if((i & 63u) == 63u && (*abort_flag || global_timer_ns() - t0 > WS_WAIT_LIMIT_NS))
            return false;
    }
    return false;
}
// The producers' form of the bounded wait: they run stages ahead of the consumers, so they can afford to be
// parked by the hardware between polls.  Every instruction a waiting warp executes is an issue slot taken from the
// FMA stream of the consumer warps on the same scheduler; a parked poll executes a handful per microsecond.
__device__ __forceinline__ bool mbar_wait_parked(uint32_t bar, uint32_t parity, volatile int* abort_flag)
{
    if(mbar_try_wait(bar, parity))
        return true;
    const uint64_t t0 = global_timer_ns();
    for(uint32_t i = 0; i < WS_SPIN_LIMIT; ++i)
    {
        if(mbar_try_wait_parked(bar, parity, 1000u))
            return true;
        if((i & 7u) == 7u && (*abort_flag || global_timer_ns() - t0 > WS_WAIT_LIMIT_NS))
            return false;
    }
    return false;
}
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p)
{
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_u32(unsigned* p, unsigned v)
{
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// tile copy global -> shared; (c0, c1) are element coordinates, c0 along the contiguous dimension
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar)
                 : "memory");
}

// (c0, c1, c2) element coordinates of a three-dimensional map
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
                 : "memory");
}

// (c0, c1, c2, c3) element coordinates of a four-dimensional map
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
                 : "memory");
}

template<class Cfg>
struct WsLayout
{
    static constexpr int    STAGE_FLOATS = (Cfg::BM + Cfg::BN) * Cfg::BK;
    static constexpr size_t TILE_BYTES   = size_t(Cfg::STAGES) * STAGE_FLOATS * sizeof(float);
    // after the tiles: full[STAGES], empty[STAGES], staging full / empty (8 bytes each), abort flag
    static constexpr int    PRODUCERS  = ws_producer_threads(Cfg::BLOCK_SIZE, Cfg::TMT * Cfg::TNT);
    static constexpr int    THREADS    = Cfg::BLOCK_SIZE + PRODUCERS;
    // staging ring of the K-contiguous operands: STG_SLOTS slots of [rows][32 floats] per staged operand behind the
    // barriers, 1024-byte aligned (the period of TMA's 128-byte swizzle), with their own full / empty barriers
    static constexpr int    STG_SLOTS  = 2;
    static constexpr size_t BAR_BYTES  = size_t(2 * Cfg::STAGES + 2 * STG_SLOTS) * 8 + 16;
    static constexpr bool   CAN_STAGE  = Cfg::BK == 32 && PRODUCERS >= 64;
    static constexpr size_t stage_slot_bytes(bool a_kmajor, bool b_kmajor)
    {
        return (a_kmajor ? size_t(Cfg::BM) * 128 : 0) + (b_kmajor ? size_t(Cfg::BN) * 128 : 0);
    }
    // dynamic shared memory of a launch that stages the given operands
    static constexpr size_t smem_bytes(bool stage_a, bool stage_b)
    {
        return TILE_BYTES + BAR_BYTES + ((stage_a || stage_b) ? 1024 + STG_SLOTS * stage_slot_bytes(stage_a, stage_b) : 0);
    }
    // k-steps unrolled back to back: the whole K tile.  A shallower unroll (compile with -DWS_KU_FORCE=8 or 16)
    // keeps the loop body of the 128-accumulator thread tiles small but measured slower on B200
    // (16x8 tile at 8192^3: 58.3 / 60.1 / 63.3 TFLOP/s for 8 / 16 / 32 steps).
#ifdef WS_KU_FORCE
    static constexpr int    KU = (Cfg::TMT * Cfg::TNT > 64 && Cfg::BK > WS_KU_FORCE) ? WS_KU_FORCE : Cfg::BK;
#else
    static constexpr int    KU = Cfg::BK;
#endif
};

// One staged operand tile moved into the stage's plain [k][x] tile by NT threads.  The staging slot holds BX rows of
// 32 k (128 bytes) as TMA wrote them with the 128-byte swizzle (the 16-byte chunk c of slot row r sits at chunk
// c ^ (r & 7); the slot is 1024-byte aligned), in the row order of the three-dimensional tensor map the host builds:
// slot row i * (BX / 4) + g holds operand row 4 g + i.  A work item is the 4 x 4 block (rows 4g .. 4g+3, k 4c .. 4c+3):
// four 128-bit reads, transposition in registers (renaming), four 128-bit writes.  The lanes of a warp take
// consecutive g: each read instruction touches 32 consecutive slot rows (all eight swizzle positions, 512 bytes in
// four wavefronts) and each write instruction one contiguous 512-byte piece of a k row: both sides run at the
// shared-memory pipe's full rate, and a tile costs 16 instructions per 4 KB - every instruction the producers issue is
// an issue slot the FMA stream of the consumers on the same scheduler does not get.
template<int NT, int BX, int BK>
struct StagedTransposer
{
    static constexpr int G     = BX / 4;
    static constexpr int ITEMS = G * (BK / 4);
    static constexpr int ITERS = (ITEMS + NT - 1) / NT;
    static_assert(G % 8 == 0, "slot rows i * G + g must keep g's low three bits");
    // byte offsets of this thread's work items inside a slot / a stage tile: fixed for the whole kernel, so the
    // per-stage work is one address addition per side and eight memory instructions with immediate offsets
    int src[ITERS], dst[ITERS];
    __device__ __forceinline__ void init(int t)
    {
#pragma unroll
        for(int it = 0; it < ITERS; ++it)
        {
            const int q = t + it * NT;
            const int g = q % G, c = q / G;
            src[it]     = (ITEMS % NT == 0 || q < ITEMS) ? g * 128 + ((c ^ (g & 7)) << 4) : -1;
            dst[it]     = ((4 * c) * BX + 4 * g) * 4;
        }
    }
    __device__ __forceinline__ void run(const char* slot, float* tile) const
    {
#pragma unroll
        for(int it = 0; it < ITERS; ++it)
        {
            if((ITEMS % NT) == 0 || src[it] >= 0)
            {
                const char*  sp = slot + src[it];
                const float4 r0 = *reinterpret_cast<const float4*>(sp + 0 * G * 128);
                const float4 r1 = *reinterpret_cast<const float4*>(sp + 1 * G * 128);
                const float4 r2 = *reinterpret_cast<const float4*>(sp + 2 * G * 128);
                const float4 r3 = *reinterpret_cast<const float4*>(sp + 3 * G * 128);
                char*        d  = reinterpret_cast<char*>(tile) + dst[it];
                *reinterpret_cast<float4*>(d + 0 * BX * 4) = make_float4(r0.x, r1.x, r2.x, r3.x);
                *reinterpret_cast<float4*>(d + 1 * BX * 4) = make_float4(r0.y, r1.y, r2.y, r3.y);
                *reinterpret_cast<float4*>(d + 2 * BX * 4) = make_float4(r0.z, r1.z, r2.z, r3.z);
                *reinterpret_cast<float4*>(d + 3 * BX * 4) = make_float4(r0.w, r1.w, r2.w, r3.w);
            }
        }
    }
};

// One block of the cooperative transposition, by one warp: rows [r0, r0 + BX) x columns [k0, k0 + BK) of src
// ([X][K], pitch ld) -> dst ([K][X], pitch ldt).  A lane takes a 4 x 4 piece at a time: four 128-bit reads along k
// (eight lanes cover 128 contiguous bytes of a row), a transposition in registers, four 128-bit writes along x (four
// lanes cover 64 contiguous bytes).  X and K are multiples of 4, so a piece is entirely inside or outside.
template<int BX, int BK>
struct CoopTransposer
{
    static constexpr int G      = BX / 4;  // row groups of four
    static constexpr int QK     = BK / 4;  // k quads of a block
    static constexpr int GP     = 32 / QK; // row groups a warp covers per pass
    static constexpr bool OK    = BK % 4 == 0 && QK <= 32 && 32 % QK == 0 && G % GP == 0;
    static constexpr int PASSES = OK ? G / GP : 1;
    static constexpr int BATCH  = PASSES % 8 == 0 ? 8 : PASSES % 4 == 0 ? 4 : PASSES % 2 == 0 ? 2 : 1; // pieces in flight per lane
    static __device__ __forceinline__ void run(const float* __restrict__ src, long long ld, float* __restrict__ dst,
                                               long long ldt, int X, int K, int r0, int k0, int lane)
    {
        const int  c  = lane % QK, gl = lane / QK;
        const int  k  = k0 + 4 * c;
        const bool k_ok = k < K;
#pragma unroll 1
        for(int pb = 0; pb < PASSES; pb += BATCH)
        {
            float4 r[BATCH][4];
#pragma unroll
            for(int b = 0; b < BATCH; ++b)
            {
                const int    x  = r0 + 4 * (gl + GP * (pb + b));
                const bool   ok = k_ok && x < X;
                const float* sp = src + (long long)x * ld + k;
#pragma unroll
                for(int i = 0; i < 4; ++i)
                    r[b][i] = ok ? __ldcs(reinterpret_cast<const float4*>(sp + i * ld)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for(int b = 0; b < BATCH; ++b)
            {
                const int x = r0 + 4 * (gl + GP * (pb + b));
                if(k_ok && x < X)
                {
                    float* dp = dst + (long long)k * ldt + x;
                    *reinterpret_cast<float4*>(dp + 0 * ldt) = make_float4(r[b][0].x, r[b][1].x, r[b][2].x, r[b][3].x);
                    *reinterpret_cast<float4*>(dp + 1 * ldt) = make_float4(r[b][0].y, r[b][1].y, r[b][2].y, r[b][3].y);
                    *reinterpret_cast<float4*>(dp + 2 * ldt) = make_float4(r[b][0].z, r[b][1].z, r[b][2].z, r[b][3].z);
                    *reinterpret_cast<float4*>(dp + 3 * ldt) = make_float4(r[b][0].w, r[b][1].w, r[b][2].w, r[b][3].w);
                }
            }
        }
    }
};

template<class Cfg, int LA, int LB, int LC, bool ALIGNED>
__global__ void __launch_bounds__(WsLayout<Cfg>::THREADS, Cfg::MIN_BLOCKS)
    sgemm_ws_kernel(const __grid_constant__ WsArgs w, const __grid_constant__ CUtensorMap map_a,
                    const __grid_constant__ CUtensorMap map_b)
{
    constexpr int  BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, STAGES = Cfg::STAGES;
    constexpr int  TM = Cfg::TM, TN = Cfg::TN, TMT = Cfg::TMT, TNT = Cfg::TNT;
    constexpr int  MODE     = Cfg::FMA_MODE;
    constexpr bool A_KMAJOR = (LA == LAYOUT_ROW); // transposed by the producers
    constexpr bool B_KMAJOR = (LB == LAYOUT_COL);
    constexpr int  CONSUMER_WARPS = Cfg::BLOCK_SIZE / 32;
    using L    = WsLayout<Cfg>;
    constexpr int KU = L::KU;
    static_assert(MODE == FMA_SCALAR || MODE == FMA_X2_DUP, "warp-specialised kernel: fma_mode 0 or 1");
    static_assert(TM % 4 == 0 && TN % 4 == 0, "warp-specialised kernel reads 128-bit fragments");
    static_assert(BK % KU == 0 && KU % 4 == 0 && KU % 2 == 0, "unroll depth must divide block_k");

    extern __shared__ __align__(128) float smem[];
    const GemmArgs& p = w.g;

    const uint32_t bar_base = smem_u32(smem) + (uint32_t)L::TILE_BYTES;
    auto           full_bar  = [&](int s) -> uint32_t { return bar_base + 8u * s; };
    auto           empty_bar = [&](int s) -> uint32_t { return bar_base + 8u * (STAGES + s); };
    auto           sfull_bar  = [&](int j) -> uint32_t { return bar_base + 8u * (2 * STAGES + j); };
    auto           sempty_bar = [&](int j) -> uint32_t { return bar_base + 8u * (2 * STAGES + L::STG_SLOTS + j); };
    volatile int*  abort_flag = reinterpret_cast<volatile int*>(reinterpret_cast<char*>(smem) + L::TILE_BYTES
                                                               + (2 * STAGES + 2 * L::STG_SLOTS) * 8);
    // the staged route is taken when every operand comes by TMA and at least one of them through the staging ring
    constexpr bool STAGE_A = L::CAN_STAGE && A_KMAJOR, STAGE_B = L::CAN_STAGE && B_KMAJOR;
    const bool     staged  = (STAGE_A || STAGE_B) && (w.stg_a || w.stg_b) && (w.tma_a || w.stg_a) && (w.tma_b || w.stg_b);
    constexpr int  TRANSPOSERS = L::PRODUCERS - 32; // producer warp 0 issues the copies
    auto tile_a = [&](int s) -> float* { return smem + s * L::STAGE_FLOATS; };
    auto tile_b = [&](int s) -> float* { return smem + s * L::STAGE_FLOATS + BM * BK; };

    const int tid = threadIdx.x;
    if(tid == Cfg::BLOCK_SIZE)
    {
        // the thread that will issue the copies fetches the descriptors while thread 0 sets up the barriers
        if(w.tma_a || w.stg_a)
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
        if(w.tma_b || w.stg_b)
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_b)) : "memory");
    }
    if(tid == 0)
    {
        for(int s = 0; s < STAGES; ++s)
        {
            // arrivals per fill: the thread that arms the byte count (and issues the TMA copies), plus one per
            // producer warp when an operand is staged by hand
            // (staged route: the issuing thread only when an operand goes straight into the stage, plus one per
            // transposing warp)
            const uint32_t arrivals = staged ? ((w.tma_a || w.tma_b) ? 1 : 0) + TRANSPOSERS / 32
                                             : (w.tma_a && w.tma_b) ? 1 : L::PRODUCERS / 32 + 1;
            mbar_init(full_bar(s), arrivals);
            mbar_init(empty_bar(s), CONSUMER_WARPS);
        }
        for(int j = 0; j < L::STG_SLOTS; ++j)
        {
            mbar_init(sfull_bar(j), 1);
            mbar_init(sempty_bar(j), TRANSPOSERS / 32);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads(); // the only block-wide barrier: everything below is role-local

    const int tiles_per_matrix = p.grid_m * p.grid_n;
    const int tiles            = tiles_per_matrix * w.batch; // the schedules walk the tiles of all matrices of a batch

    if(tid >= Cfg::BLOCK_SIZE)
    {
        // =========================== PRODUCERS ==========================================================
        const int      ptid     = tid - Cfg::BLOCK_SIZE;
        if constexpr(STAGE_A || STAGE_B)
        {
            if(staged)
            {
                constexpr uint32_t SLOT_A = STAGE_A ? BM * 128u : 0u, SLOT_B = STAGE_B ? BN * 128u : 0u;
                char* stg = reinterpret_cast<char*>(smem) + L::TILE_BYTES + L::BAR_BYTES;
                stg += (1024u - (smem_u32(stg) & 1023u)) & 1023u;
                auto slot_a = [&](int j) -> char* { return stg + j * (SLOT_A + SLOT_B); };
                auto slot_b = [&](int j) -> char* { return stg + j * (SLOT_A + SLOT_B) + SLOT_A; };
                const bool stg_a = STAGE_A && w.stg_a, stg_b = STAGE_B && w.stg_b;
                auto give_up = [&]() {
                    if(!*abort_flag)
                    {
                        *abort_flag = 1;
                        atomicCAS(w.status, 0, WS_ERR_EMPTY_TIMEOUT);
                    }
                    __nanosleep(200000); // let copies already in flight land before the CTA retires
                };
                int        s = 0, j = 0;
                uint32_t   phase = 0, jphase = 0;
                WsSchedule sch;
                sch.init(w, tiles, BK);
                if(ptid >= 32)
                {
                    // ---- transposing warps: staging slot -> stage ------------------------------------------------
                    const int tt = ptid - 32;
                    StagedTransposer<TRANSPOSERS, BM, BK> tr_a;
                    StagedTransposer<TRANSPOSERS, BN, BK> tr_b;
                    tr_a.init(tt);
                    tr_b.init(tt);
                    for(int pi = 0; pi < sch.n; ++pi)
                    {
                        const WsPiece pc     = sch.piece(pi);
                        const int     ntiles = (pc.k_end - pc.k_begin + BK - 1) / BK;
                        for(int t = 0; t < ntiles; ++t)
                        {
                            if(!mbar_wait_parked(sfull_bar(j), jphase, abort_flag)
                               || !mbar_wait_parked(empty_bar(s), phase ^ 1u, abort_flag))
                            {
                                give_up();
                                return;
                            }
                            if constexpr(STAGE_A)
                                if(stg_a)
                                    tr_a.run(slot_a(j), tile_a(s));
                            if constexpr(STAGE_B)
                                if(stg_b)
                                    tr_b.run(slot_b(j), tile_b(s));
                            __syncwarp(); // the warp is done with the slot and with the stage: one lane says so
                            if((ptid & 31) == 0)
                            {
                                mbar_arrive(full_bar(s));
                                mbar_arrive(sempty_bar(j));
                            }
                            if(++s == STAGES) { s = 0; phase ^= 1u; }
                            if(++j == L::STG_SLOTS) { j = 0; jphase ^= 1u; }
                        }
                    }
                    return;
                }
                if(ptid != 0)
                    return;
                // ---- the issuing thread: every TMA copy of the CTA --------------------------------------------------
                const uint32_t direct_bytes = (w.tma_a ? BM * BK * 4u : 0u) + (w.tma_b ? BN * BK * 4u : 0u);
                const uint32_t staged_bytes = (stg_a ? SLOT_A : 0u) + (stg_b ? SLOT_B : 0u);
                for(int pi = 0; pi < sch.n; ++pi)
                {
                    const WsPiece pc = sch.piece(pi);
                    const int     mat = pc.tile_id / tiles_per_matrix;
                    int           tile_m, tile_n;
                    map_tile<Cfg::RASTER>(pc.tile_id - mat * tiles_per_matrix, p.grid_m, p.grid_n, tile_m, tile_n);
                    const int m0 = tile_m * BM, n0 = tile_n * BN;
                    const int ntiles = (pc.k_end - pc.k_begin + BK - 1) / BK;
                    for(int t = 0; t < ntiles; ++t)
                    {
                        const int k0 = pc.k_begin + t * BK;
                        // the staging slot frees up first (the transposers run ahead of the consumers): fetch into it
                        // as early as possible; coordinates are (k, row / 4, row % 4), k a multiple of 32 elements
                        if(!mbar_wait_parked(sempty_bar(j), jphase ^ 1u, abort_flag))
                        {
                            give_up();
                            return;
                        }
                        mbar_arrive_expect_tx(sfull_bar(j), staged_bytes);
                        if(stg_a)
                            tma_load_4d(smem_u32(slot_a(j)), &map_a, k0, m0 >> 2, 0, mat * w.bstep_a, sfull_bar(j));
                        if(stg_b)
                            tma_load_4d(smem_u32(slot_b(j)), &map_b, k0, n0 >> 2, 0, mat * w.bstep_b, sfull_bar(j));
                        if(direct_bytes)
                        {
                            if(!mbar_wait_parked(empty_bar(s), phase ^ 1u, abort_flag))
                            {
                                give_up();
                                return;
                            }
                            mbar_arrive_expect_tx(full_bar(s), direct_bytes);
                            if(w.tma_a)
                                tma_load_3d(smem_u32(tile_a(s)), &map_a, m0, k0, mat * w.bstep_a, full_bar(s));
                            if(w.tma_b)
                                tma_load_3d(smem_u32(tile_b(s)), &map_b, n0, k0, mat * w.bstep_b, full_bar(s));
                        }
                        if(++s == STAGES) { s = 0; phase ^= 1u; }
                        if(++j == L::STG_SLOTS) { j = 0; jphase ^= 1u; }
                    }
                }
                return;
            }
        }
        const uint32_t tx_bytes = (w.tma_a ? BM * BK * 4u : 0u) + (w.tma_b ? BN * BK * 4u : 0u);
        OperandStager<L::PRODUCERS, BM, BK, A_KMAJOR, ALIGNED, false> stage_a;
        OperandStager<L::PRODUCERS, BN, BK, B_KMAJOR, ALIGNED, false> stage_b;
        const bool manual_a = !w.tma_a, manual_b = !w.tma_b;
        // Both operands by TMA: one thread does everything, the other producer threads leave at once.  (A warp
        // that merely polled a barrier would still take issue slots from the consumers on its scheduler.)
        if(!manual_a && !manual_b && ptid != 0)
        {
            // ---- cooperative transposition: the warps the TMA route leaves idle ---------------------------------
            constexpr int COOP_WARPS = L::PRODUCERS / 32 - 1;
            if constexpr(COOP_WARPS > 0 && CoopTransposer<BM, BK>::OK && CoopTransposer<BN, BK>::OK)
            {
                if(w.coop_flags && ptid >= 32)
                {
                    const int       lane_p = ptid & 31;
                    const int       xa = w.coop_src_a ? p.grid_m : 0, xt = xa + (w.coop_src_b ? p.grid_n : 0);
                    const long long units = (long long)w.k_tiles * xt;
                    const long long step  = (long long)gridDim.x * COOP_WARPS;
                    // blocks in the order the consumers need them (K tile by K tile), dealt round-robin to all warps
                    for(long long u = (long long)blockIdx.x * COOP_WARPS + (ptid / 32 - 1); u < units; u += step)
                    {
                        const int kt = (int)(u / xt), x = (int)(u - (long long)kt * xt);
                        if(x < xa)
                            CoopTransposer<BM, BK>::run(w.coop_src_a, w.coop_ld_a, const_cast<float*>(p.A), p.lda, p.M,
                                                        p.K, x * BM, kt * BK, lane_p);
                        else
                            CoopTransposer<BN, BK>::run(w.coop_src_b, w.coop_ld_b, const_cast<float*>(p.B), p.ldb, p.N,
                                                        p.K, (x - xa) * BN, kt * BK, lane_p);
                        __syncwarp(); // the warp's stores -> one lane's fence and gpu-scope release of the block's word
                        if(lane_p == 0)
                        {
                            __threadfence();
                            st_release_u32(w.coop_flags + u, w.epoch);
                        }
                    }
                    if(lane_p == 0)
                    {
                        __threadfence(); // (a warp without blocks counts too)
                        atomicAdd(w.coop_done, 1u);
                    }
                }
            }
            return;
        }
        // words of the transposed blocks the copy-issuing thread has to see before it may fetch a stage
        const int  coop_xa = w.coop_src_a ? p.grid_m : 0, coop_xt = coop_xa + (w.coop_src_b ? p.grid_n : 0);
        bool       coop    = w.coop_flags != nullptr && !manual_a && !manual_b;
        int      s     = 0; // ring position
        uint32_t phase = 0; // parity of the current lap
        WsSchedule sch;
        sch.init(w, tiles, BK);
        for(int pi = 0; pi < sch.n; ++pi)
        {
            const WsPiece pc  = sch.piece(pi);
            const int     mat = pc.tile_id / tiles_per_matrix;
            int           tile_m, tile_n;
            map_tile<Cfg::RASTER>(pc.tile_id - mat * tiles_per_matrix, p.grid_m, p.grid_n, tile_m, tile_n);
            const int m0 = tile_m * BM, n0 = tile_n * BN;
            const int k_begin = pc.k_begin;
            const int k_end   = pc.k_end;
            const int ntiles  = (k_end - k_begin + BK - 1) / BK;
            const float* mat_a = p.A + mat * w.stride_a;
            const float* mat_b = p.B + mat * w.stride_b;
            for(int t = 0; t < ntiles; ++t)
            {
                // the stage was released `phase` laps ago; the very first lap passes immediately
                if(!mbar_wait_parked(empty_bar(s), phase ^ 1u, abort_flag))
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
                if(w.test_omit_last_fill && pi == sch.n - 1 && t == ntiles - 1)
                    return; // self-test: this stage is never filled
                if(ptid == 0)
                {
                    if(coop)
                    {
                        // the blocks of this stage must be in place (written by some CTA's transposing warps with
                        // ordinary stores): acquire their words, then order those writes before the TMA reads
                        const unsigned* fa = w.coop_flags + (long long)(k0 / BK) * coop_xt + (w.coop_src_a ? tile_m : 0);
                        const unsigned* fb = w.coop_flags + (long long)(k0 / BK) * coop_xt + coop_xa + tile_n;
                        if(!w.coop_src_a) fa = fb;
                        if(!w.coop_src_b) fb = fa;
                        // (both reads in flight together; every eighth stage also looks whether all warps have finished:
                        // from then on nothing needs checking any more)
                        const unsigned va = ld_acquire_u32(fa), vb = ld_acquire_u32(fb);
                        bool           got = va == w.epoch && vb == w.epoch;
                        if(got && (t & 7) == 0 && ld_acquire_u32(w.coop_done) == w.coop_done_target)
                            coop = false;
                        if(!got)
                        {
                            const uint64_t t0 = global_timer_ns();
                            for(uint32_t it = 0; it < WS_SPIN_LIMIT && !got; ++it)
                            {
                                __nanosleep(100);
                                got = ld_acquire_u32(fa) == w.epoch && ld_acquire_u32(fb) == w.epoch;
                                if(!got && (it & 63u) == 63u && (*abort_flag || global_timer_ns() - t0 > WS_WAIT_LIMIT_NS))
                                    break;
                            }
                        }
                        if(!got)
                        {
                            if(!*abort_flag)
                            {
                                *abort_flag = 1;
                                atomicCAS(w.status, 0, WS_ERR_COOP_TIMEOUT);
                            }
                            __nanosleep(200000); // let copies already in flight land before the CTA retires
                            return;
                        }
                        asm volatile("fence.proxy.async;" ::: "memory");
                    }
                    if(tx_bytes)
                    {
                        mbar_arrive_expect_tx(full_bar(s), tx_bytes);
                        // tile origins are multiples of 32 elements: TMA's 16-byte start rule holds
                        if(w.tma_a)
                            tma_load_3d(smem_u32(tile_a(s)), &map_a, m0, k0, mat * w.bstep_a, full_bar(s));
                        if(w.tma_b)
                            tma_load_3d(smem_u32(tile_b(s)), &map_b, n0, k0, mat * w.bstep_b, full_bar(s));
                    }
                    else
                    {
                        mbar_arrive(full_bar(s));
                    }
                }
                if(manual_a)
                    stage_a.fetch(mat_a, p.lda, p.M, m0, k0, k_end, p.vec_a, tile_a(s), ptid);
                if(manual_b)
                    stage_b.fetch(mat_b, p.ldb, p.N, n0, k0, k_end, p.vec_b, tile_b(s), ptid);
                if(manual_a)
                    stage_a.commit(tile_a(s), ptid);
                if(manual_b)
                    stage_b.commit(tile_b(s), ptid);
                if((!A_KMAJOR && manual_a) || (!B_KMAJOR && manual_b))
                {
                    cp_async_commit();
                    cp_async_wait<0>(); // guarded-copy fallback of an operand TMA could not take
                }
                if(manual_a || manual_b)
                {
                    __syncwarp(); // the warp's stores to the stage are done; one lane publishes them
                    if((ptid & 31) == 0)
                        mbar_arrive(full_bar(s));
                }
                if(++s == STAGES)
                {
                    s = 0;
                    phase ^= 1u;
                }
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

    // fragment of k-step `kk` (relative to the pointers passed in); every operand's stage is a plain [k][x] tile
    auto load_frags = [&](int buf, const float* as, const float* bs, int kk, int /*chunk*/) {
#pragma unroll
        for(int im = 0; im < Cfg::WM_CNT; ++im)
        {
#pragma unroll
            for(int v = 0; v < TM / 4; ++v)
            {
                const float4 q = *reinterpret_cast<const float4*>(as + kk * BM + (tm0 + im * Cfg::SUB_M + 4 * v));
                float*       d = &a_frag[buf][im * TM + 4 * v];
                d[0] = q.x; d[1] = q.y; d[2] = q.z; d[3] = q.w;
            }
        }
#pragma unroll
        for(int in = 0; in < Cfg::WN_CNT; ++in)
        {
#pragma unroll
            for(int v = 0; v < TN / 4; ++v)
            {
                const float4 q = *reinterpret_cast<const float4*>(bs + kk * BN + (tn0 + in * Cfg::SUB_N + 4 * v));
                float*       d = &b_frag[buf][in * TN + 4 * v];
                d[0] = q.x; d[1] = q.y; d[2] = q.z; d[3] = q.w;
            }
        }
    };

    int      s     = 0;
    uint32_t phase = 0;
    WsSchedule sch;
    sch.init(w, tiles, BK);
    // parked accumulators: slot c is block_m x block_n floats, thread-major in 16-byte units so that the accesses of
    // a warp are contiguous; the reader is the thread with the same index in the next CTA
    constexpr int ACC_VEC = TMT * TNT / 4;
    // A parked piece is published (fence + release of the warp's flag) one K tile into the next piece: by then the
    // stores have long landed and the fence returns at once, instead of holding the warp until they are acknowledged.
    int publish = -1;
    auto publish_now = [&]() {
        __syncwarp();
        if(lane == 0)
        {
            __threadfence();
            st_release_u32(w.flags + publish * CONSUMER_WARPS + warp_id, w.epoch);
        }
        publish = -1;
    };
    for(int pi = 0; pi < sch.n; ++pi)
    {
        const WsPiece pc  = sch.piece(pi);
        const int     mat = pc.tile_id / tiles_per_matrix;
        int           tile_m, tile_n;
        map_tile<Cfg::RASTER>(pc.tile_id - mat * tiles_per_matrix, p.grid_m, p.grid_n, tile_m, tile_n);
        const int m0 = tile_m * BM, n0 = tile_n * BN;
        const int k_begin = pc.k_begin;
        const int k_end   = pc.k_end;
        const int ntiles  = (k_end - k_begin + BK - 1) / BK;

        float    acc[MODE == FMA_SCALAR ? TMT : 1][MODE == FMA_SCALAR ? TNT : 1];
        uint64_t acc2[MODE == FMA_SCALAR ? 1 : TMT][MODE == FMA_SCALAR ? 1 : TNT / 2];
        if(pc.recv >= 0)
        {
            // the chain of this tile was started by the previous CTA (first thing it did): take its accumulators over
            if(publish >= 0)
                publish_now(); // never wait for a neighbour while one's own piece is unpublished: the waits would chain
            const unsigned* flag = w.flags + pc.recv * CONSUMER_WARPS + warp_id;
            bool            got  = ld_acquire_u32(flag) == w.epoch;
            if(!got)
            {
                const uint64_t t0 = global_timer_ns();
                for(uint32_t it = 0; it < WS_SPIN_LIMIT && !got; ++it)
                {
                    __nanosleep(100);
                    got = ld_acquire_u32(flag) == w.epoch;
                    if(!got && (it & 63u) == 63u && (*abort_flag || global_timer_ns() - t0 > WS_WAIT_LIMIT_NS))
                        break;
                }
            }
            if(!got)
            {
                if(!*abort_flag)
                {
                    *abort_flag = 1;
                    atomicCAS(w.status, 0, WS_ERR_PEER_TIMEOUT);
                }
                return;
            }
            const float4* src = reinterpret_cast<const float4*>(w.handover + (size_t)pc.recv * (BM * BN)) + tid;
            float         c0[TMT][TNT];
#pragma unroll
            for(int v = 0; v < ACC_VEC; ++v)
            {
                const float4 q = __ldcg(src + v * Cfg::BLOCK_SIZE);
                float*       d = &c0[0][0] + 4 * v;
                d[0] = q.x; d[1] = q.y; d[2] = q.z; d[3] = q.w;
            }
            if constexpr(MODE == FMA_SCALAR)
            {
#pragma unroll
                for(int i = 0; i < TMT; ++i)
#pragma unroll
                    for(int j = 0; j < TNT; ++j)
                        acc[i][j] = c0[i][j];
            }
            else
            {
#pragma unroll
                for(int i = 0; i < TMT; ++i)
#pragma unroll
                    for(int j = 0; j < TNT / 2; ++j)
                        acc2[i][j] = pack2(c0[i][2 * j], c0[i][2 * j + 1]);
            }
        }
        else if constexpr(MODE == FMA_SCALAR)
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
            else
            {
                uint64_t a2[TMT];
#pragma unroll
                for(int i = 0; i < TMT; ++i)
                    a2[i] = pack2(a_frag[buf][i], a_frag[buf][i]);
#pragma unroll
                for(int j = 0; j < TNT / 2; ++j)
                {
                    const uint64_t b2 = pack2(b_frag[buf][2 * j], b_frag[buf][2 * j + 1]);
#pragma unroll
                    for(int i = 0; i < TMT; ++i)
                        fma2(acc2[i][j], a2[i], b2);
                }
            }
        };

        // first stage of this unit
        bool ok = mbar_wait(full_bar(s), phase, abort_flag);
        if(ok)
            load_frags(0, tile_a(s), tile_b(s), 0, 0);
        for(int t = 0; ok && t < ntiles; ++t)
        {
            const int      s2     = (s + 1 == STAGES) ? 0 : s + 1;
            const uint32_t phase2 = (s + 1 == STAGES) ? phase ^ 1u : phase;
            const float*   as     = tile_a(s);
            const float*   bs     = tile_b(s);
            const bool     has_next = t + 1 < ntiles;
            if constexpr(KU == BK)
            {
#pragma unroll
                for(int kk = 0; kk < BK; ++kk)
                {
                    if(kk + 1 < BK)
                    {
                        load_frags((kk + 1) & 1, as, bs, kk + 1, (kk + 1) >> 2);
                    }
                    else if(has_next)
                    {
                        // fragment 0 of the next stage is fetched under the last FMAs of this one
                        ok = mbar_wait(full_bar(s2), phase2, abort_flag);
                        if(ok)
                            load_frags(0, tile_a(s2), tile_b(s2), 0, 0);
                    }
                    fma_step(kk & 1);
                }
            }
            else
            {
#pragma unroll 1
                for(int kb = 0; kb < BK; kb += KU)
                {
                    const float* asb = as + kb * BM;
                    const float* bsb = bs + kb * BN;
                    const int    cb  = kb >> 2;
#pragma unroll
                    for(int u = 0; u < KU; ++u)
                    {
                        if(u + 1 < KU)
                        {
                            load_frags((u + 1) & 1, asb, bsb, u + 1, cb + ((u + 1) >> 2));
                        }
                        else if(kb + KU < BK)
                        {
                            load_frags(0, asb, bsb, KU, cb + (KU >> 2));
                        }
                        else if(has_next)
                        {
                            ok = mbar_wait(full_bar(s2), phase2, abort_flag);
                            if(ok)
                                load_frags(0, tile_a(s2), tile_b(s2), 0, 0);
                        }
                        fma_step(u & 1);
                    }
                }
            }
            __syncwarp();
            if(lane == 0)
                mbar_arrive(empty_bar(s)); // this warp is done reading stage s
            s     = s2;
            phase = phase2;
            if(publish >= 0)
                publish_now();
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
        else
        {
#pragma unroll
            for(int i = 0; i < TMT; ++i)
#pragma unroll
                for(int j = 0; j < TNT / 2; ++j)
                    unpack2(acc2[i][j], c[i][2 * j], c[i][2 * j + 1]);
        }
        if(pc.send >= 0)
        {
            // park the accumulators for the CTA that continues this tile, then publish them warp by warp (the reader
            // of a thread's values is the thread with the same index, so a warp only ever waits for its namesake and
            // no block-wide barrier is needed): the warp's stores -> __syncwarp -> one lane's gpu-scope release
            // (at once when this was the CTA's last piece, else after the first K tile of the next piece)
            float4* dst = reinterpret_cast<float4*>(w.handover + (size_t)pc.send * (BM * BN)) + tid;
#pragma unroll
            for(int v = 0; v < ACC_VEC; ++v)
            {
                const float* q = &c[0][0] + 4 * v;
                __stcg(dst + v * Cfg::BLOCK_SIZE, make_float4(q[0], q[1], q[2], q[3]));
            }
            publish = pc.send;
            if(pi + 1 == sch.n)
                publish_now();
            continue; // parked
        }
        if(pc.reduce >= 0)
        {
            // schedule 2: this CTA owns the last K range of the tile.  Total = ((own + p_first) + p_next) + ..., the
            // earlier pieces in ascending K order; each was parked by its CTA before that CTA did anything else.
            for(int src_cta = pc.reduce; src_cta < (int)blockIdx.x; ++src_cta)
            {
                const unsigned* flag = w.flags + src_cta * CONSUMER_WARPS + warp_id;
                bool            got  = ld_acquire_u32(flag) == w.epoch;
                if(!got)
                {
                    const uint64_t t0 = global_timer_ns();
                    for(uint32_t it = 0; it < WS_SPIN_LIMIT && !got; ++it)
                    {
                        __nanosleep(100);
                        got = ld_acquire_u32(flag) == w.epoch;
                        if(!got && (it & 63u) == 63u && (*abort_flag || global_timer_ns() - t0 > WS_WAIT_LIMIT_NS))
                            break;
                    }
                }
                if(!got)
                {
                    if(!*abort_flag)
                    {
                        *abort_flag = 1;
                        atomicCAS(w.status, 0, WS_ERR_PEER_TIMEOUT);
                    }
                    return;
                }
            }
            // all pieces are there: add them to this CTA's own chain in ascending K order, one piece at a time with
            // all of the piece's loads in flight together (the sum is ((own + p_first) + p_next) + ...)
            const float4* base = reinterpret_cast<const float4*>(w.handover) + tid;
#pragma unroll 1 // (unrolled, the compiler spills registers)
            for(int src_cta = pc.reduce; src_cta < (int)blockIdx.x; ++src_cta)
            {
                const float4* src = base + (size_t)src_cta * (BM * BN / 4);
                float4        q[ACC_VEC];
#pragma unroll
                for(int v = 0; v < ACC_VEC; ++v)
                    q[v] = __ldcg(src + v * Cfg::BLOCK_SIZE);
#pragma unroll
                for(int v = 0; v < ACC_VEC; ++v)
                {
                    float* d = &c[0][0] + 4 * v;
                    d[0] += q[v].x; d[1] += q[v].y; d[2] += q[v].z; d[3] += q[v].w;
                }
            }
        }
        // (one epilogue for both uses: alpha = 1, beta = 0 reproduce the plain store bit for bit - x * 1 is x - and a
        // second, unscaled copy of it cost two of the larger kernels a register spill)
        store_tile<Cfg, LC, ALIGNED, true>(c, p, p.C + (long long)pc.split * p.split_stride + mat * w.stride_c, m0 + tm0,
                                           n0 + tn0, w.alpha, w.beta);
        for(int d = 0; d < w.n_extra; ++d) // plain stores; to a peer GPU's memory when the pointer is a peer mapping
            store_tile<Cfg, LC, ALIGNED>(c, p, w.extra_c[d], m0 + tm0, n0 + tn0);
    }
}

} // namespace sgemm_b200
