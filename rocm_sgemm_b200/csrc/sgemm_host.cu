// b200_sgemm_host / b200_sgemm_host_submit / b200_sgemm_host_wait: the GEMM for callers whose matrices live in
// HOST memory.
//
// The reference's harnesses copy A and B to the device, call gemm(), and copy C back, one step after the
// other (test/gemm/test.cpp:50-74).  These entries do the same work end to end but overlap the phases.
// At 4096^3 the uploads (128 MiB over PCIe, about 2.4 ms) take longer than the GEMM (2.1 ms), so the aim
// is to have as much of the product as possible computed while the operands are still arriving:
//
//   * A is cut into row panels and B into column panels; they are uploaded alternately (A0 B0 A1 B1 ...).
//     A block C(i,j) needs only A_i and B_j, so after every upload one rectangular strip of C becomes
//     computable: A_k x (the B panels present) after A_k, (the A panels present) x B_k after B_k.  This
//     order maximises the computable share of C at every moment of the upload (the product of the shares
//     of A and B present is largest when the two are equal).
//   * each strip is ONE GEMM launch on the device matrices (leading dimensions = the full ones); strips
//     rotate over several compute streams so that the persistent kernels of consecutive strips fill the
//     SMs that the last wave of the previous one leaves idle;
//   * each finished strip is downloaded while the next ones are uploaded and computed (the GPU's copy
//     engines work in both directions at once).
//
// submit() only enqueues (copies, kernels, events) and returns a ticket; wait() blocks until that job's C is
// complete in host memory.  Two jobs can be in flight per device (two sets of device matrices): the uploads of
// job i+1 then run during the compute-bound second half and the downloads of job i, and a stream of jobs
// proceeds at the pace of the uploads alone.  b200_sgemm_host() is submit() followed by wait().
//
// Host buffers should be page-locked (cudaHostAlloc / cudaHostRegister); pageable memory works but the runtime
// then stages the copies and the overlap is lost.  They must stay untouched until wait() returns.  The device
// buffers come from a per-device arena owned by the library (grown on demand, released by
// b200_sgemm_shutdown_host).
#include "../../include/b200_sgemm.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <map>
#include <mutex>
#include <vector>

namespace
{
constexpr int MAX_PIECES      = 8;              // per operand
constexpr int MAX_STRIPS      = 2 * MAX_PIECES; // one strip per upload at most
constexpr int COMPUTE_STREAMS = 4;
constexpr int SLOTS           = 2;              // jobs in flight per device

struct Slot
{
    float*      dA = nullptr;
    float*      dB = nullptr;
    float*      dC = nullptr;
    size_t      bytesA = 0, bytesB = 0, bytesC = 0;
    cudaEvent_t uploaded[MAX_STRIPS] = {};
    cudaEvent_t computed[MAX_STRIPS] = {};
    cudaEvent_t done = nullptr; // recorded on the download stream after the job's last copy
    bool        busy = false;
    long long   ticket = -1;
};

struct HostCtx
{
    Slot         slot[SLOTS];
    float*       ws[COMPUTE_STREAMS] = {}; // split-K workspaces, one per compute stream (stream order protects them)
    size_t       bytesW[COMPUTE_STREAMS] = {};
    cudaStream_t up = nullptr, down = nullptr, compute[COMPUTE_STREAMS] = {};
    long long    next_ticket = 0;
    int          sms = 0;
    bool         init = false;
};
std::mutex             g_mutex;
std::map<int, HostCtx> g_ctx;

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

// Copy of the sub-matrix [o0, o0+on) x [i0, i0+in) of a packed outer x inner matrix (same shape and
// position on both sides).
cudaError_t copy_rect(float* dst, const float* src, size_t inner, size_t o0, size_t on, size_t i0, size_t in,
                      cudaMemcpyKind kind, cudaStream_t s)
{
    if(in == inner)
        return cudaMemcpyAsync(dst + o0 * inner, src + o0 * inner, on * inner * sizeof(float), kind, s);
    return cudaMemcpy2DAsync(dst + o0 * inner + i0, inner * sizeof(float), src + o0 * inner + i0, inner * sizeof(float),
                             in * sizeof(float), on, kind, s);
}

// Sub-matrix rows [r0, r0+rn) x columns [c0, c0+cn) of a packed rows x cols matrix in the given layout.
cudaError_t copy_block(float* dst, const float* src, int layout, size_t rows, size_t cols, size_t r0, size_t rn,
                       size_t c0, size_t cn, cudaMemcpyKind kind, cudaStream_t s)
{
    if(layout == B200_SGEMM_ROW_MAJOR)
        return copy_rect(dst, src, cols, r0, rn, c0, cn, kind, s);
    return copy_rect(dst, src, rows, c0, cn, r0, rn, kind, s);
}

// Pieces of one dimension: at most MAX_PIECES, multiples of 128 (the CTA tile), about `about` or more each.
void cut(size_t dim, size_t about, size_t* piece, int* count)
{
    size_t want = std::min<size_t>(MAX_PIECES, std::max<size_t>(1, dim / about));
    size_t len  = (dim + want - 1) / want;
    len         = (len + 127) / 128 * 128;
    *piece      = len;
    *count      = int((dim + len - 1) / len);
}

// Split-K factor for an m x n x K strip computed with 128 x 128 tiles on `sms` SMs.  Only the first,
// small strips are split (so that their few tiles still occupy every SM while nothing else is ready);
// larger ones run unsplit: the next strip's kernel fills the SMs their last wave leaves idle.
int pick_split(size_t m, size_t n, size_t K, int sms)
{
    const size_t tiles = ((m + 127) / 128) * ((n + 127) / 128);
    if(tiles * 2 > size_t(sms))
        return 1;
    const size_t s = std::min<size_t>({size_t(sms) / tiles, K / 512, size_t(16)});
    return int(std::max<size_t>(s, 1));
}

struct Strip
{
    size_t r0, rn, c0, cn;
    int    split;
};
struct Step
{
    bool  is_a;
    int   piece;
    bool  has_strip;
    Strip strip;
};

// The schedule of one job: the uploads in order (row panels of A and column panels of B alternately) and, for each,
// the rectangle of C it makes computable.  Pure host arithmetic (exported for tests as b200_sgemm_host_plan).
struct Plan
{
    bool              big = false; // large problem: pieces, the big-cube kernel and split-K chosen here
    size_t            pm = 0, pn = 0;
    std::vector<Step> steps;
};
// Two granularities.  A job that finds the pipeline empty is cut finely (pieces of about 512 rows / columns): its
// first strips start after a few megabytes and the call's latency is what counts.  A job submitted while another one
// is still in flight is cut coarsely (about 2048): then the uploads are the pace-maker, its strips have at least 148
// tiles each and run at the full kernel's rate - the fine strips (16 to 128 tiles, one launch each) together take
// 3.0 ms of GPU time at 4096^3, more than the 2.4 ms of the uploads they should hide behind.
Plan make_plan(size_t M, size_t N, size_t K, int sms, bool pipelined)
{
    Plan p;
    p.big = M >= 1024 && N >= 1024 && K >= 1024;
    p.pm  = M;
    p.pn  = N;
    int nm = 1, nn = 1;
    if(p.big)
    {
        cut(M, pipelined ? 2048 : 512, &p.pm, &nm);
        cut(N, pipelined ? 2048 : 512, &p.pn, &nn);
    }
    size_t rows_done = 0, cols_done = 0;
    for(int k = 0; k < std::max(nm, nn); ++k)
    {
        if(k < nm)
        {
            const size_t r0 = size_t(k) * p.pm, rn = std::min(p.pm, M - r0);
            p.steps.push_back(Step{true, k, cols_done > 0, {r0, rn, 0, cols_done, 1}});
            rows_done = r0 + rn;
        }
        if(k < nn)
        {
            const size_t c0 = size_t(k) * p.pn, cn = std::min(p.pn, N - c0);
            p.steps.push_back(Step{false, k, rows_done > 0, {0, rows_done, c0, cn, 1}});
            cols_done = c0 + cn;
        }
    }
    for(Step& s : p.steps)
        if(s.has_strip)
            s.strip.split = p.big ? pick_split(s.strip.rn, s.strip.cn, K, sms) : 1;
    return p;
}

cudaError_t init_ctx(HostCtx& x, int device)
{
    cudaError_t e;
    if((e = cudaDeviceGetAttribute(&x.sms, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess) return e;
    if((e = cudaStreamCreateWithFlags(&x.up, cudaStreamNonBlocking)) != cudaSuccess) return e;
    if((e = cudaStreamCreateWithFlags(&x.down, cudaStreamNonBlocking)) != cudaSuccess) return e;
    for(int i = 0; i < COMPUTE_STREAMS; ++i)
        if((e = cudaStreamCreateWithFlags(&x.compute[i], cudaStreamNonBlocking)) != cudaSuccess) return e;
    for(Slot& s : x.slot)
    {
        for(int i = 0; i < MAX_STRIPS; ++i)
        {
            if((e = cudaEventCreateWithFlags(&s.uploaded[i], cudaEventDisableTiming)) != cudaSuccess) return e;
            if((e = cudaEventCreateWithFlags(&s.computed[i], cudaEventDisableTiming)) != cudaSuccess) return e;
        }
        if((e = cudaEventCreateWithFlags(&s.done, cudaEventDisableTiming)) != cudaSuccess) return e;
    }
    x.init = true;
    return cudaSuccess;
}

// blocks until the job in this slot (if any) has finished
cudaError_t drain(Slot& s)
{
    if(!s.busy)
        return cudaSuccess;
    cudaError_t e = cudaEventSynchronize(s.done);
    s.busy        = false;
    return e;
}
} // namespace

extern "C" int b200_sgemm_host_submit(int layout_c, int layout_a, int layout_b, float* C, const float* A, const float* B,
                                      size_t M, size_t N, size_t K, long long* ticket)
{
    if(!C || !A || !B || !ticket || M == 0 || N == 0 || K == 0 || (layout_a | layout_b | layout_c) & ~1)
        return B200_SGEMM_INVALID_ARGUMENT;
    int         device = 0;
    cudaError_t e      = cudaGetDevice(&device);
    if(e != cudaSuccess)
        return (int)e;
    std::lock_guard<std::mutex> lock(g_mutex);
    HostCtx&                    x = g_ctx[device];
    if(!x.init && (e = init_ctx(x, device)) != cudaSuccess)
        return (int)e;
    Slot& sl = x.slot[x.next_ticket % SLOTS];
    if((e = drain(sl)) != cudaSuccess) // the job submitted two calls ago owns this slot's device matrices
        return (int)e;

    // Large problems run the table's kernel for big cubes on every strip; small ones (one piece per operand) the
    // table's kernel for their shape, unsplit.
    Slot&      other     = x.slot[(x.next_ticket + 1) % SLOTS];
    bool       pipelined = false;
    if(other.busy && cudaEventQuery(other.done) == cudaErrorNotReady)
    {
        pipelined = true;
        (void)cudaGetLastError(); // "not ready" is an answer, not an error: keep it out of later error checks
    }
    Plan                     plan  = make_plan(M, N, K, x.sms, pipelined);
    const std::vector<Step>& steps = plan.steps;
    const size_t             pm = plan.pm, pn = plan.pn;
    int                      variant = -1;
    if(plan.big && b200_sgemm_select_config(layout_c, layout_a, layout_b, 4096, 4096, 4096, nullptr, &variant) != B200_SGEMM_OK)
        variant = -1;
    size_t ws_need = 0;
    for(const Step& s : steps)
        if(s.has_strip)
            ws_need = std::max(ws_need, b200_sgemm_workspace_bytes(layout_c, layout_a, layout_b, s.strip.rn, s.strip.cn, K,
                                                                   variant, s.strip.split));

    if((e = grow(&sl.dA, &sl.bytesA, M * K * sizeof(float))) != cudaSuccess) return (int)e;
    if((e = grow(&sl.dB, &sl.bytesB, K * N * sizeof(float))) != cudaSuccess) return (int)e;
    if((e = grow(&sl.dC, &sl.bytesC, M * N * sizeof(float))) != cudaSuccess) return (int)e;
    if(ws_need > x.bytesW[0])
    {
        // a workspace may still be in use by the other slot's job: let it finish before the blocks are replaced
        if((e = drain(x.slot[(x.next_ticket + 1) % SLOTS])) != cudaSuccess) return (int)e;
        for(int i = 0; i < COMPUTE_STREAMS; ++i)
            if((e = grow(&x.ws[i], &x.bytesW[i], ws_need)) != cudaSuccess) return (int)e;
    }

    const size_t lda = layout_a == B200_SGEMM_ROW_MAJOR ? K : M;
    const size_t ldb = layout_b == B200_SGEMM_ROW_MAJOR ? N : K;
    const size_t ldc = layout_c == B200_SGEMM_ROW_MAJOR ? N : M;
    auto enqueue = [&]() -> int {
        int ev = 0;
        for(const Step& s : steps)
        {
            if(s.is_a)
            {
                const size_t r0 = size_t(s.piece) * pm, rn = std::min(pm, M - r0);
                e = copy_block(sl.dA, A, layout_a, M, K, r0, rn, 0, K, cudaMemcpyHostToDevice, x.up);
            }
            else
            {
                const size_t c0 = size_t(s.piece) * pn, cn = std::min(pn, N - c0);
                e = copy_block(sl.dB, B, layout_b, K, N, 0, K, c0, cn, cudaMemcpyHostToDevice, x.up);
            }
            if(e != cudaSuccess) return (int)e;
            if(!s.has_strip)
                continue; // the next upload's event also covers this one (same stream)
            const Strip& t = s.strip;
            if((e = cudaEventRecord(sl.uploaded[ev], x.up)) != cudaSuccess) return (int)e;
            const int    ci = ev % COMPUTE_STREAMS;
            cudaStream_t cs = x.compute[ci];
            if((e = cudaStreamWaitEvent(cs, sl.uploaded[ev], 0)) != cudaSuccess) return (int)e;
            const float* ap = layout_a == B200_SGEMM_ROW_MAJOR ? sl.dA + t.r0 * K : sl.dA + t.r0;
            const float* bp = layout_b == B200_SGEMM_ROW_MAJOR ? sl.dB + t.c0 : sl.dB + t.c0 * K;
            float*       cp = layout_c == B200_SGEMM_ROW_MAJOR ? sl.dC + t.r0 * N + t.c0 : sl.dC + t.c0 * M + t.r0;
            const int    st = b200_sgemm_ex(layout_c, layout_a, layout_b, cp, ap, bp, t.rn, t.cn, K, lda, ldb, ldc, variant,
                                            t.split, x.ws[ci], x.bytesW[ci], cs);
            if(st != B200_SGEMM_OK)
                return st;
            if((e = cudaEventRecord(sl.computed[ev], cs)) != cudaSuccess) return (int)e;
            if((e = cudaStreamWaitEvent(x.down, sl.computed[ev], 0)) != cudaSuccess) return (int)e;
            if((e = copy_block(C, sl.dC, layout_c, M, N, t.r0, t.rn, t.c0, t.cn, cudaMemcpyDeviceToHost, x.down)) != cudaSuccess)
                return (int)e;
            ++ev;
        }
        // every download waits for its GEMM, every GEMM for its uploads: the end of the download stream is the end of the job
        if((e = cudaEventRecord(sl.done, x.down)) != cudaSuccess) return (int)e;
        return B200_SGEMM_OK;
    };
    const int status = enqueue();
    if(status != B200_SGEMM_OK)
    {
        cudaDeviceSynchronize(); // whatever was enqueued before the failure must not outlive the slot's reuse
        return status;
    }
    sl.busy   = true;
    sl.ticket = x.next_ticket;
    *ticket   = x.next_ticket++;
    return B200_SGEMM_OK;
}

namespace
{
int write_plan(size_t M, size_t N, size_t K, int sm_count, size_t* rects, int* splits, int capacity, bool pipelined)
{
    if(M == 0 || N == 0 || K == 0 || sm_count < 1 || capacity < 0 || (capacity > 0 && (!rects || !splits)))
        return B200_SGEMM_INVALID_ARGUMENT;
    const Plan p = make_plan(M, N, K, sm_count, pipelined);
    int        n = 0;
    for(const Step& s : p.steps)
    {
        if(!s.has_strip)
            continue;
        if(n < capacity)
        {
            rects[4 * n + 0] = s.strip.r0;
            rects[4 * n + 1] = s.strip.rn;
            rects[4 * n + 2] = s.strip.c0;
            rects[4 * n + 3] = s.strip.cn;
            splits[n]        = s.strip.split;
        }
        ++n;
    }
    return n;
}
} // namespace

extern "C" int b200_sgemm_host_plan(size_t M, size_t N, size_t K, int sm_count, size_t* rects, int* splits, int capacity)
{
    return write_plan(M, N, K, sm_count, rects, splits, capacity, false);
}

extern "C" int b200_sgemm_host_plan_pipelined(size_t M, size_t N, size_t K, int sm_count, size_t* rects, int* splits,
                                              int capacity)
{
    return write_plan(M, N, K, sm_count, rects, splits, capacity, true);
}

extern "C" int b200_sgemm_host_wait(long long ticket)
{
    int         device = 0;
    cudaError_t e      = cudaGetDevice(&device);
    if(e != cudaSuccess)
        return (int)e;
    cudaEvent_t done = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        auto                        it = g_ctx.find(device);
        if(it == g_ctx.end() || ticket < 0 || ticket >= it->second.next_ticket)
            return B200_SGEMM_INVALID_ARGUMENT;
        Slot& sl = it->second.slot[ticket % SLOTS];
        if(sl.ticket != ticket || !sl.busy)
            return B200_SGEMM_OK; // already finished: its slot has been drained (and perhaps reused) since
        done = sl.done;
    }
    e = cudaEventSynchronize(done); // outside the lock: other threads may submit meanwhile
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        Slot&                       sl = g_ctx[device].slot[ticket % SLOTS];
        if(sl.ticket == ticket)
            sl.busy = false;
    }
    return (int)e;
}

extern "C" int b200_sgemm_host(int layout_c, int layout_a, int layout_b, float* C, const float* A, const float* B,
                               size_t M, size_t N, size_t K)
{
    long long ticket = -1;
    const int st     = b200_sgemm_host_submit(layout_c, layout_a, layout_b, C, A, B, M, N, K, &ticket);
    if(st != B200_SGEMM_OK)
        return st;
    return b200_sgemm_host_wait(ticket);
}

extern "C" int b200_sgemm_shutdown_host(void)
{
    std::lock_guard<std::mutex> lock(g_mutex);
    int                         saved = 0;
    cudaGetDevice(&saved);
    for(auto& kv : g_ctx)
    {
        HostCtx& x = kv.second;
        cudaSetDevice(kv.first);
        for(Slot& s : x.slot)
        {
            drain(s);
            cudaFree(s.dA);
            cudaFree(s.dB);
            cudaFree(s.dC);
            if(x.init)
            {
                for(int i = 0; i < MAX_STRIPS; ++i)
                {
                    cudaEventDestroy(s.uploaded[i]);
                    cudaEventDestroy(s.computed[i]);
                }
                cudaEventDestroy(s.done);
            }
        }
        for(int i = 0; i < COMPUTE_STREAMS; ++i)
            cudaFree(x.ws[i]);
        if(x.init)
        {
            cudaStreamDestroy(x.up);
            cudaStreamDestroy(x.down);
            for(int i = 0; i < COMPUTE_STREAMS; ++i)
                cudaStreamDestroy(x.compute[i]);
        }
    }
    g_ctx.clear();
    cudaSetDevice(saved);
    return B200_SGEMM_OK;
}
