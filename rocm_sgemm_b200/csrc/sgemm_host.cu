// b200_sgemm_host: the GEMM for callers whose matrices live in HOST memory.
//
// The reference's harnesses copy A and B to the device, call gemm(), and copy C back, one step after the
// other (test/gemm/test.cpp:50-74).  This entry does the same work end to end but overlaps the phases.
// At 4096^3 the uploads (128 MiB over PCIe, about 2.4 ms) take longer than the GEMM (2.1 ms), so the aim
// is to have as much of the product as possible computed while the operands are still arriving:
//
//   * A is cut into row panels and B into column panels; they are uploaded alternately (A0 B0 A1 B1 ...).
//     A block C(i,j) needs only A_i and B_j, so after every upload one rectangular strip of C becomes
//     computable: A_k x (the B panels present) after A_k, (the A panels present) x B_k after B_k.  This
//     order maximises the computable share of C at every moment of the upload (the product of the shares
//     of A and B present is largest when the two are equal).
//   * each strip is ONE GEMM launch on the device matrices (leading dimensions = the full ones), with a
//     split-K factor chosen so that tiles x splits fills the SMs in whole waves;
//   * each finished strip is downloaded while the next ones are uploaded and computed (the GPU's copy
//     engines work in both directions at once).
//
// Streams (upload, several for compute, download) ordered by events; nothing is allocated once the buffers of
// a problem size exist.  Host buffers should be page-locked (cudaHostAlloc / cudaHostRegister); pageable
// memory works but the runtime then stages the copies and the overlap is lost.  The device buffers come
// from a per-device arena owned by the library (grown on demand, released by b200_sgemm_shutdown_host).
// The call returns after C is complete in host memory.
#include "../../include/b200_sgemm.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <map>
#include <mutex>
#include <vector>
#ifdef B200_SGEMM_HOST_TRACE
#include <cstdio>
#include <cstdlib>
#endif

namespace
{
constexpr int MAX_PIECES = 8;              // per operand
constexpr int MAX_STRIPS = 2 * MAX_PIECES; // one strip per upload at most
constexpr int COMPUTE_STREAMS = 4;

struct HostCtx
{
    float*       dA = nullptr;
    float*       dB = nullptr;
    float*       dC = nullptr;
    float*       ws[COMPUTE_STREAMS] = {};
    size_t       bytesA = 0, bytesB = 0, bytesC = 0, bytesW[COMPUTE_STREAMS] = {};
    cudaStream_t up = nullptr, down = nullptr, compute[COMPUTE_STREAMS] = {};
    cudaEvent_t  uploaded[MAX_STRIPS] = {};
    cudaEvent_t  computed[MAX_STRIPS] = {};
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

// Pieces of one dimension: at most MAX_PIECES, multiples of 128 (the CTA tile), about 512 or more each.
void cut(size_t dim, size_t* piece, int* count)
{
    size_t want = std::min<size_t>(MAX_PIECES, std::max<size_t>(1, dim / 512));
#ifdef B200_SGEMM_HOST_TRACE
    if(const char* v = std::getenv("B200_HOST_PIECES"))
        want = std::min<size_t>(MAX_PIECES, std::max<size_t>(1, std::atoi(v)));
#endif
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
} // namespace

extern "C" int b200_sgemm_host(int layout_c, int layout_a, int layout_b, float* C, const float* A, const float* B,
                               size_t M, size_t N, size_t K)
{
    if(!C || !A || !B || M == 0 || N == 0 || K == 0 || (layout_a | layout_b | layout_c) & ~1)
        return B200_SGEMM_INVALID_ARGUMENT;
    int         device = 0;
    cudaError_t e      = cudaGetDevice(&device);
    if(e != cudaSuccess)
        return (int)e;
    std::lock_guard<std::mutex> lock(g_mutex); // one host-buffer call per process at a time: they share the arena
    HostCtx&                    x = g_ctx[device];
    if(!x.init)
    {
        if((e = cudaDeviceGetAttribute(&x.sms, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess) return (int)e;
        if((e = cudaStreamCreateWithFlags(&x.up, cudaStreamNonBlocking)) != cudaSuccess) return (int)e;
        if((e = cudaStreamCreateWithFlags(&x.down, cudaStreamNonBlocking)) != cudaSuccess) return (int)e;
        for(int i = 0; i < COMPUTE_STREAMS; ++i)
            if((e = cudaStreamCreateWithFlags(&x.compute[i], cudaStreamNonBlocking)) != cudaSuccess) return (int)e;
        for(int i = 0; i < MAX_STRIPS; ++i)
        {
            if((e = cudaEventCreateWithFlags(&x.uploaded[i], cudaEventDisableTiming)) != cudaSuccess) return (int)e;
            if((e = cudaEventCreateWithFlags(&x.computed[i], cudaEventDisableTiming)) != cudaSuccess) return (int)e;
        }
        x.init = true;
    }

    // Large problems: the table's kernel for big cubes, pieces and split-K chosen here.  Small ones: one
    // piece per operand and whatever the table says for the shape.
    const bool big     = M >= 1024 && N >= 1024 && K >= 1024;
    int        variant = -1;
    size_t     pm = M, pn = N;
    int        nm = 1, nn = 1;
    if(big)
    {
        if(b200_sgemm_select_config(layout_c, layout_a, layout_b, 4096, 4096, 4096, nullptr, &variant) != B200_SGEMM_OK)
            variant = -1;
        cut(M, &pm, &nm);
        cut(N, &pn, &nn);
    }

    // the schedule: uploads in order, the strip each one makes computable
    struct Step
    {
        bool  is_a;
        int   piece;
        bool  has_strip;
        Strip strip;
    };
    std::vector<Step> steps;
    size_t            rows_done = 0, cols_done = 0, ws_need = 0;
    for(int k = 0; k < std::max(nm, nn); ++k)
    {
        if(k < nm)
        {
            const size_t r0 = size_t(k) * pm, rn = std::min(pm, M - r0);
            Step         s{true, k, cols_done > 0, {r0, rn, 0, cols_done, 1}};
            rows_done = r0 + rn;
            steps.push_back(s);
        }
        if(k < nn)
        {
            const size_t c0 = size_t(k) * pn, cn = std::min(pn, N - c0);
            Step         s{false, k, rows_done > 0, {0, rows_done, c0, cn, 1}};
            cols_done = c0 + cn;
            steps.push_back(s);
        }
    }
    for(Step& s : steps)
    {
        if(!s.has_strip)
            continue;
        s.strip.split = big ? pick_split(s.strip.rn, s.strip.cn, K, x.sms) : 1;
        ws_need       = std::max(ws_need, b200_sgemm_workspace_bytes(layout_c, layout_a, layout_b, s.strip.rn, s.strip.cn,
                                                                     K, variant, s.strip.split));
    }

    if((e = grow(&x.dA, &x.bytesA, M * K * sizeof(float))) != cudaSuccess) return (int)e;
    if((e = grow(&x.dB, &x.bytesB, K * N * sizeof(float))) != cudaSuccess) return (int)e;
    if((e = grow(&x.dC, &x.bytesC, M * N * sizeof(float))) != cudaSuccess) return (int)e;
    for(int i = 0; i < COMPUTE_STREAMS; ++i)
        if((e = grow(&x.ws[i], &x.bytesW[i], ws_need)) != cudaSuccess) return (int)e;

    const size_t lda = layout_a == B200_SGEMM_ROW_MAJOR ? K : M;
    const size_t ldb = layout_b == B200_SGEMM_ROW_MAJOR ? N : K;
    const size_t ldc = layout_c == B200_SGEMM_ROW_MAJOR ? N : M;
    int          ev  = 0;
#ifdef B200_SGEMM_HOST_TRACE
    // timeline of one call: start/end of every upload, GEMM and download relative to the first upload
    std::vector<cudaEvent_t> tev;
    std::vector<const char*> tname;
    auto mark = [&](cudaStream_t st, const char* name) {
        cudaEvent_t q;
        cudaEventCreate(&q);
        cudaEventRecord(q, st);
        tev.push_back(q);
        tname.push_back(name);
    };
    mark(x.up, "start");
#else
    auto mark = [](cudaStream_t, const char*) {};
#endif
    for(const Step& s : steps)
    {
        if(s.is_a)
        {
            const size_t r0 = size_t(s.piece) * pm, rn = std::min(pm, M - r0);
            e = copy_block(x.dA, A, layout_a, M, K, r0, rn, 0, K, cudaMemcpyHostToDevice, x.up);
        }
        else
        {
            const size_t c0 = size_t(s.piece) * pn, cn = std::min(pn, N - c0);
            e = copy_block(x.dB, B, layout_b, K, N, 0, K, c0, cn, cudaMemcpyHostToDevice, x.up);
        }
        if(e != cudaSuccess) return (int)e;
        mark(x.up, s.is_a ? "A up end" : "B up end");
        if(!s.has_strip)
            continue; // the next upload's event also covers this one (same stream)
        const Strip& t = s.strip;
        if((e = cudaEventRecord(x.uploaded[ev], x.up)) != cudaSuccess) return (int)e;
        // strips rotate over several compute streams: the kernels are persistent (one CTA per SM, one or
        // two tiles each), so the CTAs of the following strips start on the SMs that the last wave of the
        // earlier ones leaves idle
        const int    ci = ev % COMPUTE_STREAMS;
        cudaStream_t cs = x.compute[ci];
        if((e = cudaStreamWaitEvent(cs, x.uploaded[ev], 0)) != cudaSuccess) return (int)e;
        const float* ap = layout_a == B200_SGEMM_ROW_MAJOR ? x.dA + t.r0 * K : x.dA + t.r0;
        const float* bp = layout_b == B200_SGEMM_ROW_MAJOR ? x.dB + t.c0 : x.dB + t.c0 * K;
        float*       cp = layout_c == B200_SGEMM_ROW_MAJOR ? x.dC + t.r0 * N + t.c0 : x.dC + t.c0 * M + t.r0;
        mark(cs, "gemm start");
        const int    st = b200_sgemm_ex(layout_c, layout_a, layout_b, cp, ap, bp, t.rn, t.cn, K, lda, ldb, ldc, variant,
                                        t.split, x.ws[ci], x.bytesW[ci], cs);
        mark(cs, "gemm end");
        if(st != B200_SGEMM_OK)
        {
            cudaDeviceSynchronize();
            return st;
        }
        if((e = cudaEventRecord(x.computed[ev], cs)) != cudaSuccess) return (int)e;
        if((e = cudaStreamWaitEvent(x.down, x.computed[ev], 0)) != cudaSuccess) return (int)e;
        if((e = copy_block(C, x.dC, layout_c, M, N, t.r0, t.rn, t.c0, t.cn, cudaMemcpyDeviceToHost, x.down)) != cudaSuccess)
            return (int)e;
        mark(x.down, "down end");
        ++ev;
    }
    if((e = cudaStreamSynchronize(x.down)) != cudaSuccess) return (int)e;
    for(int i = 0; i < COMPUTE_STREAMS; ++i)
        if((e = cudaStreamSynchronize(x.compute[i])) != cudaSuccess) return (int)e;
    if((e = cudaStreamSynchronize(x.up)) != cudaSuccess) return (int)e;
#ifdef B200_SGEMM_HOST_TRACE
    if(std::getenv("B200_HOST_TRACE"))
    {
        int si = 0;
        for(size_t i = 1; i < tev.size(); ++i)
        {
            float ms = 0;
            cudaEventElapsedTime(&ms, tev[0], tev[i]);
            std::printf("%8.3f ms  %s", ms, tname[i]);
            if(tname[i][0] == 'g' && tname[i][5] == 's')
            {
                while(!steps[si].has_strip) ++si;
                std::printf("  %zux%zu split %d", steps[si].strip.rn, steps[si].strip.cn, steps[si].strip.split);
                ++si;
            }
            std::printf("\n");
        }
    }
    for(cudaEvent_t q : tev)
        cudaEventDestroy(q);
#endif
    return B200_SGEMM_OK;
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
        cudaFree(x.dA);
        cudaFree(x.dB);
        cudaFree(x.dC);
        for(int i = 0; i < COMPUTE_STREAMS; ++i)
            cudaFree(x.ws[i]);
        if(x.init)
        {
            cudaStreamDestroy(x.up);
            cudaStreamDestroy(x.down);
            for(int i = 0; i < COMPUTE_STREAMS; ++i)
                cudaStreamDestroy(x.compute[i]);
            for(int i = 0; i < MAX_STRIPS; ++i)
            {
                cudaEventDestroy(x.uploaded[i]);
                cudaEventDestroy(x.computed[i]);
            }
        }
    }
    g_ctx.clear();
    cudaSetDevice(saved);
    return B200_SGEMM_OK;
}
