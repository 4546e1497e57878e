// b200_sgemm_host: the GEMM for callers whose matrices live in HOST memory.
//
// The reference's harnesses copy A and B to the device, call gemm(), and copy C back, one step after the
// other (test/gemm/test.cpp:50-74).  This entry does the same work end to end but overlaps it: B is
// uploaded first, then A and C are cut into row panels and the upload of panel i+1, the GEMM of panel i
// and the download of panel i-1 run concurrently on three streams (the two copy engines of the GPU work
// in both directions at once).  At 4096^3 the transfers (192 MB over PCIe) dominate, so the pipelined
// call approaches the time of the uploads alone instead of the sum of all phases.
//
// Host buffers should be page-locked (cudaHostAlloc / cudaHostRegister); pageable memory works but the
// runtime then stages the copies and the overlap is lost.  The device buffers come from a per-device
// arena owned by the library (grown on demand, released by b200_sgemm_shutdown_host or at exit).
// The call returns after C is complete in host memory.
#include "../../include/b200_sgemm.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <map>
#include <mutex>

namespace
{
struct HostCtx
{
    float*       dA = nullptr;
    float*       dB = nullptr;
    float*       dC = nullptr;
    size_t       bytesA = 0, bytesB = 0, bytesC = 0;
    cudaStream_t up = nullptr, down = nullptr, compute = nullptr;
    cudaEvent_t  b_ready = nullptr;
    cudaEvent_t  a_ready[16] = {};
    cudaEvent_t  c_ready[16] = {};
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

// copy of a sub-range [i0, i0+cnt) of the pitched dimension or of the contiguous dimension of a packed
// outer x inner matrix.  `along_outer`: the panel is a range of whole rows of the stored matrix.
cudaError_t copy_panel(float* dst, const float* src, size_t outer, size_t inner, bool along_outer, size_t i0,
                       size_t cnt, cudaMemcpyKind kind, cudaStream_t s)
{
    if(along_outer)
        return cudaMemcpyAsync(dst + i0 * inner, src + i0 * inner, cnt * inner * sizeof(float), kind, s);
    return cudaMemcpy2DAsync(dst + i0, inner * sizeof(float), src + i0, inner * sizeof(float), cnt * sizeof(float), outer,
                             kind, s);
}
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
        if((e = cudaStreamCreateWithFlags(&x.up, cudaStreamNonBlocking)) != cudaSuccess) return (int)e;
        if((e = cudaStreamCreateWithFlags(&x.down, cudaStreamNonBlocking)) != cudaSuccess) return (int)e;
        if((e = cudaStreamCreateWithFlags(&x.compute, cudaStreamNonBlocking)) != cudaSuccess) return (int)e;
        if((e = cudaEventCreateWithFlags(&x.b_ready, cudaEventDisableTiming)) != cudaSuccess) return (int)e;
        for(int i = 0; i < 16; ++i)
        {
            if((e = cudaEventCreateWithFlags(&x.a_ready[i], cudaEventDisableTiming)) != cudaSuccess) return (int)e;
            if((e = cudaEventCreateWithFlags(&x.c_ready[i], cudaEventDisableTiming)) != cudaSuccess) return (int)e;
        }
        x.init = true;
    }
    if((e = grow(&x.dA, &x.bytesA, M * K * sizeof(float))) != cudaSuccess) return (int)e;
    if((e = grow(&x.dB, &x.bytesB, K * N * sizeof(float))) != cudaSuccess) return (int)e;
    if((e = grow(&x.dC, &x.bytesC, M * N * sizeof(float))) != cudaSuccess) return (int)e;

    // row panels of A and C: multiples of 256 rows, at most 16, each worth a few hundred microseconds
    size_t panels = std::min<size_t>(16, std::max<size_t>(1, M / 1024));
    size_t rows   = (M + panels - 1) / panels;
    rows          = (rows + 255) / 256 * 256;
    panels        = (M + rows - 1) / rows;

    const bool a_outer = layout_a == B200_SGEMM_ROW_MAJOR; // A stored as M rows of K: a row panel is contiguous
    const bool c_outer = layout_c == B200_SGEMM_ROW_MAJOR;
    const size_t a_out = a_outer ? M : K, a_in = a_outer ? K : M;
    const size_t c_out = c_outer ? M : N, c_in = c_outer ? N : M;

    if((e = cudaMemcpyAsync(x.dB, B, K * N * sizeof(float), cudaMemcpyHostToDevice, x.up)) != cudaSuccess) return (int)e;
    if((e = cudaEventRecord(x.b_ready, x.up)) != cudaSuccess) return (int)e;
    if((e = cudaStreamWaitEvent(x.compute, x.b_ready, 0)) != cudaSuccess) return (int)e;
    for(size_t p = 0; p < panels; ++p)
    {
        const size_t r0 = p * rows, cnt = std::min(rows, M - r0);
        if((e = copy_panel(x.dA, A, a_out, a_in, a_outer, r0, cnt, cudaMemcpyHostToDevice, x.up)) != cudaSuccess) return (int)e;
        if((e = cudaEventRecord(x.a_ready[p], x.up)) != cudaSuccess) return (int)e;
        if((e = cudaStreamWaitEvent(x.compute, x.a_ready[p], 0)) != cudaSuccess) return (int)e;
        // the panel lives inside the full-size device matrices: leading dimensions are the full ones
        float*       cp = c_outer ? x.dC + r0 * N : x.dC + r0;
        const float* ap = a_outer ? x.dA + r0 * K : x.dA + r0;
        const int    st = b200_sgemm_ex(layout_c, layout_a, layout_b, cp, ap, x.dB, cnt, N, K, a_outer ? K : M, 0,
                                        c_outer ? N : M, -1, 1, nullptr, 0, x.compute);
        if(st != B200_SGEMM_OK)
        {
            cudaDeviceSynchronize();
            return st;
        }
        if((e = cudaEventRecord(x.c_ready[p], x.compute)) != cudaSuccess) return (int)e;
        if((e = cudaStreamWaitEvent(x.down, x.c_ready[p], 0)) != cudaSuccess) return (int)e;
        if((e = copy_panel(C, x.dC, c_out, c_in, c_outer, r0, cnt, cudaMemcpyDeviceToHost, x.down)) != cudaSuccess) return (int)e;
    }
    if((e = cudaStreamSynchronize(x.down)) != cudaSuccess) return (int)e;
    if((e = cudaStreamSynchronize(x.compute)) != cudaSuccess) return (int)e;
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
        if(x.init)
        {
            cudaStreamDestroy(x.up);
            cudaStreamDestroy(x.down);
            cudaStreamDestroy(x.compute);
            cudaEventDestroy(x.b_ready);
            for(int i = 0; i < 16; ++i)
            {
                cudaEventDestroy(x.a_ready[i]);
                cudaEventDestroy(x.c_ready[i]);
            }
        }
    }
    g_ctx.clear();
    cudaSetDevice(saved);
    return B200_SGEMM_OK;
}
