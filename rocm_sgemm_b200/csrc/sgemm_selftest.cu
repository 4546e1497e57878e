// b200_sgemm_selftest_bounded_wait: makes a bounded wait of the warp-specialised kernel run out, on purpose and
// harmlessly, so that the time-out path (status word, abort flag, every thread returning) is exercised on a GPU.
//
// This file holds a PRIVATE copy of the kernel templates (the namespace is renamed before the headers are read) built
// with a wait limit of one millisecond instead of one second.  The launch is a single 128 x 128 tile with two K tiles;
// the thread that issues the TMA copies is told to leave out the second one (no copy, no arrival on the stage's
// barrier).  The consumers compute the first K tile, wait for the second, give up after the limit, write
// WS_ERR_FULL_TIMEOUT (1) into the library's status word, raise the CTA's abort flag and return; nothing is in flight
// when they do, no memory is touched out of bounds, nothing traps.  C is not written.
#define WS_SELFTEST_LIMITS 1
#define sgemm_b200 sgemm_b200_selftest
#include "sgemm_ws_kernel.cuh"
#undef sgemm_b200

#include "../../include/b200_sgemm.h"

#include <cstring>

namespace sgemm_b200
{
int* status_word_address(); // sgemm_api.cu
}

namespace
{
using namespace sgemm_b200_selftest;
using Cfg = TileConfig<256, 128, 128, 32, 2, 2, 4, 4, 8, 4, 1, 1, 1, 1>;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

bool encode(CUtensorMap* map, const float* base, size_t inner, size_t outer, int box_inner, int box_outer)
{
    void*                           p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess
       || q != cudaDriverEntryPointSuccess)
        return false;
    // (the kernel's tensor maps carry a batch dimension: extent 1 here)
    const cuuint64_t dims[3]    = {(cuuint64_t)inner, (cuuint64_t)outer, 1};
    const cuuint64_t strides[2] = {(cuuint64_t)inner * sizeof(float), (cuuint64_t)inner * outer * sizeof(float)};
    const cuuint32_t box[3]     = {(cuuint32_t)box_inner, (cuuint32_t)box_outer, 1};
    const cuuint32_t estr[3]    = {1, 1, 1};
    return reinterpret_cast<EncodeTiledFn>(p)(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims,
                                              strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
           == CUDA_SUCCESS;
}
} // namespace

extern "C" int b200_sgemm_selftest_bounded_wait(float* C, const float* A, const float* B, void* cuda_stream)
{
    // col-major A (128 x 64), row-major B (64 x 128), row-major C (128 x 128): both operands straight by TMA
    constexpr int M = 128, N = 128, K = 64;
    if(!C || !A || !B || (reinterpret_cast<uintptr_t>(A) & 15u) || (reinterpret_cast<uintptr_t>(B) & 15u))
        return B200_SGEMM_INVALID_ARGUMENT;
    int* status = sgemm_b200::status_word_address();
    if(!status)
        return B200_SGEMM_NO_KERNEL;
    cudaSetDevice([] { int d = 0; cudaGetDevice(&d); return d; }()); // the encoder wants the context current
    WsArgs w;
    memset(&w, 0, sizeof(w));
    w.g.C = C; w.g.A = A; w.g.B = B;
    w.g.M = M; w.g.N = N; w.g.K = K;
    w.g.lda = M; w.g.ldb = N; w.g.ldc = N;
    w.g.grid_m = w.g.grid_n = 1;
    w.g.splits = 1;
    w.g.k_per_split = K;
    w.g.vec_a = w.g.vec_b = 1;
    w.g.vec_c = (reinterpret_cast<uintptr_t>(C) & 15u) == 0;
    w.total_units = 1;
    w.status = status;
    w.k_tiles = K / Cfg::BK;
    w.test_omit_last_fill = 1;
    w.batch = 1;
    w.coop_src_a = w.coop_src_b = nullptr;
    w.coop_ld_a = w.coop_ld_b = 0;
    w.coop_flags = nullptr;
    w.coop_done = nullptr;
    w.coop_done_target = 0;
    w.alpha = 1.f;
    w.beta = 0.f;
    w.range_q = 0;
    w.range_r = 0;
    CUtensorMap map_a, map_b;
    w.tma_a = encode(&map_a, A, M, K, Cfg::BM, Cfg::BK);
    w.tma_b = encode(&map_b, B, N, K, Cfg::BN, Cfg::BK);
    if(!w.tma_a || !w.tma_b)
        return B200_SGEMM_NO_KERNEL;
    auto         kernel = sgemm_ws_kernel<Cfg, LAYOUT_COL, LAYOUT_ROW, LAYOUT_ROW, true>;
    const size_t smem   = WsLayout<Cfg>::smem_bytes(false, false);
    cudaError_t  e      = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if(e != cudaSuccess)
        return (int)e;
    kernel<<<1, WsLayout<Cfg>::THREADS, smem, static_cast<cudaStream_t>(cuda_stream)>>>(w, map_a, map_b);
    e = cudaPeekAtLastError();
    return e == cudaSuccess ? B200_SGEMM_OK : (int)e;
}
