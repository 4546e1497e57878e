// b200_sgemm_splitk_static: the split-K GEMM with its partial-sum scratch inside the library image.
//
// Who needs this.  Split-K needs `splits` x M x N floats of scratch beyond the caller's A, B and C.  The
// other entry points get it from a buffer the caller allocated (b200_sgemm_ex) or from an arena that
// the library grows with cudaMalloc (b200_sgemm).  Some hosts can do neither: a process that handed
// the whole device to its own memory pool at start-up, so that a later cudaMalloc fails or eats into
// somebody else's budget; a service thread with a latency bound that must not enter the driver's
// allocator, which takes a device-wide lock and can synchronise the device; a plug-in whose host
// forbids device allocation outside an init hook that the plug-in cannot extend.  For them the scratch
// is a fixed array in device global memory that belongs to the library's own image.
//
// What it costs, and when.  B200_SGEMM_STATIC_SCRATCH_BYTES (32 MiB) of device memory on every GPU on which the
// entry point has been called, held until the process exits.  The memory is reserved when the CUDA runtime loads
// this file's module on the device.  With CUDA 12's default (lazy module loading) that happens at the first use of
// the module on that device, which is the first call of this entry point there: that one call makes the driver
// reserve the 32 MiB (free device memory drops by that much, and the call can fail with an out-of-memory error
// on a device that has none left), every later call finds the array in place and leaves free memory exactly as it
// was.  A host that may not touch the allocator later must therefore make one call per device inside its
// initialisation phase (any small problem will do), or start the process with CUDA_MODULE_LOADING=EAGER, which moves
// the reservation to the creation of the device's context.  The cached device address does not survive
// cudaDeviceReset().
//
// Rules for callers.
//   * splits x M x N x 4 bytes must fit the array; otherwise the call is rejected with
//     B200_SGEMM_SCRATCH_LIMIT and nothing is launched.
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress) and
//     caches it.  That lookup is a runtime call that loads the module on the device (see above); make the
//     first call on a device during initialisation and before starting any stream capture on it.
//   * All calls on a device share the one array, and the array keeps whatever the previous call left in
//     it.  Nothing has to start at zero: every K slice overwrites its whole M x N partial before the
//     reduction reads it.  Two calls whose kernels can overlap on the GPU (different streams, no event
//     between them) race on the array and corrupt each other's result; order them on one stream or with
//     events.
//   * No cudaMalloc, cudaFree, cudaMallocAsync or other allocating routine is reached from here; the only
//     memory the driver ever sets aside on behalf of this entry point is the array itself, once per device.
#include "../../include/b200_sgemm.h"

#include <cuda_runtime.h>
#include <mutex>

namespace
{
constexpr size_t kScratchFloats = B200_SGEMM_STATIC_SCRATCH_BYTES / sizeof(float);

// Device code could name this array directly.  Host code cannot: on the host the identifier is only a
// handle for the runtime's symbol table, not a device address, so the address is fetched per device.
static __device__ __align__(256) float g_static_scratch[kScratchFloats];

constexpr int kMaxDevices = 64;
std::mutex    g_mutex;
float*        g_scratch_ptr[kMaxDevices] = {};

// Device address of the array on the current device; looked up once per device, with that device current.
cudaError_t scratch_address(float** out)
{
    int         device = 0;
    cudaError_t e      = cudaGetDevice(&device);
    if(e != cudaSuccess)
        return e;
    if(device < 0 || device >= kMaxDevices)
        return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_mutex);
    if(!g_scratch_ptr[device])
    {
        float* ptr = nullptr;
        e          = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch);
        if(e != cudaSuccess)
            return e;
        g_scratch_ptr[device] = ptr;
    }
    *out = g_scratch_ptr[device];
    return cudaSuccess;
}
} // namespace

extern "C" int b200_sgemm_splitk_static(int layout_c, int layout_a, int layout_b, float* C, const float* A,
                                        const float* B, size_t M, size_t N, size_t K, int split_k, void* cuda_stream)
{
    if(split_k < 2)
        return B200_SGEMM_INVALID_ARGUMENT; // without a split there is no scratch: use b200_sgemm_ex
    // what the split-K launch will ask for (0 when K is too short to be split at all)
    const size_t need = b200_sgemm_workspace_bytes(layout_c, layout_a, layout_b, M, N, K, -1, split_k);
    if(need > B200_SGEMM_STATIC_SCRATCH_BYTES)
        return B200_SGEMM_SCRATCH_LIMIT;
    float*      scratch = nullptr;
    cudaError_t e       = scratch_address(&scratch);
    if(e != cudaSuccess)
        return static_cast<int>(e);
    // same kernels as the other entry points, pointed at the built-in array instead of a caller buffer
    return b200_sgemm_ex(layout_c, layout_a, layout_b, C, A, B, M, N, K, 0, 0, 0, -1, split_k, scratch,
                         B200_SGEMM_STATIC_SCRATCH_BYTES, cuda_stream);
}
