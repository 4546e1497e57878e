/* Host-only stand-in for <hip/hip_runtime.h>: just enough declarations for the reference's
 * common/hip_utils.hpp and kernel/common.hpp to parse under g++ when the reference's CPU
 * verification code is compiled into oracle/_ref/.  Nothing here is ever called. */
#ifndef ORACLE_SHIM_HIP_RUNTIME_H
#define ORACLE_SHIM_HIP_RUNTIME_H
#include <cstddef>
#include <cstdlib>
typedef int   hipError_t;
typedef void* hipEvent_t;
typedef void* hipStream_t;
static const hipError_t hipSuccess = 0;
inline const char* hipGetErrorString(hipError_t) { return "hip unavailable (host-only shim)"; }
inline hipError_t  hipEventCreate(hipEvent_t*) { return 1; }
inline hipError_t  hipEventDestroy(hipEvent_t) { return 1; }
inline hipError_t  hipEventRecord(hipEvent_t, hipStream_t) { return 1; }
inline hipError_t  hipEventSynchronize(hipEvent_t) { return 1; }
inline hipError_t  hipEventElapsedTime(float*, hipEvent_t, hipEvent_t) { return 1; }
#ifndef __host__
#define __host__
#endif
#ifndef __device__
#define __device__
#endif
#endif
