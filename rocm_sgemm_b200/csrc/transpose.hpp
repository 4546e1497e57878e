// Internal to the library: the HBM-bound transposition used to turn a K-contiguous operand into an M/N-contiguous one
// (and the other way round for the tensor-core column).  src is X rows of K contiguous floats (pitch ld_in), dst is K
// rows of X contiguous floats (pitch ld_out); defined in sgemm_api.cu.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>

namespace sgemm_b200
{
cudaError_t launch_transpose(const float* src, float* dst, size_t X, size_t K, size_t ld_in, size_t ld_out,
                             cudaStream_t stream);
}
