// Internal launch entry points of the sm_100a kernels (one translation unit per kernel family).
#pragma once
#include <cuda_runtime.h>
#include "fa2_params.h"

namespace fa2 {

// Dense and packed (varlen) forward; head_dim is 64 or 128.
cudaError_t launch_fwd(const FwdParams& p, int head_dim, bool bf16, int num_sms, cudaStream_t stream);

}  // namespace fa2
