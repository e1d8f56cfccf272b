// Internal launch entry points of the sm_100a kernels (one translation unit per kernel family).
#pragma once
#include <cuda_runtime.h>
#include "fa2_params.h"

namespace fa2 {

// Dense and packed (varlen) forward; head_dim is a multiple of 8 up to 128 (kernels for D = 64 and 128).
cudaError_t launch_fwd(const FwdParams& p, int head_dim, bool bf16, int num_sms, cudaStream_t stream);

// The same for head_dim a multiple of 8 in 136..256: one CTA per 128-row query block, 64-key tiles; p.tm_k and
// p.tm_v carry boxes of 64 rows.
cudaError_t launch_fwd_wide(const FwdParams& p, int head_dim, bool bf16, cudaStream_t stream);

// dQ / dK / dV for head_dim a multiple of 8 up to 128; the fp32 dQ accumulator behind p.tm_dqa (and the turn
// counters p.dq_turn, when given) must be zero.
cudaError_t launch_bwd(const BwdParams& p, int head_dim, bool bf16, int num_sms, cudaStream_t stream);

// The same for head_dim a multiple of 8 in 136..256: one CTA per (128 keys, half of the head dim), query blocks of
// 64 rows; p.tm_q and p.tm_do carry boxes of 64 rows, dQ goes through p.dq_acc, dK and dV through p.dk_ptr / p.dv_ptr.
cudaError_t launch_bwd_wide(const BwdParams& p, int head_dim, bool bf16, cudaStream_t stream);

// delta = rowsum(dO * O) into the padded layouts (dense [B,H,Sq_pad], packed [H,total_q+128*B]).
cudaError_t launch_bwd_preprocess(const PreprocessParams& p, cudaStream_t stream);

// Copy of a 16-bit [n0, n1, n2, d] tensor (unit last stride) between two layouts given by their outer element strides.
cudaError_t launch_copy_rows(const void* src, void* dst, int64_t n0, int64_t n1, int64_t n2, int64_t d,
                             const int64_t src_strides[3], const int64_t dst_strides[3], cudaStream_t stream);
// dst(16-bit) = src(fp32) * scale over n elements (n a multiple of 8).
cudaError_t launch_dq_convert(const float* src, void* dst, int64_t n, float scale, bool bf16, cudaStream_t stream);

}  // namespace fa2
