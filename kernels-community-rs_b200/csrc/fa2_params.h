// Kernel-side parameter blocks shared by the host launchers and the sm_100a kernels.
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace fa2 {

// Error codes a kernel leaves in its status word when a bounded wait runs out.
enum WaitSite : int {
  kWaitNone = 0,
  kWaitLoadQEmpty = 11,
  kWaitLoadKVEmpty = 12,
  kWaitMmaQFull = 21,
  kWaitMmaKVFull = 22,
  kWaitMmaPFull = 23,
  kWaitMmaOFree = 24,
  kWaitMmaSFree = 25,
  kWaitSoftmaxSFull = 31,
  kWaitSoftmaxPvDone = 32,
  kWaitEpiFinal = 41,
  kWaitEpiPvDone = 42,
  kWaitBwd = 50,
};

struct FwdParams {
  CUtensorMap tm_q, tm_k, tm_v, tm_o;  // 4-D maps: (D, heads, rows, batch), box (64, 1, 128, 1)
  void* o_ptr;                         // for the predicated (non-TMA) output path
  float* lse_ptr;
  const int32_t* cu_q;                 // packed (varlen) mode when non-null
  const int32_t* cu_k;
  const float* alibi;                  // [H] or [B,H] slopes, or null
  int64_t o_row_stride, o_head_stride, o_batch_stride;  // elements
  int64_t lse_head_stride, lse_batch_stride;            // elements
  int alibi_batch_stride;
  int batch, heads, heads_k, seqlen_q, seqlen_k;        // seqlen_* = maxima in packed mode
  int group;                           // heads / heads_k
  int num_mblk;                        // ceil(seqlen_q / 256)
  int num_tiles;                       // num_mblk * batch * heads
  int window_left, window_right;       // normalised; < 0 = open side
  int causal_alibi;                    // causal ALiBi depends on the key position only
  float scale;                         // softmax scale (applied before softcap / mask)
  float scale_log2;                    // scale * log2(e)
  float softcap;                       // 0 = off
  int* status;                         // device status word (0 = ok)
  int head_dim;                         // real head dim (<= the kernel's D; columns beyond it are padding)
};

struct BwdParams {
  CUtensorMap tm_q, tm_k, tm_v, tm_do;  // 16-bit inputs, box (64, 1, 128, 1)
  CUtensorMap tm_dk, tm_dv;             // 16-bit outputs, box (64, 1, 128, 1)
  CUtensorMap tm_dqa;                   // fp32 dQ accumulator, box (32, 1, 32, 1): one drain warp's rows
  const float* lse;
  const float* delta;
  void* dk_ptr;
  void* dv_ptr;
  const int32_t* cu_q;
  const int32_t* cu_k;
  int64_t lse_head_stride, lse_batch_stride;
  int64_t delta_head_stride, delta_batch_stride;
  int64_t dkv_row_stride, dkv_head_stride, dkv_batch_stride;  // elements
  int delta_seq_pad;                    // 128 in packed mode (sequence b starts at cu_q[b] + 128 b), else 0
  int batch, heads, heads_k, group, seqlen_q, seqlen_k;
  int num_nblk;                         // ceil(seqlen_k / 128)
  int window_left, window_right;
  int which;                            // bit 0: dQ, bit 1: dK and dV
  float scale, scale_log2;
  int* status;
  // Score transforms of the forward that the gradients have to follow (null / 0 when unused).
  const float* alibi;                   // [heads] or [batch, heads] slopes
  int alibi_batch_stride;
  int causal_alibi;                     // bias = slope * key index instead of -slope * |distance|
  float softcap;                        // scores = softcap * tanh(raw * scale / softcap)
  int head_dim;                         // real head dim (<= the kernel's D; columns beyond it are padding)
  // Ordered dQ accumulation (null = arrival order). dq_turn[((batch * heads + head) * num_mblk_q + query
  // block) * 4 + drain warp] counts the key blocks whose adds into those 32 rows have landed; it is
  // zero at launch. A CTA adds only when the count equals the number of higher key blocks that add into the
  // same rows, so every element is summed in descending key-block order and dQ is bit-reproducible.
  int* dq_turn;
  int num_mblk_q;                       // ceil(seqlen_q / 128)
  // The kernel for head dims above 128 adds into the accumulator with plain reductions:
  // dq_acc[((batch * dq_rows + row) * heads + head) * head_dim + d], dq_rows rows per batch entry.
  float* dq_acc;
  int64_t dq_rows;
  // That kernel reads V row by row from global memory (it keeps V in TMEM): element strides of [batch, row, head].
  const void* v_ptr;
  int64_t v_batch_stride, v_row_stride, v_head_stride;
};

struct PreprocessParams {
  const void* dout;
  const void* out;
  float* delta;
  const int32_t* cu_q;
  int64_t do_batch_stride, do_row_stride, do_head_stride;
  int64_t o_batch_stride, o_row_stride, o_head_stride;
  int64_t delta_head_stride, delta_batch_stride;
  int batch, heads, seqlen_q, seqlen_pad, head_dim;
  int bf16;
};

}  // namespace fa2
