/*
 * C ABI of the B200 (sm_100a) FlashAttention-2 library, libfa2_b200.so.
 *
 * Plain pointers and sizes only: device pointers are raw CUDA addresses, `stream` is a
 * cudaStream_t / CUstream passed as void*. Every call enqueues work on `stream` and returns
 * without synchronising. Return value: 0 on success, a negative FA2_E_* code on failure;
 * fa2_last_error() returns the message of the last failure on the calling thread.
 *
 * These entry points are what the host layer of the reference crate (flash-attn2-rs, Rust)
 * would bind through `extern "C"` in place of its own cuLaunchKernel calls; the tvm-ffi
 * operator symbols (__tvm_ffi_fwd, ...) in libflash_attn2_b200.so sit on top of them.
 * All tensors use the reference layouts: Q/O [B, Sq, H, D], K/V [B, Sk, Hk, D] (last stride 1),
 * LSE fp32 [B, H, Sq]; packed (varlen) Q/O [total_q, H, D], K/V [total_k, Hk, D],
 * LSE fp32 [H, total_q].
 */
#ifndef FA2_B200_H_
#define FA2_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define FA2_API __attribute__((visibility("default")))
#else
#define FA2_API
#endif

#define FA2_F16 0
#define FA2_BF16 1

#define FA2_OK 0
#define FA2_E_VALUE (-1)   /* bad shape / stride / argument value */
#define FA2_E_TYPE (-2)    /* bad dtype */
#define FA2_E_RUNTIME (-3) /* CUDA failure, or a kernel reported a stalled pipeline */

/* Strides are in elements: {batch, row, head}; the head_dim stride is 1. In packed mode
 * the batch stride is ignored. head_dim is a multiple of 8 up to 256, the reference's range
 * (flash-attn2-rs/src/host/tiles.rs:1): up to 128 on the two-stage kernels, above on kernels with
 * smaller tiles (fwd_wide_sm100.cu, bwd_wide_sm100.cu). */
typedef struct fa2_fwd_args {
  const void* q;
  const void* k;
  const void* v;
  void* out;                   /* [B, Sq, H, D] (or packed), same dtype as q */
  float* lse;                  /* contiguous fp32 [B, H, Sq] (or [H, total_q]) */
  const float* alibi_slopes;   /* fp32 [H] or [B, H], or NULL */
  int32_t alibi_batch_stride;  /* 0 for [H], H for [B, H] */
  int32_t dtype;               /* FA2_F16 or FA2_BF16 */
  int32_t batch, seqlen_q, seqlen_k, heads, heads_k, head_dim;
  int64_t q_stride[3], k_stride[3], v_stride[3], o_stride[3];
  float softmax_scale;
  int32_t causal;
  int32_t window_left, window_right; /* < 0 = unbounded, as passed by the caller */
  float softcap;                     /* 0 = off */
  /* packed (varlen) mode when cu_seqlens_q != NULL: device int32 [batch + 1] each;
   * seqlen_q / seqlen_k are then the maxima and total_q / total_k the packed row counts */
  const int32_t* cu_seqlens_q;
  const int32_t* cu_seqlens_k;
  int32_t total_q, total_k;
  int32_t zero_tensors; /* packed mode: clear out (0) and LSE (-inf) first, as the reference's flag does */
} fa2_fwd_args;

/* Dense forward. Replaces launch_forward + flash_attn_fwd of the reference
 * (flash-attn2-rs/src/host/forward/mod.rs:449-813, src/device/forward/dense.rs:472-590).
 * Empty Sk gives O = 0 and LSE = +inf (forward/mod.rs:548-582). */
FA2_API int fa2_fwd(const fa2_fwd_args* args, void* stream);

/* Packed variable-length forward driven by cu_seqlens on the device, no host read of the
 * metadata. Replaces varlen_fwd (flash-attn2-rs/src/host/varlen/mod.rs:21-630,
 * src/device/varlen/mod.rs:30-318,445-578). */
FA2_API int fa2_varlen_fwd(const fa2_fwd_args* args, void* stream);

/* delta[b,h,s] = sum_d dO*O in fp32, rows padded to a multiple of 128 and the padding zeroed:
 * delta is [B, H, ceil(Sq/128)*128]. Replaces bwd_preprocess
 * (flash-attn2-rs/src/host/backward.rs:628-737, src/device/backward/reduce.rs:40-108). */
typedef struct fa2_bwd_preprocess_args {
  const void* dout;
  const void* out;
  float* delta;
  int32_t dtype;
  int32_t batch, seqlen_q, heads, head_dim;
  int64_t do_stride[3], o_stride[3];
  /* packed mode (varlen_preprocess, src/device/varlen/backward.rs:53-132):
   * delta is [H, total_q + 128*batch], sequence b starts at cu_seqlens_q[b] + 128*b */
  const int32_t* cu_seqlens_q;
  int32_t total_q;
} fa2_bwd_preprocess_args;
FA2_API int fa2_bwd_preprocess(const fa2_bwd_preprocess_args* args, void* stream);

/* Backward: dQ, dK, dV from Q, K, V, dO, LSE and delta. dQ is accumulated in fp32 in
 * `dq_accum` (fa2_bwd_workspace_bytes() bytes, 16-byte aligned, need not be cleared) and
 * converted to the 16-bit dQ at the end. `which` selects outputs: bit 0 = dQ, bit 1 = dK and dV.
 * The workspace is the accumulator (B*Sq*H*D floats, rounded up to 256 bytes) followed by one 32-bit
 * turn counter per 32 query rows of every (batch, head). With them a dQ-only call (which = 1, the
 * deterministic bwd_dq of the reference) adds the key blocks' contributions in a fixed order, so dQ
 * is bit-reproducible; a workspace that only holds the accumulator is accepted too (arrival order).
 * dK and dV never use atomics and are always bit-reproducible. Head dims above 128 always add dQ in
 * arrival order. A dQ-only call (which = 1) may pass dk = dv = NULL, a dK/dV-only call dq = dq_accum = NULL.
 * Replaces backward_component + the `backward` and `backward_kv` kernels
 * (flash-attn2-rs/src/host/backward.rs:14-566, src/device/backward/dq.rs:12-302,438-576,
 *  src/device/backward/dkv.rs:15-266,865-1012). */
typedef struct fa2_bwd_args {
  const void* q;
  const void* k;
  const void* v;
  const void* dout;
  const float* lse;    /* [B, H, Sq] (or [H, total_q]) */
  const float* delta;  /* layout of fa2_bwd_preprocess */
  void* dq;            /* [B, Sq, H, D] contiguous, input dtype */
  void* dk;            /* [B, Sk, Hk, D] contiguous */
  void* dv;
  void* dq_accum;      /* fp32 workspace */
  int64_t dq_accum_bytes;
  int32_t dtype;
  int32_t batch, seqlen_q, seqlen_k, heads, heads_k, head_dim;
  int64_t q_stride[3], k_stride[3], v_stride[3], do_stride[3];
  float softmax_scale;
  int32_t causal;
  int32_t window_left, window_right;
  int32_t which;
  const int32_t* cu_seqlens_q;
  const int32_t* cu_seqlens_k;
  int32_t total_q, total_k;
  /* Optional cudaEvent_t handles recorded on `stream` right before and right after the main
   * dQ/dK/dV kernel (not the memset / convert around it), for per-kernel timing. May be NULL. */
  void* ev_kernel_start;
  void* ev_kernel_stop;
  /* Score transforms of the forward pass that produced `lse` (flash-attn2-rs/src/host/backward.rs:15-34
   * takes the same two): ALiBi slopes ([H] with alibi_batch_stride 0, or [B, H] with stride H; NULL
   * for none) and the softcap (0 for none). */
  const float* alibi_slopes;
  int32_t alibi_batch_stride;
  float softcap;
} fa2_bwd_args;
FA2_API int64_t fa2_bwd_workspace_bytes(const fa2_bwd_args* args);
FA2_API int fa2_bwd(const fa2_bwd_args* args, void* stream);

/* Views the kernels cannot address (base not 16-byte aligned, or an outer stride that is not a
 * multiple of 8 elements) are copied into a packed tensor first, as prepare_attention_tensor does
 * (flash-attn2-rs/src/host/layout.rs:80-100, kernel src/device/layout.rs:4-35). The C ABI does not
 * allocate: the caller tests the view with fa2_layout_is_addressable() (1 = usable as it is) and, if
 * needed, packs it into its own contiguous buffer with fa2_pack_16bit(): `shape` is [n0, n1, n2, d]
 * (use n0 = 1 for packed [total, H, D] tensors), `outer_strides` the element strides of n0, n1, n2;
 * the last dimension has stride 1. */
FA2_API int fa2_layout_is_addressable(const void* ptr, const int64_t* outer_strides, int32_t n_outer);
FA2_API int fa2_pack_16bit(const void* src, void* dst, const int64_t shape[4], const int64_t outer_strides[3],
                           void* stream);

/* Copy of a 16-bit tensor [n0, n1, n2, d] (unit last stride) between two layouts given by their outer element
 * strides: the general form of fa2_pack_16bit. The operator layer uses it to copy a result that was computed
 * into a temporary back into a supplied `out` the kernels cannot write in place (not addressable, or
 * overlapping an input), as the reference does (flash-attn2-rs/src/host/forward/mod.rs:367-375, 832-840,
 * src/host/layout.rs:458-512). */
FA2_API int fa2_copy_16bit(const void* src, const int64_t src_strides[3], void* dst, const int64_t dst_strides[3],
                           const int64_t shape[4], void* stream);

/* Backward that allocates nothing. No counterpart in the reference crate (its host layer always
 * allocates its workspaces through the tvm-ffi environment allocator).
 *
 * For callers that may not call cudaMalloc at all - a serving loop whose device memory was
 * partitioned up front, an embedding runtime that owns the device heap, a sandboxed plugin host -
 * this variant of fa2_bwd keeps the fp32 dQ accumulator (and the kernels' status word) in device
 * arrays that are part of the library image. It ignores args->dq_accum / dq_accum_bytes; the caller
 * still passes every input and output. Neither this call nor anything it reaches calls cudaMalloc,
 * cudaFree or an allocating library routine.
 *
 * Limits and rules:
 *  - dense tensors only, which = 3, head_dim up to 128, and batch * seqlen_q * heads * head_dim must not exceed
 *    FA2_BWD_STATIC_MAX_ELEMENTS (4,194,304: a 16 MiB array that every GPU which loads the
 *    library holds until the process exits); larger problems are rejected with FA2_E_VALUE;
 *  - the first call on a device looks up the arrays' device addresses (cudaGetSymbolAddress, with
 *    that device current). Make that first call outside any stream capture;
 *  - all calls share the one accumulator: each call clears the part it uses, and two calls whose
 *    GPU work overlaps (different streams, or different threads) race on it. Serialise them;
 *  - the kernels' pipeline status of these calls lands in the library image too; read it with
 *    fa2_bwd_static_status(), not fa2_device_status() (which reads the word of the allocating
 *    entry points and allocates it on first use);
 *  - lse and delta usually come from fa2_fwd and fa2_bwd_preprocess. fa2_bwd_preprocess allocates
 *    nothing; fa2_fwd (like fa2_bwd and fa2_device_status) allocates one 64-byte status block per
 *    device on its first call, so a host that cannot allocate later makes that first call while it
 *    still can. */
#define FA2_BWD_STATIC_MAX_ELEMENTS 4194304
FA2_API int fa2_bwd_static(const fa2_bwd_args* args, void* stream);

/* Status word of the fa2_bwd_static calls on `device`, with the meaning of fa2_device_status():
 * synchronises the device, returns 0 when every pipeline wait of those calls completed, else the code
 * of the first wait that ran out, and clears the word. It copies from and to the array in the
 * library image and allocates nothing. No counterpart in the reference crate. */
FA2_API int fa2_bwd_static_status(int device);

/* Message of the last failed call on this thread ("" if none). */
FA2_API const char* fa2_last_error(void);

/* Synchronises `device` and returns the kernels' status word: 0 = every pipeline wait
 * completed; otherwise the code of the first wait that ran out (the kernels bound every
 * wait instead of spinning forever). Clears the word. Negative on CUDA failure. */
FA2_API int fa2_device_status(int device);

/* Number of SMs the persistent kernels size their grids for on `device`. */
FA2_API int fa2_sm_count(int device);

#ifdef __cplusplus
}
#endif
#endif /* FA2_B200_H_ */
