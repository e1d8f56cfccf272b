// Host side of the C ABI: argument validation, TMA descriptor construction, launches.
// Mirrors the checks of the reference host layer (flash-attn2-rs/src/host/forward/mod.rs:52-447,
// src/host/layout.rs:46-125, src/host/backward.rs:14-99, src/host/varlen/mod.rs:21-630) for
// the paths this library implements.
#include "../../include/fa2_b200.h"
#include "fa2_launch.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <climits>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

namespace {

thread_local char g_error[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Per-device state, created on first use (the reference keeps the same kind of lazily built,
// never-freed per-device runtime: flash-attn2-rs/src/host/runtime.rs:68-84).
struct Runtime {
  bool ready = false;
  int sm_count = 0;
  int cc_major = 0;
  int* status = nullptr;  // device status word
};
constexpr int kMaxDevices = 64;
constexpr int kStatusWords = 16;
Runtime g_rt[kMaxDevices];
std::mutex g_mu;
EncodeTiledFn g_encode = nullptr;

int get_runtime(int device, Runtime** out) {
  if (device < 0 || device >= kMaxDevices) return fail(FA2_E_VALUE, "device index %d out of range", device);
  std::lock_guard<std::mutex> lock(g_mu);
  Runtime& rt = g_rt[device];
  if (!rt.ready) {
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return fail(FA2_E_RUNTIME, "cudaSetDevice(%d): %s", device, cudaGetErrorString(e));
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return fail(FA2_E_RUNTIME, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
    if (prop.major != 10)
      return fail(FA2_E_RUNTIME, "this library is built for sm_100a only; device %d is sm_%d%d", device, prop.major,
                  prop.minor);
    if (g_encode == nullptr) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult q;
      e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
      if (e != cudaSuccess || fn == nullptr)
        return fail(FA2_E_RUNTIME, "cuTensorMapEncodeTiled is not available from the driver");
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    // word 0: kernel status
    e = cudaMalloc(&rt.status, kStatusWords * sizeof(int));
    if (e != cudaSuccess) return fail(FA2_E_RUNTIME, "cudaMalloc(status): %s", cudaGetErrorString(e));
    cudaMemset(rt.status, 0, kStatusWords * sizeof(int));
    rt.sm_count = prop.multiProcessorCount;
    rt.cc_major = prop.major;
    rt.ready = true;
  }
  *out = &rt;
  return FA2_OK;
}

// 4-D map over [batch][rows][heads][D] with arbitrary (16-byte multiple) outer strides; the
// box is one 128-byte swizzle line wide and `box_rows` rows tall.
int make_map(CUtensorMap* m, const void* ptr, int dtype, int esize, int64_t d, int64_t heads, int64_t rows,
             int64_t batch, int64_t head_stride, int64_t row_stride, int64_t batch_stride, int box_inner, int box_rows,
             const char* name) {
  const int64_t inner_bytes = d * esize;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(d), static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(rows),
                        static_cast<cuuint64_t>(batch)};
  // Size-1 dimensions may carry arbitrary strides; give them a legal one.
  int64_t hs = heads > 1 ? head_stride * esize : inner_bytes;
  int64_t rs = rows > 1 ? row_stride * esize : inner_bytes;
  int64_t bs = batch > 1 ? batch_stride * esize : inner_bytes;
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(hs), static_cast<cuuint64_t>(rs), static_cast<cuuint64_t>(bs)};
  cuuint32_t box[4] = {static_cast<cuuint32_t>(box_inner), 1, static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUtensorMapDataType dt = dtype == 2   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                           : dtype == FA2_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = g_encode(m, dt, 4, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(FA2_E_VALUE, "cannot build a TMA descriptor for %s (CUresult %d)", name, (int)r);
  return FA2_OK;
}

// The reference copies a tensor into a packed buffer when its base is not 16-byte aligned or an
// outer stride is not a multiple of 8 elements (layout.rs:80-100); TMA has the same rule. This
// library asks the caller for such a layout instead of copying.
int check_layout(const void* ptr, const int64_t* stride, int nstride, const char* name) {
  if (ptr == nullptr) return fail(FA2_E_VALUE, "%s is null", name);
  if (reinterpret_cast<uintptr_t>(ptr) % 16 != 0) return fail(FA2_E_VALUE, "%s must be 16-byte aligned", name);
  for (int i = 0; i < nstride; ++i)
    if (stride[i] % 8 != 0 || stride[i] < 0)
      return fail(FA2_E_VALUE, "%s: outer strides must be non-negative multiples of 8 elements", name);
  return FA2_OK;
}

// Makes the device that owns `ptr` current for the lifetime of the object and restores the caller's
// device afterwards, as the reference binds the context of q before every launch
// (flash-attn2-rs/src/host/forward/mod.rs:716-718). A pointer the runtime does not know (or a null
// one) leaves the current device as it is.
class DeviceScope {
 public:
  explicit DeviceScope(const void* ptr) {
    cudaGetDevice(&prev_);
    device_ = prev_;
    cudaPointerAttributes attr;
    if (ptr != nullptr && cudaPointerGetAttributes(&attr, ptr) == cudaSuccess &&
        (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) && attr.device >= 0)
      device_ = attr.device;
    else
      cudaGetLastError();  // an unknown pointer is not an error of this call
    if (device_ != prev_) cudaSetDevice(device_);
  }
  ~DeviceScope() {
    if (device_ != prev_) cudaSetDevice(prev_);
  }
  DeviceScope(const DeviceScope&) = delete;
  DeviceScope& operator=(const DeviceScope&) = delete;
  int device() const { return device_; }

 private:
  int prev_ = 0, device_ = 0;
};

struct Windows {
  int left, right, causal_alibi;
};
// Window normalisation of the reference (forward/mod.rs:310-328, backward.rs:134-149): clamp
// sides that cover every key to "open", causal means right = 0.
Windows normalise_windows(int64_t wl, int64_t wr, bool causal, int64_t seqlen_k, bool causal_first) {
  if (causal_first && causal) wr = 0;
  if (wl >= seqlen_k) wl = -1;
  if (wr >= seqlen_k) wr = -1;
  if (causal) wr = 0;
  Windows w;
  w.causal_alibi = (wl < 0 && wr == 0) ? 1 : 0;
  w.left = wl < 0 ? -1 : static_cast<int>(wl);
  w.right = wr < 0 ? -1 : static_cast<int>(wr);
  return w;
}

__global__ void fill_empty_kernel(uint16_t* out, float* lse, int64_t rows, int heads, int d, int64_t o_row_stride,
                                  int64_t o_head_stride, int64_t o_batch_stride, int64_t rows_per_batch,
                                  int64_t lse_head_stride, int64_t lse_batch_stride, float lse_value) {
  // one thread per (row, head): zero the output row and write the LSE
  const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (idx >= rows * heads) return;
  const int64_t r = idx / heads;
  const int h = static_cast<int>(idx - r * heads);
  const int64_t b = r / rows_per_batch, s = r - b * rows_per_batch;
  uint16_t* o = out + b * o_batch_stride + s * o_row_stride + h * o_head_stride;
  for (int i = 0; i < d; ++i) o[i] = 0;
  lse[b * lse_batch_stride + h * lse_head_stride + s] = lse_value;
}

__global__ void fill_f32_kernel(float* dst, int64_t n, float value) {
  const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (i < n) dst[i] = value;
}

int fwd_common(const fa2_fwd_args* a, void* stream_v, bool packed) {
  if (a == nullptr) return fail(FA2_E_VALUE, "args is null");
  if (a->dtype != FA2_F16 && a->dtype != FA2_BF16) return fail(FA2_E_TYPE, "q, k, v must be float16 or bfloat16");
  const int d = a->head_dim;
  if (d > 256) return fail(FA2_E_VALUE, "head dim must be <= 256, got %d", d);
  if (d < 8 || d % 8 != 0) return fail(FA2_E_VALUE, "head_size must be a positive multiple of 8, got %d", d);
  if (a->heads_k <= 0 || a->heads % a->heads_k != 0)
    return fail(FA2_E_VALUE, "num_heads (%d) must be a multiple of num_heads_k (%d)", a->heads, a->heads_k);
  if (a->batch <= 0 || a->heads <= 0 || a->batch > 65535 || a->heads > 65535)
    return fail(FA2_E_VALUE, "batch and heads must each be in 1..=65535, got %d and %d", a->batch, a->heads);
  if (a->seqlen_q < 0 || a->seqlen_k < 0)
    return fail(FA2_E_VALUE, "seqlens must be non-negative, got q=%d, k=%d", a->seqlen_q, a->seqlen_k);
  if (!std::isfinite(a->softmax_scale)) return fail(FA2_E_VALUE, "softmax_scale must be finite");
  if (packed) {
    if (a->cu_seqlens_q == nullptr || a->cu_seqlens_k == nullptr)
      return fail(FA2_E_VALUE, "packed forward needs cu_seqlens_q and cu_seqlens_k");
    if (reinterpret_cast<uintptr_t>(a->cu_seqlens_q) % 4 || reinterpret_cast<uintptr_t>(a->cu_seqlens_k) % 4)
      return fail(FA2_E_VALUE, "cu_seqlens must be 4-byte aligned");
    if (a->total_q < 0 || a->total_k < 0) return fail(FA2_E_VALUE, "total_q and total_k must be non-negative");
  }
  const DeviceScope scope(a->q);
  Runtime* rt = nullptr;
  int rc = get_runtime(scope.device(), &rt);
  if (rc != FA2_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

  const int64_t rows_q = packed ? a->total_q : a->seqlen_q;
  const int64_t rows_k = packed ? a->total_k : a->seqlen_k;
  const int64_t nbatch = packed ? 1 : a->batch;
  if (rows_q == 0 || a->seqlen_q == 0) return FA2_OK;

  fa2::FwdParams p;
  memset(&p, 0, sizeof(p));
  p.o_ptr = a->out;
  p.lse_ptr = a->lse;
  p.o_batch_stride = packed ? 0 : a->o_stride[0];
  p.o_row_stride = a->o_stride[1];
  p.o_head_stride = a->o_stride[2];
  if (packed) {
    p.lse_head_stride = a->total_q;
    p.lse_batch_stride = 0;
    p.cu_q = a->cu_seqlens_q;
    p.cu_k = a->cu_seqlens_k;
  } else {
    p.lse_head_stride = a->seqlen_q;
    p.lse_batch_stride = static_cast<int64_t>(a->heads) * a->seqlen_q;
  }
  if (a->out == nullptr || a->lse == nullptr) return fail(FA2_E_VALUE, "out and lse must be non-null");

  if (packed && a->zero_tensors && a->seqlen_k != 0 && rows_k != 0) {
    // zero_tensors of the reference: out = 0, LSE = -inf before the kernel (varlen/mod.rs:419-444).
    const int64_t n = rows_q * a->heads;
    if (a->o_stride[2] == d && a->o_stride[1] == static_cast<int64_t>(a->heads) * d) {
      cudaMemsetAsync(a->out, 0, static_cast<size_t>(n) * d * 2, stream);
      fill_f32_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(a->lse, n, -INFINITY);
    } else {  // a strided output view: clear only the elements that belong to it
      fill_empty_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(
          static_cast<uint16_t*>(a->out), a->lse, rows_q, a->heads, d, a->o_stride[1], a->o_stride[2], 0, rows_q,
          a->total_q, 0, -INFINITY);
    }
  }
  if (rows_k == 0 || a->seqlen_k == 0) {
    // No keys at all: O = 0, LSE = +inf (forward/mod.rs:548-582).
    const int64_t n = rows_q * nbatch * a->heads;
    fill_empty_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(
        static_cast<uint16_t*>(a->out), a->lse, rows_q * nbatch, a->heads, d, p.o_row_stride, p.o_head_stride,
        p.o_batch_stride, rows_q, p.lse_head_stride, p.lse_batch_stride, INFINITY);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(FA2_E_RUNTIME, "launch failed: %s", cudaGetErrorString(e));
    return FA2_OK;
  }

  const int ns = packed ? 2 : 3;
  const int64_t* qs = a->q_stride + (packed ? 1 : 0);
  const int64_t* ks = a->k_stride + (packed ? 1 : 0);
  const int64_t* vs = a->v_stride + (packed ? 1 : 0);
  const int64_t* os = a->o_stride + (packed ? 1 : 0);
  if ((rc = check_layout(a->q, qs, ns, "q")) != FA2_OK) return rc;
  if ((rc = check_layout(a->k, ks, ns, "k")) != FA2_OK) return rc;
  if ((rc = check_layout(a->v, vs, ns, "v")) != FA2_OK) return rc;
  if ((rc = check_layout(a->out, os, ns, "out")) != FA2_OK) return rc;

  if ((rc = make_map(&p.tm_q, a->q, a->dtype, 2, d, a->heads, rows_q, nbatch, a->q_stride[2], a->q_stride[1],
                     a->q_stride[0], 64, 128, "q")) != FA2_OK)
    return rc;
  // Head dims above 128 run on the kernel with 64-key tiles (fwd_wide_sm100.cu); the others take 128 keys a tile.
  const int kv_box_rows = d > 128 ? 64 : 128;
  if ((rc = make_map(&p.tm_k, a->k, a->dtype, 2, d, a->heads_k, rows_k, nbatch, a->k_stride[2], a->k_stride[1],
                     a->k_stride[0], 64, kv_box_rows, "k")) != FA2_OK)
    return rc;
  if ((rc = make_map(&p.tm_v, a->v, a->dtype, 2, d, a->heads_k, rows_k, nbatch, a->v_stride[2], a->v_stride[1],
                     a->v_stride[0], 64, kv_box_rows, "v")) != FA2_OK)
    return rc;
  if ((rc = make_map(&p.tm_o, a->out, a->dtype, 2, d, a->heads, rows_q, nbatch, a->o_stride[2], a->o_stride[1],
                     a->o_stride[0], 64, 128, "out")) != FA2_OK)
    return rc;

  p.alibi = a->alibi_slopes;
  p.alibi_batch_stride = a->alibi_batch_stride;
  p.batch = a->batch;
  p.heads = a->heads;
  p.heads_k = a->heads_k;
  p.group = a->heads / a->heads_k;
  p.seqlen_q = a->seqlen_q;
  p.seqlen_k = a->seqlen_k;
  p.num_mblk = (a->seqlen_q + 255) / 256;
  p.num_tiles = p.num_mblk * a->batch * a->heads;
  // Packed mode applies `causal` before clamping against max_seqlen_k (varlen/mod.rs:253-268).
  const Windows w = normalise_windows(a->window_left, a->window_right, a->causal != 0, a->seqlen_k, packed);
  p.window_left = w.left;
  p.window_right = w.right;
  p.causal_alibi = w.causal_alibi;
  p.scale = a->softmax_scale;
  p.scale_log2 = a->softmax_scale * 1.4426950408889634f;
  p.softcap = a->softcap > 0.f ? a->softcap : 0.f;
  p.status = rt->status;

  p.head_dim = d;
  cudaError_t e = d > 128 ? fa2::launch_fwd_wide(p, d, a->dtype == FA2_BF16, stream)
                          : fa2::launch_fwd(p, d, a->dtype == FA2_BF16, rt->sm_count, stream);
  if (e != cudaSuccess) return fail(FA2_E_RUNTIME, "forward launch failed: %s", cudaGetErrorString(e));
  return FA2_OK;
}

int bwd_preprocess_impl(const fa2_bwd_preprocess_args* a, void* stream_v) {
  if (a == nullptr) return fail(FA2_E_VALUE, "args is null");
  if (a->dtype != FA2_F16 && a->dtype != FA2_BF16) return fail(FA2_E_TYPE, "dout and out must be float16 or bfloat16");
  const int d = a->head_dim;
  const bool packed = a->cu_seqlens_q != nullptr;
  if (a->batch <= 0 || a->heads <= 0 || a->batch > 65535 || a->heads > 65535 || a->seqlen_q < 0 || d < 8 || d > 256 ||
      d % 8 != 0)
    return fail(FA2_E_VALUE, "unsupported backward tensor dimensions");
  if (a->seqlen_q == 0 || (packed && a->total_q == 0)) return FA2_OK;
  if (a->dout == nullptr || a->out == nullptr || a->delta == nullptr)
    return fail(FA2_E_VALUE, "dout, out and delta must be non-null");
  const int ns = packed ? 2 : 3;
  int rc;
  const DeviceScope scope(a->dout);
  if ((rc = check_layout(a->dout, a->do_stride + (packed ? 1 : 0), ns, "dout")) != FA2_OK) return rc;
  if ((rc = check_layout(a->out, a->o_stride + (packed ? 1 : 0), ns, "out")) != FA2_OK) return rc;
  fa2::PreprocessParams p;
  memset(&p, 0, sizeof(p));
  p.dout = a->dout;
  p.out = a->out;
  p.delta = a->delta;
  p.cu_q = a->cu_seqlens_q;
  p.do_batch_stride = packed ? 0 : a->do_stride[0];
  p.do_row_stride = a->do_stride[1];
  p.do_head_stride = a->do_stride[2];
  p.o_batch_stride = packed ? 0 : a->o_stride[0];
  p.o_row_stride = a->o_stride[1];
  p.o_head_stride = a->o_stride[2];
  p.batch = a->batch;
  p.heads = a->heads;
  p.seqlen_q = a->seqlen_q;
  p.seqlen_pad = (a->seqlen_q + 127) / 128 * 128;
  p.head_dim = d;
  p.bf16 = a->dtype == FA2_BF16;
  if (packed) {
    p.delta_head_stride = static_cast<int64_t>(a->total_q) + 128LL * a->batch;
    p.delta_batch_stride = 0;
  } else {
    p.delta_head_stride = p.seqlen_pad;
    p.delta_batch_stride = static_cast<int64_t>(a->heads) * p.seqlen_pad;
  }
  if (packed)  // the 128-row gaps between packed sequences read as zero
    cudaMemsetAsync(a->delta, 0, static_cast<size_t>(p.delta_head_stride) * a->heads * 4, static_cast<cudaStream_t>(stream_v));
  cudaError_t e = fa2::launch_bwd_preprocess(p, static_cast<cudaStream_t>(stream_v));
  if (e != cudaSuccess) return fail(FA2_E_RUNTIME, "preprocess launch failed: %s", cudaGetErrorString(e));
  return FA2_OK;
}

int64_t bwd_rows(const fa2_bwd_args* a) {
  return a->cu_seqlens_q != nullptr ? static_cast<int64_t>(a->total_q)
                                    : static_cast<int64_t>(a->batch) * a->seqlen_q;
}

// Bytes of the fp32 dQ accumulator, rounded so that what follows it is 256-byte aligned.
int64_t bwd_accum_bytes(const fa2_bwd_args* a) {
  return (bwd_rows(a) * a->heads * a->head_dim * 4 + 255) / 256 * 256;
}

// One counter per (batch, head, 128-row query block, 32-row slab of a drain warp).
int64_t bwd_turn_counters(const fa2_bwd_args* a) {
  return static_cast<int64_t>(a->batch) * a->heads * ((a->seqlen_q + 127) / 128) * 4;
}

int bwd_impl(const fa2_bwd_args* a, void* stream_v) {
  if (a == nullptr) return fail(FA2_E_VALUE, "args is null");
  if (a->dtype != FA2_F16 && a->dtype != FA2_BF16) return fail(FA2_E_TYPE, "q, k, v must be float16 or bfloat16");
  const bool packed = a->cu_seqlens_q != nullptr;
  const int d = a->head_dim;
  if (d > 256 || d < 8 || d % 8 != 0) return fail(FA2_E_VALUE, "unsupported backward tensor dimensions");
  if (a->heads_k <= 0 || a->heads % a->heads_k != 0)
    return fail(FA2_E_VALUE, "num_heads (%d) must be a multiple of num_heads_k (%d)", a->heads, a->heads_k);
  if (a->batch <= 0 || a->heads <= 0 || a->batch > 65535 || a->heads > 65535 || a->seqlen_q < 0 || a->seqlen_k < 0)
    return fail(FA2_E_VALUE, "unsupported backward tensor dimensions");
  if ((a->which & 3) == 0) return fail(FA2_E_VALUE, "`which` selects no output");
  if (packed && a->cu_seqlens_k == nullptr) return fail(FA2_E_VALUE, "packed backward needs cu_seqlens_k");
  const DeviceScope scope(a->q);
  Runtime* rt = nullptr;
  int rc = get_runtime(scope.device(), &rt);
  if (rc != FA2_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const int64_t rows_q = packed ? a->total_q : a->seqlen_q;
  const int64_t rows_k = packed ? a->total_k : a->seqlen_k;
  const int64_t nbatch = packed ? 1 : a->batch;
  const bool want_dq = (a->which & 1) != 0, want_dkv = (a->which & 2) != 0;
  const int64_t n_dq = bwd_rows(a) * a->heads * d;
  const int64_t n_dkv = (packed ? rows_k : static_cast<int64_t>(a->batch) * a->seqlen_k) * a->heads_k * d;
  cudaError_t e;
  if (rows_q == 0 || a->seqlen_q == 0 || rows_k == 0 || a->seqlen_k == 0) {
    // Nothing attends: every gradient that exists is zero.
    if (want_dq && n_dq > 0 && (e = cudaMemsetAsync(a->dq, 0, n_dq * 2, stream)) != cudaSuccess)
      return fail(FA2_E_RUNTIME, "memset failed: %s", cudaGetErrorString(e));
    if (want_dkv && n_dkv > 0) {
      cudaMemsetAsync(a->dk, 0, n_dkv * 2, stream);
      cudaMemsetAsync(a->dv, 0, n_dkv * 2, stream);
    }
    return FA2_OK;
  }
  if (want_dq) {
    if (a->dq == nullptr || a->dq_accum == nullptr) return fail(FA2_E_VALUE, "dq and dq_accum must be non-null");
    if (a->dq_accum_bytes < n_dq * 4) return fail(FA2_E_VALUE, "dq_accum is smaller than fa2_bwd_workspace_bytes()");
    if (reinterpret_cast<uintptr_t>(a->dq_accum) % 16 || reinterpret_cast<uintptr_t>(a->dq) % 16)
      return fail(FA2_E_VALUE, "dq and dq_accum must be 16-byte aligned");
  }
  if (want_dkv && (a->dk == nullptr || a->dv == nullptr)) return fail(FA2_E_VALUE, "dk and dv must be non-null");
  if (a->lse == nullptr || a->delta == nullptr) return fail(FA2_E_VALUE, "lse and delta must be non-null");
  const int ns = packed ? 2 : 3;
  const int so = packed ? 1 : 0;
  if ((rc = check_layout(a->q, a->q_stride + so, ns, "q")) != FA2_OK) return rc;
  if ((rc = check_layout(a->k, a->k_stride + so, ns, "k")) != FA2_OK) return rc;
  if ((rc = check_layout(a->v, a->v_stride + so, ns, "v")) != FA2_OK) return rc;
  if ((rc = check_layout(a->dout, a->do_stride + so, ns, "dout")) != FA2_OK) return rc;
  if (want_dkv && (reinterpret_cast<uintptr_t>(a->dk) % 16 || reinterpret_cast<uintptr_t>(a->dv) % 16))
    return fail(FA2_E_VALUE, "dk and dv must be 16-byte aligned");

  fa2::BwdParams p;
  memset(&p, 0, sizeof(p));
  const int64_t hd = static_cast<int64_t>(a->heads) * d, hkd = static_cast<int64_t>(a->heads_k) * d;
  // Head dims above 128 run on the kernel that takes query rows 64 at a time (bwd_wide_sm100.cu).
  const bool wide = d > 128;
  const int q_box_rows = wide ? 64 : 128;
  if ((rc = make_map(&p.tm_q, a->q, a->dtype, 2, d, a->heads, rows_q, nbatch, a->q_stride[2], a->q_stride[1],
                     a->q_stride[0], 64, q_box_rows, "q")) != FA2_OK) return rc;
  if ((rc = make_map(&p.tm_do, a->dout, a->dtype, 2, d, a->heads, rows_q, nbatch, a->do_stride[2], a->do_stride[1],
                     a->do_stride[0], 64, q_box_rows, "dout")) != FA2_OK) return rc;
  if ((rc = make_map(&p.tm_k, a->k, a->dtype, 2, d, a->heads_k, rows_k, nbatch, a->k_stride[2], a->k_stride[1],
                     a->k_stride[0], 64, 128, "k")) != FA2_OK) return rc;
  if ((rc = make_map(&p.tm_v, a->v, a->dtype, 2, d, a->heads_k, rows_k, nbatch, a->v_stride[2], a->v_stride[1],
                     a->v_stride[0], 64, 128, "v")) != FA2_OK) return rc;
  if (want_dkv) {
    if ((rc = make_map(&p.tm_dk, a->dk, a->dtype, 2, d, a->heads_k, rows_k, nbatch, d, hkd, rows_k * hkd, 64, 128,
                       "dk")) != FA2_OK) return rc;
    if ((rc = make_map(&p.tm_dv, a->dv, a->dtype, 2, d, a->heads_k, rows_k, nbatch, d, hkd, rows_k * hkd, 64, 128,
                       "dv")) != FA2_OK) return rc;
  } else {  // a dQ-only call writes neither: the kernels never touch these maps
    p.tm_dk = p.tm_k;
    p.tm_dv = p.tm_v;
  }
  if (want_dq) {
    // one reduce-add box: 32 columns of 32 query rows (64 on the kernel for head dims above 128)
    if ((rc = make_map(&p.tm_dqa, a->dq_accum, 2, 4, d, a->heads, rows_q, nbatch, d, hd, rows_q * hd, 32, wide ? 64 : 32,
                       "dq_accum")) != FA2_OK) return rc;
  } else {
    p.tm_dqa = p.tm_q;
  }
  p.lse = a->lse;
  p.delta = a->delta;
  p.dk_ptr = a->dk;
  p.dv_ptr = a->dv;
  p.cu_q = a->cu_seqlens_q;
  p.cu_k = a->cu_seqlens_k;
  const int64_t sq_pad = (a->seqlen_q + 127) / 128 * 128;
  if (packed) {
    p.lse_head_stride = a->total_q;
    p.lse_batch_stride = 0;
    p.delta_head_stride = static_cast<int64_t>(a->total_q) + 128LL * a->batch;
    p.delta_batch_stride = 0;
    p.delta_seq_pad = 128;
  } else {
    p.lse_head_stride = a->seqlen_q;
    p.lse_batch_stride = static_cast<int64_t>(a->heads) * a->seqlen_q;
    p.delta_head_stride = sq_pad;
    p.delta_batch_stride = static_cast<int64_t>(a->heads) * sq_pad;
    p.delta_seq_pad = 0;
  }
  p.dkv_row_stride = hkd;
  p.dkv_head_stride = d;
  p.dkv_batch_stride = rows_k * hkd;
  p.batch = a->batch;
  p.heads = a->heads;
  p.heads_k = a->heads_k;
  p.group = a->heads / a->heads_k;
  p.seqlen_q = a->seqlen_q;
  p.seqlen_k = a->seqlen_k;
  p.num_nblk = (a->seqlen_k + 127) / 128;
  const Windows w = normalise_windows(a->window_left, a->window_right, a->causal != 0, a->seqlen_k, packed);
  p.window_left = w.left;
  p.window_right = w.right;
  p.which = a->which;
  p.alibi = a->alibi_slopes;
  p.alibi_batch_stride = a->alibi_batch_stride;
  p.causal_alibi = w.causal_alibi;
  p.softcap = a->softcap > 0.f ? a->softcap : 0.f;
  p.scale = a->softmax_scale;
  p.scale_log2 = a->softmax_scale * 1.4426950408889634f;
  p.status = rt->status;

  // A dQ-only call (the deterministic pair bwd_dq + bwd_dkv of the reference, whose dQ kernel sums in
  // registers in key order) accumulates in a fixed key-block order when the workspace holds the
  // turn counters; otherwise, and in the combined call, the adds land in arrival order.
  const int64_t acc_bytes = bwd_accum_bytes(a), n_turn = bwd_turn_counters(a);
  const bool ordered = !wide && a->which == 1 && a->dq_accum_bytes >= acc_bytes + n_turn * 4;
  p.dq_turn = ordered ? reinterpret_cast<int*>(static_cast<char*>(a->dq_accum) + acc_bytes) : nullptr;
  p.num_mblk_q = (a->seqlen_q + 127) / 128;
  if (want_dq && (e = cudaMemsetAsync(a->dq_accum, 0, ordered ? acc_bytes + n_turn * 4 : n_dq * 4, stream)) != cudaSuccess)
    return fail(FA2_E_RUNTIME, "memset failed: %s", cudaGetErrorString(e));
  if (a->ev_kernel_start != nullptr) cudaEventRecord(static_cast<cudaEvent_t>(a->ev_kernel_start), stream);
  p.head_dim = d;
  p.dq_acc = static_cast<float*>(a->dq_accum);
  p.dq_rows = rows_q;
  p.v_ptr = a->v;
  p.v_batch_stride = packed ? 0 : a->v_stride[0];
  p.v_row_stride = a->v_stride[1];
  p.v_head_stride = a->v_stride[2];
  e = wide ? fa2::launch_bwd_wide(p, d, a->dtype == FA2_BF16, stream)
           : fa2::launch_bwd(p, d, a->dtype == FA2_BF16, rt->sm_count, stream);
  if (a->ev_kernel_stop != nullptr) cudaEventRecord(static_cast<cudaEvent_t>(a->ev_kernel_stop), stream);
  if (e != cudaSuccess) return fail(FA2_E_RUNTIME, "backward launch failed: %s", cudaGetErrorString(e));
  if (want_dq && (e = fa2::launch_dq_convert(static_cast<const float*>(a->dq_accum), a->dq, n_dq, a->softmax_scale,
                                             a->dtype == FA2_BF16, stream)) != cudaSuccess)
    return fail(FA2_E_RUNTIME, "dq convert launch failed: %s", cudaGetErrorString(e));
  return FA2_OK;
}

// ------------------------------------------------------------------------------------------------
// Backward for callers that cannot allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off limits: inside a real-time or
// latency-critical serving loop whose memory was carved up front, under a framework that owns
// every byte of the device heap, or in a sandbox where the allocation calls are simply not
// permitted. fa2_bwd needs a caller-provided fp32 dQ accumulator, and this library's own set-up
// allocates a status word; fa2_bwd_static needs neither. Its accumulator and its status word are
// file-scope device arrays that live in the module image: every GPU that loads the library holds
// them (16 MiB + 4 bytes) until the process exits.
//
// The array name below is only a host-side handle: passing it to a kernel from host code would
// hand the kernel a host address. The device address is fetched with cudaGetSymbolAddress, once per
// device, with that device current.
constexpr int64_t kStaticDqFloats = FA2_BWD_STATIC_MAX_ELEMENTS;  // 16 MiB of fp32
static __device__ __align__(256) float g_static_dq_accum[kStaticDqFloats];
static __device__ __align__(256) int g_static_status[64];

struct StaticRuntime {
  bool ready = false;
  float* accum = nullptr;
  int* status = nullptr;
  int sm_count = 0;
};
StaticRuntime g_static_rt[kMaxDevices];

int get_static_runtime(int device, StaticRuntime** out) {
  if (device < 0 || device >= kMaxDevices) return fail(FA2_E_VALUE, "device index %d out of range", device);
  std::lock_guard<std::mutex> lock(g_mu);
  StaticRuntime& rt = g_static_rt[device];
  if (!rt.ready) {
    int cc_major = 0;
    cudaError_t e = cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, device);
    if (e != cudaSuccess) return fail(FA2_E_RUNTIME, "cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
    if (cc_major != 10) return fail(FA2_E_RUNTIME, "this library is built for sm_100a only");
    if (g_encode == nullptr) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult q;
      e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
      if (e != cudaSuccess || fn == nullptr)
        return fail(FA2_E_RUNTIME, "cuTensorMapEncodeTiled is not available from the driver");
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    void* accum = nullptr;
    void* status = nullptr;
    e = cudaGetSymbolAddress(&accum, g_static_dq_accum);
    if (e != cudaSuccess) return fail(FA2_E_RUNTIME, "cudaGetSymbolAddress(accumulator): %s", cudaGetErrorString(e));
    e = cudaGetSymbolAddress(&status, g_static_status);
    if (e != cudaSuccess) return fail(FA2_E_RUNTIME, "cudaGetSymbolAddress(status): %s", cudaGetErrorString(e));
    e = cudaDeviceGetAttribute(&rt.sm_count, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess) return fail(FA2_E_RUNTIME, "cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
    rt.accum = static_cast<float*>(accum);
    rt.status = static_cast<int*>(status);
    rt.ready = true;
  }
  *out = &rt;
  return FA2_OK;
}

int bwd_static_impl(const fa2_bwd_args* a, void* stream_v) {
  if (a == nullptr) return fail(FA2_E_VALUE, "args is null");
  if (a->dtype != FA2_F16 && a->dtype != FA2_BF16) return fail(FA2_E_TYPE, "q, k, v must be float16 or bfloat16");
  if (a->cu_seqlens_q != nullptr || a->cu_seqlens_k != nullptr)
    return fail(FA2_E_VALUE, "fa2_bwd_static takes dense [B, S, H, D] tensors only");
  const int d = a->head_dim;
  if (d < 8 || d % 8 != 0 || d > 128)
    return fail(FA2_E_VALUE, "head dim %d is not built for sm_100a (multiples of 8 up to 128 are)", d);
  if (a->heads_k <= 0 || a->heads % a->heads_k != 0)
    return fail(FA2_E_VALUE, "num_heads (%d) must be a multiple of num_heads_k (%d)", a->heads, a->heads_k);
  if (a->batch <= 0 || a->heads <= 0 || a->batch > 65535 || a->heads > 65535 || a->seqlen_q <= 0 || a->seqlen_k <= 0)
    return fail(FA2_E_VALUE, "fa2_bwd_static needs positive batch, heads and sequence lengths");
  if ((a->which & 3) != 3) return fail(FA2_E_VALUE, "fa2_bwd_static always produces dQ, dK and dV (which = 3)");
  const int64_t n_dq = static_cast<int64_t>(a->batch) * a->seqlen_q * a->heads * d;
  if (n_dq > kStaticDqFloats)
    return fail(FA2_E_VALUE,
                "fa2_bwd_static: B*Sq*H*D = %lld exceeds the built-in accumulator of %lld elements; use fa2_bwd with "
                "a caller-provided dq_accum",
                static_cast<long long>(n_dq), static_cast<long long>(kStaticDqFloats));
  if (a->q == nullptr || a->k == nullptr || a->v == nullptr || a->dout == nullptr || a->lse == nullptr ||
      a->delta == nullptr || a->dq == nullptr || a->dk == nullptr || a->dv == nullptr)
    return fail(FA2_E_VALUE, "q, k, v, dout, lse, delta, dq, dk and dv must be non-null");
  int rc;
  if ((rc = check_layout(a->q, a->q_stride, 3, "q")) != FA2_OK) return rc;
  if ((rc = check_layout(a->k, a->k_stride, 3, "k")) != FA2_OK) return rc;
  if ((rc = check_layout(a->v, a->v_stride, 3, "v")) != FA2_OK) return rc;
  if ((rc = check_layout(a->dout, a->do_stride, 3, "dout")) != FA2_OK) return rc;
  if (reinterpret_cast<uintptr_t>(a->dq) % 16 || reinterpret_cast<uintptr_t>(a->dk) % 16 ||
      reinterpret_cast<uintptr_t>(a->dv) % 16)
    return fail(FA2_E_VALUE, "dq, dk and dv must be 16-byte aligned");
  const DeviceScope scope(a->q);
  StaticRuntime* rt = nullptr;
  if ((rc = get_static_runtime(scope.device(), &rt)) != FA2_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

  fa2::BwdParams p;
  memset(&p, 0, sizeof(p));
  const int64_t rows_q = a->seqlen_q, rows_k = a->seqlen_k, nbatch = a->batch;
  const int64_t hd = static_cast<int64_t>(a->heads) * d, hkd = static_cast<int64_t>(a->heads_k) * d;
  if ((rc = make_map(&p.tm_q, a->q, a->dtype, 2, d, a->heads, rows_q, nbatch, a->q_stride[2], a->q_stride[1],
                     a->q_stride[0], 64, 128, "q")) != FA2_OK) return rc;
  if ((rc = make_map(&p.tm_do, a->dout, a->dtype, 2, d, a->heads, rows_q, nbatch, a->do_stride[2], a->do_stride[1],
                     a->do_stride[0], 64, 128, "dout")) != FA2_OK) return rc;
  if ((rc = make_map(&p.tm_k, a->k, a->dtype, 2, d, a->heads_k, rows_k, nbatch, a->k_stride[2], a->k_stride[1],
                     a->k_stride[0], 64, 128, "k")) != FA2_OK) return rc;
  if ((rc = make_map(&p.tm_v, a->v, a->dtype, 2, d, a->heads_k, rows_k, nbatch, a->v_stride[2], a->v_stride[1],
                     a->v_stride[0], 64, 128, "v")) != FA2_OK) return rc;
  if ((rc = make_map(&p.tm_dk, a->dk, a->dtype, 2, d, a->heads_k, rows_k, nbatch, d, hkd, rows_k * hkd, 64, 128,
                     "dk")) != FA2_OK) return rc;
  if ((rc = make_map(&p.tm_dv, a->dv, a->dtype, 2, d, a->heads_k, rows_k, nbatch, d, hkd, rows_k * hkd, 64, 128,
                     "dv")) != FA2_OK) return rc;
  if ((rc = make_map(&p.tm_dqa, rt->accum, 2, 4, d, a->heads, rows_q, nbatch, d, hd, rows_q * hd, 32, 32,
                     "static dq accumulator")) != FA2_OK) return rc;
  p.lse = a->lse;
  p.delta = a->delta;
  p.dk_ptr = a->dk;
  p.dv_ptr = a->dv;
  const int64_t sq_pad = (a->seqlen_q + 127) / 128 * 128;
  p.lse_head_stride = a->seqlen_q;
  p.lse_batch_stride = static_cast<int64_t>(a->heads) * a->seqlen_q;
  p.delta_head_stride = sq_pad;
  p.delta_batch_stride = static_cast<int64_t>(a->heads) * sq_pad;
  p.dkv_row_stride = hkd;
  p.dkv_head_stride = d;
  p.dkv_batch_stride = rows_k * hkd;
  p.batch = a->batch;
  p.heads = a->heads;
  p.heads_k = a->heads_k;
  p.group = a->heads / a->heads_k;
  p.seqlen_q = a->seqlen_q;
  p.seqlen_k = a->seqlen_k;
  p.num_nblk = (a->seqlen_k + 127) / 128;
  const Windows w = normalise_windows(a->window_left, a->window_right, a->causal != 0, a->seqlen_k, false);
  p.window_left = w.left;
  p.window_right = w.right;
  p.which = 3;
  p.dq_turn = nullptr;
  p.num_mblk_q = (a->seqlen_q + 127) / 128;
  p.alibi = a->alibi_slopes;
  p.alibi_batch_stride = a->alibi_batch_stride;
  p.causal_alibi = w.causal_alibi;
  p.softcap = a->softcap > 0.f ? a->softcap : 0.f;
  p.scale = a->softmax_scale;
  p.scale_log2 = a->softmax_scale * 1.4426950408889634f;
  p.status = rt->status;

  // The array keeps whatever the previous call left: the part this call adds into starts at zero.
  cudaError_t e = cudaMemsetAsync(rt->accum, 0, static_cast<size_t>(n_dq) * 4, stream);
  if (e != cudaSuccess) return fail(FA2_E_RUNTIME, "memset failed: %s", cudaGetErrorString(e));
  p.head_dim = d;
  if ((e = fa2::launch_bwd(p, d, a->dtype == FA2_BF16, rt->sm_count, stream)) != cudaSuccess)
    return fail(FA2_E_RUNTIME, "backward launch failed: %s", cudaGetErrorString(e));
  if ((e = fa2::launch_dq_convert(rt->accum, a->dq, n_dq, a->softmax_scale, a->dtype == FA2_BF16, stream)) != cudaSuccess)
    return fail(FA2_E_RUNTIME, "dq convert launch failed: %s", cudaGetErrorString(e));
  return FA2_OK;
}

}  // namespace

extern "C" {

int fa2_bwd_preprocess(const fa2_bwd_preprocess_args* args, void* stream) { return bwd_preprocess_impl(args, stream); }

int64_t fa2_bwd_workspace_bytes(const fa2_bwd_args* args) {
  if (args == nullptr || (args->which & 1) == 0) return 0;
  // The fp32 accumulator, then (used by dQ-only calls) one turn counter per 32 query rows of every
  // (batch, head) for the ordered accumulation.
  return bwd_accum_bytes(args) + bwd_turn_counters(args) * 4;
}

int fa2_bwd(const fa2_bwd_args* args, void* stream) { return bwd_impl(args, stream); }

int fa2_layout_is_addressable(const void* ptr, const int64_t* outer_strides, int32_t n_outer) {
  if (ptr == nullptr || reinterpret_cast<uintptr_t>(ptr) % 16 != 0) return 0;
  for (int i = 0; i < n_outer; ++i)
    if (outer_strides[i] % 8 != 0 || outer_strides[i] < 0) return 0;
  return 1;
}

int fa2_copy_16bit(const void* src, const int64_t src_strides[3], void* dst, const int64_t dst_strides[3],
                   const int64_t shape[4], void* stream) {
  if (shape == nullptr || src_strides == nullptr || dst_strides == nullptr)
    return fail(FA2_E_VALUE, "fa2_copy_16bit: null argument");
  for (int i = 0; i < 4; ++i)
    if (shape[i] < 0 || shape[i] > INT32_MAX) return fail(FA2_E_VALUE, "fa2_copy_16bit: unsupported shape");
  // An empty tensor has nothing to copy and may come without storage.
  if (shape[0] == 0 || shape[1] == 0 || shape[2] == 0 || shape[3] == 0) return FA2_OK;
  if (src == nullptr || dst == nullptr) return fail(FA2_E_VALUE, "fa2_copy_16bit: null tensor");
  const DeviceScope scope(src);
  cudaError_t e = fa2::launch_copy_rows(src, dst, shape[0], shape[1], shape[2], shape[3], src_strides, dst_strides,
                                        static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(FA2_E_RUNTIME, "copy launch failed: %s", cudaGetErrorString(e));
  return FA2_OK;
}

int fa2_pack_16bit(const void* src, void* dst, const int64_t shape[4], const int64_t outer_strides[3], void* stream) {
  if (shape == nullptr || outer_strides == nullptr) return fail(FA2_E_VALUE, "fa2_pack_16bit: null argument");
  const int64_t packed[3] = {shape[1] * shape[2] * shape[3], shape[2] * shape[3], shape[3]};
  return fa2_copy_16bit(src, outer_strides, dst, packed, shape, stream);
}

int fa2_bwd_static(const fa2_bwd_args* args, void* stream) { return bwd_static_impl(args, stream); }

int fa2_bwd_static_status(int device) {
  int prev = 0;
  cudaGetDevice(&prev);
  if (device != prev && cudaSetDevice(device) != cudaSuccess) {
    cudaGetLastError();
    return fail(FA2_E_VALUE, "device index %d cannot be selected", device);
  }
  StaticRuntime* rt = nullptr;
  int rc = get_static_runtime(device, &rt);
  int word = 0;
  if (rc == FA2_OK) {
    // Plain copies from and to the array inside the library image: nothing is allocated.
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpy(&word, rt->status, sizeof(int), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && word != 0) {
      const int zero = 0;
      e = cudaMemcpy(rt->status, &zero, sizeof(int), cudaMemcpyHostToDevice);
    }
    if (e != cudaSuccess) rc = fail(FA2_E_RUNTIME, "static status: %s", cudaGetErrorString(e));
  }
  if (device != prev) cudaSetDevice(prev);
  return rc != FA2_OK ? rc : word;
}


int fa2_fwd(const fa2_fwd_args* args, void* stream) { return fwd_common(args, stream, false); }

int fa2_varlen_fwd(const fa2_fwd_args* args, void* stream) { return fwd_common(args, stream, true); }

const char* fa2_last_error(void) { return g_error; }

int fa2_device_status(int device) {
  Runtime* rt = nullptr;
  int rc = get_runtime(device, &rt);
  if (rc != FA2_OK) return rc;
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(device);
  int word = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(&word, rt->status, sizeof(int), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess && word != 0) e = cudaMemset(rt->status, 0, sizeof(int));
  cudaSetDevice(prev);
  if (e != cudaSuccess) return fail(FA2_E_RUNTIME, "device status: %s", cudaGetErrorString(e));
  return word;
}

int fa2_sm_count(int device) {
  Runtime* rt = nullptr;
  int rc = get_runtime(device, &rt);
  if (rc != FA2_OK) return rc;
  return rt->sm_count;
}

}  // extern "C"
