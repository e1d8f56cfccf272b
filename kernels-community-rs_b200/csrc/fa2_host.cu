// Host side of the C ABI: argument validation, TMA descriptor construction, launches.
// Mirrors the checks of the reference host layer (flash-attn2-rs/src/host/forward/mod.rs:52-447,
// src/host/layout.rs:46-125, src/host/backward.rs:14-99, src/host/varlen/mod.rs:21-630) for
// the paths this library implements.
#include "../../include/fa2_b200.h"
#include "fa2_launch.h"

#include <cuda.h>
#include <cuda_runtime.h>
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
    e = cudaMalloc(&rt.status, sizeof(int));
    if (e != cudaSuccess) return fail(FA2_E_RUNTIME, "cudaMalloc(status): %s", cudaGetErrorString(e));
    cudaMemset(rt.status, 0, sizeof(int));
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

int fwd_common(const fa2_fwd_args* a, void* stream_v, bool packed) {
  if (a == nullptr) return fail(FA2_E_VALUE, "args is null");
  if (a->dtype != FA2_F16 && a->dtype != FA2_BF16) return fail(FA2_E_TYPE, "q, k, v must be float16 or bfloat16");
  const int d = a->head_dim;
  if (d > 256) return fail(FA2_E_VALUE, "head dim must be <= 256, got %d", d);
  if (d < 8 || d % 8 != 0) return fail(FA2_E_VALUE, "head_size must be a positive multiple of 8, got %d", d);
  if (d != 64 && d != 128)
    return fail(FA2_E_VALUE, "head dim %d is not built for sm_100a yet (64 and 128 are)", d);
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
  int device = 0;
  cudaGetDevice(&device);
  Runtime* rt = nullptr;
  int rc = get_runtime(device, &rt);
  if (rc != FA2_OK) return rc;
  cudaSetDevice(device);
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
  if ((rc = make_map(&p.tm_k, a->k, a->dtype, 2, d, a->heads_k, rows_k, nbatch, a->k_stride[2], a->k_stride[1],
                     a->k_stride[0], 64, 128, "k")) != FA2_OK)
    return rc;
  if ((rc = make_map(&p.tm_v, a->v, a->dtype, 2, d, a->heads_k, rows_k, nbatch, a->v_stride[2], a->v_stride[1],
                     a->v_stride[0], 64, 128, "v")) != FA2_OK)
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

  cudaError_t e = fa2::launch_fwd(p, d, a->dtype == FA2_BF16, rt->sm_count, stream);
  if (e != cudaSuccess) return fail(FA2_E_RUNTIME, "forward launch failed: %s", cudaGetErrorString(e));
  return FA2_OK;
}

}  // namespace

extern "C" {

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
