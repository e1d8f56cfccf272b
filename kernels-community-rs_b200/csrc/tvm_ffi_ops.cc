// tvm-ffi operator boundary: the packed-call symbols the reference crate exports
// (`#[no_mangle] extern "C" fn __tvm_ffi_*` in flash-attn2-rs/src/host/**), re-implemented in C++
// on top of the C ABI in include/fa2_b200.h. Argument order, optional arguments, returned
// containers, allocation through TVMFFIEnvTensorAlloc, the caller's stream from
// TVMFFIEnvGetStream and the error kinds follow the reference:
//   fwd / fwd_lse            host/forward/mod.rs:52-447,815-853
//   bwd_preprocess           host/backward.rs:628-757
//   bwd_dq / bwd_dkv / bwd_all   host/backward.rs:14-626
//   varlen_fwd_explicit      host/varlen/mod.rs:21-650
//   varlen_bwd_explicit      host/varlen/backward.rs:15-546
// The remaining exports of the reference (dropout RNG state, KV-cache, paged decode) are present
// as symbols that raise RuntimeError, so the Python package imports and fails loudly.
#include <tvm/ffi/any.h>
#include <tvm/ffi/container/array.h>
#include <tvm/ffi/container/tensor.h>
#include <tvm/ffi/error.h>
#include <tvm/ffi/extra/c_env_api.h>
#include <tvm/ffi/function.h>
#include <tvm/ffi/optional.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <string>
#include <vector>

#include "fa2_b200.h"

namespace {

using tvm::ffi::Any;
using tvm::ffi::AnyView;
using tvm::ffi::Array;
using tvm::ffi::Optional;
using tvm::ffi::Tensor;

constexpr DLDataType kF32{kDLFloat, 32, 1};

template <typename T>
T arg(const AnyView* args, int i, const char* name) {
  auto v = args[i].try_cast<T>();
  if (!v.has_value()) {
    TVM_FFI_THROW(TypeError) << "argument '" << name << "' (#" << i << ") has the wrong type: got "
                             << args[i].GetTypeKey();
  }
  return *v;
}

[[noreturn]] void raise_from_cabi(int rc) {
  const std::string msg = fa2_last_error();
  if (rc == FA2_E_TYPE) TVM_FFI_THROW(TypeError) << msg;
  if (rc == FA2_E_VALUE) TVM_FFI_THROW(ValueError) << msg;
  TVM_FFI_THROW(RuntimeError) << msg;
}

void check(int rc) {
  if (rc != FA2_OK) raise_from_cabi(rc);
}

int dtype_code(const Tensor& t, const char* name) {
  const DLDataType dt = t.dtype();
  if (dt.lanes == 1 && dt.bits == 16 && dt.code == kDLFloat) return FA2_F16;
  if (dt.lanes == 1 && dt.bits == 16 && dt.code == kDLBfloat) return FA2_BF16;
  TVM_FFI_THROW(TypeError) << name << " must be float16 or bfloat16";
}

// Rank / device / last-stride checks of prepare_qkv (host/layout.rs:51-79).
void check_attention_tensor(const Tensor& t, const char* name, int rank_lo, int rank_hi) {
  if (t.device().device_type != kDLCUDA) TVM_FFI_THROW(ValueError) << name << " must be a CUDA tensor";
  if (t.ndim() < rank_lo || t.ndim() > rank_hi)
    TVM_FFI_THROW(ValueError) << name << " must have rank " << rank_hi << ", got " << t.ndim();
  if (t.strides()[t.ndim() - 1] != 1 && t.shape()[t.ndim() - 1] > 1)
    TVM_FFI_THROW(ValueError) << name << " must have unit last stride";
}

void fill_strides(const Tensor& t, int64_t out[3]) {
  const auto s = t.strides();
  if (t.ndim() == 4) {
    out[0] = s[0];
    out[1] = s[1];
    out[2] = s[2];
  } else {
    out[0] = 0;
    out[1] = s[0];
    out[2] = s[1];
  }
}

Tensor alloc(std::initializer_list<int64_t> shape, DLDataType dtype, DLDevice dev) {
  std::vector<int64_t> s(shape);
  return Tensor::FromEnvAlloc(TVMFFIEnvTensorAlloc, tvm::ffi::ShapeView(s.data(), s.size()), dtype, dev);
}

void* stream_of(DLDevice dev) { return TVMFFIEnvGetStream(dev.device_type, dev.device_id); }

bool is_contiguous(const Tensor& t) {
  int64_t expect = 1;
  const auto sh = t.shape();
  const auto st = t.strides();
  for (int i = t.ndim() - 1; i >= 0; --i) {
    if (sh[i] != 1 && st[i] != expect) return false;
    expect *= sh[i];
  }
  return true;
}

// A view the kernels cannot address (base not 16-byte aligned or an outer stride that is not a
// multiple of 8 elements) is packed into a fresh contiguous tensor from the environment allocator,
// as prepare_attention_tensor does (host/layout.rs:80-100); anything else is returned as it is.
Tensor addressable(const Tensor& t, DLDevice dev) {
  int64_t strides[3];
  const auto st = t.strides();
  const auto sh = t.shape();
  const int nd = t.ndim();
  for (int i = 0; i < nd - 1; ++i) strides[i] = sh[i] > 1 ? st[i] : 0;  // the stride of a size-1 dimension is never used
  if (fa2_layout_is_addressable(t.data_ptr(), strides, nd - 1)) return t;
  int64_t shape4[4] = {1, 1, 1, 1}, outer[3] = {0, 0, 0};
  for (int i = 0; i < nd; ++i) shape4[4 - nd + i] = sh[i];
  for (int i = 0; i < nd - 1; ++i) outer[3 - (nd - 1) + i] = st[i];
  std::vector<int64_t> shp(sh.begin(), sh.end());
  Tensor packed = Tensor::FromEnvAlloc(TVMFFIEnvTensorAlloc, tvm::ffi::ShapeView(shp.data(), shp.size()), t.dtype(), dev);
  check(fa2_pack_16bit(t.data_ptr(), packed.data_ptr(), shape4, outer, stream_of(dev)));
  return packed;
}

// ---- layout predicates of a caller-supplied output (the reference: host/layout.rs:127-172, 145-456)
// Number of elements between the first and one past the last element of the view.
uint64_t element_span(const Tensor& t) {
  uint64_t span = 1;
  for (int i = 0; i < t.ndim(); ++i) {
    if (t.shape()[i] == 0) return 0;
    span += static_cast<uint64_t>(t.shape()[i] - 1) * static_cast<uint64_t>(t.strides()[i]);
  }
  return span;
}

// Do the address ranges of two 16-bit tensors intersect?
bool ranges_overlap(const Tensor& a, const Tensor& b) {
  const uint64_t x = reinterpret_cast<uint64_t>(a.data_ptr()), y = reinterpret_cast<uint64_t>(b.data_ptr());
  return x < y + element_span(b) * 2 && y < x + element_span(a) * 2;
}

// True when no two index tuples of the view name the same element. Strides that nest (every stride at least
// the extent of the faster axes) prove it at once. Otherwise the axes above the contiguous run are
// enumerated, up to a bound, and their offsets must keep at least that run's length apart; a view that is too
// large for the bounded check is refused as "cannot be proved", like the reference refuses what its own
// bounded checks cannot prove.
bool elements_are_disjoint(const Tensor& t) {
  std::vector<std::pair<int64_t, int64_t>> dims;  // (stride, extent) of the axes that matter
  for (int i = 0; i < t.ndim(); ++i) {
    if (t.shape()[i] == 0) return true;
    if (t.strides()[i] < 0) return false;
    if (t.shape()[i] > 1) dims.emplace_back(t.strides()[i], t.shape()[i]);
  }
  std::sort(dims.begin(), dims.end());
  int64_t span = 1;
  bool nested = true;
  for (const auto& [stride, n] : dims) {
    if (stride < span) {
      nested = false;
      break;
    }
    span += (n - 1) * stride;
  }
  if (nested) return true;
  // the contiguous run at the bottom, then every other axis by enumeration
  int64_t run = 1;
  size_t i = 0;
  while (i < dims.size() && dims[i].first == run) run *= dims[i++].second;
  int64_t count = 1;
  for (size_t j = i; j < dims.size(); ++j) {
    if (dims[j].first <= 0) return false;
    count *= dims[j].second;
    if (count > (int64_t{1} << 22)) return false;
  }
  std::vector<int64_t> offsets{0};
  offsets.reserve(static_cast<size_t>(count));
  for (size_t j = i; j < dims.size(); ++j) {
    const size_t before = offsets.size();
    for (int64_t k = 1; k < dims[j].second; ++k)
      for (size_t m = 0; m < before; ++m) offsets.push_back(offsets[m] + k * dims[j].first);
  }
  std::sort(offsets.begin(), offsets.end());
  for (size_t m = 1; m < offsets.size(); ++m)
    if (offsets[m] - offsets[m - 1] < run) return false;
  return true;
}

void unsupported(const char* what) {
  TVM_FFI_THROW(ValueError) << what << " is not built in the sm_100a library";
}

const float* alibi_ptr(const Optional<Tensor>& alibi, int64_t b, int64_t h, DLDevice dev, int32_t* batch_stride) {
  *batch_stride = 0;
  if (!alibi.has_value()) return nullptr;
  const Tensor& t = alibi.value();
  if (t.device().device_type != kDLCUDA || t.device().device_id != dev.device_id)
    TVM_FFI_THROW(TypeError) << "alibi_slopes must be a CUDA tensor on q's device";
  const DLDataType dt = t.dtype();
  if (dt.code != kDLFloat || dt.bits != 32 || dt.lanes != 1) TVM_FFI_THROW(TypeError) << "alibi_slopes must be float32";
  if (!is_contiguous(t)) TVM_FFI_THROW(ValueError) << "alibi_slopes must be contiguous";
  if (t.ndim() == 1 && t.shape()[0] == h) {
    *batch_stride = 0;
  } else if (t.ndim() == 2 && t.shape()[0] == b && t.shape()[1] == h) {
    *batch_stride = static_cast<int32_t>(h);
  } else {
    TVM_FFI_THROW(ValueError) << "alibi_slopes must be [" << h << "] or [" << b << ", " << h << "]";
  }
  return static_cast<const float*>(t.data_ptr());
}

void check_dropout_zero(double p) {
  if (!std::isfinite(p) || p < 0.0 || p >= 1.0 || static_cast<float>(p) >= 1.0f)
    TVM_FFI_THROW(ValueError) << "p_dropout must be finite and in [0, 1) as float32";
  if (static_cast<float>(p) > 0.f) unsupported("dropout (p_dropout > 0)");
}

// ------------------------------------------------------------------------------------ forward
Any fwd_impl(const AnyView* args, int32_t n, bool lse_only) {
  if (!(n == 9 || n == 10 || n == 12 || n == 13 || n == 14 || n == 16 || n == 18))
    TVM_FFI_THROW(ValueError)
        << "fwd expects 9 positional arguments (q, k, v, alibi_slopes, softmax_scale, is_causal, window_size_left, "
           "window_size_right, softcap), optionally followed by p_dropout, seed, offset, and/or an output tensor; got "
        << n;
  Tensor q = arg<Tensor>(args, 0, "q"), k = arg<Tensor>(args, 1, "k"), v = arg<Tensor>(args, 2, "v");
  Optional<Tensor> alibi = arg<Optional<Tensor>>(args, 3, "alibi_slopes");
  Optional<double> scale_opt = arg<Optional<double>>(args, 4, "softmax_scale");
  const bool causal = arg<bool>(args, 5, "is_causal");
  const int64_t wl = arg<int64_t>(args, 6, "window_size_left");
  const int64_t wr = arg<int64_t>(args, 7, "window_size_right");
  const double softcap = arg<double>(args, 8, "softcap");
  if (n >= 12) check_dropout_zero(arg<double>(args, 9, "p_dropout"));
  if (n >= 14 && arg<bool>(args, 13, "return_softmax")) unsupported("return_softmax");

  check_attention_tensor(q, "q", 4, 4);
  check_attention_tensor(k, "k", 4, 4);
  check_attention_tensor(v, "v", 4, 4);
  const int dt = dtype_code(q, "q");
  if (dtype_code(k, "k") != dt || dtype_code(v, "v") != dt)
    TVM_FFI_THROW(TypeError) << "q, k, v must share dtype (all f16 or all bf16)";
  const int64_t b = q.shape()[0], sq = q.shape()[1], h = q.shape()[2], d = q.shape()[3];
  const int64_t sk = k.shape()[1], hk = k.shape()[2];
  if (k.shape()[0] != b || k.shape()[3] != d)
    TVM_FFI_THROW(ValueError) << "k must be [B, Sk, Hk, D] with q's batch and head dim";
  for (int i = 0; i < 4; ++i)
    if (v.shape()[i] != k.shape()[i]) TVM_FFI_THROW(ValueError) << "v must have k's shape [B, Sk, Hk, D]";
  const DLDevice dev = q.device();
  if (k.device().device_id != dev.device_id || v.device().device_id != dev.device_id)
    TVM_FFI_THROW(ValueError) << "k and v must be on the same device as q";
  if (wl < INT32_MIN || wl > INT32_MAX || wr < INT32_MIN || wr > INT32_MAX)
    TVM_FFI_THROW(ValueError) << "window sizes must fit int32";
  q = addressable(q, dev);
  k = addressable(k, dev);
  v = addressable(v, dev);

  Optional<Tensor> supplied;
  if (n == 10 || n == 13 || n == 14 || n == 16 || n == 18)
    supplied = arg<Optional<Tensor>>(args, (n == 14 || n == 16 || n == 18) ? 12 : n - 1, "out");
  if (lse_only && !supplied.has_value()) TVM_FFI_THROW(ValueError) << "LSE-only forward requires a supplied output";
  Tensor out = supplied.has_value() ? supplied.value() : alloc({b, sq, h, d}, q.dtype(), dev);
  if (supplied.has_value()) {
    const Tensor& o = supplied.value();
    bool same = o.ndim() == 4 && o.dtype().code == q.dtype().code && o.dtype().bits == q.dtype().bits &&
                o.device().device_type == dev.device_type && o.device().device_id == dev.device_id;
    for (int i = 0; same && i < 4; ++i) same = o.shape()[i] == q.shape()[i];
    if (!same) TVM_FFI_THROW(ValueError) << "out must match q's shape, dtype and device";
    if ((o.strides()[3] != 1 && d > 1) || !elements_are_disjoint(o))
      TVM_FFI_THROW(ValueError) << "out must have unit last stride and nonoverlapping non-negative strides; unsupported "
                                   "writable layout: elements overlap or the bounded safety checks cannot prove they are "
                                   "disjoint. Use a separately allocated contiguous output.";
  }
  // A supplied output is written in place when the kernels can address it and it shares no memory with an input;
  // otherwise the result goes to a temporary and is copied into it afterwards (host/forward/mod.rs:367-375,832-840).
  bool copy_out = false;
  if (supplied.has_value()) {
    const Tensor& o = supplied.value();
    int64_t os[3] = {b > 1 ? o.strides()[0] : 0, sq > 1 ? o.strides()[1] : 0, h > 1 ? o.strides()[2] : 0};
    copy_out = !fa2_layout_is_addressable(o.data_ptr(), os, 3) || ranges_overlap(o, q) || ranges_overlap(o, k) ||
               ranges_overlap(o, v);
    if (copy_out) out = alloc({b, sq, h, d}, q.dtype(), dev);
  }
  Tensor lse = alloc({b, h, sq}, kF32, dev);

  fa2_fwd_args a{};
  a.q = q.data_ptr();
  a.k = k.data_ptr();
  a.v = v.data_ptr();
  a.out = out.data_ptr();
  a.lse = static_cast<float*>(lse.data_ptr());
  a.alibi_slopes = alibi_ptr(alibi, b, h, dev, &a.alibi_batch_stride);
  a.dtype = dt;
  a.batch = static_cast<int32_t>(b);
  a.seqlen_q = static_cast<int32_t>(sq);
  a.seqlen_k = static_cast<int32_t>(sk);
  a.heads = static_cast<int32_t>(h);
  a.heads_k = static_cast<int32_t>(hk);
  a.head_dim = static_cast<int32_t>(d);
  fill_strides(q, a.q_stride);
  fill_strides(k, a.k_stride);
  fill_strides(v, a.v_stride);
  fill_strides(out, a.o_stride);
  a.softmax_scale = static_cast<float>(scale_opt.has_value() ? scale_opt.value() : 1.0 / std::sqrt(static_cast<double>(d)));
  a.causal = causal;
  a.window_left = static_cast<int32_t>(wl);
  a.window_right = static_cast<int32_t>(wr);
  a.softcap = static_cast<float>(softcap);
  check(fa2_fwd(&a, stream_of(dev)));
  if (copy_out) {
    const Tensor& o = supplied.value();
    const int64_t shape4[4] = {b, sq, h, d};
    const int64_t from[3] = {sq * h * d, h * d, d};
    const int64_t to[3] = {o.strides()[0], o.strides()[1], o.strides()[2]};
    check(fa2_copy_16bit(out.data_ptr(), from, o.data_ptr(), to, shape4, stream_of(dev)));
    out = o;
  }
  if (lse_only) return Any(lse);
  if (n >= 14) return Any(Array<Tensor>{out, lse, alloc({0}, q.dtype(), dev)});
  return Any(Array<Tensor>{out, lse});
}

// ------------------------------------------------------------------------------------ backward
Any bwd_preprocess_impl(const AnyView* args, int32_t n) {
  if (n != 3) TVM_FFI_THROW(ValueError) << "bwd_preprocess expects dout, out, p_dropout";
  check_dropout_zero(arg<double>(args, 2, "p_dropout"));
  Tensor dout = arg<Tensor>(args, 0, "dout"), out = arg<Tensor>(args, 1, "out");
  check_attention_tensor(dout, "dout", 4, 4);
  check_attention_tensor(out, "out", 4, 4);
  const int dt = dtype_code(dout, "dout");
  bool same = dtype_code(out, "out") == dt && dout.device().device_id == out.device().device_id;
  for (int i = 0; same && i < 4; ++i) same = dout.shape()[i] == out.shape()[i];
  if (!same) TVM_FFI_THROW(ValueError) << "dout and out must share shape, dtype and device";
  dout = addressable(dout, dout.device());
  out = addressable(out, out.device());
  const int64_t b = out.shape()[0], s = out.shape()[1], h = out.shape()[2], d = out.shape()[3];
  if (b <= 0 || h <= 0 || b > 65535 || h > 65535 || s < 0 || d < 8 || d > 256 || d % 8 != 0)
    TVM_FFI_THROW(ValueError) << "unsupported backward tensor dimensions";
  const int64_t s_pad = (s + 127) / 128 * 128;
  Tensor delta = alloc({b, h, s_pad}, kF32, out.device());
  if (s == 0) return Any(delta);
  fa2_bwd_preprocess_args a{};
  a.dout = dout.data_ptr();
  a.out = out.data_ptr();
  a.delta = static_cast<float*>(delta.data_ptr());
  a.dtype = dt;
  a.batch = static_cast<int32_t>(b);
  a.seqlen_q = static_cast<int32_t>(s);
  a.heads = static_cast<int32_t>(h);
  a.head_dim = static_cast<int32_t>(d);
  fill_strides(dout, a.do_stride);
  fill_strides(out, a.o_stride);
  check(fa2_bwd_preprocess(&a, stream_of(out.device())));
  return Any(delta);
}

// which: 1 = dq, 2 = dk and dv, 3 = all
Any bwd_impl(const AnyView* args, int32_t n, int which) {
  if (n != 14)
    TVM_FFI_THROW(ValueError) << "backward expects q, k, v, dout, lse, delta, alibi_slopes, softmax_scale, is_causal, "
                                 "window_size_left, window_size_right, softcap, p_dropout, rng_state; got "
                              << n;
  Tensor q = arg<Tensor>(args, 0, "q"), k = arg<Tensor>(args, 1, "k"), v = arg<Tensor>(args, 2, "v");
  Tensor dout = arg<Tensor>(args, 3, "dout"), lse = arg<Tensor>(args, 4, "lse"), delta = arg<Tensor>(args, 5, "delta");
  Optional<Tensor> alibi = arg<Optional<Tensor>>(args, 6, "alibi_slopes");
  Optional<double> scale_opt = arg<Optional<double>>(args, 7, "softmax_scale");
  const bool causal = arg<bool>(args, 8, "is_causal");
  const int64_t wl = arg<int64_t>(args, 9, "window_size_left"), wr = arg<int64_t>(args, 10, "window_size_right");
  const double softcap = arg<double>(args, 11, "softcap");
  check_dropout_zero(arg<double>(args, 12, "p_dropout"));
  for (auto [t, name] : {std::pair<const Tensor&, const char*>{q, "q"}, {k, "k"}, {v, "v"}, {dout, "dout"}})
    check_attention_tensor(t, name, 4, 4);
  const int dt = dtype_code(q, "q");
  if (dtype_code(k, "k") != dt || dtype_code(v, "v") != dt || dtype_code(dout, "dout") != dt)
    TVM_FFI_THROW(TypeError) << "q, k, v, dout must share dtype (all f16 or all bf16)";
  const int64_t b = q.shape()[0], sq = q.shape()[1], h = q.shape()[2], d = q.shape()[3];
  const int64_t sk = k.shape()[1], hk = k.shape()[2];
  bool ok = k.shape()[0] == b && k.shape()[3] == d;
  for (int i = 0; ok && i < 4; ++i) ok = v.shape()[i] == k.shape()[i] && dout.shape()[i] == q.shape()[i];
  if (!ok) TVM_FFI_THROW(ValueError) << "dout must match q, and k, v must be [B, Sk, Hk, D] with q's batch and head dim";
  const DLDevice dev = q.device();
  q = addressable(q, dev);
  k = addressable(k, dev);
  v = addressable(v, dev);
  dout = addressable(dout, dev);
  const int64_t sq_pad = (sq + 127) / 128 * 128;
  auto f32_on_dev = [&](const Tensor& t) {
    return t.dtype().code == kDLFloat && t.dtype().bits == 32 && t.device().device_type == kDLCUDA &&
           t.device().device_id == dev.device_id && is_contiguous(t);
  };
  if (!f32_on_dev(lse) || lse.ndim() != 3 || lse.shape()[0] != b || lse.shape()[1] != h || lse.shape()[2] != sq)
    TVM_FFI_THROW(ValueError) << "lse must be contiguous float32 [B, H, Sq] on q's device";
  if (!f32_on_dev(delta) || delta.ndim() != 3 || delta.shape()[0] != b || delta.shape()[1] != h ||
      delta.shape()[2] != sq_pad)
    TVM_FFI_THROW(ValueError) << "delta must be contiguous float32 [B, H, ceil(Sq/128)*128] on q's device";
  if (wl < INT32_MIN || wl > INT32_MAX || wr < INT32_MIN || wr > INT32_MAX)
    TVM_FFI_THROW(ValueError) << "window sizes must fit int32";

  fa2_bwd_args a{};
  a.q = q.data_ptr();
  a.k = k.data_ptr();
  a.v = v.data_ptr();
  a.dout = dout.data_ptr();
  a.lse = static_cast<const float*>(lse.data_ptr());
  a.delta = static_cast<const float*>(delta.data_ptr());
  a.dtype = dt;
  a.batch = static_cast<int32_t>(b);
  a.seqlen_q = static_cast<int32_t>(sq);
  a.seqlen_k = static_cast<int32_t>(sk);
  a.heads = static_cast<int32_t>(h);
  a.heads_k = static_cast<int32_t>(hk);
  a.head_dim = static_cast<int32_t>(d);
  fill_strides(q, a.q_stride);
  fill_strides(k, a.k_stride);
  fill_strides(v, a.v_stride);
  fill_strides(dout, a.do_stride);
  a.alibi_slopes = alibi_ptr(alibi, b, h, dev, &a.alibi_batch_stride);
  a.softcap = static_cast<float>(softcap);
  a.softmax_scale = static_cast<float>(scale_opt.has_value() ? scale_opt.value() : 1.0 / std::sqrt(static_cast<double>(d)));
  a.causal = causal;
  a.window_left = static_cast<int32_t>(wl);
  a.window_right = static_cast<int32_t>(wr);
  a.which = which;
  // Gradients are allocated like the inputs (backward.rs:199-204); the fp32 dQ accumulator is a
  // workspace tensor from the same stream-ordered allocator.
  // Only what the call returns is allocated (bwd_dq: dQ; bwd_dkv: dK and dV).
  Optional<Tensor> dq, dk, dv;
  if (which & 1) {
    dq = alloc({b, sq, h, d}, q.dtype(), dev);
    a.dq = dq.value().data_ptr();
  }
  if (which & 2) {
    dk = alloc({b, sk, hk, d}, k.dtype(), dev);
    dv = alloc({b, sk, hk, d}, v.dtype(), dev);
    a.dk = dk.value().data_ptr();
    a.dv = dv.value().data_ptr();
  }
  Optional<Tensor> accum;
  const int64_t ws = fa2_bwd_workspace_bytes(&a);
  if (ws > 0) {
    accum = alloc({ws / 4}, kF32, dev);
    a.dq_accum = accum.value().data_ptr();
    a.dq_accum_bytes = ws;
  }
  check(fa2_bwd(&a, stream_of(dev)));
  if (which == 1) return Any(dq.value());
  if (which == 2) return Any(Array<Tensor>{dk.value(), dv.value()});
  return Any(Array<Tensor>{dq.value(), dk.value(), dv.value()});
}

// ------------------------------------------------------------------------------------ packed (varlen)
struct Packed {
  int64_t total, heads, d;
  int64_t row_stride, head_stride;
};
Packed packed_shape(const Tensor& t, const char* name) {
  check_attention_tensor(t, name, 3, 4);
  Packed p{};
  const auto sh = t.shape();
  const auto st = t.strides();
  if (t.ndim() == 4) {
    if (sh[0] != 1) TVM_FFI_THROW(ValueError) << "inconsistent packed attention inputs";
    p = {sh[1], sh[2], sh[3], st[1], st[2]};
  } else {
    p = {sh[0], sh[1], sh[2], st[0], st[1]};
  }
  return p;
}

const int32_t* metadata(const Tensor& t, int64_t len, DLDevice dev, const char* name) {
  const DLDataType dt = t.dtype();
  if (t.device().device_type != kDLCUDA || t.device().device_id != dev.device_id || dt.code != kDLInt ||
      dt.bits != 32 || dt.lanes != 1 || t.ndim() != 1 || t.shape()[0] != len || !is_contiguous(t) ||
      reinterpret_cast<uintptr_t>(t.data_ptr()) % 4 != 0)
    TVM_FFI_THROW(ValueError) << name << " must be a contiguous CUDA int32 tensor of shape [" << len << "]";
  return static_cast<const int32_t*>(t.data_ptr());
}

Any varlen_fwd_impl(const AnyView* args, int32_t n) {
  if (n != 19 && n != 20 && !(n >= 22 && n <= 24))
    TVM_FFI_THROW(ValueError) << "varlen_fwd expects q, k, v, cuq, cuk, used, leftpad, alibi, scale, causal, left, "
                                 "right, cap, dropout, state, max_q, max_k, return_softmax, zero_tensors";
  if (n >= 22) unsupported("the KV-cache form of varlen_fwd");
  Tensor q = arg<Tensor>(args, 0, "q"), k = arg<Tensor>(args, 1, "k"), v = arg<Tensor>(args, 2, "v");
  Optional<Tensor> cuq = arg<Optional<Tensor>>(args, 3, "cu_seqlens_q");
  Optional<Tensor> cuk = arg<Optional<Tensor>>(args, 4, "cu_seqlens_k");
  Optional<Tensor> used = arg<Optional<Tensor>>(args, 5, "seqused_k");
  Optional<Tensor> leftpad = arg<Optional<Tensor>>(args, 6, "leftpad_k");
  Optional<Tensor> alibi = arg<Optional<Tensor>>(args, 7, "alibi");
  Optional<double> scale_opt = arg<Optional<double>>(args, 8, "scale");
  bool causal = arg<bool>(args, 9, "causal");
  const int64_t wl = arg<int64_t>(args, 10, "left"), wr = arg<int64_t>(args, 11, "right");
  const double cap = arg<double>(args, 12, "cap");
  check_dropout_zero(arg<double>(args, 13, "dropout"));
  const int64_t max_q = arg<int64_t>(args, 15, "max_q"), max_k = arg<int64_t>(args, 16, "max_k");
  if (arg<bool>(args, 17, "return_softmax")) unsupported("return_softmax");
  const bool zero_tensors = arg<bool>(args, 18, "zero_tensors");
  if (n == 20 && arg<Optional<Tensor>>(args, 19, "block_table").has_value()) unsupported("paged K/V (block_table)");
  if (used.has_value()) unsupported("seqused_k");
  if (leftpad.has_value()) unsupported("leftpad_k");
  if (!cuq.has_value()) TVM_FFI_THROW(ValueError) << "cu_seqlens_q is required";
  if (!cuk.has_value()) TVM_FFI_THROW(ValueError) << "cu_seqlens_k is required";
  if (cuq.value().ndim() != 1 || cuq.value().shape()[0] < 2)
    TVM_FFI_THROW(ValueError) << "cu_seqlens_q must have shape [batch + 1]";
  const int64_t batch = cuq.value().shape()[0] - 1;

  for (Tensor* t : {&q, &k, &v}) {
    check_attention_tensor(*t, "q, k, v", 3, 4);
    dtype_code(*t, "q, k, v");
    *t = addressable(*t, t->device());
  }
  const Packed pq = packed_shape(q, "q"), pk = packed_shape(k, "k"), pv = packed_shape(v, "v");
  const int dt = dtype_code(q, "q");
  const DLDevice dev = q.device();
  if (pk.total != pv.total || pk.heads != pv.heads || pk.d != pv.d || pk.d != pq.d || dtype_code(k, "k") != dt ||
      dtype_code(v, "v") != dt || k.device().device_id != dev.device_id || v.device().device_id != dev.device_id)
    TVM_FFI_THROW(ValueError) << "inconsistent packed attention inputs";
  const int64_t h = pq.heads, hk = pk.heads, d = pq.d;
  if (batch <= 0 || h <= 0 || hk <= 0 || h % hk != 0 || batch > 65535 || h > 65535 || d < 8 || d > 256 || d % 8 != 0 ||
      pq.total > INT32_MAX || pk.total > INT32_MAX || max_q < 0 || max_k < 0 || max_q > INT32_MAX - 127 ||
      max_k > INT32_MAX - 127)
    TVM_FFI_THROW(ValueError) << "unsupported packed attention dimensions";
  const int32_t* cu_q = metadata(cuq.value(), batch + 1, dev, "cu_seqlens_q");
  const int32_t* cu_k = metadata(cuk.value(), batch + 1, dev, "cu_seqlens_k");
  if (max_q == 1 && !alibi.has_value()) causal = false;  // single-query convention (varlen/mod.rs:250-252)

  Tensor out = q.ndim() == 4 ? alloc({1, pq.total, h, d}, q.dtype(), dev) : alloc({pq.total, h, d}, q.dtype(), dev);
  Tensor lse = alloc({h, pq.total}, kF32, dev);
  Tensor probs = alloc({0}, q.dtype(), dev);
  void* stream = stream_of(dev);

  fa2_fwd_args a{};
  a.q = q.data_ptr();
  a.k = k.data_ptr();
  a.v = v.data_ptr();
  a.out = out.data_ptr();
  a.lse = static_cast<float*>(lse.data_ptr());
  int32_t abs = 0;
  a.alibi_slopes = alibi_ptr(alibi, batch, h, dev, &abs);
  a.alibi_batch_stride = abs;
  a.dtype = dt;
  a.batch = static_cast<int32_t>(batch);
  a.seqlen_q = static_cast<int32_t>(max_q);
  a.seqlen_k = static_cast<int32_t>(max_k);
  a.heads = static_cast<int32_t>(h);
  a.heads_k = static_cast<int32_t>(hk);
  a.head_dim = static_cast<int32_t>(d);
  a.q_stride[1] = pq.row_stride;
  a.q_stride[2] = pq.head_stride;
  a.k_stride[1] = pk.row_stride;
  a.k_stride[2] = pk.head_stride;
  a.v_stride[1] = pv.row_stride;
  a.v_stride[2] = pv.head_stride;
  a.o_stride[1] = h * d;
  a.o_stride[2] = d;
  a.softmax_scale = static_cast<float>(scale_opt.has_value() ? scale_opt.value() : 1.0 / std::sqrt(static_cast<double>(d)));
  a.causal = causal;
  a.window_left = static_cast<int32_t>(wl);
  a.window_right = static_cast<int32_t>(wr);
  a.softcap = static_cast<float>(cap);
  a.cu_seqlens_q = cu_q;
  a.cu_seqlens_k = cu_k;
  a.total_q = static_cast<int32_t>(pq.total);
  a.total_k = static_cast<int32_t>(pk.total);
  a.zero_tensors = zero_tensors ? 1 : 0;
  check(fa2_varlen_fwd(&a, stream));
  return Any(Array<Tensor>{out, lse, probs});
}

Any varlen_bwd_impl(const AnyView* args, int32_t n) {
  if (n != 19)
    TVM_FFI_THROW(ValueError) << "varlen_bwd expects q,k,v,dout,out,lse,cuq,cuk,alibi,scale,causal,left,right,cap,"
                                 "dropout,state,max_q,max_k,zero_tensors";
  Tensor q = arg<Tensor>(args, 0, "q"), k = arg<Tensor>(args, 1, "k"), v = arg<Tensor>(args, 2, "v");
  Tensor dout = arg<Tensor>(args, 3, "dout"), out = arg<Tensor>(args, 4, "out"), lse = arg<Tensor>(args, 5, "lse");
  Tensor cuq = arg<Tensor>(args, 6, "cu_seqlens_q"), cuk = arg<Tensor>(args, 7, "cu_seqlens_k");
  Optional<Tensor> alibi = arg<Optional<Tensor>>(args, 8, "alibi");
  Optional<double> scale_opt = arg<Optional<double>>(args, 9, "scale");
  const bool causal = arg<bool>(args, 10, "causal");
  const int64_t wl = arg<int64_t>(args, 11, "left"), wr = arg<int64_t>(args, 12, "right");
  const double cap = arg<double>(args, 13, "cap");
  check_dropout_zero(arg<double>(args, 14, "dropout"));
  const int64_t max_q = arg<int64_t>(args, 16, "max_q"), max_k = arg<int64_t>(args, 17, "max_k");
  if (cuq.ndim() != 1 || cuq.shape()[0] < 2) TVM_FFI_THROW(ValueError) << "cu_seqlens_q must have shape [batch + 1]";
  const int64_t batch = cuq.shape()[0] - 1;
  for (Tensor* t : {&q, &k, &v, &dout, &out}) {
    check_attention_tensor(*t, "q, k, v, dout, out", 3, 4);
    dtype_code(*t, "q, k, v, dout, out");
    *t = addressable(*t, t->device());
  }
  const Packed pq = packed_shape(q, "q"), pk = packed_shape(k, "k"), pv = packed_shape(v, "v");
  const Packed pd = packed_shape(dout, "dout"), po = packed_shape(out, "out");
  const int dt = dtype_code(q, "q");
  const DLDevice dev = q.device();
  if (pk.total != pv.total || pk.heads != pv.heads || pk.d != pv.d || pk.d != pq.d || dtype_code(k, "k") != dt ||
      dtype_code(v, "v") != dt || dtype_code(dout, "dout") != dt || dtype_code(out, "out") != dt ||
      pd.total != pq.total || pd.heads != pq.heads || pd.d != pq.d || po.total != pq.total || po.heads != pq.heads ||
      po.d != pq.d)
    TVM_FFI_THROW(ValueError) << "inconsistent packed attention inputs";
  const int64_t h = pq.heads, hk = pk.heads, d = pq.d;
  if (batch <= 0 || h <= 0 || hk <= 0 || h % hk != 0 || d < 8 || d > 256 || d % 8 != 0 || max_q < 0 || max_k < 0)
    TVM_FFI_THROW(ValueError) << "unsupported packed attention dimensions";
  const int32_t* cu_q = metadata(cuq, batch + 1, dev, "cu_seqlens_q");
  const int32_t* cu_k = metadata(cuk, batch + 1, dev, "cu_seqlens_k");
  if (lse.dtype().code != kDLFloat || lse.dtype().bits != 32 || lse.ndim() != 2 || lse.shape()[0] != h ||
      lse.shape()[1] != pq.total || !is_contiguous(lse))
    TVM_FFI_THROW(ValueError) << "lse must be contiguous float32 [H, total_q]";
  void* stream = stream_of(dev);

  Tensor delta = alloc({h, pq.total + 128 * batch}, kF32, dev);
  fa2_bwd_preprocess_args pa{};
  pa.dout = dout.data_ptr();
  pa.out = out.data_ptr();
  pa.delta = static_cast<float*>(delta.data_ptr());
  pa.dtype = dt;
  pa.batch = static_cast<int32_t>(batch);
  pa.seqlen_q = static_cast<int32_t>(max_q);
  pa.heads = static_cast<int32_t>(h);
  pa.head_dim = static_cast<int32_t>(d);
  pa.do_stride[1] = pd.row_stride;
  pa.do_stride[2] = pd.head_stride;
  pa.o_stride[1] = po.row_stride;
  pa.o_stride[2] = po.head_stride;
  pa.cu_seqlens_q = cu_q;
  pa.total_q = static_cast<int32_t>(pq.total);
  check(fa2_bwd_preprocess(&pa, stream));

  auto like = [&](const Tensor& t, const Packed& p) {
    return t.ndim() == 4 ? alloc({1, p.total, p.heads, p.d}, t.dtype(), dev) : alloc({p.total, p.heads, p.d}, t.dtype(), dev);
  };
  Tensor dq = like(q, pq), dk = like(k, pk), dv = like(v, pk);
  fa2_bwd_args a{};
  a.q = q.data_ptr();
  a.k = k.data_ptr();
  a.v = v.data_ptr();
  a.dout = dout.data_ptr();
  a.lse = static_cast<const float*>(lse.data_ptr());
  a.delta = static_cast<const float*>(delta.data_ptr());
  a.dq = dq.data_ptr();
  a.dk = dk.data_ptr();
  a.dv = dv.data_ptr();
  a.dtype = dt;
  a.batch = static_cast<int32_t>(batch);
  a.seqlen_q = static_cast<int32_t>(max_q);
  a.seqlen_k = static_cast<int32_t>(max_k);
  a.heads = static_cast<int32_t>(h);
  a.heads_k = static_cast<int32_t>(hk);
  a.head_dim = static_cast<int32_t>(d);
  a.alibi_slopes = alibi_ptr(alibi, batch, h, dev, &a.alibi_batch_stride);
  a.softcap = static_cast<float>(cap);
  a.q_stride[1] = pq.row_stride;
  a.q_stride[2] = pq.head_stride;
  a.k_stride[1] = pk.row_stride;
  a.k_stride[2] = pk.head_stride;
  a.v_stride[1] = pv.row_stride;
  a.v_stride[2] = pv.head_stride;
  a.do_stride[1] = pd.row_stride;
  a.do_stride[2] = pd.head_stride;
  a.softmax_scale = static_cast<float>(scale_opt.has_value() ? scale_opt.value() : 1.0 / std::sqrt(static_cast<double>(d)));
  a.causal = causal;
  a.window_left = static_cast<int32_t>(wl);
  a.window_right = static_cast<int32_t>(wr);
  a.which = 3;
  a.cu_seqlens_q = cu_q;
  a.cu_seqlens_k = cu_k;
  a.total_q = static_cast<int32_t>(pq.total);
  a.total_k = static_cast<int32_t>(pk.total);
  Optional<Tensor> accum;
  const int64_t ws = fa2_bwd_workspace_bytes(&a);
  if (ws > 0) {
    accum = alloc({ws / 4}, kF32, dev);
    a.dq_accum = accum.value().data_ptr();
    a.dq_accum_bytes = ws;
  }
  check(fa2_bwd(&a, stream));
  return Any(Array<Tensor>{dq, dk, dv, delta});
}

}  // namespace

#define FA2_EXPORT_PACKED(name, expr)                                                                          \
  extern "C" TVM_FFI_DLL_EXPORT int __tvm_ffi_##name(void* self, const TVMFFIAny* raw_args, int32_t num_args, \
                                                     TVMFFIAny* result) {                                     \
    TVM_FFI_SAFE_CALL_BEGIN();                                                                                 \
    const AnyView* args = reinterpret_cast<const AnyView*>(raw_args);                                          \
    (void)args;                                                                                                \
    *reinterpret_cast<Any*>(result) = (expr);                                                                  \
    TVM_FFI_SAFE_CALL_END();                                                                                   \
  }

static Any not_built(const char* name) {
  TVM_FFI_THROW(RuntimeError) << name << " is not implemented in the B200 build";
  return Any();
}

FA2_EXPORT_PACKED(fwd, fwd_impl(args, num_args, false))
FA2_EXPORT_PACKED(fwd_lse, fwd_impl(args, num_args, true))
FA2_EXPORT_PACKED(bwd_preprocess, bwd_preprocess_impl(args, num_args))
FA2_EXPORT_PACKED(bwd_dq, bwd_impl(args, num_args, 1))
FA2_EXPORT_PACKED(bwd_dkv, bwd_impl(args, num_args, 2))
FA2_EXPORT_PACKED(bwd_all, bwd_impl(args, num_args, 3))
FA2_EXPORT_PACKED(varlen_fwd_explicit, varlen_fwd_impl(args, num_args))
FA2_EXPORT_PACKED(varlen_bwd_explicit, varlen_bwd_impl(args, num_args))
FA2_EXPORT_PACKED(varlen_fwd_descriptor, not_built("varlen_fwd_descriptor"))
FA2_EXPORT_PACKED(rng_state, not_built("rng_state"))
FA2_EXPORT_PACKED(cache_merge_explicit, not_built("cache_merge_explicit"))
FA2_EXPORT_PACKED(cache_update_explicit, not_built("cache_update_explicit"))
FA2_EXPORT_PACKED(cache_validate_layouts, not_built("cache_validate_layouts"))
