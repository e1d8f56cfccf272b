// HBM-bound helpers of the backward pass:
//   * delta = rowsum(dO * O) in fp32, written into the padded layouts the reference uses
//     (flash-attn2-rs/src/device/backward/reduce.rs:40-108, src/device/varlen/backward.rs:53-132);
//   * the final dQ = 16-bit(scale * fp32 accumulator) conversion
//     (same shape as the reference's backward_dq_merge, reduce.rs:164-197).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "fa2_params.h"
#include "fa2_launch.h"

namespace fa2 {

namespace {

template <bool BF16>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
  if constexpr (BF16) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  } else {
    const __half2 h = *reinterpret_cast<const __half2*>(&w);
    return __half22float2(h);
  }
}

// One group of LANES threads handles kRows consecutive (batch, row, head) units; each thread reads 16 bytes
// of dO and of O per unit, and all of a thread's loads are issued before the first is used, which keeps
// enough bytes in flight to run at HBM speed. Rows are enumerated over the padded length so the padding
// is written as zero.
constexpr int kRows = 4;

template <bool BF16, int LANES, typename IDX>
__global__ void __launch_bounds__(256) preprocess_kernel(const PreprocessParams p) {
  // IDX is 32-bit whenever the number of (batch, row, head) units allows: the 64-bit divisions of the index
  // arithmetic otherwise take longer than the loads they lead to.
  const IDX group = static_cast<IDX>((blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x) / LANES);
  const int lane = threadIdx.x % LANES;
  const IDX total = static_cast<IDX>(static_cast<uint64_t>(p.batch) * p.seqlen_pad * p.heads);
  const int chunks = p.head_dim / 8;  // 16-byte chunks per row; LANES >= chunks
  uint4 x[kRows], y[kRows];
  bool store[kRows];
  int64_t dst[kRows];
  // The first unit is split into (batch, row, head) once; the following ones are reached by counting up.
  const IDX gid0 = group * kRows;
  const bool any = gid0 < total;
  int h = static_cast<int>((any ? gid0 : 0) % static_cast<IDX>(p.heads));
  const IDX bs0 = (any ? gid0 : 0) / static_cast<IDX>(p.heads);
  int s = static_cast<int>(bs0 % static_cast<IDX>(p.seqlen_pad));
  int b = static_cast<int>(bs0 / static_cast<IDX>(p.seqlen_pad));
  // No thread leaves before the shuffles below: a warp holds 32 / LANES groups, some of which may lie past
  // the end.
#pragma unroll
  for (int r = 0; r < kRows; ++r) {
    const bool in_range = any && (gid0 + r < total);
    int64_t row = s;     // row inside the input tensors
    int64_t drow = s;    // row inside delta
    bool live = in_range && s < p.seqlen_q;
    store[r] = in_range;
    int bq = b;
    if (p.cu_q != nullptr) {
      const int bb = in_range ? b : 0;
      const int q0 = p.cu_q[bb];
      const int len = p.cu_q[bb + 1] - q0;
      live = in_range && s < len;
      row = q0 + s;
      drow = q0 + 128 * bb + s;
      bq = 0;
      // Padding of a packed sequence: only the 128-row tail that belongs to it.
      if (s >= (len + 127) / 128 * 128) store[r] = false;
    }
    dst[r] = bq * p.delta_batch_stride + h * p.delta_head_stride + drow;
    x[r] = make_uint4(0, 0, 0, 0);
    y[r] = make_uint4(0, 0, 0, 0);
    if (live && lane < chunks) {
      x[r] = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.dout) + bq * p.do_batch_stride +
                                            row * p.do_row_stride + h * p.do_head_stride)[lane];
      y[r] = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.out) + bq * p.o_batch_stride +
                                            row * p.o_row_stride + h * p.o_head_stride)[lane];
    }
    if (++h == p.heads) {
      h = 0;
      if (++s == p.seqlen_pad) {
        s = 0;
        ++b;
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kRows; ++r) {
    const uint32_t xs[4] = {x[r].x, x[r].y, x[r].z, x[r].w}, ys[4] = {y[r].x, y[r].y, y[r].z, y[r].w};
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 fx = unpack2<BF16>(xs[k]), fy = unpack2<BF16>(ys[k]);
      sum = fmaf(fx.x, fy.x, sum);
      sum = fmaf(fx.y, fy.y, sum);
    }
#pragma unroll
    for (int d = LANES / 2; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d, LANES);
    if (lane == 0 && store[r]) p.delta[dst[r]] = sum;
  }
}

template <bool BF16>
__global__ void __launch_bounds__(256) dq_convert_kernel(const float4* __restrict__ src, uint4* __restrict__ dst,
                                                         int64_t n8, float scale) {
  // From the end of the accumulator to its start: the backward kernel walks the heads in ascending order, so
  // what it touched last (and the L2 still holds) sits at the end.
  for (int64_t j = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; j < n8;
       j += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t i = n8 - 1 - j;
    const float4 a = src[2 * i], b = src[2 * i + 1];
    uint4 w;
    if constexpr (BF16) {
      __nv_bfloat162 t0 = __floats2bfloat162_rn(a.x * scale, a.y * scale), t1 = __floats2bfloat162_rn(a.z * scale, a.w * scale);
      __nv_bfloat162 t2 = __floats2bfloat162_rn(b.x * scale, b.y * scale), t3 = __floats2bfloat162_rn(b.z * scale, b.w * scale);
      w = make_uint4(*reinterpret_cast<uint32_t*>(&t0), *reinterpret_cast<uint32_t*>(&t1),
                     *reinterpret_cast<uint32_t*>(&t2), *reinterpret_cast<uint32_t*>(&t3));
    } else {
      __half2 t0 = __floats2half2_rn(a.x * scale, a.y * scale), t1 = __floats2half2_rn(a.z * scale, a.w * scale);
      __half2 t2 = __floats2half2_rn(b.x * scale, b.y * scale), t3 = __floats2half2_rn(b.z * scale, b.w * scale);
      w = make_uint4(*reinterpret_cast<uint32_t*>(&t0), *reinterpret_cast<uint32_t*>(&t1),
                     *reinterpret_cast<uint32_t*>(&t2), *reinterpret_cast<uint32_t*>(&t3));
    }
    dst[i] = w;
  }
}

}  // namespace

cudaError_t launch_bwd_preprocess(const PreprocessParams& p, cudaStream_t stream) {
  const int64_t units = static_cast<int64_t>(p.batch) * p.seqlen_pad * p.heads;
  if (units == 0) return cudaSuccess;
  const int64_t groups = (units + kRows - 1) / kRows;
  const int lanes = p.head_dim <= 64 ? 8 : p.head_dim <= 128 ? 16 : 32;  // one 16-byte chunk of the row per lane
  const int64_t threads = groups * lanes;
  const unsigned grid = static_cast<unsigned>((threads + 255) / 256);
  const bool small = units < (1ll << 31);
#define FA2_LAUNCH_PRE(BF, L)                                                      \
  do {                                                                             \
    if (small) preprocess_kernel<BF, L, uint32_t><<<grid, 256, 0, stream>>>(p);    \
    else preprocess_kernel<BF, L, uint64_t><<<grid, 256, 0, stream>>>(p);          \
  } while (0)
  if (p.bf16) {
    if (lanes == 8) FA2_LAUNCH_PRE(true, 8);
    else if (lanes == 16) FA2_LAUNCH_PRE(true, 16);
    else FA2_LAUNCH_PRE(true, 32);
  } else {
    if (lanes == 8) FA2_LAUNCH_PRE(false, 8);
    else if (lanes == 16) FA2_LAUNCH_PRE(false, 16);
    else FA2_LAUNCH_PRE(false, 32);
  }
#undef FA2_LAUNCH_PRE
  return cudaGetLastError();
}

// Copy of a 16-bit tensor [n0, n1, n2, d] with unit last stride between two layouts with arbitrary outer
// strides. Stands in for the reference's packing kernel (flash-attn2-rs/src/device/layout.rs:4-35), which
// runs when a view cannot be addressed by the main kernels (there: 16-byte alignment of the row starts), and
// for its copy-out of a result computed into a temporary (src/host/layout.rs:458-512). VEC = 8 moves 16 bytes
// per thread and needs both layouts to keep every row start 16-byte aligned; VEC = 1 is the general case.
template <int VEC>
__global__ void __launch_bounds__(256) copy_rows_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst,
                                                        int64_t total, int n1, int n2, int dv, int64_t a0, int64_t a1,
                                                        int64_t a2, int64_t b0, int64_t b1, int64_t b2) {
  const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;  // one group of VEC elements
  if (i >= total) return;
  const int c = static_cast<int>(i % dv) * VEC;
  int64_t r = i / dv;
  const int i2 = static_cast<int>(r % n2);
  r /= n2;
  const int i1 = static_cast<int>(r % n1);
  const int64_t i0 = r / n1;
  const uint16_t* s = src + i0 * a0 + i1 * a1 + i2 * a2 + c;
  uint16_t* d = dst + i0 * b0 + i1 * b1 + i2 * b2 + c;
  if constexpr (VEC == 8) {
    *reinterpret_cast<uint4*>(d) = *reinterpret_cast<const uint4*>(s);
  } else {
    *d = *s;
  }
}

cudaError_t launch_copy_rows(const void* src, void* dst, int64_t n0, int64_t n1, int64_t n2, int64_t d,
                             const int64_t src_strides[3], const int64_t dst_strides[3], cudaStream_t stream) {
  if (n0 * n1 * n2 * d == 0) return cudaSuccess;
  bool vec = d % 8 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0;
  for (int i = 0; i < 3; ++i) vec = vec && src_strides[i] % 8 == 0 && dst_strides[i] % 8 == 0;
  const int64_t dv = vec ? d / 8 : d;
  const int64_t total = n0 * n1 * n2 * dv;
  const unsigned grid = static_cast<unsigned>((total + 255) / 256);
  const uint16_t* s = static_cast<const uint16_t*>(src);
  uint16_t* t = static_cast<uint16_t*>(dst);
  if (vec)
    copy_rows_kernel<8><<<grid, 256, 0, stream>>>(s, t, total, static_cast<int>(n1), static_cast<int>(n2), static_cast<int>(dv),
                                                  src_strides[0], src_strides[1], src_strides[2], dst_strides[0],
                                                  dst_strides[1], dst_strides[2]);
  else
    copy_rows_kernel<1><<<grid, 256, 0, stream>>>(s, t, total, static_cast<int>(n1), static_cast<int>(n2), static_cast<int>(dv),
                                                  src_strides[0], src_strides[1], src_strides[2], dst_strides[0],
                                                  dst_strides[1], dst_strides[2]);
  return cudaGetLastError();
}

cudaError_t launch_dq_convert(const float* src, void* dst, int64_t n, float scale, bool bf16, cudaStream_t stream) {
  const int64_t n8 = n / 8;
  if (n8 == 0) return cudaSuccess;
  const int64_t want = (n8 + 255) / 256;
  const unsigned grid = static_cast<unsigned>(want < 148 * 16 ? want : 148 * 16);
  if (bf16) dq_convert_kernel<true><<<grid, 256, 0, stream>>>(reinterpret_cast<const float4*>(src), reinterpret_cast<uint4*>(dst), n8, scale);
  else dq_convert_kernel<false><<<grid, 256, 0, stream>>>(reinterpret_cast<const float4*>(src), reinterpret_cast<uint4*>(dst), n8, scale);
  return cudaGetLastError();
}

}  // namespace fa2
