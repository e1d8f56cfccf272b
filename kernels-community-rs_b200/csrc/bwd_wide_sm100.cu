// FlashAttention-2 backward for sm_100a (B200), head dims above 128 (136 ... 256): dQ, dK, dV in one kernel.
//
// dK and dV of 128 keys at head dim 256 would fill all 512 TMEM columns, so a CTA owns 128 keys of one
// (batch, kv head) and one HALF of the head dim (columns [128 c, 128 c + 128)): it accumulates that half of dK
// and dV, and adds that half of dQ. S^T and dP^T contract over the whole head dim and are computed by both
// halves' CTAs. Query rows go by in blocks of 64 (all query heads of the GQA group, one after the other):
//
//   S^T   = K Q^T                 smem x smem -> TMEM [128 keys x 64 q], over the whole head dim
//   dP^T  = V dO^T                TMEM x smem: V sits in TMEM as a 16-bit A operand, written there once by the
//                                 compute warps straight from global memory, which leaves its 64 KB of shared
//                                 memory to a second Q / dO stage
//   P^T   = exp2(S^T c - lse)     compute warps, written back over S^T as 16-bit
//   dV_c += P^T dO_c              TMEM x smem (dO as an MN-major operand)
//   dS^T  = P^T (dP^T - delta)    compute warps -> swizzled smem [128 keys x 64 q]
//   dK_c += dS^T Q_c              smem x smem (Q as an MN-major operand)
//   dQ_c^T = K_c^T dS^T           smem x smem, both MN-major -> TMEM [128 d x 64 q] over the dP^T columns; the
//                                 compute warps transpose it into the retired Q stage (one d column per thread,
//                                 [64 q x 32 d] fp32 per warp) and add it into the fp32 dQ accumulator with one
//                                 cp.reduce.async.bulk per warp (64 plain reductions per thread took 3500 cycles
//                                 an iteration and set its pace)
//
// TMEM columns: dK_c [0,128) dV_c [128,256) S^T/P^T [256,320) dP^T/dQ_c^T [320,384) V [384,512).
// Shared memory: K whole (64 KB), two stages of a Q and a dO tile of 64 rows (32 KB each), dS^T (16 KB).
// Warps: 0-3 compute (one key row per thread; one d row per thread for dQ^T), 4 loader, 5 MMA issuer,
// 6 fixer (packed batches: clears the rows of K, Q and dO tiles that lie past the end of the sequence).
//
// Stands in, for these head dims, for the reference kernels `backward` and `backward_kv`
// (flash-attn2-rs/src/device/backward/dq.rs:12-302, dkv.rs:15-266, common.rs:121-152) and their packed
// variants (src/device/varlen/backward.rs:134-648). dQ is summed in arrival order.
#include "sm100_ptx.cuh"
#include "fa2_params.h"
#include "fa2_launch.h"

namespace fa2 {

namespace {

constexpr int kBK = 128;  // keys per CTA
constexpr int kBQ = 64;   // query rows per iteration
constexpr int kBWThreads = 256;
constexpr int kBWLoadWarp = 4;
constexpr int kBWMmaWarp = 5;
constexpr int kBWFixWarp = 6;
constexpr float kBWLog2e = 1.4426950408889634f;

struct BwdWideCfg {
  static constexpr int kAtomK = kBK * 128;   // bytes of one 64-column atom of K
  static constexpr int kAtomQ = kBQ * 128;   // bytes of one 64-column atom of Q or dO
  static constexpr int kMaxAtoms = 4;
  static constexpr int kStageBytes = kMaxAtoms * kAtomQ;
  static constexpr int kKOff = 0;
  static constexpr int kQOff = kMaxAtoms * kAtomK;        // 2 stages
  static constexpr int kDOOff = kQOff + 2 * kStageBytes;  // 2 stages
  static constexpr int kDSOff = kDOOff + 2 * kStageBytes; // [128 keys x 64 q] 16-bit, one atom
  static constexpr int kBarOff = kDSOff + kAtomK;
  static constexpr int kNumBars = 23;
  static constexpr int kMiscOff = (kBarOff + kNumBars * 8 + 15) / 16 * 16;
  static constexpr int kStatOff = kMiscOff + 32;   // lse / delta: [2 buffers][2][64] fp32
  static constexpr int kSmemBytes = kStatOff + 2 * 2 * kBQ * 4;
  static_assert(kStatOff % 16 == 0, "lse / delta are read as float4");
  static constexpr uint32_t kTmemDK = 0, kTmemDV = 128, kTmemS = 256, kTmemDP = 320, kTmemV = 384;
};

struct WKvTile {
  int b, hk, n0, half;
  int sq, sk, q_row0, k_row0, bq, off;
  int m_start, n_m, n_iter;
  bool valid;
};

struct WWalk {
  int g, mi;
};
__device__ __forceinline__ WWalk wwalk_next(WWalk w, int n_m) {
  if (++w.mi == n_m) {
    w.mi = 0;
    ++w.g;
  }
  return w;
}

__device__ __forceinline__ float bw_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// The two halves of a key block are neighbours in the grid (they read the same tiles), and consecutive pairs
// walk the key blocks of one (batch, kv head), heaviest first under a causal mask.
__device__ __forceinline__ WKvTile get_wkv_tile(const BwdParams& p, int t) {
  WKvTile ti;
  ti.half = t & 1;
  t >>= 1;
  const int bh = t / p.num_nblk;
  const int nblk = t - bh * p.num_nblk;
  ti.b = bh / p.heads_k;
  ti.hk = bh - ti.b * p.heads_k;
  ti.n0 = nblk * kBK;
  if (p.cu_q != nullptr) {
    ti.q_row0 = p.cu_q[ti.b];
    ti.sq = p.cu_q[ti.b + 1] - ti.q_row0;
    ti.k_row0 = p.cu_k[ti.b];
    ti.sk = p.cu_k[ti.b + 1] - ti.k_row0;
    ti.bq = 0;
    if (ti.sq < 0 || ti.sk < 0 || ti.sq > p.seqlen_q || ti.sk > p.seqlen_k) ti.sk = 0;
  } else {
    ti.q_row0 = 0;
    ti.k_row0 = 0;
    ti.sq = p.seqlen_q;
    ti.sk = p.seqlen_k;
    ti.bq = ti.b;
  }
  ti.off = ti.sk - ti.sq;
  ti.valid = ti.n0 < ti.sk;
  // Query rows [q_lo, q_hi) can see a key of [n0, n0 + 127].
  int q_lo = 0, q_hi = ti.sq;
  const int n_last = min(ti.n0 + kBK - 1, ti.sk - 1);
  if (p.window_right >= 0) q_lo = max(0, ti.n0 - ti.off - p.window_right);
  if (p.window_left >= 0) q_hi = min(ti.sq, n_last - ti.off + p.window_left + 1);
  ti.m_start = q_lo / kBQ;
  ti.n_m = (q_hi > q_lo) ? ((q_hi + kBQ - 1) / kBQ - ti.m_start) : 0;
  ti.n_iter = ti.n_m * p.group;
  return ti;
}

// ATOMS: 64-column atoms of the head dim that are loaded (3 for head dims up to 192, else 4). TMA fills what lies
// past the real head dim inside them with zeros, so every contraction runs over ATOMS * 64 columns with
// compile-time operand offsets: a runtime bound in the issuing thread's loops doubles the cost of an MMA issue.
// FANCY (softcap or ALiBi in use) and PACKED (cu_seqlens batches) are compile-time: the plain dense kernel carries
// none of their code, which keeps its loops within reach of the SM's instruction cache.
template <bool BF16, int ATOMS, bool FANCY, bool PACKED>
__global__ void __launch_bounds__(kBWThreads, 1) bwd_wide_kernel(const __grid_constant__ BwdParams p) {
  using Cfg = BwdWideCfg;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0u) {
    if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, kWaitNone + 1);
    return;
  }
  uint8_t* s_k = smem + Cfg::kKOff;
  uint8_t* s_q = smem + Cfg::kQOff;
  uint8_t* s_do = smem + Cfg::kDOOff;
  uint8_t* s_ds = smem + Cfg::kDSOff;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kBarOff);
  uint64_t* k_full = bars + 0;
  uint64_t* q_full = bars + 1;     // [2]
  uint64_t* do_full = bars + 3;    // [2]
  uint64_t* q_free = bars + 5;     // [2] S^T and dK have read the Q stage and the dQ reductions staged in it have left
  uint64_t* do_free = bars + 7;    // [2] dP^T and dV, the readers of the dO stage, have completed
  uint64_t* s_full = bars + 9;
  uint64_t* p_full = bars + 10;
  uint64_t* dp_full = bars + 11;
  uint64_t* ds_full = bars + 12;
  uint64_t* dq_full = bars + 13;
  uint64_t* dq_free = bars + 14;   // dQ^T has been read out of TMEM: the next dP^T may overwrite its columns
  uint64_t* dkv_done = bars + 15;
  uint64_t* stat_full = bars + 16;
  uint64_t* v_ready = bars + 17;   // V sits in TMEM
  uint64_t* k_fixed = bars + 18;   // packed batches: the fixer warp has cleared the rows past the sequence
  uint64_t* q_fixed = bars + 19;   // [2]
  uint64_t* do_fixed = bars + 21;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Cfg::kMiscOff + 8);
  float* s_stat = reinterpret_cast<float*>(smem + Cfg::kStatOff);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const WaitCtl ctl{abort_flag, p.status};
  const WKvTile ti = get_wkv_tile(p, blockIdx.x);
  if (!ti.valid) return;
  constexpr int atoms = ATOMS;
  const int ncol = min(128, atoms * 64 - ti.half * 128);     // columns of this CTA's half (128 or 64)
  const int n_iter = ti.n_iter;
  const bool want_dq = (p.which & 1) != 0;
  constexpr bool packed = PACKED;

  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(k_full, 1);
    for (int st = 0; st < 2; ++st) {
      mbar_init(&q_full[st], 1);
      mbar_init(&do_full[st], 1);
      mbar_init(&q_free[st], 5);  // the dK commit and the four compute warps
      mbar_init(&do_free[st], 1);
      mbar_init(&q_fixed[st], 1);
      mbar_init(&do_fixed[st], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, kBK);
    mbar_init(dp_full, 1);
    mbar_init(ds_full, kBK);
    mbar_init(dq_full, 1);
    mbar_init(dq_free, kBK);
    mbar_init(dkv_done, 1);
    mbar_init(stat_full, kBK);
    mbar_init(v_ready, kBK);
    mbar_init(k_fixed, 1);
    mbar_fence_init();
  }
  if (warp == kBWMmaWarp) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (warp == kBWLoadWarp && lane == 0) {
    tma_prefetch_desc(&p.tm_q);
    tma_prefetch_desc(&p.tm_k);
    tma_prefetch_desc(&p.tm_do);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp < 4) {
    // ------------------------------------------------------------------ compute
    const int key_in = tid;
    const int kpos = ti.n0 + key_in;
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t t_s = tmem + lane_addr + Cfg::kTmemS;
    const uint32_t t_dp = tmem + lane_addr + Cfg::kTmemDP;
    bool ok = true;
    if (n_iter > 0) {
      // V of this key row goes from global memory into TMEM as the 16-bit A operand of dP^T: column c holds the
      // elements 2c and 2c + 1, which is the row's own memory layout. Rows past the sequence and columns past the
      // head dim are zero.
      const uint4* vrow = reinterpret_cast<const uint4*>(
          reinterpret_cast<const uint16_t*>(p.v_ptr) + ti.bq * p.v_batch_stride +
          static_cast<int64_t>(ti.k_row0 + kpos) * p.v_row_stride + ti.hk * p.v_head_stride);
      const int chunks = (kpos < ti.sk) ? p.head_dim / 8 : 0;
#pragma unroll
      for (int part = 0; part < 4; ++part) {
        uint32_t vr[32];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint4 x = make_uint4(0, 0, 0, 0);
          if (part * 8 + c < chunks) x = vrow[part * 8 + c];
          vr[4 * c] = x.x;
          vr[4 * c + 1] = x.y;
          vr[4 * c + 2] = x.z;
          vr[4 * c + 3] = x.w;
        }
        tmem_st32(tmem + lane_addr + Cfg::kTmemV + part * 32, vr);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(v_ready);
    }
    // LSE (log2 domain) and delta of one query block: thread t < 64 loads LSE of row t, the others delta of
    // row t - 64; rows past the sequence give P = 0. The value for iteration it + 1 is requested while
    // iteration it computes.
    auto load_stat = [&](WWalk w) -> float {
      const int hq = ti.hk * p.group + w.g;
      const int q = (ti.m_start + w.mi) * kBQ + (tid & (kBQ - 1));
      if (tid < kBQ) {
        float v = INFINITY;
        if (q < ti.sq) v = p.lse[ti.bq * p.lse_batch_stride + hq * p.lse_head_stride + ti.q_row0 + q] * kBWLog2e;
        return v;
      }
      float v = 0.f;
      if (q < ti.sq)
        v = p.delta[ti.bq * p.delta_batch_stride + hq * p.delta_head_stride + ti.q_row0 + ti.b * p.delta_seq_pad + q];
      return v;
    };
    const float inv_cap = (p.softcap > 0.f) ? p.scale / p.softcap : 0.f;
    const float cap_l2 = p.softcap * kBWLog2e;
    constexpr bool fancy = FANCY;
    WWalk w{0, 0};
    float stat_next = n_iter > 0 ? load_stat(w) : 0.f;
    for (int it = 0; it < n_iter; ++it) {
      const int m0 = (ti.m_start + w.mi) * kBQ;
      const int hq = ti.hk * p.group + w.g;
      w = wwalk_next(w, ti.n_m);
      float* stat = s_stat + (it & 1) * (2 * kBQ);
      stat[tid] = stat_next;
      if (it + 1 < n_iter) stat_next = load_stat(w);
      mbar_arrive(stat_full);
      const bool stat_ok = mbar_wait(stat_full, it & 1, ctl, kWaitBwd + 15);  // voted on with s_full below
      if (it > 0) {
        // The reductions of the previous iteration have read their staging area by now: its Q stage goes back
        // to the loader.
        if (lane == 0) {
          tma_wait_group_read<0>();
          mbar_arrive(&q_free[(it - 1) & 1]);
        }
        __syncwarp();
      }
      const float* lse_s = stat;
      const float* dl_s = stat + kBQ;

      // ---- phase A: P^T = exp2(S^T c - lse)
      if (!__all_sync(0xffffffffu, mbar_wait(s_full, it & 1, ctl, kWaitBwd + 11) && stat_ok)) { ok = false; break; }
      tc_fence_after();
      uint32_t sr[kBQ];
      tmem_ld32(t_s, sr);
      tmem_ld32(t_s + 32, sr + 32);
      tmem_wait_ld();
      // Columns [c_lo, c_hi) of this key row are visible.
      int c_lo = 0, c_hi = kBQ;
      if (p.window_right >= 0) c_lo = kpos - ti.off - p.window_right - m0;
      if (p.window_left >= 0) c_hi = kpos - ti.off + p.window_left + 1 - m0;
      if (kpos >= ti.sk) c_hi = -1;
      const float slope = (p.alibi != nullptr) ? p.alibi[ti.b * p.alibi_batch_stride + hq] * kBWLog2e : 0.f;
      float pr[kBQ];  // P times the derivative of the score transform: what goes on to dS
      if (!fancy) {
#pragma unroll
        for (int i = 0; i < kBQ; i += 2) {
          float pv0 = ex2(fmaf(__uint_as_float(sr[i]), p.scale_log2, -lse_s[i]));
          float pv1 = ex2(fmaf(__uint_as_float(sr[i + 1]), p.scale_log2, -lse_s[i + 1]));
          if (i < c_lo || i >= c_hi) pv0 = 0.f;
          if (i + 1 < c_lo || i + 1 >= c_hi) pv1 = 0.f;
          pr[i] = pv0;
          pr[i + 1] = pv1;
          sr[i / 2] = pack2<BF16>(pv0, pv1);
        }
      } else {
#pragma unroll
        for (int i = 0; i < kBQ; i += 2) {
          float pp[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float raw = __uint_as_float(sr[i + e]);
            float x, deriv = 1.f;
            if (p.softcap > 0.f) {
              const float t = bw_tanh(raw * inv_cap);
              x = cap_l2 * t;
              deriv = fmaf(-t, t, 1.f);
            } else {
              x = raw * p.scale_log2;
            }
            if (p.alibi != nullptr)
              x += p.causal_alibi ? slope * static_cast<float>(kpos)
                                  : -slope * fabsf(static_cast<float>(m0 + i + e + ti.off - kpos));
            float pv = ex2(x - lse_s[i + e]);
            if (i + e < c_lo || i + e >= c_hi) pv = 0.f;
            pp[e] = pv;
            pr[i + e] = pv * deriv;
          }
          sr[i / 2] = pack2<BF16>(pp[0], pp[1]);
        }
      }
      tmem_st32(t_s, sr);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(p_full);

      // ---- phase B: dS^T = P^T (dP^T - delta)
      if (!warp_wait(dp_full, it & 1, ctl, kWaitBwd + 12)) { ok = false; break; }
      tc_fence_after();
      tmem_ld32(t_dp, sr);
      tmem_ld32(t_dp + 32, sr + 32);
      tmem_wait_ld();
      tc_fence_before();
      // The dS^T buffer is free: dq_full (or q_free) of the previous iteration has been seen in phase C.
      uint8_t* ds_row = s_ds + key_in * 128;
#pragma unroll
      for (int c = 0; c < kBQ / 8; ++c) {
        const int i = c * 8;
        uint4 wv;
        wv.x = pack2<BF16>(pr[i] * (__uint_as_float(sr[i]) - dl_s[i]), pr[i + 1] * (__uint_as_float(sr[i + 1]) - dl_s[i + 1]));
        wv.y = pack2<BF16>(pr[i + 2] * (__uint_as_float(sr[i + 2]) - dl_s[i + 2]), pr[i + 3] * (__uint_as_float(sr[i + 3]) - dl_s[i + 3]));
        wv.z = pack2<BF16>(pr[i + 4] * (__uint_as_float(sr[i + 4]) - dl_s[i + 4]), pr[i + 5] * (__uint_as_float(sr[i + 5]) - dl_s[i + 5]));
        wv.w = pack2<BF16>(pr[i + 6] * (__uint_as_float(sr[i + 6]) - dl_s[i + 6]), pr[i + 7] * (__uint_as_float(sr[i + 7]) - dl_s[i + 7]));
        *reinterpret_cast<uint4*>(ds_row + ((c ^ (key_in & 7)) << 4)) = wv;
      }
      fence_proxy_async_smem();
      mbar_arrive(ds_full);

      // ---- phase C: this half of dQ^T [128 d x 64 q] (in the dP^T columns) into the fp32 accumulator: every
      // thread holds one d column; a warp writes its [64 q x 32 d] block, rows of 128 bytes with the 16-byte
      // chunks swizzled as the tensor map expects, into the Q stage that dK has finished with, and one bulk
      // reduce-add takes it from there. dq_full also tells that dK has read dS^T.
      if (!warp_wait(dq_full, it & 1, ctl, kWaitBwd + 14)) { ok = false; break; }
      if (want_dq) {
        tc_fence_after();
        tmem_ld32(t_dp, sr);
        tmem_ld32(t_dp + 32, sr + 32);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(dq_free);
        // Rows past the sequence (the 64-row box reaches the next sequence of a packed batch) add exact zeros.
        const int rows = min(kBQ, ti.sq - m0);
        uint8_t* buf = s_q + (it & 1) * Cfg::kStageBytes + warp * (kBQ * 128);
        const uint32_t col_byte = static_cast<uint32_t>(lane & 3) * 4;
        const uint32_t chunk = static_cast<uint32_t>(lane >> 2);
#pragma unroll
        for (int i = 0; i < kBQ; ++i)
          *reinterpret_cast<uint32_t*>(buf + i * 128 + ((chunk ^ (i & 7)) << 4) + col_byte) = (i < rows) ? sr[i] : 0u;
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          const int d0 = ti.half * 128 + warp * 32;
          if (d0 < p.head_dim) tma_reduce_add_4d(&p.tm_dqa, buf, d0, hq, ti.q_row0 + m0, ti.bq);
          tma_commit_group();
        }
        __syncwarp();
      }
    }
    if (n_iter > 0) {
      // The last iteration's reductions: see them read their staging area before the CTA may end.
      if (lane == 0) {
        tma_wait_group_read<0>();
        mbar_arrive(&q_free[(n_iter - 1) & 1]);
      }
      __syncwarp();
    }
    // ---- epilogue: this half of dK (scaled) and of dV, 32 columns at a time, straight to global memory
    if (ok && (p.which & 2) != 0) {
      bool done = true;
      if (n_iter > 0) done = warp_wait(dkv_done, 0, ctl, kWaitBwd + 13);
      if (done) {
        tc_fence_after();
        const int64_t row_off = ti.bq * p.dkv_batch_stride + static_cast<int64_t>(ti.k_row0 + kpos) * p.dkv_row_stride +
                                ti.hk * p.dkv_head_stride + ti.half * 128;
        for (int o = 0; o < 2; ++o) {
          const float mul = (o == 0) ? p.scale : 1.f;
          uint16_t* grow = reinterpret_cast<uint16_t*>(o == 0 ? p.dk_ptr : p.dv_ptr) + row_off;
          const uint32_t t_acc = tmem + lane_addr + (o == 0 ? Cfg::kTmemDK : Cfg::kTmemDV);
          for (int c = 0; c < ncol / 32; ++c) {
            uint32_t acc[32];
            if (n_iter > 0) {
              tmem_ld32(t_acc + c * 32, acc);
              tmem_wait_ld();
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) acc[i] = 0u;
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 wv;
              wv.x = pack2<BF16>(__uint_as_float(acc[8 * q]) * mul, __uint_as_float(acc[8 * q + 1]) * mul);
              wv.y = pack2<BF16>(__uint_as_float(acc[8 * q + 2]) * mul, __uint_as_float(acc[8 * q + 3]) * mul);
              wv.z = pack2<BF16>(__uint_as_float(acc[8 * q + 4]) * mul, __uint_as_float(acc[8 * q + 5]) * mul);
              wv.w = pack2<BF16>(__uint_as_float(acc[8 * q + 6]) * mul, __uint_as_float(acc[8 * q + 7]) * mul);
              const int col = c * 32 + q * 8;
              if (kpos < ti.sk && ti.half * 128 + col < p.head_dim) *reinterpret_cast<uint4*>(grow + col) = wv;
            }
          }
        }
        tc_fence_before();
      }
    } else if (ok && n_iter > 0) {
      // dQ-only call: still see the last commits land before the CTA ends.
      warp_wait(dkv_done, 0, ctl, kWaitBwd + 13);
    }
    __syncwarp();
  } else if (warp == kBWLoadWarp) {
    if (n_iter > 0 && elect_one()) {
      // ---------------------------------------------------------------- loader
      mbar_expect_tx(k_full, atoms * Cfg::kAtomK);
      for (int a = 0; a < atoms; ++a) tma_load_4d(s_k + a * Cfg::kAtomK, &p.tm_k, k_full, a * 64, ti.hk, ti.k_row0 + ti.n0, ti.bq);
      bool ok = true;
      WWalk w{0, 0};
      for (int it = 0; it < n_iter && ok; ++it, w = wwalk_next(w, ti.n_m)) {
        const int hq = ti.hk * p.group + w.g;
        const int m0 = (ti.m_start + w.mi) * kBQ;
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        // A stage is free once the MMAs of its previous use that read it have completed.
        ok = mbar_wait(&q_free[st], ph ^ 1, ctl, kWaitBwd + 1);
        if (!ok) break;
        mbar_expect_tx(&q_full[st], atoms * Cfg::kAtomQ);
        for (int a = 0; a < atoms; ++a)
          tma_load_4d(s_q + st * Cfg::kStageBytes + a * Cfg::kAtomQ, &p.tm_q, &q_full[st], a * 64, hq, ti.q_row0 + m0, ti.bq);
        ok = mbar_wait(&do_free[st], ph ^ 1, ctl, kWaitBwd + 2);
        if (!ok) break;
        mbar_expect_tx(&do_full[st], atoms * Cfg::kAtomQ);
        for (int a = 0; a < atoms; ++a)
          tma_load_4d(s_do + st * Cfg::kStageBytes + a * Cfg::kAtomQ, &p.tm_do, &do_full[st], a * 64, hq, ti.q_row0 + m0, ti.bq);
      }
      // The loader leaves last: the commits on the free barriers of each stage's last use have landed.
      for (int st = 0; st < 2 && ok; ++st) {
        const int uses = (n_iter - st + 1) / 2;  // iterations st, st + 2, ...
        if (uses > 0) {
          ok = mbar_wait(&q_free[st], (uses - 1) & 1, ctl, kWaitBwd + 1);
          if (ok) ok = mbar_wait(&do_free[st], (uses - 1) & 1, ctl, kWaitBwd + 2);
        }
      }
    }
  } else if (warp == kBWFixWarp) {
    // ---------------------------------------------------------------- fixer (packed batches)
    // The reference zero-fills the rows of a tile that lie past the end of the sequence while staging it; the
    // TMA boxes here carry the next sequence's rows instead, and a zero probability times a NaN or Inf of a
    // neighbour would still poison the gradients. This warp waits for every Q and dO tile and clears the stray
    // rows of those that need it, and of K once (V is written to TMEM row by row, with zeros past the sequence).
    if (packed && n_iter > 0) {
      auto clear_rows = [&](uint8_t* tile, int atom_bytes, int first, int rows) {
        for (int r = first + (lane >> 3); r < rows; r += 4)
          for (int a = 0; a < atoms; ++a)
            *reinterpret_cast<uint4*>(tile + a * atom_bytes + r * 128 + (lane & 7) * 16) = make_uint4(0, 0, 0, 0);
      };
      auto publish = [&](uint64_t* bar) {
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar);
        __syncwarp();
      };
      bool ok = true;
      const int k_first = ti.sk - ti.n0;
      if (k_first < kBK) {
        ok = __all_sync(0xffffffffu, mbar_wait(k_full, 0, ctl, kWaitBwd + 3));
        if (ok) {
          clear_rows(s_k, Cfg::kAtomK, k_first, kBK);
          publish(k_fixed);
        }
      }
      WWalk w{0, 0};
      for (int it = 0; it < n_iter && ok; ++it, w = wwalk_next(w, ti.n_m)) {
        const int first = ti.sq - (ti.m_start + w.mi) * kBQ;
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(&q_full[st], ph, ctl, kWaitBwd + 4));
        if (ok && first < kBQ) {
          clear_rows(s_q + st * Cfg::kStageBytes, Cfg::kAtomQ, first, kBQ);
          publish(&q_fixed[st]);
        }
        ok = ok && __all_sync(0xffffffffu, mbar_wait(&do_full[st], ph, ctl, kWaitBwd + 5));
        if (ok && first < kBQ) {
          clear_rows(s_do + st * Cfg::kStageBytes, Cfg::kAtomQ, first, kBQ);
          publish(&do_fixed[st]);
        }
      }
    }
  } else if (warp == kBWMmaWarp && n_iter > 0 && elect_one()) {
    // ---------------------------------------------------------------- mma issuer
    const uint32_t fmt = BF16 ? 1u : 0u;
    const uint32_t kBase = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(kBK >> 4) << 24);
    const uint32_t idesc_qk = kBase | (static_cast<uint32_t>(kBQ >> 3) << 17);                      // S^T, dP^T
    const uint32_t idesc_dv = kBase | (static_cast<uint32_t>(ncol >> 3) << 17) | (1u << 16);        // dV, dK: B MN-major
    const uint32_t idesc_dq = kBase | (static_cast<uint32_t>(kBQ >> 3) << 17) | (1u << 15) | (1u << 16);  // dQ^T: both MN-major
    constexpr uint32_t kAtomK16 = Cfg::kAtomK >> 4;
    constexpr uint32_t kAtomQ16 = Cfg::kAtomQ >> 4;
    constexpr uint32_t kStage16 = Cfg::kStageBytes >> 4;
    const uint64_t k_kmaj = make_smem_desc(smem_u32(s_k), 16, 1024);
    const uint64_t q_kmaj = make_smem_desc(smem_u32(s_q), 16, 1024);
    const uint64_t do_kmaj = make_smem_desc(smem_u32(s_do), 16, 1024);
    const uint64_t ds_kmaj = make_smem_desc(smem_u32(s_ds), 16, 1024);
    // MN-major views: the leading offset is the distance between 64-element chunks along M / N (one atom).
    const uint64_t q_mn = make_smem_desc(smem_u32(s_q + ti.half * 2 * Cfg::kAtomQ), Cfg::kAtomQ, 1024);
    const uint64_t do_mn = make_smem_desc(smem_u32(s_do + ti.half * 2 * Cfg::kAtomQ), Cfg::kAtomQ, 1024);
    const uint64_t k_mn = make_smem_desc(smem_u32(s_k + ti.half * 2 * Cfg::kAtomK), Cfg::kAtomK, 1024);
    const uint64_t ds_mn = make_smem_desc(smem_u32(s_ds), Cfg::kAtomK, 1024);
    constexpr int n_ks = ATOMS * 4;  // steps of 16 over the loaded columns
    // S^T [keys x q] = K[keys x d] Q[q x d]^T, both K-major in shared memory, over the head dim in steps of 16;
    // compile-time operand offsets keep the issuing thread lean.
    auto issue_st = [&](uint64_t q_stage) {
      static_for<n_ks>([&](auto ks) {
        constexpr uint32_t in_atom = (ks.value & 3) * 2;
        mma_ss_o<(ks.value >> 2) * kAtomK16 + in_atom, (ks.value >> 2) * kAtomQ16 + in_atom>(
            tmem + Cfg::kTmemS, k_kmaj, q_stage, idesc_qk, ks.value > 0 ? 1u : 0u);
      });
    };
    // dP^T [keys x q] = V[keys x d] dO[q x d]^T with V in TMEM: 16 elements of a row are 8 columns.
    auto issue_dp = [&](uint64_t do_stage) {
      static_for<n_ks>([&](auto ks) {
        constexpr uint32_t in_atom = (ks.value & 3) * 2;
        mma_ts_o<ks.value * 8, (ks.value >> 2) * kAtomQ16 + in_atom>(tmem + Cfg::kTmemDP, tmem + Cfg::kTmemV, do_stage,
                                                                     idesc_qk, ks.value > 0 ? 1u : 0u);
      });
    };
    // Packed batches: a tile that reaches past the end of its sequence holds rows of the next sequence; it is
    // usable once the fixer warp has cleared them. bit st of *_par: parity of the stage's next fix.
    uint32_t qfix_par = 0, dofix_par = 0;
    auto ragged_q = [&](int mi) { return packed && (ti.m_start + mi) * kBQ + kBQ > ti.sq; };
    auto q_ready = [&](int mi, uint32_t st, uint32_t ph, int code) -> bool {
      if (!mbar_wait(&q_full[st], ph, ctl, code)) return false;
      if (!ragged_q(mi)) return true;
      const uint32_t par = (qfix_par >> st) & 1;
      qfix_par ^= 1u << st;
      return mbar_wait(&q_fixed[st], par, ctl, kWaitBwd + 21);
    };
    auto do_ready = [&](int mi, uint32_t st, uint32_t ph, int code) -> bool {
      if (!mbar_wait(&do_full[st], ph, ctl, code)) return false;
      if (!ragged_q(mi)) return true;
      const uint32_t par = (dofix_par >> st) & 1;
      dofix_par ^= 1u << st;
      return mbar_wait(&do_fixed[st], par, ctl, kWaitBwd + 22);
    };
    bool ok = mbar_wait(k_full, 0, ctl, kWaitBwd + 3);
    if (ok && packed && ti.n0 + kBK > ti.sk) ok = mbar_wait(k_fixed, 0, ctl, kWaitBwd + 20);
    if (ok) ok = q_ready(0, 0, 0, kWaitBwd + 4);  // iteration 0 is query block m_start
    if (ok) {
      tc_fence_after();
      issue_st(q_kmaj);
      mma_commit(s_full);
      ok = do_ready(0, 0, 0, kWaitBwd + 5);
    }
    if (ok) ok = mbar_wait(v_ready, 0, ctl, kWaitBwd + 23);
    if (ok) {
      tc_fence_after();
      issue_dp(do_kmaj);
      mma_commit(dp_full);
    }
    WWalk wn{0, 0};  // position of iteration it + 1
    for (int it = 0; it < n_iter && ok; ++it) {
      wn = wwalk_next(wn, ti.n_m);
      const uint32_t st = it & 1;
      const uint32_t nph = ((it + 1) >> 1) & 1;  // phase of the stage barriers of iteration it + 1
      const bool has_next = it + 1 < n_iter;
      const uint32_t acc = it > 0 ? 1u : 0u;
      // dV_c += P^T dO_c (P^T: 32 packed columns at S^T; 16 query rows of dO are 2048 bytes)
      ok = mbar_wait(p_full, it & 1, ctl, kWaitBwd + 6);
      if (!ok) break;
      tc_fence_after();
      {
        const uint64_t b = do_mn + st * kStage16;
        static_for<kBQ / 16>([&](auto ks) {
          mma_ts_o<ks.value * 8, ks.value * (2048 >> 4)>(tmem + Cfg::kTmemDV, tmem + Cfg::kTmemS, b, idesc_dv,
                                                         ks.value > 0 ? 1u : acc);
        });
      }
      mma_commit(&do_free[st]);
      // dK_c += dS^T Q_c, then dQ_c^T = K_c^T dS^T over the 128 keys into the dP^T columns (the compute warps
      // have read dP^T). They go before the next S^T: the compute warps wait for dQ^T next.
      ok = mbar_wait(ds_full, it & 1, ctl, kWaitBwd + 7);
      if (!ok) break;
      tc_fence_after();
      {
        const uint64_t b = q_mn + st * kStage16;
        static_for<kBQ / 16>([&](auto ks) {
          mma_ss_o<ks.value * 2, ks.value * (2048 >> 4)>(tmem + Cfg::kTmemDK, ds_kmaj, b, idesc_dv, ks.value > 0 ? 1u : acc);
        });
      }
      mma_commit(&q_free[st]);
      if (want_dq) {
        static_for<kBK / 16>([&](auto ks) {
          mma_ss_o<ks.value * (2048 >> 4), ks.value * (2048 >> 4)>(tmem + Cfg::kTmemDP, k_mn, ds_mn, idesc_dq,
                                                                    ks.value > 0 ? 1u : 0u);
        });
      }
      mma_commit(dq_full);
      if (has_next) {
        // S^T of the next iteration (dV, the last reader of P^T, was issued above), then its dP^T once dQ^T has
        // left the columns.
        ok = q_ready(wn.mi, st ^ 1, nph, kWaitBwd + 8);
        if (!ok) break;
        tc_fence_after();
        issue_st(q_kmaj + (st ^ 1) * kStage16);
        mma_commit(s_full);
        ok = do_ready(wn.mi, st ^ 1, nph, kWaitBwd + 9);
        if (ok && want_dq) ok = mbar_wait(dq_free, it & 1, ctl, kWaitBwd + 10);
        if (!ok) break;
        tc_fence_after();
        issue_dp(do_kmaj + (st ^ 1) * kStage16);
        mma_commit(dp_full);
      }
    }
    if (ok) mma_commit(dkv_done);
  }
  __syncwarp();
  if (*abort_flag) {
    // A wait ran out somewhere in this CTA. MMAs, commits and copies may still be in flight: give them
    // about a millisecond to land before the barriers' memory and the TMEM columns are given back.
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) {
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kBWMmaWarp) tmem_dealloc(tmem, 512);
}

template <bool BF16, int ATOMS, bool FANCY, bool PACKED>
cudaError_t launch_bwd_wide_one(const BwdParams& p, cudaStream_t stream) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(bwd_wide_kernel<BF16, ATOMS, FANCY, PACKED>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, BwdWideCfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int64_t blocks = 2LL * p.num_nblk * p.batch * p.heads_k;
  if (blocks <= 0) return cudaSuccess;
  if (blocks > 0x7fffffffLL) return cudaErrorInvalidValue;
  bwd_wide_kernel<BF16, ATOMS, FANCY, PACKED>
      <<<static_cast<unsigned>(blocks), kBWThreads, BwdWideCfg::kSmemBytes, stream>>>(p);
  return cudaGetLastError();
}

template <bool BF16, int ATOMS>
cudaError_t pick_features(const BwdParams& p, cudaStream_t stream) {
  const bool fancy = (p.softcap > 0.f) || (p.alibi != nullptr);
  const bool packed = p.cu_q != nullptr;
  if (fancy) {
    return packed ? launch_bwd_wide_one<BF16, ATOMS, true, true>(p, stream)
                  : launch_bwd_wide_one<BF16, ATOMS, true, false>(p, stream);
  }
  return packed ? launch_bwd_wide_one<BF16, ATOMS, false, true>(p, stream)
                : launch_bwd_wide_one<BF16, ATOMS, false, false>(p, stream);
}

}  // namespace

cudaError_t launch_bwd_wide(const BwdParams& p, int head_dim, bool bf16, cudaStream_t stream) {
  if (head_dim <= 128 || head_dim > 256 || head_dim % 8 != 0) return cudaErrorInvalidValue;
  if (head_dim <= 192) return bf16 ? pick_features<true, 3>(p, stream) : pick_features<false, 3>(p, stream);
  return bf16 ? pick_features<true, 4>(p, stream) : pick_features<false, 4>(p, stream);
}

}  // namespace fa2
