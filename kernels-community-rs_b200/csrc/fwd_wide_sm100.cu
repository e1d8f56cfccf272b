// FlashAttention-2 forward for sm_100a (B200), head dims above 128 (136 ... 256, the reference's 192 and 256
// buckets, flash-attn2-rs/src/host/tiles.rs:1).
//
// The O accumulator of one 128-row query block takes up to 256 of the 512 TMEM columns and a 128-key K or V
// tile would take 64 KB of shared memory, so this kernel is laid out differently from the one for head dims
// up to 128: one CTA per 128-row query block of one (batch, head), 64-key tiles, one softmax warpgroup.
//
//   warps 0-3   softmax + epilogue: one S row per thread out of TMEM (two 64-column S buffers, so Q K^T of the
//               next key tile runs under this one's softmax), mask, row max, exp2, row sum, P as 16-bit into
//               shared memory (K-major swizzled A operand of P V), lazy rescale of O in TMEM; at the end
//               O / l and LSE straight to global memory
//   warp 4      loader: TMA of Q (up to four 64-column atoms) and of the K/V ring (four 32 KB slots) in the
//               order K(0) K(1) V(0) K(2) V(1) ...; leaves last, after every commit on its barriers has landed
//   warp 5      MMA issuer: S = Q K^T (M 128, N 64, head dim / 16 steps), O += P V (M 128, N = the padded head
//               dim, 4 steps of 16 keys, V as an MN-major operand)
//   warp 6      fixer, packed batches only: clears the rows of a V tile that lie past the end of the sequence
//               (they belong to the next sequence; P is exactly zero there but 0 x NaN is NaN), as the reference
//               zero-fills them while staging (flash-attn2-rs/src/device/forward/mod.rs:171-175,200)
//
// Conventions as in the kernel for the smaller head dims: bottom-right aligned masks, fully masked rows give
// O = 0 and LSE = +inf, natural-log LSE, kv_head = head / group; every wait is bounded.
#include "sm100_ptx.cuh"
#include "fa2_params.h"
#include "fa2_launch.h"

namespace fa2 {

namespace {

constexpr int kWM = 128;        // query rows per CTA
constexpr int kWN = 64;         // keys per tile
constexpr int kWThreads = 256;
constexpr int kWLoadWarp = 4;
constexpr int kWMmaWarp = 5;
constexpr int kWFixWarp = 6;
constexpr int kWSlots = 4;      // K/V ring depth
constexpr float kWRescaleThreshold = 8.0f;  // log2 domain

struct WideCfg {
  static constexpr int kAtomQ = kWM * 128;    // bytes of one 64-column atom of Q (and of P)
  static constexpr int kAtomKV = kWN * 128;   // bytes of one 64-column atom of a K or V tile
  static constexpr int kMaxAtoms = 4;
  static constexpr int kQOff = 0;
  static constexpr int kKVTile = kMaxAtoms * kAtomKV;
  static constexpr int kKVOff = kMaxAtoms * kAtomQ;
  static constexpr int kPOff = kKVOff + kWSlots * kKVTile;
  static constexpr int kBarOff = kPOff + kAtomQ;
  static constexpr int kNumBars = 3 * kWSlots + 7;
  static constexpr int kMiscOff = (kBarOff + kNumBars * 8 + 15) / 16 * 16;
  static constexpr int kSmemBytes = kMiscOff + 32;
  static constexpr uint32_t kTmemS = 0, kTmemO = 128;  // S buffers at columns 0 and 64
};

struct WTile {
  int b, h, hk;
  int m0;              // first query row of the block (within the sequence)
  int sq, sk;
  int q_row0, k_row0;  // row offsets of the sequence inside the packed tensors (0 when dense)
  int bq;              // batch coordinate for TMA (0 when packed)
  int off;             // sk - sq (bottom-right alignment)
  int nb, ne;          // key-tile range; nb == ne means no key is visible
  bool valid;
};

// Blocks are listed longest first (last query block of every head first, for causal masks).
__device__ __forceinline__ WTile get_wtile(const FwdParams& p, int t) {
  WTile ti;
  const int num_mblk = (p.seqlen_q + kWM - 1) / kWM;
  const int bh = p.batch * p.heads;
  const int mrev = t / bh;
  const int rem = t - mrev * bh;
  ti.b = rem / p.heads;
  ti.h = rem - ti.b * p.heads;
  ti.hk = ti.h / p.group;
  ti.m0 = (num_mblk - 1 - mrev) * kWM;
  if (p.cu_q != nullptr) {
    ti.q_row0 = p.cu_q[ti.b];
    ti.sq = p.cu_q[ti.b + 1] - ti.q_row0;
    ti.k_row0 = p.cu_k[ti.b];
    ti.sk = p.cu_k[ti.b + 1] - ti.k_row0;
    ti.bq = 0;
    // Inconsistent metadata is skipped, as the reference kernel does.
    if (ti.sq < 0 || ti.sk < 0 || ti.sq > p.seqlen_q || ti.sk > p.seqlen_k || ti.q_row0 < 0 || ti.k_row0 < 0) ti.sq = 0;
  } else {
    ti.q_row0 = 0;
    ti.k_row0 = 0;
    ti.sq = p.seqlen_q;
    ti.sk = p.seqlen_k;
    ti.bq = ti.b;
  }
  ti.off = ti.sk - ti.sq;
  ti.valid = ti.m0 < ti.sq;
  ti.nb = 0;
  ti.ne = 0;
  if (ti.valid) {
    const int r_hi = min(ti.m0 + kWM - 1, ti.sq - 1);
    int hi_col = ti.sk;
    if (p.window_right >= 0) hi_col = min(ti.sk, r_hi + ti.off + p.window_right + 1);
    int lo_col = 0;
    if (p.window_left >= 0) lo_col = max(0, ti.m0 + ti.off - p.window_left);
    if (hi_col > lo_col) {
      ti.nb = lo_col / kWN;
      ti.ne = (hi_col + kWN - 1) / kWN;
    }
  }
  return ti;
}

// First row of key tile j that lies past the end of a packed sequence (kWN = none). Dense tensors need
// nothing: the TMA unit fills rows past the tensor with zeros.
template <bool PACKED>
__device__ __forceinline__ int wide_ragged_row(int sk, int j) {
  if (!PACKED) return kWN;
  const int left = sk - j * kWN;
  return left < kWN ? max(left, 0) : kWN;
}

__device__ __forceinline__ float wide_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ATOMS: 64-column atoms of the head dim that are loaded (3 for head dims up to 192, else 4). TMA fills what lies
// past the real head dim inside them with zeros, so Q K^T runs over ATOMS * 64 columns with compile-time operand
// offsets: a runtime bound in the issuing thread's loop doubles the cost of an MMA issue.
// FANCY (softcap or ALiBi in use) and PACKED (cu_seqlens batches) are compile-time: the plain dense kernel carries
// none of their code, which keeps its loops within reach of the SM's instruction cache.
template <bool BF16, int ATOMS, bool FANCY, bool PACKED>
__global__ void __launch_bounds__(kWThreads, 1) fwd_wide_kernel(const __grid_constant__ FwdParams p) {
  using Cfg = WideCfg;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0u) {
    // 128-byte swizzled tiles need a 1024-byte aligned base; report instead of computing garbage.
    if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, kWaitNone + 1);
    return;
  }
  uint8_t* s_q = smem + Cfg::kQOff;
  uint8_t* s_kv = smem + Cfg::kKVOff;
  uint8_t* s_p = smem + Cfg::kPOff;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kBarOff);
  uint64_t* kv_full = bars;
  uint64_t* kv_empty = bars + kWSlots;
  uint64_t* kv_fixed = bars + 2 * kWSlots;
  uint64_t* q_full = bars + 3 * kWSlots;
  uint64_t* s_full = q_full + 1;   // [2]
  uint64_t* s_free = q_full + 3;   // [2] the scores have been read out of TMEM
  uint64_t* p_full = q_full + 5;   // P of this key tile is in shared memory (and O has been rescaled)
  uint64_t* pv_done = q_full + 6;  // P V of this key tile has completed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Cfg::kMiscOff + 8);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const WaitCtl ctl{abort_flag, p.status};
  const WTile ti = get_wtile(p, blockIdx.x);
  if (!ti.valid) return;
  constexpr int atoms = ATOMS;
  constexpr int n_cols = atoms * 64;         // columns of O in TMEM
  const int n_tiles = ti.ne - ti.nb;

  if (n_tiles == 0) {
    // No key is visible to this block: O = 0, LSE = +inf.
    if (tid < kWM && ti.m0 + tid < ti.sq) {
      const int row = ti.m0 + tid;
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.o_ptr) + ti.bq * p.o_batch_stride +
                       static_cast<int64_t>(ti.q_row0 + row) * p.o_row_stride + ti.h * p.o_head_stride;
      for (int c = 0; c * 8 < p.head_dim; ++c) *reinterpret_cast<uint4*>(orow + c * 8) = make_uint4(0, 0, 0, 0);
      p.lse_ptr[ti.bq * p.lse_batch_stride + ti.h * p.lse_head_stride + ti.q_row0 + row] = INFINITY;
    }
    return;
  }

  if (tid == 0) {
    *abort_flag = 0;
    for (int i = 0; i < kWSlots; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&kv_fixed[i], 1);
    }
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_free[s], kWM);
    }
    mbar_init(p_full, kWM);
    mbar_init(pv_done, 1);
    mbar_fence_init();
  }
  if (warp == kWMmaWarp) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (warp == kWLoadWarp && lane == 0) {
    tma_prefetch_desc(&p.tm_q);
    tma_prefetch_desc(&p.tm_k);
    tma_prefetch_desc(&p.tm_v);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp < 4) {
    // ------------------------------------------------------------------ softmax + epilogue
    const int row_in = tid;
    const int row = ti.m0 + row_in;
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t t_s = tmem + lane_addr + Cfg::kTmemS;
    const uint32_t t_o = tmem + lane_addr + Cfg::kTmemO;
    // P as the K-major, 128-byte swizzled A operand of P V: key chunk c (8 keys, 16 bytes) of row r sits at
    // byte 128 r + 16 (c ^ (r % 8)) of the single atom.
    uint8_t* p_row = s_p + row_in * 128;
    const int p_swz = row_in & 7;
    float m = -INFINITY, l = 0.f;
    float slope = 0.f;
    if (p.alibi != nullptr) slope = p.alibi[ti.b * p.alibi_batch_stride + ti.h] * 1.4426950408889634f;
    const float inv_cap = (p.softcap > 0.f) ? p.scale / p.softcap : 0.f;
    const float cap_l2 = p.softcap * 1.4426950408889634f;
    constexpr bool fancy = FANCY;
    bool ok = true;
    for (int i = 0; i < n_tiles; ++i) {
      const int j = ti.nb + i;
      const int buf = i & 1;
      if (!warp_wait(&s_full[buf], (i >> 1) & 1, ctl, kWaitSoftmaxSFull)) { ok = false; break; }
      tc_fence_after();
      uint32_t sr[kWN];
      tmem_ld32(t_s + buf * kWN, sr);
      tmem_ld32(t_s + buf * kWN + 32, sr + 32);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(&s_free[buf]);  // the scores live in registers from here on
      const int col0 = j * kWN;
      // Scores into the log2 domain: scale (or softcap), ALiBi, then the mask.
      if (fancy) {
#pragma unroll
        for (int c = 0; c < kWN; ++c) {
          float x = __uint_as_float(sr[c]);
          x = (p.softcap > 0.f) ? cap_l2 * wide_tanh(x * inv_cap) : x * p.scale_log2;
          if (p.alibi != nullptr) {
            const int col = col0 + c;
            x += p.causal_alibi ? slope * static_cast<float>(col) : -slope * fabsf(static_cast<float>(row + ti.off - col));
          }
          sr[c] = __float_as_uint(x);
        }
      } else {
#pragma unroll
        for (int c = 0; c < kWN; ++c) sr[c] = __float_as_uint(__uint_as_float(sr[c]) * p.scale_log2);
      }
      {
        int hi = ti.sk;
        if (p.window_right >= 0) hi = min(hi, row + ti.off + p.window_right + 1);
        int lo = 0;
        if (p.window_left >= 0) lo = row + ti.off - p.window_left;
        hi -= col0;
        lo -= col0;
        if (lo > 0 || hi < kWN) {
#pragma unroll
          for (int c = 0; c < kWN; ++c)
            if (c < lo || c >= hi) sr[c] = __float_as_uint(-INFINITY);
        }
      }
      float mx0 = __uint_as_float(sr[0]), mx1 = __uint_as_float(sr[1]);
      float mx2 = __uint_as_float(sr[2]), mx3 = __uint_as_float(sr[3]);
#pragma unroll
      for (int c = 4; c < kWN; c += 4) {
        mx0 = fmaxf(mx0, __uint_as_float(sr[c]));
        mx1 = fmaxf(mx1, __uint_as_float(sr[c + 1]));
        mx2 = fmaxf(mx2, __uint_as_float(sr[c + 2]));
        mx3 = fmaxf(mx3, __uint_as_float(sr[c + 3]));
      }
      const float m_new = fmaxf(m, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)));
      // Keep the stale max unless it grew by more than 2^8: the final O / l is exact either way.
      const bool grow = (m_new - m) > kWRescaleThreshold;
      float alpha = 1.f;
      if (grow) {
        alpha = ex2(m - m_new);  // m = -inf gives 0
        m = m_new;
        l *= alpha;
      }
      // A row that has seen no key yet has m = -inf and only -inf scores: keep x = -inf (not NaN).
      const float neg_m = (m == -INFINITY) ? 0.f : -m;
      float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
#pragma unroll
      for (int c = 0; c < kWN; c += 4) {
        const float p0 = ex2(__uint_as_float(sr[c]) + neg_m);
        const float p1 = ex2(__uint_as_float(sr[c + 1]) + neg_m);
        const float p2 = ex2(__uint_as_float(sr[c + 2]) + neg_m);
        const float p3 = ex2(__uint_as_float(sr[c + 3]) + neg_m);
        l0 += p0;
        l1 += p1;
        l2 += p2;
        l3 += p3;
        sr[c / 2] = pack2<BF16>(p0, p1);
        sr[c / 2 + 1] = pack2<BF16>(p2, p3);
      }
      l += (l0 + l1) + (l2 + l3);
      // P V of the previous key tile has to be complete: it reads the P buffer that is overwritten next, and
      // it is the only operation that touches O.
      bool waited = true;
      if (i > 0) waited = mbar_wait(pv_done, (i - 1) & 1, ctl, kWaitSoftmaxPvDone);
      // One warp reduction reconverges the lanes after the wait and carries both warp-uniform decisions.
      const unsigned votes = __reduce_or_sync(0xffffffffu, (grow ? 1u : 0u) | (waited ? 0u : 2u));
      if (votes & 2u) { ok = false; break; }
      if (i > 0 && (votes & 1u)) {
        tc_fence_after();
        for (int c = 0; c < n_cols / 16; ++c) {
          uint32_t orr[16];
          tmem_ld16(t_o + c * 16, orr);
          tmem_wait_ld();
#pragma unroll
          for (int q = 0; q < 16; ++q) orr[q] = __float_as_uint(__uint_as_float(orr[q]) * alpha);
          tmem_st16(t_o + c * 16, orr);
        }
        // The rescaled O must be in TMEM before p_full lets the next P V accumulate onto it.
        tmem_wait_st();
        tc_fence_before();
      }
#pragma unroll
      for (int c = 0; c < kWN / 8; ++c)
        *reinterpret_cast<uint4*>(p_row + ((c ^ p_swz) << 4)) = make_uint4(sr[4 * c], sr[4 * c + 1], sr[4 * c + 2], sr[4 * c + 3]);
      fence_proxy_async_smem();
      mbar_arrive(p_full);
    }
    if (ok && warp_wait(pv_done, (n_tiles - 1) & 1, ctl, kWaitEpiPvDone)) {
      // ---- epilogue: O / l -> 16-bit -> global memory, 32 columns at a time; LSE = (m + log2 l) ln 2
      tc_fence_after();
      const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.o_ptr) + ti.bq * p.o_batch_stride +
                       static_cast<int64_t>(ti.q_row0 + row) * p.o_row_stride + ti.h * p.o_head_stride;
      for (int c = 0; c < n_cols / 32; ++c) {
        uint32_t orr[32];
        tmem_ld32(t_o + c * 32, orr);
        tmem_wait_ld();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 w;
          w.x = pack2<BF16>(__uint_as_float(orr[8 * q]) * inv_l, __uint_as_float(orr[8 * q + 1]) * inv_l);
          w.y = pack2<BF16>(__uint_as_float(orr[8 * q + 2]) * inv_l, __uint_as_float(orr[8 * q + 3]) * inv_l);
          w.z = pack2<BF16>(__uint_as_float(orr[8 * q + 4]) * inv_l, __uint_as_float(orr[8 * q + 5]) * inv_l);
          w.w = pack2<BF16>(__uint_as_float(orr[8 * q + 6]) * inv_l, __uint_as_float(orr[8 * q + 7]) * inv_l);
          const int col = c * 32 + q * 8;
          if (row < ti.sq && col < p.head_dim) *reinterpret_cast<uint4*>(orow + col) = w;
        }
      }
      tc_fence_before();
      if (row < ti.sq) {
        const float lse = (l > 0.f) ? (m + lg2(l)) * 0.6931471805599453f : INFINITY;
        p.lse_ptr[ti.bq * p.lse_batch_stride + ti.h * p.lse_head_stride + ti.q_row0 + row] = lse;
      }
    }
    __syncwarp();
  } else if (warp == kWLoadWarp) {
    if (elect_one()) {
      // ---------------------------------------------------------------- loader
      uint32_t slot = 0, ring_phase = 0;
      bool ok = true;
      auto load_kv = [&](const CUtensorMap* tm, int row) -> bool {
        if (!mbar_wait(&kv_empty[slot], ring_phase ^ 1, ctl, kWaitLoadKVEmpty)) return false;
        mbar_expect_tx(&kv_full[slot], atoms * Cfg::kAtomKV);
        uint8_t* dst = s_kv + slot * Cfg::kKVTile;
        for (int a = 0; a < atoms; ++a) tma_load_4d(dst + a * Cfg::kAtomKV, tm, &kv_full[slot], a * 64, ti.hk, row, ti.bq);
        if (++slot == kWSlots) {
          slot = 0;
          ring_phase ^= 1;
        }
        return true;
      };
      mbar_expect_tx(q_full, atoms * Cfg::kAtomQ);
      for (int a = 0; a < atoms; ++a)
        tma_load_4d(s_q + a * Cfg::kAtomQ, &p.tm_q, q_full, a * 64, ti.h, ti.q_row0 + ti.m0, ti.bq);
      // Ring order K(nb), K(nb+1), V(nb), K(nb+2), V(nb+1), ...: Q K^T runs one key tile ahead of P V.
      ok = load_kv(&p.tm_k, ti.k_row0 + ti.nb * kWN);
      for (int j = ti.nb; j < ti.ne && ok; ++j) {
        if (j + 1 < ti.ne) ok = load_kv(&p.tm_k, ti.k_row0 + (j + 1) * kWN);
        if (ok) ok = load_kv(&p.tm_v, ti.k_row0 + j * kWN);
      }
      // The loader leaves last: it waits until the issuer's commits on every ring slot have landed, so that no
      // asynchronous arrival is still on its way when the CTA gives back its shared memory. A slot that was
      // never used passes at once.
      for (int i = 0; i < kWSlots && ok; ++i) {
        ok = mbar_wait(&kv_empty[slot], ring_phase ^ 1, ctl, kWaitLoadKVEmpty);
        if (++slot == kWSlots) {
          slot = 0;
          ring_phase ^= 1;
        }
      }
    }
  } else if (warp == kWFixWarp) {
    // ---------------------------------------------------------------- fixer (packed batches)
    // Walks the ring in the loader's order and waits for every tile, which keeps it within one ring pass of
    // the issuer; it acts on V tiles that reach past the end of their sequence.
    if (PACKED) {
      uint32_t slot = 0, ring_phase = 0;
      bool ok = true;
      auto step = [&](int first_stray) -> bool {
        if (!__all_sync(0xffffffffu, mbar_wait(&kv_full[slot], ring_phase, ctl, kWaitMmaKVFull))) return false;
        if (first_stray < kWN) {
          uint8_t* tile = s_kv + slot * Cfg::kKVTile;
          // 8 lanes clear one 128-byte row of an atom (the swizzle only permutes 16-byte chunks inside it)
          for (int r = first_stray + (lane >> 3); r < kWN; r += 4)
            for (int a = 0; a < atoms; ++a)
              *reinterpret_cast<uint4*>(tile + a * Cfg::kAtomKV + r * 128 + (lane & 7) * 16) = make_uint4(0, 0, 0, 0);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&kv_fixed[slot]);
          __syncwarp();
        }
        if (++slot == kWSlots) {
          slot = 0;
          ring_phase ^= 1;
        }
        return true;
      };
      ok = step(kWN);
      for (int j = ti.nb; j < ti.ne && ok; ++j) {
        if (j + 1 < ti.ne) ok = step(kWN);
        if (ok) ok = step(wide_ragged_row<PACKED>(ti.sk, j));
      }
    }
  } else if (warp == kWMmaWarp && elect_one()) {
    // ---------------------------------------------------------------- mma issuer
    const uint32_t fmt = BF16 ? 1u : 0u;
    const uint32_t idesc_qk = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(kWN >> 3) << 17) |
                              (static_cast<uint32_t>(kWM >> 4) << 24);
    const uint32_t idesc_pv = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) |
                              (static_cast<uint32_t>(n_cols >> 3) << 17) | (static_cast<uint32_t>(kWM >> 4) << 24);
    constexpr uint32_t kTile16 = Cfg::kKVTile >> 4;
    constexpr uint32_t kAtomQ16 = Cfg::kAtomQ >> 4;
    constexpr uint32_t kAtomKV16 = Cfg::kAtomKV >> 4;
    const uint64_t q_desc = make_smem_desc(smem_u32(s_q), 16, 1024);               // K-major A
    const uint64_t k_desc = make_smem_desc(smem_u32(s_kv), 16, 1024);              // K-major B
    const uint64_t v_desc = make_smem_desc(smem_u32(s_kv), Cfg::kAtomKV, 1024);    // MN-major B
    const uint64_t p_desc = make_smem_desc(smem_u32(s_p), 16, 1024);               // K-major A
    constexpr int n_ks = ATOMS * 4;  // steps of 16 over the loaded columns
    const uint32_t t_s = tmem + Cfg::kTmemS;
    const uint32_t t_o = tmem + Cfg::kTmemO;
    uint32_t slot = 0, ring_phase = 0;
    uint32_t fix_par = 0;  // bit i: parity of the next kv_fixed phase of slot i
    bool ok = true;
    auto advance = [&]() {
      mma_commit(&kv_empty[slot]);
      if (++slot == kWSlots) {
        slot = 0;
        ring_phase ^= 1;
      }
    };
    // S_buf = Q K_i^T; the S buffer is free as soon as the softmax warps hold its previous scores in registers.
    auto do_k = [&](const int i) -> bool {
      if (!mbar_wait(&kv_full[slot], ring_phase, ctl, kWaitMmaKVFull)) return false;
      if (i == 0 && !mbar_wait(q_full, 0, ctl, kWaitMmaQFull)) return false;
      const int buf = i & 1;
      if (!mbar_wait(&s_free[buf], ((i >> 1) & 1) ^ 1, ctl, kWaitMmaSFree)) return false;
      tc_fence_after();
      const uint64_t b = k_desc + slot * kTile16;
      // Compile-time operand offsets: a rolled loop that builds descriptors costs the issuing thread about twice
      // the 54 cycles such an MMA takes.
      const uint32_t d_s = t_s + buf * kWN;
      static_for<n_ks>([&](auto ks) {
        constexpr uint32_t in_atom = (ks.value & 3) * 2;
        mma_ss_o<(ks.value >> 2) * kAtomQ16 + in_atom, (ks.value >> 2) * kAtomKV16 + in_atom>(d_s, q_desc, b, idesc_qk,
                                                                                           ks.value > 0 ? 1u : 0u);
      });
      mma_commit(&s_full[buf]);
      advance();
      return true;
    };
    // O (+)= P V_i: per step of 16 keys, 32 bytes of a P row inside its atom and 16 rows of 128 bytes of V.
    auto do_v = [&](const int i) -> bool {
      if (!mbar_wait(&kv_full[slot], ring_phase, ctl, kWaitMmaKVFull)) return false;
      if (wide_ragged_row<PACKED>(ti.sk, ti.nb + i) < kWN) {
        // A V tile that reaches past its sequence is usable once the fixer has cleared the stray rows.
        if (!mbar_wait(&kv_fixed[slot], (fix_par >> slot) & 1, ctl, kWaitMmaKVFull)) return false;
        fix_par ^= 1u << slot;
      }
      if (!mbar_wait(p_full, i & 1, ctl, kWaitMmaPFull)) return false;
      tc_fence_after();
      const uint64_t b = v_desc + slot * kTile16;
      static_for<kWN / 16>([&](auto ks) {
        mma_ss_o<ks.value * 2, ks.value * (2048 >> 4)>(t_o, p_desc, b, idesc_pv, (i == 0 && ks.value == 0) ? 0u : 1u);
      });
      mma_commit(pv_done);
      advance();
      return true;
    };
    ok = do_k(0);
    for (int i = 0; i < n_tiles && ok; ++i) {
      if (i + 1 < n_tiles) ok = do_k(i + 1);
      if (ok) ok = do_v(i);
    }
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
  if (warp == kWMmaWarp) tmem_dealloc(tmem, 512);
}

template <bool BF16, int ATOMS, bool FANCY, bool PACKED>
cudaError_t launch_wide(const FwdParams& p, cudaStream_t stream) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(fwd_wide_kernel<BF16, ATOMS, FANCY, PACKED>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, WideCfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int64_t blocks = static_cast<int64_t>((p.seqlen_q + kWM - 1) / kWM) * p.batch * p.heads;
  if (blocks <= 0) return cudaSuccess;
  if (blocks > 0x7fffffffLL) return cudaErrorInvalidValue;
  fwd_wide_kernel<BF16, ATOMS, FANCY, PACKED>
      <<<static_cast<unsigned>(blocks), kWThreads, WideCfg::kSmemBytes, stream>>>(p);
  return cudaGetLastError();
}

template <bool BF16, int ATOMS>
cudaError_t pick_features(const FwdParams& p, cudaStream_t stream) {
  const bool fancy = (p.softcap > 0.f) || (p.alibi != nullptr);
  const bool packed = p.cu_q != nullptr;
  if (fancy) {
    return packed ? launch_wide<BF16, ATOMS, true, true>(p, stream) : launch_wide<BF16, ATOMS, true, false>(p, stream);
  }
  return packed ? launch_wide<BF16, ATOMS, false, true>(p, stream) : launch_wide<BF16, ATOMS, false, false>(p, stream);
}

}  // namespace

cudaError_t launch_fwd_wide(const FwdParams& p, int head_dim, bool bf16, cudaStream_t stream) {
  if (head_dim <= 128 || head_dim > 256 || head_dim % 8 != 0) return cudaErrorInvalidValue;
  if (head_dim <= 192) return bf16 ? pick_features<true, 3>(p, stream) : pick_features<false, 3>(p, stream);
  return bf16 ? pick_features<true, 4>(p, stream) : pick_features<false, 4>(p, stream);
}

}  // namespace fa2
