// FlashAttention-2 forward for sm_100a (B200).
//
// One persistent CTA per SM walks a longest-first list of work tiles. A work tile is 256 query
// rows of one (batch, head): two 128-row "stages" that ping-pong so the tensor core always has
// one stage's MMA to run while the other stage's softmax is in flight.
//
//   warp 13      loader   : TMA (cp.async.bulk.tensor, 128B swizzle) Q stages + K/V ring
//   warp 12      mma      : one thread issues tcgen05.mma; S = Q K^T (smem x smem) into TMEM,
//                           O += P V (P read from TMEM, V from smem as an MN-major operand)
//   warps 0-3    softmax of stage 0: tcgen05.ld S row -> mask, row max, exp2, row sum ->
//   warps 4-7    softmax of stage 1: bf16/fp16 P written back over S in TMEM (tcgen05.st);
//                           rescales O in TMEM only when the row max grew by more than 2^8
//   warps 8-11   epilogue : O / l -> 16-bit -> swizzled smem -> TMA store (or predicated
//                           stores on ragged packed tiles), LSE = (m + log2 l) ln 2
//
// Replaces the reference kernels flash_attn_fwd / varlen_fwd
// (flash-attn2-rs/src/device/forward/dense.rs:472-590, forward/mod.rs:1162-1407,
//  varlen/mod.rs:30-318,445-578) and keeps their conventions: bottom-right aligned masks,
// fully masked rows give O = 0 and LSE = +inf, natural-log LSE, kv_head = head / group.
#include "sm100_ptx.cuh"
#include "fa2_params.h"
#include "fa2_launch.h"

namespace fa2 {

namespace {

constexpr int kBlockM = 128;
constexpr int kBlockN = 128;
constexpr int kThreads = 512;
constexpr int kSoftmaxRegs = 192;
constexpr int kEpilogueRegs = 64;
constexpr int kOtherRegs = 64;
constexpr float kRescaleThreshold = 8.0f;  // log2 domain

template <int D>
struct FwdCfg {
  static constexpr int kAtoms = D / 64;                    // 128-byte swizzle atoms along D
  static constexpr int kTileBytes = kBlockN * D * 2;       // one Q stage / K / V tile
  static constexpr int kSlots = (D == 128) ? 4 : 6;        // K/V ring depth
  static constexpr int kQOff = 0;
  static constexpr int kKVOff = 2 * kTileBytes;
  static constexpr int kBarOff = kKVOff + kSlots * kTileBytes;
  static constexpr int kNumBars = 2 * kSlots + 16;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;  // tmem slot, abort flag
  static constexpr int kStatOff = kMiscOff + 32;           // l and m exchange: [2 stages][128][2]
  static constexpr int kSmemBytes = kStatOff + 2 * 128 * 2 * 4 + 1024;  // + alignment slack
  static constexpr uint32_t kTmemS0 = 0, kTmemS1 = 128, kTmemO0 = 256, kTmemO1 = 256 + D;
};

struct Tile {
  int b, h, hk;
  int m0;              // first query row of the 256-row block (within the sequence)
  int sq, sk;          // lengths of this sequence
  int q_row0, k_row0;  // row offsets of the sequence inside the packed tensors (0 when dense)
  int bq;              // batch coordinate for TMA (0 when packed)
  int off;             // sk - sq (bottom-right alignment)
  int nb[2], ne[2];    // key-tile range per stage; nb == ne means no work
  int jlo, jhi;
  bool valid;
};

__device__ __forceinline__ Tile get_tile(const FwdParams& p, int t) {
  Tile ti;
  const int bh = p.batch * p.heads;
  const int mrev = t / bh;
  const int rem = t - mrev * bh;
  ti.b = rem / p.heads;
  ti.h = rem - ti.b * p.heads;
  ti.hk = ti.h / p.group;
  ti.m0 = (p.num_mblk - 1 - mrev) * (2 * kBlockM);
  if (p.cu_q != nullptr) {
    ti.q_row0 = p.cu_q[ti.b];
    ti.sq = p.cu_q[ti.b + 1] - ti.q_row0;
    ti.k_row0 = p.cu_k[ti.b];
    ti.sk = p.cu_k[ti.b + 1] - ti.k_row0;
    ti.bq = 0;
    // Inconsistent metadata is skipped, as the reference kernel does.
    if (ti.sq < 0 || ti.sk < 0 || ti.sq > p.seqlen_q || ti.sk > p.seqlen_k) ti.sq = 0;
  } else {
    ti.q_row0 = 0;
    ti.k_row0 = 0;
    ti.sq = p.seqlen_q;
    ti.sk = p.seqlen_k;
    ti.bq = ti.b;
  }
  ti.off = ti.sk - ti.sq;
  ti.valid = ti.m0 < ti.sq;
  ti.jlo = 0x7fffffff;
  ti.jhi = 0;
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    const int r_lo = ti.m0 + s * kBlockM;
    int nb = 0, ne = 0;
    if (r_lo < ti.sq) {
      const int r_hi = min(r_lo + kBlockM - 1, ti.sq - 1);
      int hi_col = ti.sk;
      if (p.window_right >= 0) hi_col = min(ti.sk, r_hi + ti.off + p.window_right + 1);
      int lo_col = 0;
      if (p.window_left >= 0) lo_col = max(0, r_lo + ti.off - p.window_left);
      if (hi_col > lo_col) {
        nb = lo_col / kBlockN;
        ne = (hi_col + kBlockN - 1) / kBlockN;
      }
    }
    ti.nb[s] = nb;
    ti.ne[s] = ne;
    if (ne > nb) {
      ti.jlo = min(ti.jlo, nb);
      ti.jhi = max(ti.jhi, ne);
    }
  }
  if (ti.jhi == 0) ti.jlo = 0;
  return ti;
}

__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D, bool BF16>
__global__ void __launch_bounds__(kThreads, 1) fwd_kernel(const __grid_constant__ FwdParams p) {
  using Cfg = FwdCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_q = smem + Cfg::kQOff;
  uint8_t* s_kv = smem + Cfg::kKVOff;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kBarOff);
  uint64_t* kv_full = bars;
  uint64_t* kv_empty = bars + Cfg::kSlots;
  uint64_t* q_full = bars + 2 * Cfg::kSlots;  // [2]
  uint64_t* q_empty = q_full + 2;
  uint64_t* s_full = q_full + 4;
  uint64_t* p_full = q_full + 6;
  uint64_t* pv_done = q_full + 8;
  uint64_t* sm_final = q_full + 10;
  uint64_t* o_free = q_full + 12;
  uint64_t* epi_full = q_full + 14;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Cfg::kMiscOff + 8);
  float* s_stat = reinterpret_cast<float*>(smem + Cfg::kStatOff);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const WaitCtl ctl{abort_flag, p.status};

  if (tid == 0) {
    *abort_flag = 0;
    for (int i = 0; i < Cfg::kSlots; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], kBlockM);
      mbar_init(&pv_done[s], 1);
      mbar_init(&sm_final[s], kBlockM);
      mbar_init(&o_free[s], kBlockM);
      mbar_init(&epi_full[s], kBlockM);
    }
    mbar_fence_init();
  }
  if (warp == 12) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (warp == 13 && lane == 0) {
    tma_prefetch_desc(&p.tm_q);
    tma_prefetch_desc(&p.tm_k);
    tma_prefetch_desc(&p.tm_v);
    tma_prefetch_desc(&p.tm_o);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp < 8) {
    // ------------------------------------------------------------------ softmax
    reg_alloc<kSoftmaxRegs>();
    const int s = warp >> 2;
    const int row_in = tid & 127;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem + lane_addr + (s == 0 ? Cfg::kTmemS0 : Cfg::kTmemS1);
    const uint32_t t_o = tmem + lane_addr + (s == 0 ? Cfg::kTmemO0 : Cfg::kTmemO1);
    const bool fancy = (p.softcap > 0.f) || (p.alibi != nullptr) || (p.scale_log2 < 0.f);
    uint32_t n_sfull = 0, n_pv = 0, n_tile = 0;
    for (int t = blockIdx.x; t < p.num_tiles; t += gridDim.x) {
      const Tile ti = get_tile(p, t);
      if (!ti.valid) continue;
      const int row = ti.m0 + s * kBlockM + row_in;
      const int nb_s = s ? ti.nb[1] : ti.nb[0];
      const int ne_s = s ? ti.ne[1] : ti.ne[0];
      float m = -INFINITY, l = 0.f;
      float slope = 0.f;
      if (p.alibi != nullptr) slope = p.alibi[ti.b * p.alibi_batch_stride + ti.h] * 1.4426950408889634f;
      bool ok = true;
      for (int j = nb_s; j < ne_s; ++j) {
        if (!mbar_wait(&s_full[s], n_sfull & 1, ctl, kWaitSoftmaxSFull)) { ok = false; break; }
        ++n_sfull;
        tc_fence_after();
        uint32_t sr[kBlockN];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(t_s + c * 32, sr + c * 32);
        tmem_wait_ld();
        float cs = p.scale_log2;
        const int col0 = j * kBlockN;
        if (fancy) {
          // Scores leave this block already in the log2 domain.
          const float inv_cap = (p.softcap > 0.f) ? p.scale / p.softcap : 0.f;
          const float cap_l2 = p.softcap * 1.4426950408889634f;
#pragma unroll
          for (int i = 0; i < kBlockN; ++i) {
            float x = __uint_as_float(sr[i]);
            x = (p.softcap > 0.f) ? cap_l2 * tanh_approx(x * inv_cap) : x * p.scale_log2;
            if (p.alibi != nullptr) {
              const int col = col0 + i;
              x += p.causal_alibi ? slope * static_cast<float>(col)
                                  : -slope * fabsf(static_cast<float>(row + ti.off - col));
            }
            sr[i] = __float_as_uint(x);
          }
          cs = 1.f;
        }
        // Mask only tiles that touch a boundary (warp-uniform test on the stage's row range).
        const int r_lo = ti.m0 + s * kBlockM;
        const int r_hi = r_lo + kBlockM - 1;
        bool need_mask = (col0 + kBlockN > ti.sk);
        if (p.window_right >= 0) need_mask |= (col0 + kBlockN - 1 > r_lo + ti.off + p.window_right);
        if (p.window_left >= 0) need_mask |= (col0 < r_hi + ti.off - p.window_left);
        if (need_mask) {
          int hi = ti.sk;
          if (p.window_right >= 0) hi = min(hi, row + ti.off + p.window_right + 1);
          int lo = 0;
          if (p.window_left >= 0) lo = row + ti.off - p.window_left;
          hi -= col0;
          lo -= col0;
#pragma unroll
          for (int i = 0; i < kBlockN; ++i)
            if (i < lo || i >= hi) sr[i] = __float_as_uint(-INFINITY);
        }
        float mx0 = __uint_as_float(sr[0]), mx1 = __uint_as_float(sr[1]);
        float mx2 = __uint_as_float(sr[2]), mx3 = __uint_as_float(sr[3]);
#pragma unroll
        for (int i = 4; i < kBlockN; i += 4) {
          mx0 = fmaxf(mx0, __uint_as_float(sr[i]));
          mx1 = fmaxf(mx1, __uint_as_float(sr[i + 1]));
          mx2 = fmaxf(mx2, __uint_as_float(sr[i + 2]));
          mx3 = fmaxf(mx3, __uint_as_float(sr[i + 3]));
        }
        const float m_tile = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * cs;
        const float m_new = fmaxf(m, m_tile);
        // Keep the stale max unless it grew by more than 2^8: the final O / l is exact either way.
        const bool grow = (m_new - m) > kRescaleThreshold;
        float alpha = 1.f;
        if (grow) {
          alpha = ex2(m - m_new);  // m = -inf gives 0
          m = m_new;
          l *= alpha;
        }
        if (j > nb_s && __any_sync(0xffffffffu, grow)) {
          // O of this stage is only touched by PV(j-1), which has to be complete.
          if (!mbar_wait(&pv_done[s], (n_pv - 1) & 1, ctl, kWaitSoftmaxPvDone)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < D / 16; ++c) {
            uint32_t orr[16];
            tmem_ld16(t_o + c * 16, orr);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
            tmem_st16(t_o + c * 16, orr);
          }
        }
        const float neg_m = (m == -INFINITY) ? 0.f : -m;
        float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
#pragma unroll
        for (int i = 0; i < kBlockN; i += 4) {
          const float p0 = ex2(fmaf(__uint_as_float(sr[i]), cs, neg_m));
          const float p1 = ex2(fmaf(__uint_as_float(sr[i + 1]), cs, neg_m));
          const float p2 = ex2(fmaf(__uint_as_float(sr[i + 2]), cs, neg_m));
          const float p3 = ex2(fmaf(__uint_as_float(sr[i + 3]), cs, neg_m));
          l0 += p0;
          l1 += p1;
          l2 += p2;
          l3 += p3;
          sr[i / 2] = pack2<BF16>(p0, p1);
          sr[i / 2 + 1] = pack2<BF16>(p2, p3);
        }
        l += (l0 + l1) + (l2 + l3);
        tmem_st32(t_s, sr);
        tmem_st32(t_s + 32, sr + 32);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&p_full[s]);
        ++n_pv;
      }
      if (!ok) break;
      // Hand the row statistics to the epilogue once it is done with the previous tile.
      if (!mbar_wait(&o_free[s], (n_tile & 1) ^ 1, ctl, kWaitSoftmaxPvDone)) break;
      s_stat[(s * kBlockM + row_in) * 2] = l;
      s_stat[(s * kBlockM + row_in) * 2 + 1] = m;
      mbar_arrive(&sm_final[s]);
      ++n_tile;
    }
  } else if (warp < 12) {
    // ------------------------------------------------------------------ epilogue
    reg_dealloc<kEpilogueRegs>();
    const int row_in = tid & 127;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    uint32_t n_tile = 0;
    uint32_t n_pv[2] = {0, 0};
    uint32_t n_epi[2] = {0, 0};
    bool ok = true;
    for (int t = blockIdx.x; t < p.num_tiles && ok; t += gridDim.x) {
      const Tile ti = get_tile(p, t);
      if (!ti.valid) continue;
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        const int r_lo = ti.m0 + s * kBlockM;
        const int row = r_lo + row_in;
        const int iters = ti.ne[s] - ti.nb[s];
        if (!mbar_wait(&sm_final[s], n_tile & 1, ctl, kWaitEpiFinal)) { ok = false; break; }
        const float l = s_stat[(s * kBlockM + row_in) * 2];
        const float m = s_stat[(s * kBlockM + row_in) * 2 + 1];
        const bool tma_store = (p.cu_q == nullptr) || (r_lo + kBlockM <= ti.sq);
        uint8_t* stage_smem = s_q + s * Cfg::kTileBytes;
        if (iters > 0) {
          n_pv[s] += iters;
          if (!mbar_wait(&pv_done[s], (n_pv[s] - 1) & 1, ctl, kWaitEpiPvDone)) { ok = false; break; }
          tc_fence_after();
          const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
          const uint32_t t_o = tmem + lane_addr + (s == 0 ? Cfg::kTmemO0 : Cfg::kTmemO1);
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t orr[32];
            tmem_ld32(t_o + c * 32, orr);
            tmem_wait_ld();
            uint32_t w[16];
#pragma unroll
            for (int i = 0; i < 16; ++i)
              w[i] = pack2<BF16>(__uint_as_float(orr[2 * i]) * inv_l, __uint_as_float(orr[2 * i + 1]) * inv_l);
            if (tma_store) {
              // 32 columns = 64 bytes = four 16-byte chunks of the row's 128-byte swizzle line.
              uint8_t* rowp = stage_smem + (c / 2) * (kBlockM * 128) + row_in * 128;
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const int chunk = (c & 1) * 4 + q;
                *reinterpret_cast<uint4*>(rowp + ((chunk ^ (row_in & 7)) << 4)) =
                    make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
              }
            } else if (row < ti.sq) {
              uint16_t* dst = reinterpret_cast<uint16_t*>(p.o_ptr) + ti.bq * p.o_batch_stride +
                              static_cast<int64_t>(ti.q_row0 + row) * p.o_row_stride + ti.h * p.o_head_stride + c * 32;
#pragma unroll
              for (int q = 0; q < 4; ++q)
                *reinterpret_cast<uint4*>(dst + q * 8) = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
            }
          }
        } else if (row < ti.sq) {
          // No key is visible to this stage: O = 0.
          uint16_t* dst = reinterpret_cast<uint16_t*>(p.o_ptr) + ti.bq * p.o_batch_stride +
                          static_cast<int64_t>(ti.q_row0 + row) * p.o_row_stride + ti.h * p.o_head_stride;
#pragma unroll
          for (int q = 0; q < D / 8; ++q) *reinterpret_cast<uint4*>(dst + q * 8) = make_uint4(0, 0, 0, 0);
        }
        tc_fence_before();
        mbar_arrive(&o_free[s]);
        if (row < ti.sq) {
          const float lse = (l > 0.f) ? (m + lg2(l)) * 0.6931471805599453f : INFINITY;
          p.lse_ptr[ti.bq * p.lse_batch_stride + ti.h * p.lse_head_stride + ti.q_row0 + row] = lse;
        }
        if (iters > 0 && tma_store) {
          // All 128 rows staged -> one thread stores the tile.
          fence_proxy_async_smem();
          mbar_arrive(&epi_full[s]);
          if (row_in == 0) {
            if (!mbar_wait(&epi_full[s], n_epi[s] & 1, ctl, kWaitEpiFinal)) { ok = false; break; }
#pragma unroll
            for (int a = 0; a < Cfg::kAtoms; ++a)
              tma_store_4d(&p.tm_o, stage_smem + a * (kBlockM * 128), a * 64, ti.h, ti.q_row0 + r_lo, ti.bq);
            tma_commit_group();
            tma_wait_group_read<0>();
          }
          ++n_epi[s];
        }
        if (row_in == 0) mbar_arrive(&q_empty[s]);
      }
      ++n_tile;
    }
    if (row_in == 0) tma_wait_group<0>();
  } else {
    reg_dealloc<kOtherRegs>();
    if (warp == 13 && lane == 0) {
      // ---------------------------------------------------------------- loader
      uint32_t n_tile = 0, kv_it = 0;
      bool ok = true;
      auto load_kv = [&](const CUtensorMap* tm, int row, int head, int bcoord) -> bool {
        const uint32_t slot = kv_it % Cfg::kSlots;
        const uint32_t ph = (kv_it / Cfg::kSlots) & 1;
        if (!mbar_wait(&kv_empty[slot], ph ^ 1, ctl, kWaitLoadKVEmpty)) return false;
        mbar_expect_tx(&kv_full[slot], Cfg::kTileBytes);
        uint8_t* dst = s_kv + slot * Cfg::kTileBytes;
#pragma unroll
        for (int a = 0; a < Cfg::kAtoms; ++a)
          tma_load_4d(dst + a * (kBlockN * 128), tm, &kv_full[slot], a * 64, head, row, bcoord);
        ++kv_it;
        return true;
      };
      for (int t = blockIdx.x; t < p.num_tiles && ok; t += gridDim.x) {
        const Tile ti = get_tile(p, t);
        if (!ti.valid) continue;
        auto load_q = [&](int s) -> bool {
          if (ti.ne[s] <= ti.nb[s]) return true;
          if (!mbar_wait(&q_empty[s], (n_tile & 1) ^ 1, ctl, kWaitLoadQEmpty)) return false;
          mbar_expect_tx(&q_full[s], Cfg::kTileBytes);
#pragma unroll
          for (int a = 0; a < Cfg::kAtoms; ++a)
            tma_load_4d(s_q + s * Cfg::kTileBytes + a * (kBlockM * 128), &p.tm_q, &q_full[s], a * 64, ti.h,
                        ti.q_row0 + ti.m0 + s * kBlockM, ti.bq);
          return true;
        };
        ok = load_q(0);
        for (int j = ti.jlo; j < ti.jhi && ok; ++j) {
          ok = load_kv(&p.tm_k, ti.k_row0 + j * kBlockN, ti.hk, ti.bq);
          if (j == ti.jlo && ok) ok = load_q(1);
          if (ok) ok = load_kv(&p.tm_v, ti.k_row0 + j * kBlockN, ti.hk, ti.bq);
        }
        if (ti.jlo >= ti.jhi && ok) ok = load_q(1);
        ++n_tile;
      }
      if (!ok) {
        // Give copies that are still in flight time to land before the CTA exits.
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) {
        }
      }
    } else if (warp == 12 && lane == 0) {
      // ---------------------------------------------------------------- mma issuer
      const uint32_t idesc_qk = make_idesc(BF16, kBlockM, kBlockN, false, false);
      const uint32_t idesc_pv = make_idesc(BF16, kBlockM, D, false, true);
      const uint32_t q_addr = smem_u32(s_q);
      const uint32_t kv_addr = smem_u32(s_kv);
      uint32_t n_tile = 0, kv_it = 0;
      uint32_t n_p[2] = {0, 0};
      uint32_t n_q[2] = {0, 0};  // Q loads seen per stage (a stage without work loads nothing)
      bool ok = true;
      for (int t = blockIdx.x; t < p.num_tiles && ok; t += gridDim.x) {
        const Tile ti = get_tile(p, t);
        if (!ti.valid) continue;
        bool q_ready[2] = {false, false};
        // S_s = Q_s K^T over D in steps of 16 (32 bytes inside the 128-byte swizzle atom).
        auto issue_qk = [&](int s, uint32_t k_base) -> bool {
          if (!q_ready[s]) {
            if (!mbar_wait(&q_full[s], n_q[s] & 1, ctl, kWaitMmaQFull)) return false;
            ++n_q[s];
            q_ready[s] = true;
          }
          tc_fence_after();
          const uint32_t a_base = q_addr + s * Cfg::kTileBytes;
          const uint32_t d_tmem = tmem + (s == 0 ? Cfg::kTmemS0 : Cfg::kTmemS1);
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t o = (ks / 4) * (kBlockM * 128) + (ks % 4) * 32;
            mma_ss(d_tmem, make_smem_desc(a_base + o, 16, 1024), make_smem_desc(k_base + o, 16, 1024), idesc_qk,
                   ks > 0);
          }
          mma_commit(&s_full[s]);
          return true;
        };
        // O_s (+)= P_s V over the 128 keys in steps of 16 (P: 8 TMEM columns, V: 16 rows of 128 bytes).
        auto issue_pv = [&](int s, uint32_t v_base, bool first) -> bool {
          if (!mbar_wait(&p_full[s], n_p[s] & 1, ctl, kWaitMmaPFull)) return false;
          ++n_p[s];
          if (first && !mbar_wait(&o_free[s], (n_tile & 1) ^ 1, ctl, kWaitMmaOFree)) return false;
          tc_fence_after();
          const uint32_t d_tmem = tmem + (s == 0 ? Cfg::kTmemO0 : Cfg::kTmemO1);
          const uint32_t a_tmem = tmem + (s == 0 ? Cfg::kTmemS0 : Cfg::kTmemS1);
#pragma unroll
          for (int ks = 0; ks < kBlockN / 16; ++ks)
            mma_ts(d_tmem, a_tmem + ks * 8, make_smem_desc(v_base + ks * 2048, kBlockN * 128, 1024), idesc_pv,
                   (!first) || ks > 0);
          mma_commit(&pv_done[s]);
          return true;
        };
        auto wait_kv = [&](uint32_t it) -> bool {
          return mbar_wait(&kv_full[it % Cfg::kSlots], (it / Cfg::kSlots) & 1, ctl, kWaitMmaKVFull);
        };
        auto slot_addr = [&](uint32_t it) -> uint32_t { return kv_addr + (it % Cfg::kSlots) * Cfg::kTileBytes; };
        auto act = [&](int s, int j) -> bool { return j >= ti.nb[s] && j < ti.ne[s]; };

        if (ti.jlo < ti.jhi) {
          // Ring order is K(jlo), V(jlo), K(jlo+1), V(jlo+1), ...
          ok = wait_kv(kv_it);
          if (ok && act(0, ti.jlo)) ok = issue_qk(0, slot_addr(kv_it));
          if (ok && act(1, ti.jlo)) ok = issue_qk(1, slot_addr(kv_it));
          if (ok) mma_commit(&kv_empty[kv_it % Cfg::kSlots]);
          ++kv_it;
          for (int j = ti.jlo; j < ti.jhi && ok; ++j) {
            const uint32_t it_v = kv_it, it_k = kv_it + 1;
            const bool has_next = (j + 1 < ti.jhi);
            ok = wait_kv(it_v);
            if (ok && act(0, j)) ok = issue_pv(0, slot_addr(it_v), j == ti.nb[0]);
            if (ok && has_next) ok = wait_kv(it_k);
            if (ok && has_next && act(0, j + 1)) ok = issue_qk(0, slot_addr(it_k));
            if (ok && act(1, j)) ok = issue_pv(1, slot_addr(it_v), j == ti.nb[1]);
            if (ok) mma_commit(&kv_empty[it_v % Cfg::kSlots]);
            if (ok && has_next && act(1, j + 1)) ok = issue_qk(1, slot_addr(it_k));
            if (ok && has_next) mma_commit(&kv_empty[it_k % Cfg::kSlots]);
            kv_it += has_next ? 2 : 1;
          }
        }
        ++n_tile;
      }
    }
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 12) tmem_dealloc(tmem, 512);
}

template <int D, bool BF16>
cudaError_t launch_one(const FwdParams& p, int num_sms, cudaStream_t stream) {
  using Cfg = FwdCfg<D>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(fwd_kernel<D, BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int grid = p.num_tiles < num_sms ? p.num_tiles : num_sms;
  fwd_kernel<D, BF16><<<grid, kThreads, Cfg::kSmemBytes, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_fwd(const FwdParams& p, int head_dim, bool bf16, int num_sms, cudaStream_t stream) {
  if (p.num_tiles <= 0) return cudaSuccess;
  if (head_dim == 128) return bf16 ? launch_one<128, true>(p, num_sms, stream) : launch_one<128, false>(p, num_sms, stream);
  if (head_dim == 64) return bf16 ? launch_one<64, true>(p, num_sms, stream) : launch_one<64, false>(p, num_sms, stream);
  return cudaErrorInvalidValue;
}

}  // namespace fa2
