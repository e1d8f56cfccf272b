// FlashAttention-2 backward for sm_100a (B200): dQ, dK, dV in one kernel.
//
// One CTA owns 128 keys of one (batch, kv head) and walks every 128-row query block (and every
// query head of the GQA group) that can see those keys. Everything is computed transposed, keys
// on the TMEM lanes, so that P^T feeds the dV MMA straight from TMEM:
//
//   S^T  = K Q^T            smem x smem  -> TMEM [keys x q]
//   dP^T = V dO^T           smem x smem  -> TMEM [keys x q]
//   P^T  = exp2(S^T c - lse)             compute warps, written back over S^T as 16-bit
//   dV  += P^T dO           TMEM x smem (dO as MN-major operand)
//   dS^T = P^T (dP^T - delta)            compute warps -> swizzled smem [keys x q]
//   dK  += dS^T Q           smem (K-major view of dS^T) x smem (Q MN-major)
//   dQ   = dS K             smem (MN-major view of dS^T) x smem (K MN-major) -> TMEM, aliasing dP^T
//   dQ tile -> registers -> smem -> cp.reduce.async.bulk (fp32 add) into the dQ accumulator
//
// TMEM: dK [0,D) dV [D,2D) S^T/P^T [256,384) dP^T/dQ [384,512).
// Warps: 0 loader (TMA), 1 MMA issuer, 4-11 compute (two warpgroups, 64 query columns each),
// 12-15 dQ drain. dK and dV are accumulated over the whole loop in TMEM and written once, so they
// need no atomics; the GQA heads are walked serially like the reference kernel does.
//
// Replaces the reference kernels `backward` (dQ) and `backward_kv`
// (flash-attn2-rs/src/device/backward/dq.rs:12-302,438-576, dkv.rs:15-266,865-1012,
//  common.rs:121-152) and their packed variants (src/device/varlen/backward.rs:134-648), with
// fp32 dQ accumulation in global memory as in the reference's fused kernel (common.rs:248-252).
#include "sm100_ptx.cuh"
#include "fa2_params.h"
#include "fa2_launch.h"

namespace fa2 {

namespace {

constexpr int kBlk = 128;  // keys per CTA and query rows per iteration
constexpr int kThreads = 512;
constexpr int kComputeRegs = 152;
constexpr int kDrainRegs = 152;
constexpr int kMiscRegs = 56;
// setmaxnreg moves registers inside the CTA's own allocation (128 per thread at launch: 65536 / 512). What the
// compute and drain warps take must not exceed what warps 0-3 give back: an increase beyond it never returns.
static_assert(8 * (kComputeRegs - 128) + 4 * (kDrainRegs - 128) <= 4 * (128 - kMiscRegs), "setmaxnreg: more registers asked for than released");
constexpr float kLog2e = 1.4426950408889634f;

template <int D>
struct BwdCfg {
  static constexpr int kAtoms = D / 64;
  static constexpr int kTileBytes = kBlk * D * 2;
  static constexpr int kKOff = 0;
  static constexpr int kVOff = kTileBytes;
  static constexpr int kQOff = 2 * kTileBytes;     // 2 stages
  static constexpr int kDOOff = 4 * kTileBytes;    // 2 stages; a retired stage doubles as dQ staging
  static constexpr int kDSOff = 6 * kTileBytes;    // [128 keys x 128 q] 16-bit
  static constexpr int kDSBytes = kBlk * kBlk * 2;
  static constexpr int kBarOff = kDSOff + kDSBytes;
  static constexpr int kNumBars = 28;
  static constexpr int kMiscOff = (kBarOff + kNumBars * 8 + 15) / 16 * 16;  // what follows is read as float4
  static constexpr int kStatOff = kMiscOff + 32;       // lse / delta: [2 buffers][2][128] fp32
  static constexpr int kSmemBytes = kStatOff + 2 * 2 * kBlk * 4;  // the dynamic window must start 1024-aligned
  static_assert(kStatOff % 16 == 0, "lse / delta are read as float4");
  static constexpr int kPieceBytes = kBlk * 128;       // dQ staging piece: [128 rows x 32 fp32]
  static constexpr uint32_t kTmemDK = 0, kTmemDV = D, kTmemS = 256, kTmemDP = 384;
};

struct KvTile {
  int b, hk, n0;
  int sq, sk, q_row0, k_row0, bq, off;
  int m_start, n_m, n_iter;
  bool valid;
};

__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Query blocks [m_start, m_start + n_m) whose rows can see a key of [n0, n0 + 127].
__device__ __forceinline__ void q_block_range(const BwdParams& p, int sq, int sk, int n0, int& m_start, int& n_m) {
  int q_lo = 0, q_hi = sq;  // [q_lo, q_hi)
  const int off = sk - sq;
  const int n_last = min(n0 + kBlk - 1, sk - 1);
  if (p.window_right >= 0) q_lo = max(0, n0 - off - p.window_right);
  if (p.window_left >= 0) q_hi = min(sq, n_last - off + p.window_left + 1);
  m_start = q_lo / kBlk;
  n_m = (q_hi > q_lo) ? ((q_hi + kBlk - 1) / kBlk - m_start) : 0;
}

// Position of an iteration in the CTA's walk over (query head of the GQA group, query block), advanced
// without integer divisions: iteration it is head g = it / n_m of the group, query block m_start + it % n_m.
struct Walk {
  int g, mi;
};
__device__ __forceinline__ Walk walk_next(Walk w, int n_m) {
  if (++w.mi == n_m) {
    w.mi = 0;
    ++w.g;
  }
  return w;
}

__device__ __forceinline__ KvTile get_kv_tile(const BwdParams& p, int t) {
  KvTile ti;
  // Consecutive CTAs walk the key blocks of one (batch, kv head): the head's Q, dO and its fp32
  // dQ accumulator stay in L2 while the 16-odd CTAs that add into it run side by side. With a
  // causal mask the first key blocks see the most query rows, so each head starts with its
  // heaviest CTAs.
  const int bh = t / p.num_nblk;
  int nblk = t - bh * p.num_nblk;
  // Ordered dQ accumulation waits for the higher key blocks of the same head. CTAs start in grid order, so
  // there the highest key block comes first: a CTA only ever waits for CTAs that were started before it,
  // whatever the number of key blocks and of resident CTAs.
  if (p.dq_turn != nullptr) nblk = p.num_nblk - 1 - nblk;
  ti.b = bh / p.heads_k;
  ti.hk = bh - ti.b * p.heads_k;
  ti.n0 = nblk * kBlk;
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
  q_block_range(p, ti.sq, ti.sk, ti.n0, ti.m_start, ti.n_m);
  ti.n_iter = ti.n_m * p.group;
  return ti;
}

// FANCY: softcap or ALiBi in use; PACKED: cu_seqlens batches. Both are compile-time so that the plain dense
// kernel carries none of their code: at 156 KB the all-in-one kernel missed the SM's instruction cache on a
// quarter of its fetches and ran 6-9 % slower than the 62 KB one.
template <int D, bool BF16, bool FANCY, bool PACKED>
__global__ void __launch_bounds__(kThreads, 1) bwd_kernel(const __grid_constant__ BwdParams p) {
  using Cfg = BwdCfg<D>;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0u) {
    if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, kWaitNone + 1);
    return;
  }
  uint8_t* s_k = smem + Cfg::kKOff;
  uint8_t* s_v = smem + Cfg::kVOff;
  uint8_t* s_q = smem + Cfg::kQOff;
  uint8_t* s_do = smem + Cfg::kDOOff;
  uint8_t* s_ds = smem + Cfg::kDSOff;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kBarOff);
  uint64_t* kv_full = bars + 0;    // K has landed (V has a barrier of its own: the first S^T needs only K and Q)
  uint64_t* q_full = bars + 1;    // [2]
  uint64_t* q_empty = bars + 3;   // [2]
  uint64_t* do_full = bars + 5;   // [2]
  uint64_t* do_empty = bars + 7;  // [2] dV has read the stage and the dQ drain is done staging in it
  uint64_t* s_full = bars + 9;
  uint64_t* p_full = bars + 10;
  uint64_t* dp_full = bars + 11;
  uint64_t* ds_full = bars + 12;
  uint64_t* dq_full = bars + 13;
  uint64_t* dq_free = bars + 14;
  uint64_t* dkv_done = bars + 15;
  uint64_t* stat_full = bars + 16;
  uint64_t* stage_free = bars + 17;
  uint64_t* stage_full = bars + 18;
  uint64_t* epi_full = bars + 19;  // [2]
  uint64_t* kv_fixed = bars + 21;  // packed batches: the fixer warp has cleared the rows past the sequence
  uint64_t* q_fixed = bars + 22;   // [2]
  uint64_t* do_fixed = bars + 24;  // [2]
  uint64_t* dv_done = bars + 26;   // the last dV MMA has completed (dK still has one GEMM to go)
  uint64_t* v_full = bars + 27;    // V has landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Cfg::kMiscOff + 8);
  float* s_stat = reinterpret_cast<float*>(smem + Cfg::kStatOff);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const WaitCtl ctl{abort_flag, p.status};
  const KvTile ti = get_kv_tile(p, blockIdx.x);
  if (!ti.valid) return;
  const bool want_dq = (p.which & 1) != 0;
  const bool want_dkv = (p.which & 2) != 0;  // a dQ-only call skips the dV and dK GEMMs (their commits still hand the stages back)

  // Descriptor fetches start first: they are the head of the latency chain of the first loads.
  if (warp == 2 && lane == 0) {
    tma_prefetch_desc(&p.tm_k);
    tma_prefetch_desc(&p.tm_q);
    tma_prefetch_desc(&p.tm_v);
    tma_prefetch_desc(&p.tm_do);
    tma_prefetch_desc(&p.tm_dqa);
  }
  if (warp == 0) {
    // One barrier per lane: arrival counts by index (see the list above).
    if (lane < Cfg::kNumBars) {
      uint32_t count = 1;
      if (lane == 10 || lane == 12 || lane == 16) count = 256;            // p_full, ds_full, stat_full
      if (lane == 14 || lane == 18 || lane == 19 || lane == 20) count = kBlk;  // dq_free, stage_full, epi_full[2]
      if ((lane == 7 || lane == 8) && want_dq) count = 5;  // do_empty: the dV commit and, with dQ, the four drain warps
      mbar_init(bars + lane, count);
    }
    if (lane == 0) *abort_flag = 0;
    mbar_fence_init();
    __syncwarp();
  }
  if (tid == 0) {
    // The first loads go out before the rest of the CTA is set up (TMEM allocation, the block-wide
    // barrier): their latency is the longest item of a CTA's start.
    if (ti.n_iter > 0) {
      const int hq0 = ti.hk * p.group;
      const int m00 = ti.m_start * kBlk;
      mbar_expect_tx(kv_full, Cfg::kTileBytes);
      mbar_expect_tx(v_full, Cfg::kTileBytes);
      mbar_expect_tx(&q_full[0], Cfg::kTileBytes);
      mbar_expect_tx(&do_full[0], Cfg::kTileBytes);
#pragma unroll
      for (int a = 0; a < Cfg::kAtoms; ++a) {
        tma_load_4d(s_k + a * (kBlk * 128), &p.tm_k, kv_full, a * 64, ti.hk, ti.k_row0 + ti.n0, ti.bq);
        tma_load_4d(s_q + a * (kBlk * 128), &p.tm_q, &q_full[0], a * 64, hq0, ti.q_row0 + m00, ti.bq);
      }
#pragma unroll
      for (int a = 0; a < Cfg::kAtoms; ++a) {
        tma_load_4d(s_v + a * (kBlk * 128), &p.tm_v, v_full, a * 64, ti.hk, ti.k_row0 + ti.n0, ti.bq);
        tma_load_4d(s_do + a * (kBlk * 128), &p.tm_do, &do_full[0], a * 64, hq0, ti.q_row0 + m00, ti.bq);
      }
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int n_iter = ti.n_iter;

  if (warp < 4) {
    reg_dealloc<kMiscRegs>();
    if (warp == 0 && elect_one()) {
      // ---------------------------------------------------------------- loader
      // K, V and the first Q / dO tiles were requested during set-up.
      bool ok = true;
      Walk w{0, 0};
      for (int it = 1; it < n_iter && ok; ++it) {
        w = walk_next(w, ti.n_m);
        const int hq = ti.hk * p.group + w.g;
        const int m0 = (ti.m_start + w.mi) * kBlk;
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        ok = mbar_wait(&q_empty[st], ph ^ 1, ctl, kWaitBwd + 1);
        if (!ok) break;
        mbar_expect_tx(&q_full[st], Cfg::kTileBytes);
#pragma unroll
        for (int a = 0; a < Cfg::kAtoms; ++a)
          tma_load_4d(s_q + st * Cfg::kTileBytes + a * (kBlk * 128), &p.tm_q, &q_full[st], a * 64, hq,
                      ti.q_row0 + m0, ti.bq);
        ok = mbar_wait(&do_empty[st], ph ^ 1, ctl, kWaitBwd + 2);
        if (!ok) break;
        mbar_expect_tx(&do_full[st], Cfg::kTileBytes);
#pragma unroll
        for (int a = 0; a < Cfg::kAtoms; ++a)
          tma_load_4d(s_do + st * Cfg::kTileBytes + a * (kBlk * 128), &p.tm_do, &do_full[st], a * 64, hq,
                      ti.q_row0 + m0, ti.bq);
      }
      if (!ok) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) {
        }
      }
    } else if (warp == 1 && elect_one()) {
      // ---------------------------------------------------------------- mma issuer
      // Descriptors are built once; in the loops an operand address is one 64-bit add of a constant
      // (the descriptor's address field counts 16-byte units).
      constexpr uint32_t kBase = (1u << 4) | ((BF16 ? 1u : 0u) << 7) | ((BF16 ? 1u : 0u) << 10) |
                                 (static_cast<uint32_t>(kBlk >> 4) << 24);
      constexpr uint32_t idesc_qk = kBase | (static_cast<uint32_t>(kBlk >> 3) << 17);             // S^T, dP^T
      constexpr uint32_t idesc_dv = kBase | (static_cast<uint32_t>(D >> 3) << 17) | (1u << 16);   // dV, dK: B MN-major
      constexpr uint32_t idesc_dq = idesc_dv | (1u << 15);                                        // dQ: A and B MN-major
      constexpr uint32_t kTile16 = Cfg::kTileBytes >> 4;
      constexpr uint32_t kAtom16 = (kBlk * 128) >> 4;
      // One base descriptor (K-major view of the start of shared memory); every operand is that
      // plus a constant: its byte offset / 16, and for the MN-major views the larger leading offset.
      const uint64_t base = make_smem_desc(smem_u32(smem), 16, 1024);
      constexpr uint64_t kMn = static_cast<uint64_t>(((kBlk * 128) >> 4) - 1) << 16;
      const uint64_t k_kmaj = base + (Cfg::kKOff >> 4), k_mn = k_kmaj + kMn;
      const uint64_t v_kmaj = base + (Cfg::kVOff >> 4);
      const uint64_t q_kmaj = base + (Cfg::kQOff >> 4), q_mn = q_kmaj + kMn;
      const uint64_t do_kmaj = base + (Cfg::kDOOff >> 4), do_mn = do_kmaj + kMn;
      const uint64_t ds_kmaj = base + (Cfg::kDSOff >> 4), ds_mn = ds_kmaj + kMn;
      // [keys x q] = A[keys x d] B[q x d]^T, both K-major, over d in steps of 16
      auto kmajor_pair = [&](uint32_t d_tmem, uint64_t a, uint64_t b) {
        static_for<D / 16>([&](auto ks) {
          constexpr uint32_t o = (ks.value / 4) * kAtom16 + (ks.value % 4) * 2;
          mma_ss_o<o, o>(d_tmem, a, b, idesc_qk, ks.value > 0 ? 1u : 0u);
        });
      };
      // Packed batches: a tile that reaches past the end of its sequence holds rows of the next sequence; it
      // is usable once the fixer warp has cleared them. bit st of *_par: parity of the stage's next fix.
      constexpr bool packed = PACKED;
      uint32_t qfix_par = 0, dofix_par = 0;
      auto ragged_q = [&](int mi) { return packed && (ti.m_start + mi) * kBlk + kBlk > ti.sq; };
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
      bool ok = n_iter > 0;
      if (ok) ok = mbar_wait(kv_full, 0, ctl, kWaitBwd + 3);
      if (ok && packed && ti.n0 + kBlk > ti.sk) ok = mbar_wait(kv_fixed, 0, ctl, kWaitBwd + 20);
      if (ok) ok = q_ready(0, 0, 0, kWaitBwd + 4);  // iteration 0 is query block m_start
      if (ok) {
        tc_fence_after();
        kmajor_pair(tmem + Cfg::kTmemS, k_kmaj, q_kmaj);
        mma_commit(s_full);
        ok = do_ready(0, 0, 0, kWaitBwd + 5);
        if (ok) ok = mbar_wait(v_full, 0, ctl, kWaitBwd + 3);
      }
      if (ok) {
        tc_fence_after();
        kmajor_pair(tmem + Cfg::kTmemDP, v_kmaj, do_kmaj);
        mma_commit(dp_full);
      }
      Walk wn{0, 0};  // position of iteration it + 1
      for (int it = 0; it < n_iter && ok; ++it) {
        wn = walk_next(wn, ti.n_m);
        const uint32_t st = it & 1;
        const uint32_t nph = ((it + 1) >> 1) & 1;  // phase of the stage barriers of iteration it + 1
        const bool has_next = it + 1 < n_iter;
        const uint32_t acc = it > 0 ? 1u : 0u;
        // dV += P^T dO   (P^T: two 32-column halves at S + 0 and S + 64)
        ok = mbar_wait(p_full, it & 1, ctl, kWaitBwd + 6);
        if (!ok) break;
        tc_fence_after();
        if (want_dkv) {
          const uint64_t b = do_mn + st * kTile16;
          static_for<kBlk / 16>([&](auto ks) {
            mma_ts_o<(ks.value / 4) * 64 + (ks.value % 4) * 8, ks.value * (2048 >> 4)>(
                tmem + Cfg::kTmemDV, tmem + Cfg::kTmemS, b, idesc_dv, ks.value > 0 ? 1u : acc);
          });
        }
        mma_commit(&do_empty[st]);
        if (!has_next) mma_commit(dv_done);  // dV is final: its epilogue runs beside the last dQ and dK GEMMs
        // S^T of the next iteration right behind dV, the last reader of P^T: the scores are there when the
        // compute warps come out of phase B.
        if (has_next) {
          ok = q_ready(wn.mi, st ^ 1, nph, kWaitBwd + 8);
          if (!ok) break;
          tc_fence_after();
          kmajor_pair(tmem + Cfg::kTmemS, k_kmaj, q_kmaj + (st ^ 1) * kTile16);
          mma_commit(s_full);
        }
        // dQ = dS K   (into the dP^T columns, which the compute warps have drained)
        ok = mbar_wait(ds_full, it & 1, ctl, kWaitBwd + 7);
        if (!ok) break;
        tc_fence_after();
        if (want_dq) {
          static_for<kBlk / 16>([&](auto ks) {
            mma_ss_o<ks.value * (2048 >> 4), ks.value * (2048 >> 4)>(tmem + Cfg::kTmemDP, ds_mn, k_mn, idesc_dq,
                                                                      ks.value > 0 ? 1u : 0u);
          });
          mma_commit(dq_full);
        }
        // dK += dS^T Q
        if (want_dkv) {
          const uint64_t b = q_mn + st * kTile16;
          static_for<kBlk / 16>([&](auto ks) {
            mma_ss_o<(ks.value / 4) * kAtom16 + (ks.value % 4) * 2, ks.value * (2048 >> 4)>(
                tmem + Cfg::kTmemDK, ds_kmaj, b, idesc_dv, ks.value > 0 ? 1u : acc);
          });
        }
        mma_commit(&q_empty[st]);
        // dP^T of the next iteration, once the dQ tile has left TMEM
        if (has_next) {
          ok = do_ready(wn.mi, st ^ 1, nph, kWaitBwd + 9);
          if (ok && want_dq) ok = mbar_wait(dq_free, it & 1, ctl, kWaitBwd + 10);
          if (!ok) break;
          tc_fence_after();
          kmajor_pair(tmem + Cfg::kTmemDP, v_kmaj, do_kmaj + (st ^ 1) * kTile16);
          mma_commit(dp_full);
        }
      }
      if (ok) mma_commit(dkv_done);
    } else if (PACKED && warp == 2 && n_iter > 0) {
      // ---------------------------------------------------------------- fixer (packed batches)
      // The reference zero-fills the rows of a tile that lie past the end of the sequence while staging it
      // (flash-attn2-rs/src/device/varlen/backward.rs:134-648 through the zfill copies of
      // src/device/forward/mod.rs:171-175); the TMA boxes here carry the next sequence's rows instead, and
      // a zero probability times a NaN or Inf of a neighbour would still poison dK, dV and dQ. This warp
      // waits for every Q and dO tile (which keeps it in step with the loader) and clears the stray rows
      // of those that need it, and of K and V once.
      auto clear_rows = [&](uint8_t* tile, int first) {
        for (int r = first + (lane >> 3); r < kBlk; r += 4)
#pragma unroll
          for (int a = 0; a < Cfg::kAtoms; ++a)
            *reinterpret_cast<uint4*>(tile + a * (kBlk * 128) + r * 128 + (lane & 7) * 16) = make_uint4(0, 0, 0, 0);
      };
      auto publish = [&](uint64_t* bar) {
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar);
        __syncwarp();
      };
      bool ok = true;
      const int kv_first = ti.sk - ti.n0;
      if (kv_first < kBlk) {
        ok = __all_sync(0xffffffffu, mbar_wait(kv_full, 0, ctl, kWaitBwd + 3) && mbar_wait(v_full, 0, ctl, kWaitBwd + 3));
        if (ok) {
          clear_rows(s_k, kv_first);
          clear_rows(s_v, kv_first);
          publish(kv_fixed);
        }
      }
      Walk w{0, 0};
      for (int it = 0; it < n_iter && ok; ++it, w = walk_next(w, ti.n_m)) {
        const int first = ti.sq - (ti.m_start + w.mi) * kBlk;
        const uint32_t st = it & 1, ph = (it >> 1) & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(&q_full[st], ph, ctl, kWaitBwd + 4));
        if (ok && first < kBlk) {
          clear_rows(s_q + st * Cfg::kTileBytes, first);
          publish(&q_fixed[st]);
        }
        ok = ok && __all_sync(0xffffffffu, mbar_wait(&do_full[st], ph, ctl, kWaitBwd + 5));
        if (ok && first < kBlk) {
          clear_rows(s_do + st * Cfg::kTileBytes, first);
          publish(&do_fixed[st]);
        }
      }
    }
  } else if (warp < 12) {
    // ------------------------------------------------------------------ compute
    reg_alloc<kComputeRegs>();
    const int cw = warp - 4;
    const int wg = cw >> 2;                 // which 64 query columns
    const int key_in = (cw & 3) * 32 + lane;
    const int ct = tid - 128;               // 0..255
    const uint32_t lane_addr = static_cast<uint32_t>((cw & 3) * 32) << 16;
    const uint32_t t_s = tmem + lane_addr + Cfg::kTmemS + wg * 64;
    const uint32_t t_dp = tmem + lane_addr + Cfg::kTmemDP + wg * 64;
    const int kpos = ti.n0 + key_in;
    bool ok = true;
    // LSE (log2 domain) and delta of one query block: thread ct < 128 loads LSE of row ct, the others
    // delta of row ct - 128; rows past the sequence give P = 0. The value for iteration it + 1 is
    // requested while iteration it computes, so its latency never sits in front of phase A.
    auto load_stat = [&](Walk w) -> float {
      const int hq = ti.hk * p.group + w.g;
      const int q = (ti.m_start + w.mi) * kBlk + (ct & 127);
      if (ct < kBlk) {
        float v = INFINITY;
        if (q < ti.sq) v = p.lse[ti.bq * p.lse_batch_stride + hq * p.lse_head_stride + ti.q_row0 + q] * kLog2e;
        return v;
      }
      float v = 0.f;
      if (q < ti.sq)
        v = p.delta[ti.bq * p.delta_batch_stride + hq * p.delta_head_stride + ti.q_row0 + ti.b * p.delta_seq_pad + q];
      return v;
    };
    constexpr bool fancy = FANCY;
    Walk w{0, 0};
    float stat_next = n_iter > 0 ? load_stat(w) : 0.f;
    for (int it = 0; it < n_iter; ++it) {
      const int m0 = (ti.m_start + w.mi) * kBlk;
      const int g_cur = w.g;
      w = walk_next(w, ti.n_m);
      float* stat = s_stat + (it & 1) * (2 * kBlk);
      stat[ct] = stat_next;
      if (it + 1 < n_iter) stat_next = load_stat(w);
      mbar_arrive(stat_full);
      const bool stat_ok = mbar_wait(stat_full, it & 1, ctl, kWaitBwd + 15);  // voted on with s_full below
      const float4* lse4 = reinterpret_cast<const float4*>(stat + wg * 64);
      const float4* dl4 = reinterpret_cast<const float4*>(stat + kBlk + wg * 64);

      // ---- phase A: P^T = exp2(S^T c - lse)
      if (!__all_sync(0xffffffffu, mbar_wait(s_full, it & 1, ctl, kWaitBwd + 11) && stat_ok)) { ok = false; break; }
      tc_fence_after();
      uint32_t sr[64];
      tmem_ld32(t_s, sr);
      tmem_ld32(t_s + 32, sr + 32);
      tmem_wait_ld();
      const int qbase = m0 + wg * 64;
      bool need_mask = (ti.n0 + kBlk > ti.sk);
      if (p.window_right >= 0) need_mask |= (ti.n0 + kBlk - 1 > m0 + ti.off + p.window_right);
      if (p.window_left >= 0) need_mask |= (ti.n0 < m0 + kBlk - 1 + ti.off - p.window_left);
      int c_lo = 0, c_hi = 64;
      if (need_mask) {
        if (p.window_right >= 0) c_lo = kpos - ti.off - p.window_right - qbase;
        if (p.window_left >= 0) c_hi = kpos - ti.off + p.window_left + 1 - qbase;
        if (kpos >= ti.sk) c_hi = -1;
      }
      float pr[64];
      if (!fancy) {
#pragma unroll
        for (int i = 0; i < 64; i += 4) {
          const float4 l4 = lse4[i / 4];
          pr[i] = ex2(fmaf(__uint_as_float(sr[i]), p.scale_log2, -l4.x));
          pr[i + 1] = ex2(fmaf(__uint_as_float(sr[i + 1]), p.scale_log2, -l4.y));
          pr[i + 2] = ex2(fmaf(__uint_as_float(sr[i + 2]), p.scale_log2, -l4.z));
          pr[i + 3] = ex2(fmaf(__uint_as_float(sr[i + 3]), p.scale_log2, -l4.w));
        }
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (i < c_lo || i >= c_hi) pr[i] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) sr[i] = pack2<BF16>(pr[2 * i], pr[2 * i + 1]);
      } else {
        // softcap / ALiBi: P follows the transformed scores of the forward; what goes on to dS is
        // P times the derivative of the transform, 1 - tanh^2 (the ALiBi bias is a constant).
        const int hq = ti.hk * p.group + g_cur;
        const float slope = (p.alibi != nullptr) ? p.alibi[ti.b * p.alibi_batch_stride + hq] * kLog2e : 0.f;
        const float inv_cap = (p.softcap > 0.f) ? p.scale / p.softcap : 0.f;
        const float cap_l2 = p.softcap * kLog2e;
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          float pp[2], dd[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float raw = __uint_as_float(sr[i + e]);
            float x, deriv = 1.f;
            if (p.softcap > 0.f) {
              const float t = tanh_approx(raw * inv_cap);
              x = cap_l2 * t;
              deriv = fmaf(-t, t, 1.f);
            } else {
              x = raw * p.scale_log2;
            }
            if (p.alibi != nullptr)
              x += p.causal_alibi ? slope * static_cast<float>(kpos)
                                  : -slope * fabsf(static_cast<float>(qbase + i + e + ti.off - kpos));
            const float l = reinterpret_cast<const float*>(lse4)[i + e];
            float pv = ex2(x - l);
            if (need_mask && (i + e < c_lo || i + e >= c_hi)) pv = 0.f;
            pp[e] = pv;
            dd[e] = pv * deriv;
          }
          sr[i / 2] = pack2<BF16>(pp[0], pp[1]);
          pr[i] = dd[0];
          pr[i + 1] = dd[1];
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
      uint8_t* ds_row = s_ds + wg * (kBlk * 128) + key_in * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float4 d0 = dl4[2 * c], d1 = dl4[2 * c + 1];
        const int i = c * 8;
        uint4 w;
        w.x = pack2<BF16>(pr[i] * (__uint_as_float(sr[i]) - d0.x), pr[i + 1] * (__uint_as_float(sr[i + 1]) - d0.y));
        w.y = pack2<BF16>(pr[i + 2] * (__uint_as_float(sr[i + 2]) - d0.z), pr[i + 3] * (__uint_as_float(sr[i + 3]) - d0.w));
        w.z = pack2<BF16>(pr[i + 4] * (__uint_as_float(sr[i + 4]) - d1.x), pr[i + 5] * (__uint_as_float(sr[i + 5]) - d1.y));
        w.w = pack2<BF16>(pr[i + 6] * (__uint_as_float(sr[i + 6]) - d1.z), pr[i + 7] * (__uint_as_float(sr[i + 7]) - d1.w));
        *reinterpret_cast<uint4*>(ds_row + ((c ^ (key_in & 7)) << 4)) = w;
      }
      fence_proxy_async_smem();
      mbar_arrive(ds_full);
    }
    // ---- epilogue: warpgroup 0 writes dK (scaled), warpgroup 1 writes dV
    if (ok) {
      const uint32_t t_acc = tmem + lane_addr + (wg == 0 ? Cfg::kTmemDK : Cfg::kTmemDV);
      const float mul = (wg == 0) ? p.scale : 1.f;
      const CUtensorMap* tm = (wg == 0) ? &p.tm_dk : &p.tm_dv;
      uint16_t* gptr = reinterpret_cast<uint16_t*>(wg == 0 ? p.dk_ptr : p.dv_ptr);
      const bool store = (p.which & 2) != 0;
      const bool tma_store = !PACKED || (ti.n0 + kBlk <= ti.sk);
      // Staging tile of the bulk store: the K tile for dK, the V tile for dV (their last readers have completed
      // with dkv_done; the Q and dO stages may still hold dQ pieces of the last iteration's drain).
      uint8_t* stage = (wg == 0) ? s_k : s_v;
      bool done = true;
      if (n_iter > 0) done = warp_wait(wg == 0 ? dkv_done : dv_done, 0, ctl, kWaitBwd + 13);
      if (done && store) {
        tc_fence_after();
        uint16_t* grow = gptr + ti.bq * p.dkv_batch_stride + static_cast<int64_t>(ti.k_row0 + kpos) * p.dkv_row_stride +
                         ti.hk * p.dkv_head_stride;
        uint32_t acc[D];
        if (n_iter > 0) {
#pragma unroll
          for (int c = 0; c < D / 32; ++c) tmem_ld32(t_acc + c * 32, acc + c * 32);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < D; ++i) acc[i] = 0;
        }
#pragma unroll
        for (int c = 0; c < D / 8; ++c) {  // 16-byte chunks of the row
          uint4 w;
          w.x = pack2<BF16>(__uint_as_float(acc[8 * c]) * mul, __uint_as_float(acc[8 * c + 1]) * mul);
          w.y = pack2<BF16>(__uint_as_float(acc[8 * c + 2]) * mul, __uint_as_float(acc[8 * c + 3]) * mul);
          w.z = pack2<BF16>(__uint_as_float(acc[8 * c + 4]) * mul, __uint_as_float(acc[8 * c + 5]) * mul);
          w.w = pack2<BF16>(__uint_as_float(acc[8 * c + 6]) * mul, __uint_as_float(acc[8 * c + 7]) * mul);
          if (tma_store) {
            *reinterpret_cast<uint4*>(stage + (c / 8) * (kBlk * 128) + key_in * 128 + (((c & 7) ^ (key_in & 7)) << 4)) = w;
          } else if (kpos < ti.sk && c * 8 < p.head_dim) {
            *reinterpret_cast<uint4*>(grow + c * 8) = w;
          }
        }
        if (tma_store) {
          fence_proxy_async_smem();
          mbar_arrive(&epi_full[wg]);
          if ((ct & 127) == 0 && mbar_wait(&epi_full[wg], 0, ctl, kWaitBwd + 16)) {
#pragma unroll
            for (int a = 0; a < Cfg::kAtoms; ++a)
              if (a * 64 < p.head_dim) tma_store_4d(tm, stage + a * (kBlk * 128), a * 64, ti.hk, ti.k_row0 + ti.n0, ti.bq);
            tma_commit_group();
            tma_wait_group_read<0>();  // the staging tile must outlive the copy's reads, not its writes
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ dQ drain
    // The whole 128 x D fp32 tile goes to registers at once so that the dP^T / dQ columns are free
    // for the next iteration right away; it then leaves through the dO stage and the Q stage this
    // iteration has retired as cp.reduce.async.bulk adds into the accumulator.
    reg_alloc<kDrainRegs>();
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_dq = tmem + lane_addr + Cfg::kTmemDP;
    if (want_dq) {
      bool ok = true;
      Walk w{0, 0};
      for (int it = 0; it < n_iter && ok; ++it, w = walk_next(w, ti.n_m)) {
        const int hq = ti.hk * p.group + w.g;
        const int m0 = (ti.m_start + w.mi) * kBlk;
        const uint32_t st = it & 1;
        if (!warp_wait(dq_full, it & 1, ctl, kWaitBwd + 14)) break;
        tc_fence_after();
        uint32_t acc[D];
#pragma unroll
        for (int c = 0; c < D / 32; ++c) tmem_ld32(t_dq + c * 32, acc + c * 32);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(dq_free);
        // Packed batches: the 32-row boxes of the reduce-adds below reach past the end of the sequence into
        // the next sequence's rows. Rows past the end hold nothing of this sequence (and possibly NaN, when this
        // sequence's own data is not finite): they add exact zeros.
        if (PACKED && m0 + (warp & 3) * 32 + lane >= ti.sq) {
#pragma unroll
          for (int i = 0; i < D; ++i) acc[i] = 0u;
        }
        // Each warp drains its own 32 rows in pieces of 32 fp32 columns (4 KB). The reduce engine is bound by
        // the latency of the L2 adds, not by bandwidth: with only the dO stage as staging (half of the tile in
        // flight) a tile took 4000-4800 cycles and paced the whole loop. The first half of the pieces goes
        // through the warp's share of the retired dO stage at once, the second half through its share of the
        // Q stage as soon as dK has read it, so the whole tile is in flight together. Nothing but the warp
        // itself has to be synchronised.
        constexpr int kPieces = D / 32;
        constexpr int kHalf = kPieces / 2;              // pieces per staging area
        constexpr int kWarpPiece = Cfg::kPieceBytes / 4;
        static_assert(kHalf * Cfg::kPieceBytes <= Cfg::kTileBytes, "half of the dQ tile fits one stage");
        uint8_t* stage_do = s_do + st * Cfg::kTileBytes + (warp & 3) * (kHalf * kWarpPiece);
        int* turn = nullptr;
        if (p.dq_turn != nullptr) {
          // Ordered mode: the key blocks that add into these rows take their turns in descending order,
          // which is the order in which they get there under a causal or sliding-window mask (a higher key
          // block starts at a later query block). This block's turn is the number of higher key blocks
          // that cover the rows; a bounded wait for the slab's counter to reach it follows. In this mode the
          // grid lists a head's key blocks highest first (get_kv_tile), so the blocks waited for started earlier.
          const int mq = m0 / kBlk;
          int rank = 0;
          for (int nb = ti.n0 / kBlk + 1; nb < p.num_nblk; nb += 32) {
            const int n = nb + lane;
            bool covers = false;
            if (n < p.num_nblk && n * kBlk < ti.sk) {
              int ms, nm;
              q_block_range(p, ti.sq, ti.sk, n * kBlk, ms, nm);
              covers = (mq >= ms) && (mq < ms + nm);
            }
            rank += __popc(__ballot_sync(0xffffffffu, covers));
          }
          turn = p.dq_turn + ((static_cast<int64_t>(ti.b) * p.heads + hq) * p.num_mblk_q + mq) * 4 + (warp & 3);
          if (lane == 0) {
            const long long t0 = clock64();
            while (*reinterpret_cast<volatile int*>(turn) != rank) {
              __nanosleep(200);
              if (*abort_flag || clock64() - t0 > FA2_WAIT_LIMIT_CYCLES) {
                if (!*abort_flag) {
                  *abort_flag = 1;
                  if (p.status != nullptr) atomicCAS(p.status, 0, kWaitBwd + 19);
                }
                ok = false;
                break;
              }
            }
            __threadfence();
          }
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
          if (!ok) break;
        }
#pragma unroll
        for (int k = 0; k < kPieces; ++k) {
          // dO stage only: piece k reuses the buffer of piece k - kHalf once its reduce has read it
          if (k >= kHalf) {
            if (lane == 0) tma_wait_group_read<kHalf - 1>();
            __syncwarp();
          }
          uint8_t* buf = stage_do + (k % kHalf) * kWarpPiece;
          uint8_t* rowp = buf + lane * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c)
            *reinterpret_cast<uint4*>(rowp + ((c ^ (lane & 7)) << 4)) =
                make_uint4(acc[k * 32 + 4 * c], acc[k * 32 + 4 * c + 1], acc[k * 32 + 4 * c + 2], acc[k * 32 + 4 * c + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (k * 32 < p.head_dim) tma_reduce_add_4d(&p.tm_dqa, buf, k * 32, hq, ti.q_row0 + m0 + (warp & 3) * 32, ti.bq);
            tma_commit_group();
          }
        }
        if (!ok) break;
        // Hand both stages back to the loader once the reduces have read them.
        if (lane == 0) {
          tma_wait_group_read<0>();
          mbar_arrive(&do_empty[st]);
          if (turn != nullptr) {
            // The adds have to be in memory before the next key block may start on these rows.
            tma_wait_group<0>();
            asm volatile("fence.proxy.async.global;" ::: "memory");
            __threadfence();
            atomicAdd(turn, 1);
          }
        }
      }
      if (lane == 0) tma_wait_group_read<0>();
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
  if (warp == 1) tmem_dealloc(tmem, 512);
}

template <int D, bool BF16, bool FANCY, bool PACKED>
cudaError_t launch_one(const BwdParams& p, int num_ctas, cudaStream_t stream) {
  using Cfg = BwdCfg<D>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(bwd_kernel<D, BF16, FANCY, PACKED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  bwd_kernel<D, BF16, FANCY, PACKED><<<num_ctas, kThreads, Cfg::kSmemBytes, stream>>>(p);
  return cudaGetLastError();
}

template <int D, bool BF16>
cudaError_t pick_features(const BwdParams& p, bool fancy, bool packed, int num_ctas, cudaStream_t stream) {
  if (fancy) {
    return packed ? launch_one<D, BF16, true, true>(p, num_ctas, stream)
                  : launch_one<D, BF16, true, false>(p, num_ctas, stream);
  }
  return packed ? launch_one<D, BF16, false, true>(p, num_ctas, stream)
                : launch_one<D, BF16, false, false>(p, num_ctas, stream);
}

template <int D>
cudaError_t pick_dtype(const BwdParams& p, bool bf16, bool fancy, bool packed, int num_ctas, cudaStream_t stream) {
  return bf16 ? pick_features<D, true>(p, fancy, packed, num_ctas, stream)
              : pick_features<D, false>(p, fancy, packed, num_ctas, stream);
}

}  // namespace

cudaError_t launch_bwd(const BwdParams& p, int head_dim, bool bf16, int /*num_sms*/, cudaStream_t stream) {
  const int num_ctas = p.num_nblk * p.batch * p.heads_k;
  if (num_ctas <= 0) return cudaSuccess;
  if (head_dim <= 0 || head_dim > 128) return cudaErrorInvalidValue;
  const bool fancy = (p.softcap > 0.f) || (p.alibi != nullptr);
  const bool packed = p.cu_q != nullptr;
  return head_dim > 64 ? pick_dtype<128>(p, bf16, fancy, packed, num_ctas, stream)
                       : pick_dtype<64>(p, bf16, fancy, packed, num_ctas, stream);
}

}  // namespace fa2
