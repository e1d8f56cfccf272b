// FlashAttention-2 forward for sm_100a (B200).
//
// One persistent CTA per SM walks a longest-first list of work tiles. A work tile is 256 query
// rows of one (batch, head): two 128-row "stages" that run independently of each other and share
// the K/V tiles in shared memory.
//
//   warps 0-3    stage 0 } softmax: tcgen05.ld one S row per thread (the S region of TMEM is handed back
//   warps 4-7    stage 1 }   to the MMA warp at once, so the next Q K^T runs under this softmax) -> mask,
//                            row max, exp2, row sum -> bf16/fp16 P written to shared memory in pieces, as the
//                            K-major swizzled A operand of P V; O in TMEM is rescaled only when the row max
//                            grew by more than 2^8. At the end of a tile the same warps run the stage's
//                            epilogue: O / l -> 16-bit -> swizzled smem (the P buffer) -> TMA store
//                            (predicated stores on ragged packed tiles), LSE = (m + log2 l) ln 2.
//   warp 8, 10   mma      : one thread per stage issues tcgen05.mma; S = Q K^T (smem x smem) into TMEM one
//                           key tile ahead, O += P V (smem x smem, V as an MN-major operand) piece by piece
//   warp 9       loader   : TMA (cp.async.bulk.tensor, 128B swizzle) Q stages + K/V ring in the order
//                           K(0) K(1) V(0) K(2) V(1) ...; it leaves last, after every commit on its
//                           barriers has landed
//   warp 11      fixer    : packed batches only. The rows of a V tile that lie past the end of the sequence
//                           belong to the next sequence (P is exactly zero there, but 0 x NaN is NaN); it
//                           clears them in shared memory once the tile has landed, before the MMA threads
//                           may read it (the reference zero-fills them while staging,
//                           flash-attn2-rs/src/device/forward/mod.rs:171-175,200). Stray K rows only reach
//                           score columns that the mask replaces.
//
// A stage never waits for the other one: each has its own issuing thread, barriers and counters, and a
// K/V ring slot is released by one commit of each issuer, so stage 0 may already work on the next tile
// while stage 1 finishes the current one. Every asynchronous arrival (TMA bytes, tcgen05.commit, bulk
// stores) has a waiter before the CTA ends.
//
// A variant with a separate epilogue warpgroup (O read and stored by four more warps while the softmax
// warps go on) was built and measured slower at S = 2048: O is single-buffered in TMEM, so the epilogue's
// latency stays on the path to the next tile's first P V, and the softmax warps lose 24 registers to it.
//
// Replaces the reference kernels flash_attn_fwd / varlen_fwd
// (flash-attn2-rs/src/device/forward/dense.rs:472-590, forward/mod.rs:1162-1407,
//  varlen/mod.rs:30-318,445-578) and keeps their conventions: bottom-right aligned masks,
// fully masked rows give O = 0 and LSE = +inf, natural-log LSE, kv_head = head / group.
#include "sm100_ptx.cuh"
#include "fa2_params.h"
#include "fa2_launch.h"

#ifndef FA2_PQ
#define FA2_PQ 4
#endif
#ifndef FA2_FWD_SPIN
#define FA2_FWD_SPIN 1  // 1: the hand-offs inside a stage's epilogue spin on the barrier instead of parking
#endif

namespace fa2 {

namespace {

constexpr int kBlockM = 128;
constexpr int kBlockN = 128;
constexpr int kThreads = 384;   // 8 softmax warps + one warpgroup holding the MMA and the loader warp
constexpr int kMmaWarp = 8;   // issues the MMAs of stage 0
constexpr int kMmaWarp1 = 10;  // issues the MMAs of stage 1
constexpr int kLoadWarp = 9;
constexpr int kFixWarp = 11;
constexpr int kSoftmaxRegs = 200;
constexpr int kOtherRegs = 104;
// setmaxnreg moves registers inside the CTA's own allocation (168 per thread at launch: 65536 / 384 rounded down
// to a multiple of 8). What the softmax warps take must not exceed what the other warps give back: an increase
// beyond it never returns (a build with 208 / 96 hung the kernel), and no bounded wait can cover that instruction.
static_assert(8 * (kSoftmaxRegs - 168) <= 4 * (168 - kOtherRegs), "setmaxnreg: the softmax warps ask for more than the others release");
constexpr int kPQ = FA2_PQ;                        // P is handed to the MMA warp in kPQ pieces of kBlockN / kPQ keys
constexpr float kRescaleThreshold = 8.0f;  // log2 domain

template <int D>
struct FwdCfg {
  static constexpr int kAtoms = D / 64;                    // 128-byte swizzle atoms along D
  static constexpr int kTileBytes = kBlockN * D * 2;       // one Q stage / K / V tile
  static constexpr int kSlots = (D == 128) ? 3 : 6;        // K/V ring depth
  static constexpr int kQOff = 0;
  static constexpr int kKVOff = 2 * kTileBytes;
  // One buffer per stage that holds P (128 x 128 16-bit, the A operand of P V) during the key loop and
  // the output tile for the TMA store in the epilogue.
  static constexpr int kPBytes = kBlockM * kBlockN * 2;
  static constexpr int kStageBufBytes = kTileBytes > kPBytes ? kTileBytes : kPBytes;
  static constexpr int kOOff = kKVOff + kSlots * kTileBytes;
  static constexpr int kBarOff = kOOff + 2 * kStageBufBytes;
  static constexpr int kNumBars = 3 * kSlots + 18 + 2 * kPQ;  // kv_full, kv_empty, kv_fixed + per stage
  static constexpr int kMiscOff = (kBarOff + kNumBars * 8 + 15) / 16 * 16;  // tmem slot, abort flag
  static constexpr int kSmemBytes = kMiscOff + 48;  // tmem slot, abort flag, ListDiv; the dynamic window must start 1024-aligned
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
  int flip;            // 1: stage 0 takes the upper 128 rows of the block and stage 1 the lower ones
  bool valid;
};

// Divisors of the work-list index as fixed-point reciprocals floor(2^40 / d) + 1: an integer division is a long
// dependent chain, every role walks the list, and the softmax warps do so between two tiles. The quotient is one
// 64-bit multiply, a shift and a correction on the integer pipes; going through float reciprocals instead put
// int <-> float conversions on the MUFU unit, behind the other stage's exponentials (1000-3500 cycles a tile).
// n / d for 0 <= n < 2^24; the four constants live in shared memory (written once by thread 0).
struct ListDiv {
  unsigned long long grid, bh, heads, group;
};
__device__ __forceinline__ void make_list_div(const FwdParams& p, volatile ListDiv* d) {
  d->grid = (1ull << 40) / gridDim.x + 1;
  d->bh = (1ull << 40) / static_cast<unsigned>(p.batch * p.heads) + 1;
  d->heads = (1ull << 40) / static_cast<unsigned>(p.heads) + 1;
  d->group = (1ull << 40) / static_cast<unsigned>(p.group) + 1;
}
__device__ __forceinline__ int div_small(int n, int d, unsigned long long m) {
  if (n >= (1 << 24)) return n / d;
  int q = static_cast<int>((static_cast<unsigned long long>(static_cast<unsigned>(n)) * m) >> 40);
  if (q * d > n) --q;  // the reciprocal is rounded up: the estimate can be one too large for d >= 2^16
  return q;
}

__device__ __forceinline__ Tile get_tile(const FwdParams& p, const volatile ListDiv* ldp, int t) {
  const ListDiv ld{ldp->grid, ldp->bh, ldp->heads, ldp->group};
  Tile ti;
  // Work tiles are listed longest first; CTA c takes list entries c, 2G-1-c, 2G+c, 4G-1-c, ... (G CTAs):
  // reversing every other round evens out the work per CTA when the sizes fall off in plateaus.
  const int grid = static_cast<int>(gridDim.x);
  const int round = div_small(t, grid, ld.grid);
  const int pos = (round & 1) ? round * grid + (grid - 1 - (t - round * grid)) : t;
  // Under a causal mask the upper half of a block sees one key tile more than the lower one. The stages run
  // independently through the CTA's list, so they take the halves in turns: otherwise stage 1 would end up with
  // about 6 % more key tiles than stage 0 at S = 2048 and the CTA would wait for it.
  ti.flip = round & 1;
  if (pos >= p.num_tiles) {
    ti.valid = false;
    return ti;
  }
  const int bh = p.batch * p.heads;
  const int mrev = div_small(pos, bh, ld.bh);
  const int rem = pos - mrev * bh;
  ti.b = div_small(rem, p.heads, ld.heads);
  ti.h = rem - ti.b * p.heads;
  ti.hk = div_small(ti.h, p.group, ld.group);
  ti.m0 = (p.num_mblk - 1 - mrev) * (2 * kBlockM);
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
  ti.jlo = 0x7fffffff;
  ti.jhi = 0;
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    const int r_lo = ti.m0 + (s ^ ti.flip) * kBlockM;
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

// First row of key tile j that lies past the end of a packed sequence (kBlockN = none). Dense tensors need
// nothing: the TMA unit fills rows past the tensor with zeros.
template <bool PACKED>
__device__ __forceinline__ int ragged_row(int sk, int j) {
  if (!PACKED) return kBlockN;
  const int left = sk - j * kBlockN;
  return left < kBlockN ? max(left, 0) : kBlockN;
}

__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// FANCY: softcap, ALiBi or a negative scale in use; PACKED: cu_seqlens batches. Both are compile-time so that the
// plain dense kernel carries none of their code and stays within reach of the SM's instruction cache: without the
// score transforms the kernel is a third smaller and ran 3-4 % faster.
template <int D, bool BF16, bool FANCY, bool PACKED>
__global__ void __launch_bounds__(kThreads, 1) fwd_kernel(const __grid_constant__ FwdParams p) {
  using Cfg = FwdCfg<D>;
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0u) {
    // 128-byte swizzled tiles need a 1024-byte aligned base; report instead of computing garbage.
    if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, kWaitNone + 1);
    return;
  }
  uint8_t* s_q = smem + Cfg::kQOff;
  uint8_t* s_kv = smem + Cfg::kKVOff;
  uint8_t* s_o = smem + Cfg::kOOff;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kBarOff);
  uint64_t* kv_full = bars;
  uint64_t* kv_empty = bars + Cfg::kSlots;
  uint64_t* kv_fixed = bars + 2 * Cfg::kSlots;  // the fixer has cleared the stray rows of a ragged V tile
  uint64_t* q_full = bars + 3 * Cfg::kSlots;    // every array below is [2], one per stage
  uint64_t* q_empty = q_full + 2;
  uint64_t* s_full = q_full + 4;
  uint64_t* s_free = q_full + 16;        // S_s has been read out of TMEM: the next Q K^T may overwrite it
  uint64_t* p_full = q_full + 18;        // [2][kPQ]: piece q of P_s is in shared memory
  uint64_t* pv_done = q_full + 8;
  uint64_t* o_free = q_full + 10;        // O_s has been read out of TMEM
  uint64_t* epi_full = q_full + 12;      // all 128 rows of O_s are staged in smem
  uint64_t* o_stage_free = q_full + 14;  // the previous TMA store of stage s has read its staging tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Cfg::kMiscOff + 8);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const WaitCtl ctl{abort_flag, p.status};
  volatile ListDiv* ld = reinterpret_cast<volatile ListDiv*>(smem + Cfg::kMiscOff + 16);

  if (tid == 0) {
    *abort_flag = 0;
    make_list_div(p, ld);
    for (int i = 0; i < Cfg::kSlots; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 2);  // one commit per issuer
      mbar_init(&kv_fixed[i], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
      mbar_init(&s_full[s], 1);
      for (int q = 0; q < kPQ; ++q) mbar_init(&p_full[s * kPQ + q], kBlockM);
      mbar_init(&pv_done[s], 1);
      mbar_init(&o_free[s], kBlockM);
      mbar_init(&s_free[s], kBlockM);
      mbar_init(&epi_full[s], kBlockM);
      mbar_init(&o_stage_free[s], 1);
    }
    mbar_fence_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (warp == kLoadWarp && lane == 0) {
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
    // ------------------------------------------------------------------ softmax + epilogue of stage s
    reg_alloc<kSoftmaxRegs>();
    const int s = warp >> 2;
    const int row_in = tid & 127;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem + lane_addr + (s == 0 ? Cfg::kTmemS0 : Cfg::kTmemS1);
    const uint32_t t_o = tmem + lane_addr + (s == 0 ? Cfg::kTmemO0 : Cfg::kTmemO1);
    uint8_t* stage_smem = s_o + s * Cfg::kStageBufBytes;
    // P of this stage as the K-major, 128-byte swizzled A operand of P V: key chunk c (8 keys, 16 bytes) of
    // row r sits in atom c / 8 at byte 128 r + 16 ((c % 8) ^ (r % 8)).
    const uint32_t p_row = smem_u32(stage_smem) + row_in * 128;
    const uint32_t p_swz = static_cast<uint32_t>(row_in & 7) << 4;
    auto store_p_chunk = [&](const int c, uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3) {
      const uint32_t addr = p_row + (c >> 3) * (kBlockM * 128) + ((static_cast<uint32_t>(c & 7) << 4) ^ p_swz);
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
    };
    constexpr bool fancy = FANCY;
    uint32_t n_sfull = 0, n_pv = 0, n_store = 0, n_first = 0;
    for (int t = blockIdx.x; t - static_cast<int>(blockIdx.x) < p.num_tiles; t += gridDim.x) {
      const Tile ti = get_tile(p, ld, t);
      if (!ti.valid) continue;
      const int r_lo = ti.m0 + (s ^ ti.flip) * kBlockM;
      const int row = r_lo + row_in;
      const int nb_s = s ? ti.nb[1] : ti.nb[0];
      const int ne_s = s ? ti.ne[1] : ti.ne[0];
      float m = -INFINITY, l = 0.f;
      float slope = 0.f;
      if (p.alibi != nullptr) slope = p.alibi[ti.b * p.alibi_batch_stride + ti.h] * 1.4426950408889634f;
      bool ok = true;
      for (int j = nb_s; j < ne_s; ++j) {
        if (!warp_wait(&s_full[s], n_sfull & 1, ctl, kWaitSoftmaxSFull)) { ok = false; break; }
        ++n_sfull;
        tc_fence_after();
        uint32_t sr[kBlockN];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(t_s + c * 32, sr + c * 32);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(&s_free[s]);  // the scores live in registers from here on
        float cs = p.scale_log2;
        const int col0 = j * kBlockN;
        // Tiles that touch no mask boundary (warp-uniform test on the stage's row range) and need
        // no score transform take the fast path.
        const int r_hi = r_lo + kBlockM - 1;
        bool need_mask = (col0 + kBlockN > ti.sk);
        if (p.window_right >= 0) need_mask |= (col0 + kBlockN - 1 > r_lo + ti.off + p.window_right);
        if (p.window_left >= 0) need_mask |= (col0 < r_hi + ti.off - p.window_left);
        bool grow;
        float alpha = 1.f;
        if (!fancy) {
          // ---- fast path (also for tiles that touch a mask boundary: masked scores become -inf first):
          // row max with 3-input max, then the O rescale decision
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
          float mx0 = max3(__uint_as_float(sr[0]), __uint_as_float(sr[1]), __uint_as_float(sr[2]));
          float mx1 = max3(__uint_as_float(sr[3]), __uint_as_float(sr[4]), __uint_as_float(sr[5]));
          float mx2 = max3(__uint_as_float(sr[6]), __uint_as_float(sr[7]), __uint_as_float(sr[8]));
          float mx3 = max3(__uint_as_float(sr[9]), __uint_as_float(sr[10]), __uint_as_float(sr[11]));
#pragma unroll
          for (int i = 12; i < kBlockN - 4; i += 8) {
            mx0 = max3(mx0, __uint_as_float(sr[i]), __uint_as_float(sr[i + 1]));
            mx1 = max3(mx1, __uint_as_float(sr[i + 2]), __uint_as_float(sr[i + 3]));
            mx2 = max3(mx2, __uint_as_float(sr[i + 4]), __uint_as_float(sr[i + 5]));
            mx3 = max3(mx3, __uint_as_float(sr[i + 6]), __uint_as_float(sr[i + 7]));
          }
          mx0 = max3(mx0, __uint_as_float(sr[kBlockN - 4]), __uint_as_float(sr[kBlockN - 3]));
          mx1 = max3(mx1, __uint_as_float(sr[kBlockN - 2]), __uint_as_float(sr[kBlockN - 1]));
          const float m_new = fmaxf(m, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2);
          grow = (m_new - m) > kRescaleThreshold;
          if (grow) {
            alpha = ex2(m - m_new);
            m = m_new;
            l *= alpha;
          }
        } else {
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
          grow = (m_new - m) > kRescaleThreshold;
          if (grow) {
            alpha = ex2(m - m_new);  // m = -inf gives 0
            m = m_new;
            l *= alpha;
          }
        }
        bool waited;
        if (j > nb_s) {
          // P V(j-1) has to be complete: it reads the P buffer that this iteration overwrites, and it is the
          // only operation that touches O of this stage.
          waited = mbar_wait(&pv_done[s], (n_pv - 1) & 1, ctl, kWaitSoftmaxPvDone);
        } else {
          // First iteration of a tile: the TMA store of the previous tile must have read the buffer.
          if (row_in == 0) {
            tma_wait_group_read<0>();
            mbar_arrive(&o_stage_free[s]);
          }
          __syncwarp();
          waited = FA2_FWD_SPIN ? mbar_wait_spin(&o_stage_free[s], n_first & 1, ctl, kWaitEpiFinal)
                                : mbar_wait(&o_stage_free[s], n_first & 1, ctl, kWaitEpiFinal);
          ++n_first;
        }
        // One warp reduction reconverges the lanes after the wait and carries both warp-uniform
        // decisions: bit 1 = a lane's wait ran out, bit 0 = a lane's row maximum grew.
        const unsigned votes = __reduce_or_sync(0xffffffffu, (grow ? 1u : 0u) | (waited ? 0u : 2u));
        if (votes & 2u) { ok = false; break; }
        if (j > nb_s && (votes & 1u)) {
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
          // The rescaled O must be in TMEM before p_full lets the next P V accumulate onto it.
          tmem_wait_st();
          tc_fence_before();
        }
        if (!fancy) {
          // ---- fast path: x = s * c - m with packed FMAs, exp2 on the MUFU unit, packed row-sum accumulation.
          const uint64_t c2 = pack_f32x2(p.scale_log2, p.scale_log2);
          // A row that has seen no key yet has m = -inf and only -inf scores: keep x = -inf (not NaN).
          const float neg_m = (m == -INFINITY) ? 0.f : -m;
          const uint64_t nm2 = pack_f32x2(neg_m, neg_m);
          uint64_t acc0 = pack_f32x2(0.f, 0.f), acc1 = acc0;
          constexpr int kPieceCols = kBlockN / kPQ;
#pragma unroll
          for (int i = 0; i < kBlockN; i += 8) {
            float x[8];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint64_t v = fma2(pack_f32x2(__uint_as_float(sr[i + 2 * q]), __uint_as_float(sr[i + 2 * q + 1])), c2, nm2);
              unpack_f32x2(v, x[2 * q], x[2 * q + 1]);
            }
#pragma unroll
            for (int q = 0; q < 8; ++q) x[q] = ex2(x[q]);
            acc0 = add2(acc0, pack_f32x2(x[0], x[1]));
            acc1 = add2(acc1, pack_f32x2(x[2], x[3]));
            acc0 = add2(acc0, pack_f32x2(x[4], x[5]));
            acc1 = add2(acc1, pack_f32x2(x[6], x[7]));
#pragma unroll
            for (int q = 0; q < 4; ++q) sr[i / 2 + q] = pack2<BF16>(x[2 * q], x[2 * q + 1]);
            // The eight probabilities just packed are one 16-byte chunk of this row of P; a piece is
            // announced to the MMA warp as soon as its last chunk is written.
            store_p_chunk(i / 8, sr[i / 2], sr[i / 2 + 1], sr[i / 2 + 2], sr[i / 2 + 3]);
            if (i % kPieceCols == kPieceCols - 8) {
              fence_proxy_async_smem();
              mbar_arrive(&p_full[s * kPQ + i / kPieceCols]);
            }
          }
          float a0, a1;
          unpack_f32x2(add2(acc0, acc1), a0, a1);
          l += a0 + a1;
        } else {
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
        }
        if (fancy) {
#pragma unroll
          for (int c = 0; c < kBlockN / 8; ++c) store_p_chunk(c, sr[4 * c], sr[4 * c + 1], sr[4 * c + 2], sr[4 * c + 3]);
          fence_proxy_async_smem();
#pragma unroll
          for (int q = 0; q < kPQ; ++q) mbar_arrive(&p_full[s * kPQ + q]);
        }
        ++n_pv;
      }
      if (!ok) break;
      // ---- epilogue of this stage: O / l -> 16-bit -> swizzled smem -> one TMA store.
      // A ragged tile of a packed batch (rows of the next sequence follow) uses predicated stores.
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.o_ptr) + ti.bq * p.o_batch_stride +
                       static_cast<int64_t>(ti.q_row0 + row) * p.o_row_stride + ti.h * p.o_head_stride;
      const bool tma_store = !PACKED || (r_lo + kBlockM <= ti.sq);
      if (ne_s > nb_s) {
        const float inv_l = (l > 0.f) ? 1.f / l : 0.f;  // before the wait: the reciprocal queues behind the other stage's exp2 stream
        if (!warp_wait(&pv_done[s], (n_pv - 1) & 1, ctl, kWaitEpiPvDone)) break;
        tc_fence_after();
        uint32_t orr[D];
#pragma unroll
        for (int c = 0; c < D / 32; ++c) tmem_ld32(t_o + c * 32, orr + c * 32);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(&o_free[s]);
        // The other stage's softmax warp shares this scheduler and rarely stalls, so every instruction here
        // is dear: packed multiplies, one conversion per pair, st.shared with a precomputed row address.
        const uint64_t il2 = pack_f32x2(inv_l, inv_l);
        const uint32_t o_row = smem_u32(stage_smem) + row_in * 128;
#pragma unroll
        for (int c = 0; c < D / 8; ++c) {  // 16-byte chunks of the row
          uint32_t w[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float a, b;
            unpack_f32x2(mul2(pack_f32x2(__uint_as_float(orr[8 * c + 2 * q]), __uint_as_float(orr[8 * c + 2 * q + 1])), il2), a, b);
            w[q] = pack2<BF16>(a, b);
          }
          if (tma_store) {
            // chunk c lives in swizzle atom c / 8, at position (c % 8) ^ (row % 8) of the row's 128-byte line
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(o_row + (c / 8) * (kBlockM * 128) +
                                                                             (((c & 7) ^ (row_in & 7)) << 4)),
                         "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                         : "memory");
          } else if (row < ti.sq && c * 8 < p.head_dim) {
            *reinterpret_cast<uint4*>(orow + c * 8) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
        if (tma_store) {
          fence_proxy_async_smem();
          mbar_arrive(&epi_full[s]);
          // A wait that runs out here sets the abort flag; the warp then leaves together at its next
          // warp_wait, which is also where the lanes meet again after this single-lane section.
          if (row_in == 0 && (FA2_FWD_SPIN ? mbar_wait_spin(&epi_full[s], n_store & 1, ctl, kWaitEpiFinal)
                                           : mbar_wait(&epi_full[s], n_store & 1, ctl, kWaitEpiFinal))) {
#pragma unroll
            for (int a = 0; a < Cfg::kAtoms; ++a)
              if (a * 64 < p.head_dim)
                tma_store_4d(&p.tm_o, stage_smem + a * (kBlockM * 128), a * 64, ti.h, ti.q_row0 + r_lo, ti.bq);
            tma_commit_group();
          }
          __syncwarp();
          ++n_store;
        }
      } else {
        mbar_arrive(&o_free[s]);
        if (row < ti.sq) {
          // No key is visible to this stage: O = 0.
#pragma unroll
          for (int q = 0; q < D / 8; ++q)
            if (q * 8 < p.head_dim) *reinterpret_cast<uint4*>(orow + q * 8) = make_uint4(0, 0, 0, 0);
        }
      }
      if (row < ti.sq) {
        const float lse = (l > 0.f) ? (m + lg2(l)) * 0.6931471805599453f : INFINITY;
        p.lse_ptr[ti.bq * p.lse_batch_stride + ti.h * p.lse_head_stride + ti.q_row0 + row] = lse;
      }
      // Rows past the end of a packed sequence skipped the stores above.
      __syncwarp();
    }
    // The last bulk store has read its staging tile, and the last P V of this stage has completed: nothing of
    // this stage is still on its way when the CTA ends.
    if (row_in == 0) tma_wait_group_read<0>();
    __syncwarp();
  } else {
    reg_dealloc<kOtherRegs>();
    if (warp == kLoadWarp && elect_one()) {
      // ---------------------------------------------------------------- loader
      uint32_t slot = 0, ring_phase = 0, n_q0 = 0, n_q1 = 0;
      bool ok = true;
      auto load_kv = [&](const CUtensorMap* tm, int row, int head, int bcoord) -> bool {
        if (!mbar_wait(&kv_empty[slot], ring_phase ^ 1, ctl, kWaitLoadKVEmpty)) return false;
        mbar_expect_tx(&kv_full[slot], Cfg::kTileBytes);
        uint8_t* dst = s_kv + slot * Cfg::kTileBytes;
#pragma unroll
        for (int a = 0; a < Cfg::kAtoms; ++a)
          tma_load_4d(dst + a * (kBlockN * 128), tm, &kv_full[slot], a * 64, head, row, bcoord);
        if (++slot == Cfg::kSlots) {
          slot = 0;
          ring_phase ^= 1;
        }
        return true;
      };
      for (int t = blockIdx.x; t - static_cast<int>(blockIdx.x) < p.num_tiles && ok; t += gridDim.x) {
        const Tile ti = get_tile(p, ld, t);
        if (!ti.valid) continue;
        auto load_q = [&](int s) -> bool {
          if (ti.ne[s] <= ti.nb[s]) return true;
          uint32_t& nq = s ? n_q1 : n_q0;
          if (!mbar_wait(&q_empty[s], (nq & 1) ^ 1, ctl, kWaitLoadQEmpty)) return false;
          ++nq;
          mbar_expect_tx(&q_full[s], Cfg::kTileBytes);
#pragma unroll
          for (int a = 0; a < Cfg::kAtoms; ++a)
            tma_load_4d(s_q + s * Cfg::kTileBytes + a * (kBlockM * 128), &p.tm_q, &q_full[s], a * 64, ti.h,
                        ti.q_row0 + ti.m0 + (s ^ ti.flip) * kBlockM, ti.bq);
          return true;
        };
        // Ring order K(jlo), K(jlo+1), V(jlo), K(jlo+2), V(jlo+1), ...: Q K^T runs one key tile ahead of P V.
        // (one loop from jlo - 1 instead of a peeled first step: each helper is inlined once)
        ok = load_q(0);
        for (int j = ti.jlo - 1; j < ti.jhi && ok; ++j) {
          if (j + 1 < ti.jhi) ok = load_kv(&p.tm_k, ti.k_row0 + (j + 1) * kBlockN, ti.hk, ti.bq);
          if (j < ti.jlo) {
            if (ok) ok = load_q(1);
          } else if (ok) {
            ok = load_kv(&p.tm_v, ti.k_row0 + j * kBlockN, ti.hk, ti.bq);
          }
        }
      }
      // The loader leaves last: it waits until the issuers' commits on every ring slot and on both Q stages
      // have landed, so that no asynchronous arrival is still on its way when the CTA gives back its shared
      // memory. A slot or stage that was never used passes at once.
      for (int i = 0; i < Cfg::kSlots && ok; ++i) {
        ok = mbar_wait(&kv_empty[slot], ring_phase ^ 1, ctl, kWaitLoadKVEmpty);
        if (++slot == Cfg::kSlots) {
          slot = 0;
          ring_phase ^= 1;
        }
      }
      if (ok) ok = mbar_wait(&q_empty[0], (n_q0 & 1) ^ 1, ctl, kWaitLoadQEmpty);
      if (ok) ok = mbar_wait(&q_empty[1], (n_q1 & 1) ^ 1, ctl, kWaitLoadQEmpty);
    } else if (warp == kFixWarp) {
      // ---------------------------------------------------------------- fixer (packed batches)
      // Walks the ring in the loader's order and waits for every tile, which keeps it within one ring
      // pass of the consumers; it acts on V tiles that reach past the end of their sequence.
      if (PACKED) {
        uint32_t slot = 0, ring_phase = 0;
        bool ok = true;
        auto step = [&](int first_stray) -> bool {
          if (!__all_sync(0xffffffffu, mbar_wait(&kv_full[slot], ring_phase, ctl, kWaitMmaKVFull))) return false;
          if (first_stray < kBlockN) {
            uint8_t* tile = s_kv + slot * Cfg::kTileBytes;
            // 8 lanes clear one 128-byte row of an atom (the swizzle only permutes 16-byte chunks inside it)
            for (int r = first_stray + (lane >> 3); r < kBlockN; r += 4)
#pragma unroll
              for (int a = 0; a < Cfg::kAtoms; ++a)
                *reinterpret_cast<uint4*>(tile + a * (kBlockN * 128) + r * 128 + (lane & 7) * 16) = make_uint4(0, 0, 0, 0);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&kv_fixed[slot]);
            __syncwarp();
          }
          if (++slot == Cfg::kSlots) {
            slot = 0;
            ring_phase ^= 1;
          }
          return true;
        };
        for (int t = blockIdx.x; t - static_cast<int>(blockIdx.x) < p.num_tiles && ok; t += gridDim.x) {
          const Tile ti = get_tile(p, ld, t);
          if (!ti.valid) continue;
          if (ti.jlo < ti.jhi) ok = step(kBlockN);
          for (int j = ti.jlo; j < ti.jhi && ok; ++j) {
            if (j + 1 < ti.jhi) ok = step(kBlockN);
            if (ok) ok = step(ragged_row<PACKED>(ti.sk, j));
          }
        }
      }
    } else if ((warp == kMmaWarp || warp == kMmaWarp1) && elect_one()) {
      // ---------------------------------------------------------------- mma issuer
      // Descriptors are built once; inside the loops an operand address is one 64-bit add of a
      // compile-time constant (descriptor address field is in 16-byte units), so that the single
      // issuing thread keeps the tensor pipe fed.
      constexpr uint32_t idesc_qk = (1u << 4) | ((BF16 ? 1u : 0u) << 7) | ((BF16 ? 1u : 0u) << 10) |
                                    (static_cast<uint32_t>(kBlockN >> 3) << 17) | (static_cast<uint32_t>(kBlockM >> 4) << 24);
      constexpr uint32_t idesc_pv = (1u << 4) | ((BF16 ? 1u : 0u) << 7) | ((BF16 ? 1u : 0u) << 10) | (1u << 16) |
                                    (static_cast<uint32_t>(D >> 3) << 17) | (static_cast<uint32_t>(kBlockM >> 4) << 24);
      constexpr uint32_t kTile16 = Cfg::kTileBytes >> 4;
      const uint64_t q_desc = make_smem_desc(smem_u32(s_q), 16, 1024);                 // K-major A
      const uint64_t k_desc = make_smem_desc(smem_u32(s_kv), 16, 1024);                // K-major B
      const uint64_t v_desc = make_smem_desc(smem_u32(s_kv), kBlockN * 128, 1024);     // MN-major B
      // Each stage has its own issuing warp, and both walk the same sequence of tiles and K/V ring
      // positions. A stage never waits for the other one: stage 0 may already run the next tile while
      // stage 1 finishes the current one, and a piece of P V is issued while the other stage's
      // exponentials are still in flight. A K/V slot is released by two commits, one per issuer.
      const int s = (warp == kMmaWarp) ? 0 : 1;
      const uint64_t a_q = q_desc + s * kTile16;
      const uint32_t t_s = tmem + (s == 0 ? Cfg::kTmemS0 : Cfg::kTmemS1);
      const uint32_t t_o = tmem + (s == 0 ? Cfg::kTmemO0 : Cfg::kTmemO1);
      const uint64_t a_p = make_smem_desc(smem_u32(s_o + s * Cfg::kStageBufBytes), 16, 1024);  // P: K-major A
      uint32_t slot = 0, ring_phase = 0;  // K/V ring position of the next tile to consume
      uint32_t fix_par = 0;               // bit i: parity of the next kv_fixed phase of slot i
      uint32_t n_qk = 0, n_p = 0, n_q = 0, n_tile = 0;
      bool ok = true;
      auto advance = [&]() {
        mma_commit(&kv_empty[slot]);
        if (++slot == Cfg::kSlots) {
          slot = 0;
          ring_phase ^= 1;
        }
      };
      for (int t = blockIdx.x; t - static_cast<int>(blockIdx.x) < p.num_tiles && ok; t += gridDim.x) {
        const Tile ti = get_tile(p, ld, t);
        if (!ti.valid) continue;
        const int nb = s ? ti.nb[1] : ti.nb[0], ne = s ? ti.ne[1] : ti.ne[0];
        bool q_ready = false;
        // S_s = Q_s K_j^T over D in steps of 16 (32 bytes inside the 128-byte swizzle atom). The S region
        // is free as soon as the softmax warps hold the previous scores in registers.
        auto do_k = [&](const int j) -> bool {
          if (!mbar_wait(&kv_full[slot], ring_phase, ctl, kWaitMmaKVFull)) return false;
          if (j >= nb && j < ne) {
            if (!q_ready) {
              if (!mbar_wait(&q_full[s], n_q & 1, ctl, kWaitMmaQFull)) return false;
              ++n_q;
              q_ready = true;
            }
            if (!mbar_wait(&s_free[s], (n_qk & 1) ^ 1, ctl, kWaitMmaSFree)) return false;
            ++n_qk;
            tc_fence_after();
            const uint64_t b = k_desc + slot * kTile16;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
              constexpr uint32_t kAtom16 = (kBlockM * 128) >> 4;
              const uint32_t o = (ks / 4) * kAtom16 + (ks % 4) * 2;
              mma_ss(t_s, a_q + o, b + o, idesc_qk, ks > 0 ? 1u : 0u);
            }
            mma_commit(&s_full[s]);
            if (j == ne - 1) mma_commit(&q_empty[s]);  // the Q stage may be refilled for the next tile
          }
          advance();
          return true;
        };
        // O_s (+)= P_s V_j, one piece of kBlockN / kPQ keys at a time (per step of 16 keys: 32 bytes of a
        // P row inside its swizzle atom, 16 rows of 128 bytes of V).
        auto do_v = [&](const int j) -> bool {
          if (!mbar_wait(&kv_full[slot], ring_phase, ctl, kWaitMmaKVFull)) return false;
          if (ragged_row<PACKED>(ti.sk, j) < kBlockN) {
            // A V tile that reaches past its sequence is usable once the fixer has cleared the stray rows.
            if (!mbar_wait(&kv_fixed[slot], (fix_par >> slot) & 1, ctl, kWaitMmaKVFull)) return false;
            fix_par ^= 1u << slot;
          }
          if (j >= nb && j < ne) {
            const bool first = (j == nb);
            const uint64_t b = v_desc + slot * kTile16;
            constexpr int kStepsPerPiece = kBlockN / 16 / kPQ;
#pragma unroll
            for (int q = 0; q < kPQ; ++q) {
              if (!mbar_wait(&p_full[s * kPQ + q], n_p & 1, ctl, kWaitMmaPFull)) return false;
              if (q == 0 && first && !mbar_wait(&o_free[s], (n_tile & 1) ^ 1, ctl, kWaitMmaOFree)) return false;
              tc_fence_after();
#pragma unroll
              for (int ks = q * kStepsPerPiece; ks < (q + 1) * kStepsPerPiece; ++ks) {
                constexpr uint32_t kAtom16 = (kBlockM * 128) >> 4;
                const uint32_t o = (ks / 4) * kAtom16 + (ks % 4) * 2;
                mma_ss(t_o, a_p + o, b + ks * (2048 >> 4), idesc_pv, (first && ks == 0) ? 0u : 1u);
              }
            }
            ++n_p;
            mma_commit(&pv_done[s]);
          }
          advance();
          return true;
        };
        for (int j = ti.jlo - 1; j < ti.jhi && ok; ++j) {
          if (j + 1 < ti.jhi) ok = do_k(j + 1);
          if (ok && j >= ti.jlo) ok = do_v(j);
        }
        ++n_tile;
      }
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
  if (warp == kMmaWarp) tmem_dealloc(tmem, 512);
}

template <int D, bool BF16, bool FANCY, bool PACKED>
cudaError_t launch_one(const FwdParams& p, int num_sms, cudaStream_t stream) {
  using Cfg = FwdCfg<D>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(fwd_kernel<D, BF16, FANCY, PACKED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int grid = p.num_tiles < num_sms ? p.num_tiles : num_sms;
  fwd_kernel<D, BF16, FANCY, PACKED><<<grid, kThreads, Cfg::kSmemBytes, stream>>>(p);
  return cudaGetLastError();
}

template <int D, bool BF16>
cudaError_t pick_features(const FwdParams& p, bool fancy, bool packed, int num_sms, cudaStream_t stream) {
  if (fancy) {
    return packed ? launch_one<D, BF16, true, true>(p, num_sms, stream)
                  : launch_one<D, BF16, true, false>(p, num_sms, stream);
  }
  return packed ? launch_one<D, BF16, false, true>(p, num_sms, stream)
                : launch_one<D, BF16, false, false>(p, num_sms, stream);
}

template <int D>
cudaError_t pick_dtype(const FwdParams& p, bool bf16, bool fancy, bool packed, int num_sms, cudaStream_t stream) {
  return bf16 ? pick_features<D, true>(p, fancy, packed, num_sms, stream)
              : pick_features<D, false>(p, fancy, packed, num_sms, stream);
}

}  // namespace

cudaError_t launch_fwd(const FwdParams& p, int head_dim, bool bf16, int num_sms, cudaStream_t stream) {
  if (p.num_tiles <= 0) return cudaSuccess;
  // Head dims below the kernel's D ride on TMA: loads past the real head dim read zeros, stores are clipped.
  if (head_dim <= 0 || head_dim > 128) return cudaErrorInvalidValue;
  const bool fancy = (p.softcap > 0.f) || (p.alibi != nullptr) || (p.scale_log2 < 0.f);
  const bool packed = p.cu_q != nullptr;
  return head_dim > 64 ? pick_dtype<128>(p, bf16, fancy, packed, num_sms, stream)
                       : pick_dtype<64>(p, bf16, fancy, packed, num_sms, stream);
}

}  // namespace fa2
