// Tensor-core backward of the Universal Attention operator for sm_100a, keys-on-lanes form
// (bf16, key chunk = 128, head_dim 64 or 128).  Needs the log-sum-exp of the forward.
//
// One thread block owns one key chunk (b, h, i) and sweeps the rows that see it DOWNWARDS in
// half tiles of 64 rows, so that the reverse cumulative sum of the decay gradient is carried
// per key in a register (universal_attention_autograd.py:232-259).  Every 128 x 64 plane of
// the sweep has the chunk's KEYS on the TMEM lanes and the 64 rows in the columns:
//
//   G    = K_i K_j^T        decay recomputation: log-retention, scan ALONG the columns, thread-local
//   S_r  = K_i Q_rj^T,  dP_r = V_i dO_rj^T
//        P  = exp(S + C - lse_row)          (lse: the forward's per-chunk log-sum-exp, or the row's
//                                             log-sum-exp over all keys in "merged" mode)
//        dS = P (dP - sum_k P dP + g_denom) (the sum over the keys is the one cross-lane step: a
//                                             32 x 32 shuffle transpose per warp, then shared-memory adds)
//        dC += dS                           stays in registers for the whole half tile
//   dV_i += P dO      (P as bf16 in TMEM: the A operand)      dK_i += dS Q     (dS as bf16 in shared memory)
//   dQ_rj = dS^T K_i  (the same shared-memory tile read MN-major)
//   decay gradient from dC (reverse scan along the columns, thread-local), dG (bf16, shared memory)
//   dK_j  = dG^T K_i      dK_i += dG K_j
//
// so the decay prefix and its gradient never change orientation: no transposed copy of C, no
// transposing MMAs, 16 KB of shared memory per bf16 operand tile instead of 64 + 64 KB.  What is freed
// holds a ring of (Q, dO) slots and, at head_dim 64, a second (S, dP) pair in TMEM: the loads and the
// MMAs of the next head run under the element-wise work of the current one.
//
// Warps: 0 = TMA producer + "front" MMA issuer (G, S, dP: everything that only needs loaded tiles),
// 1 = "back" MMA issuer (dV, dK, dQ, dK_j: everything that needs a tile the workers wrote), 2..9 = workers:
// two column groups of 128 threads (thread = key, 32 of the 64 columns each, held in registers).
// dQ_rj / dK_j (64 rows, M = 128 MMAs whose upper 64 lanes compute on whatever the next buffer holds and are
// never read) leave as TMA reduce-adds into fp32 accumulators.  Rows BEFORE the chunk are not handled here.
//
// Every mbarrier wait is bounded; on a timeout the block raises a shared abort flag, every role
// leaves, TMEM is freed and status[0] is set (status[1]: where the first block gave up).
#pragma once
#include "ua_bwd_sm100.cuh"

namespace ua {
namespace sm100 {

struct Bwd2Params {
  Shape s;
  const void* ssrc;
  const void* sdest;
  const void* g_denom;       // (b,h,n,r,L) fp32 or bf16                     [mode 1]
  int g_denom_is_f32;
  const float* lse;          // (b,h,n,r,L) fp32: the forward's log-sum-exp   [mode 1]
  const float* row_lse;      // (b,h,r,L) fp32: log-sum-exp over all keys     [mode 2]
  const float* row_delta;    // (b,h,r,L) fp32: g . merged                    [mode 2]
  const float* carry;        // (b*h*n, n, 2, 128): decay prefix of key k at the start of each 64-row half tile
  float* acc_dk;             // (b*h, L, D) fp32, zeroed (or holding the masked-block part)
  float* acc_dq;             // (b*h, r, L, D) fp32, likewise
  float* acc_dt;             // (b*h, L) fp32, zeroed
  const float* acc_dv_in;    // optional (b*h, L, D) fp32: added to dV_i before it is written (masked-block part)
  __nv_bfloat16* dvc;
  void* dss;
  int* status;
};

template <int D>
struct Bwd2Cfg {
  static constexpr int kNB = (D == 64) ? 2 : 1;            // (S, dP) buffers in TMEM
  static constexpr int kNS = (D == 64) ? 4 : 2;            // (Q, dO) slots
  static constexpr int kKj = (D == 64) ? 2 : 1;            // K_j slots
  static constexpr int kDs = (D == 64) ? 2 : 1;            // dS buffers
  static constexpr int kHalf = 64 * D * 2;                 // [64][D] bf16
  static constexpr int kFull = 128 * D * 2;                // [128][D] bf16
  static constexpr int kBoxes = D / 64;
  static constexpr int oKi = 0;
  static constexpr int oVi = kFull;
  static constexpr int oKj = 2 * kFull;
  static constexpr int oSlot = oKj + kKj * kHalf;          // slot: Q half tile, then dO half tile
  static constexpr int kSlot = 2 * kHalf;
  static constexpr int oDs = oSlot + kNS * kSlot;          // kDs x 16 KB [128 keys][64 rows] bf16, then dG, then the staging tile
  static constexpr int oDg = oDs + kDs * 16384;
  static constexpr int oStage = oDg + 16384;               // [64][D] fp32 as D/32 boxes of [64][32], 128-byte swizzle
  static constexpr int oT3 = oStage + 256 * D;             // float [2][64]
  static constexpr int oLse = oT3 + 512;                   // float [3][64]  lse * log2(e) of the head's rows
  static constexpr int oCc = oLse + 768;                   // float [3][64]  g_denom - sum_k P dP  (or -delta)
  static constexpr int oXch = oCc + 768;                   // float [3][128] totals crossing the two column groups
  static constexpr int oBar = oXch + 1536;
  static constexpr int oMisc = oBar + 256;
  static constexpr int kSmemBytes = oMisc + 64 + 1024;     // + slack to align the base to 1024 B
  // TMEM columns
  static constexpr uint32_t tDV = 0, tDK = D, tY = 2 * D;
  static constexpr uint32_t tS0 = (D == 64) ? 192 : 384, tP0 = tS0 + 64, tS1 = tS0 + 128, tP1 = tS0 + 192;
  static_assert(D == 64 || D == 128, "head_dim 64 or 128");
  static_assert(D == 64 ? (tP1 + 64 <= 512) : (tP0 + 64 <= 512), "TMEM budget");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

enum Bwd2Bar {
  qKvFull = 0,
  qKjFull = 1, qKjFree = 3,        // [2]
  qInFull = 5, qInFree = 9,        // [4]
  qSFull = 13, qLdDone = 15, qMmaDone = 17,   // [2] per (S, dP) buffer
  qDsReady = 19, qDsFree = 21,     // [2] per dS buffer
  qYFull = 23, qYFree = 24, qDgReady = 25, qDgFree = 26, qFinal = 27, qNumBars = 28
};

struct Bwd2Ctx {
  uint8_t* smem;
  uint32_t bars;
  uint32_t tmem;
  volatile int* abort_flag;
  int i, bh, nht;
  __device__ __forceinline__ uint32_t bar(int idx) const { return bars + 8u * idx; }
  __device__ __forceinline__ void note_failure(int idx, uint32_t parity) const {
    atomicCAS(const_cast<int*>(abort_flag) + 1, 0, (idx + 1) | ((int)threadIdx.x << 8) | ((int)(parity & 0x7ff) << 20));
  }
  __device__ __forceinline__ bool wait(int idx, uint32_t parity) const {
    const bool ok = mbar_wait(bar(idx), parity & 1u, abort_flag);
    if (!ok) note_failure(idx, parity);
    return ok;
  }
  __device__ __forceinline__ bool wait_w(int idx, uint32_t parity) const {
    const bool ok = mbar_wait_warp(bar(idx), parity & 1u, abort_flag);
    if (!ok && (threadIdx.x & 31) == 0) note_failure(idx, parity);
    return ok;
  }
  __device__ __forceinline__ void arrive_w(int idx) const { mbar_arrive_warp(bar(idx)); }
  // half tile ht of the sweep: row tile j (descending), upper half first
  __device__ __forceinline__ int tile_j(int ht, int N) const { return N - 1 - (ht >> 1); }
  __device__ __forceinline__ int half_of(int ht) const { return 1 - (ht & 1); }
};

// ------------------------------------------------- producer + front MMA issuer --
template <int D, int kMode>
__device__ __forceinline__ void bwd2_front(const Bwd2Ctx& c, const Bwd2Params& p, const CUtensorMap* tmK, const CUtensorMap* tmV,
                                           const CUtensorMap* tmQ, const CUtensorMap* tmG) {
  using Cfg = Bwd2Cfg<D>;
  const int L = p.s.L, R = p.s.R, N = p.s.N;
  const uint32_t sb = smem_u32(c.smem);
  const int krow = c.bh * L + c.i * 128;
  const size_t chunk_id = (size_t)c.bh * N + c.i;
  constexpr uint32_t id_g = idesc_bf16(128, 64, 0, 0);

  mbar_expect_tx(c.bar(qKvFull), 2 * Cfg::kFull);
#pragma unroll
  for (int b = 0; b < Cfg::kBoxes; ++b)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      tma_load_2d(sb + Cfg::oKi + b * 16384 + h * 8192, tmK, b * 64, krow + h * 64, c.bar(qKvFull));
      tma_load_2d(sb + Cfg::oVi + b * 16384 + h * 8192, tmV, b * 64, krow + h * 64, c.bar(qKvFull));
    }

  auto row0_of = [&](int ht) { return c.tile_j(ht, N) * 128 + 64 * c.half_of(ht); };
  auto load_kj = [&](int ht) -> bool {
    const int sl = ht % Cfg::kKj, use = ht / Cfg::kKj;
    if (use >= 1 && !c.wait(qKjFree + sl, use - 1)) return false;
    mbar_expect_tx(c.bar(qKjFull + sl), Cfg::kHalf);
#pragma unroll
    for (int b = 0; b < Cfg::kBoxes; ++b)
      tma_load_2d(sb + Cfg::oKj + sl * Cfg::kHalf + b * 8192, tmK, b * 64, c.bh * L + row0_of(ht), c.bar(qKjFull + sl));
    return true;
  };
  const int total_heads = c.nht * R;
  int next_load = 0;
  auto load_head = [&](int hc) -> bool {
    const int ht = hc / R, r = hc - ht * R;
    const int sl = hc % Cfg::kNS, use = hc / Cfg::kNS;
    if (use >= 1 && !c.wait(qInFree + sl, use - 1)) return false;
    const int qrow = (c.bh * R + r) * L + row0_of(ht);
    const int grow = (kMode == 2) ? qrow : (int)((chunk_id * R + r) * L + row0_of(ht));
    const uint32_t dst = sb + Cfg::oSlot + sl * Cfg::kSlot;
    mbar_expect_tx(c.bar(qInFull + sl), 2 * Cfg::kHalf);
#pragma unroll
    for (int b = 0; b < Cfg::kBoxes; ++b) {
      tma_load_2d(dst + b * 8192, tmQ, b * 64, qrow, c.bar(qInFull + sl));
      tma_load_2d(dst + Cfg::kHalf + b * 8192, tmG, b * 64, grow, c.bar(qInFull + sl));
    }
    return true;
  };
  auto topup = [&](int upto) -> bool {
    while (next_load < total_heads && next_load <= upto) {
      if (!load_head(next_load)) return false;
      ++next_load;
    }
    return true;
  };

  // D[128 keys x 64 rows] = A[128][D] B[64][D]^T, both K-major; A boxes 16 KB apart, B boxes 8 KB apart
  auto mma_kk = [&](uint32_t d, uint32_t a_lo, uint32_t b_lo) {
    mma_ss_c<false>(d, desc_from_lo(a_lo), desc_from_lo(b_lo), id_g);
#pragma unroll
    for (int ks = 1; ks < D / 16; ++ks)
      mma_ss_c<true>(d, desc_from_lo(a_lo + (ks >> 2) * 1024 + (ks & 3) * 2), desc_from_lo(b_lo + (ks >> 2) * 512 + (ks & 3) * 2), id_g);
  };
  const uint32_t kKi = desc_lo(sb + Cfg::oKi, 16), kVi = desc_lo(sb + Cfg::oVi, 16);

  // (S, dP) buffer b is free again when its previous unit has been consumed: a G unit once the workers have loaded it,
  // a head unit once the dV MMA has read the probabilities the workers wrote over S.
  int u = 0, head_uses[2] = {0, 0};
  bool last_was_head[2] = {false, false};
  auto acquire = [&](int b) -> bool {
    const int uses = (u - b + Cfg::kNB - 1) / Cfg::kNB;            // units before u that used buffer b
    if (uses == 0) return true;
    if (last_was_head[b]) return c.wait(qMmaDone + b, head_uses[b] - 1);
    return c.wait(qLdDone + b, uses - 1);
  };
  auto unit_g = [&](int ht) -> bool {
    const int b = u % Cfg::kNB;
    if (!acquire(b)) return false;
    tc_fence_after();
    mma_kk(c.tmem + (b ? Cfg::tS1 : Cfg::tS0), kKi, desc_lo(sb + Cfg::oKj + (ht % Cfg::kKj) * Cfg::kHalf, 16));
    tc_commit(c.bar(qSFull + b));
    last_was_head[b] = false;
    ++u;
    return true;
  };

  if (!c.wait(qKvFull, 0)) return;
  if (!load_kj(0)) return;
  if (!topup(Cfg::kNS - 1)) return;
  int hc = 0;
  for (int ht = 0; ht < c.nht; ++ht) {
    if (!c.wait(qKjFull + ht % Cfg::kKj, ht / Cfg::kKj)) return;
    if (!unit_g(ht)) return;                                        // G for the decay recomputation
    if (Cfg::kKj > 1 && ht + 1 < c.nht && !load_kj(ht + 1)) return;
    for (int r = 0; r < R; ++r, ++hc) {
      const int sl = hc % Cfg::kNS, b = u % Cfg::kNB;
      if (!c.wait(qInFull + sl, hc / Cfg::kNS)) return;
      if (!acquire(b)) return;
      tc_fence_after();
      const uint32_t slot = sb + Cfg::oSlot + sl * Cfg::kSlot;
      mma_kk(c.tmem + (b ? Cfg::tS1 : Cfg::tS0), kKi, desc_lo(slot, 16));                    // S^T  = K_i Q^T
      mma_kk(c.tmem + (b ? Cfg::tP1 : Cfg::tP0), kVi, desc_lo(slot + Cfg::kHalf, 16));       // dP^T = V_i dO^T
      tc_commit(c.bar(qSFull + b));
      last_was_head[b] = true;
      ++head_uses[b];
      ++u;
      if (!topup(hc + Cfg::kNS - 1)) return;
    }
    if (!unit_g(ht)) return;                                        // G again for the decay gradient
    if (Cfg::kKj == 1 && ht + 1 < c.nht && !load_kj(ht + 1)) return;
  }
}

// ------------------------------------------------------------ back MMA issuer --
template <int D>
__device__ __forceinline__ void bwd2_back(const Bwd2Ctx& c, const Bwd2Params& p) {
  using Cfg = Bwd2Cfg<D>;
  const int R = p.s.R;
  const uint32_t sb = smem_u32(c.smem);
  constexpr uint32_t id_kn = idesc_bf16(128, D, 0, 1);     // A K-major (or TMEM), B MN-major
  constexpr uint32_t id_tn = idesc_bf16(128, D, 1, 1);     // A MN-major, B MN-major
  const uint32_t DV = c.tmem + Cfg::tDV, DK = c.tmem + Cfg::tDK, Y = c.tmem + Cfg::tY;
  const uint32_t mKi = desc_lo(sb + Cfg::oKi, 16384);      // K_i as [K = keys][N = D] (MN-major, 64-wide groups 16 KB apart)
  const uint32_t kdG = desc_lo(sb + Cfg::oDg, 16), mdG = desc_lo(sb + Cfg::oDg, 16384);
  bool have_dv = false, have_dk = false;
  int yc = 0, hc = 0;
  // Y[rows][D] = T^T K_i with T a [128 keys][64 rows] bf16 tile read MN-major; M = 128: lanes 64..127 come from the 16 KB
  // after the tile and are never read
  auto mma_rows_out = [&](uint32_t t_mn) {
    mma_ss_c<false>(Y, desc_from_lo(t_mn), desc_from_lo(mKi), id_tn);
#pragma unroll
    for (int ks = 1; ks < 8; ++ks) mma_ss_c<true>(Y, desc_from_lo(t_mn + ks * 128), desc_from_lo(mKi + ks * 128), id_tn);
  };
  for (int ht = 0; ht < c.nht; ++ht) {
    const int u0 = ht * (R + 2);
    for (int r = 0; r < R; ++r, ++hc) {
      const int b = (u0 + 1 + r) % Cfg::kNB, sl = hc % Cfg::kNS, db = hc % Cfg::kDs;
      if (!c.wait(qInFull + sl, hc / Cfg::kNS)) return;
      if (!c.wait(qDsReady + db, hc / Cfg::kDs)) return;
      tc_fence_after();
      const uint32_t slot = sb + Cfg::oSlot + sl * Cfg::kSlot;
      const uint32_t mQ = desc_lo(slot, 8192), mGo = desc_lo(slot + Cfg::kHalf, 8192);
      const uint32_t tS = c.tmem + (b ? Cfg::tS1 : Cfg::tS0);
      const uint32_t kdS = desc_lo(sb + Cfg::oDs + db * 16384, 16), mdS = desc_lo(sb + Cfg::oDs + db * 16384, 16384);
      // dV_i += P dO: P^T as bf16 pairs in TMEM, group g's 32 rows at columns [32 g, 32 g + 16)
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const uint32_t acol = (uint32_t)((ks >> 1) * 32 + (ks & 1) * 8);
        if (ks == 0 && !have_dv) mma_ts_c<false>(DV, tS + acol, desc_from_lo(mGo + ks * 128), id_kn);
        else mma_ts_c<true>(DV, tS + acol, desc_from_lo(mGo + ks * 128), id_kn);
      }
      have_dv = true;
      // dK_i += dS Q
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        if (ks == 0 && !have_dk) mma_ss_c<false>(DK, desc_from_lo(kdS + ks * 2), desc_from_lo(mQ + ks * 128), id_kn);
        else mma_ss_c<true>(DK, desc_from_lo(kdS + ks * 2), desc_from_lo(mQ + ks * 128), id_kn);
      }
      have_dk = true;
      tc_commit(c.bar(qMmaDone + b));
      tc_commit(c.bar(qInFree + sl));
      if (yc >= 1 && !c.wait(qYFree, yc - 1)) return;
      tc_fence_after();
      mma_rows_out(mdS);                                            // dQ_rj = dS^T K_i
      ++yc;
      tc_commit(c.bar(qYFull));
      tc_commit(c.bar(qDsFree + db));
    }
    if (!c.wait(qDgReady, ht)) return;
    if (yc >= 1 && !c.wait(qYFree, yc - 1)) return;
    tc_fence_after();
    mma_rows_out(mdG);                                              // dK_j = dG^T K_i
    ++yc;
    tc_commit(c.bar(qYFull));
    const uint32_t mKj = desc_lo(sb + Cfg::oKj + (ht % Cfg::kKj) * Cfg::kHalf, 8192);
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {                                // dK_i += dG K_j
      if (ks == 0 && !have_dk) mma_ss_c<false>(DK, desc_from_lo(kdG + ks * 2), desc_from_lo(mKj + ks * 128), id_kn);
      else mma_ss_c<true>(DK, desc_from_lo(kdG + ks * 2), desc_from_lo(mKj + ks * 128), id_kn);
    }
    have_dk = true;
    tc_commit(c.bar(qKjFree + ht % Cfg::kKj));
    tc_commit(c.bar(qDgFree));
  }
  tc_commit(c.bar(qFinal));
}

// --------------------------------------------------------------------- workers --
constexpr int kBarAll = 1, kBarGroup = 2, kBarDrain = 4;     // named barriers (0 is __syncthreads)

template <int D, typename TG, int kMode>
__device__ __forceinline__ void bwd2_worker(const Bwd2Ctx& c, const Bwd2Params& p, const CUtensorMap* tmDQ,
                                            const CUtensorMap* tmDK) {
  using Cfg = Bwd2Cfg<D>;
  const int L = p.s.L, R = p.s.R, N = p.s.N;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = (warp - 2) >> 2;                 // column group: columns [32 g, 32 g + 32) of a half tile
  const int quad = warp & 3;                     // TMEM lane quadrant this warp may touch
  const int slotw = (warp - 2) & 3;              // position of the warp inside its group (helper duties)
  const int key = quad * 32 + lane;
  const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
  const int col0 = 32 * g;
  const bool is_drain = quad < 2;                // the 64 result rows of dQ / dK_j sit on lanes 0..63
  const bool drain_leader = (g == 0 && quad == 0 && lane == 0);
  const float kLog2e = 1.4426950408889634f;
  const size_t chunk_id = (size_t)c.bh * N + c.i;
  const TG* ss = static_cast<const TG*>(p.ssrc) + (size_t)c.bh * L;
  const TG* sd = static_cast<const TG*>(p.sdest) + (size_t)c.bh * L;
  const float s3 = cbrtf(Num<TG>::ld(ss + c.i * 128 + key));
  float* sT3 = reinterpret_cast<float*>(c.smem + Cfg::oT3);
  float* sLse = reinterpret_cast<float*>(c.smem + Cfg::oLse);
  float* sCc = reinterpret_cast<float*>(c.smem + Cfg::oCc);
  float* sXch = reinterpret_cast<float*>(c.smem + Cfg::oXch);
  uint8_t* sStage = c.smem + Cfg::oStage;
  const uint32_t swz = (uint32_t)(key & 7);
  const int total_heads = c.nht * R;

  auto row0_of = [&](int ht) { return c.tile_j(ht, N) * 128 + 64 * c.half_of(ht); };
  auto carry_at = [&](int ht) -> float {
    return p.carry[((chunk_id * N + c.tile_j(ht, N)) * 2 + c.half_of(ht)) * 128 + key];
  };
  // helper duties, one warp of each group per table, lane = column: values of head hc for the group's 32 columns
  auto fetch_lse = [&](int hc) -> float {
    const int ht = hc / R, r = hc - ht * R;
    const int row = row0_of(ht) + col0 + lane;
    return (kMode == 2) ? p.row_lse[((size_t)c.bh * R + r) * L + row] : p.lse[(chunk_id * R + r) * L + row];
  };
  auto fetch_cc = [&](int hc) -> float {
    const int ht = hc / R, r = hc - ht * R;
    const int row = row0_of(ht) + col0 + lane;
    if (kMode == 2) return -p.row_delta[((size_t)c.bh * R + r) * L + row];
    const size_t o = (chunk_id * R + r) * L + row;
    return p.g_denom_is_f32 ? static_cast<const float*>(p.g_denom)[o]
                            : __bfloat162float(static_cast<const __nv_bfloat16*>(p.g_denom)[o]);
  };
  auto fetch_t3 = [&](int ht) -> float { return cbrtf(Num<TG>::ld(sd + row0_of(ht) + col0 + lane)); };

  // this thread's 32 columns of row `key` of a [128 keys][64 rows] bf16 tile (128-byte swizzled rows): chunks 4g .. 4g+3
  auto store_row = [&](uint8_t* base, const uint32_t* v) {
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const uint32_t ch = (uint32_t)(4 * g + x);
      *reinterpret_cast<uint4*>(base + key * 128 + (((ch ^ swz) & 7) << 4)) = make_uint4(v[4 * x], v[4 * x + 1], v[4 * x + 2], v[4 * x + 3]);
    }
  };

  // The 64 x D fp32 tile in Y (dQ_rj or dK_j, rows on lanes 0..63) is added to rows [y, y + 64) of a global accumulator:
  // the four warps of lanes 0..63 move it into the staging tile (boxes of [64][32] floats) and their leader issues
  // TMA reduce-adds, which run behind whatever follows.
  int yc = 0;
  bool pending = false;
  const CUtensorMap* pend_map = nullptr;
  int pend_row = 0;
  auto drain = [&]() -> bool {
    if (!pending) return true;
    pending = false;
    const int use = yc++;
    if (!is_drain) return true;
    if (!c.wait_w(qYFull, use)) return false;
    tc_fence_after();
    if (drain_leader) bulk_wait_read_all();           // the previous reduce-add has read the staging tile
    named_bar_sync(kBarDrain, 128);
    constexpr int kBlk = D / 64;                      // 32-column blocks per thread
#pragma unroll
    for (int hb = 0; hb < kBlk; ++hb) {
      uint32_t o[32];
      tmem_ld32(c.tmem + Cfg::tY + lane_base + (D / 2) * g + 32 * hb, o);
      tc_wait_ld();
      if (hb == kBlk - 1) {
        tc_fence_before();
        c.arrive_w(qYFree);
      }
      uint8_t* box = sStage + (kBlk * g + hb) * 8192 + key * 128;
#pragma unroll
      for (int x = 0; x < 8; ++x)
        *reinterpret_cast<uint4*>(box + ((((uint32_t)x ^ swz) & 7) << 4)) = make_uint4(o[4 * x], o[4 * x + 1], o[4 * x + 2], o[4 * x + 3]);
    }
    fence_proxy_async();
    named_bar_sync(kBarDrain, 128);
    if (drain_leader) {
#pragma unroll
      for (int bx = 0; bx < D / 32; ++bx) tma_reduce_add_2d(pend_map, 32 * bx, pend_row, smem_u32(sStage) + bx * 8192);
      bulk_commit_group();
    }
    __syncwarp();
    return true;
  };

  // ---- prologue: tables of the first half tile / first head ----
  if (slotw == 0) sLse[col0 + lane] = fetch_lse(0) * kLog2e;
  if (slotw == 1) sCc[col0 + lane] = fetch_cc(0);
  if (slotw == 2) sT3[col0 + lane] = fetch_t3(0);
  float carry_next = carry_at(0);
  float suffix = 0.f, ds_acc = 0.f;
  named_bar_sync(kBarAll, 256);

  int u = 0, hc = 0;
  for (int ht = 0; ht < c.nht; ++ht) {
    const int j = c.tile_j(ht, N), half = c.half_of(ht), row0 = j * 128 + 64 * half;
    const bool diag = (j == c.i);
    const int qbase = 64 * half + col0;            // row of this thread's first column inside the 128-row tile
    const float* t3v = sT3 + (ht & 1) * 64 + col0;

    // ================= decay recomputation: C2 = log2(e) * decay prefix of (key, 32 rows) =================
    float c2[32];
    {
      const float carry = carry_next;
      const int b = u % Cfg::kNB;
      if (!c.wait_w(qSFull + b, u / Cfg::kNB)) return;
      tc_fence_after();
      uint32_t gr[32];
      tmem_ld32(c.tmem + (b ? Cfg::tS1 : Cfg::tS0) + lane_base + col0, gr);
      tc_wait_ld();
      tc_fence_before();
      c.arrive_w(qLdDone + b);
      ++u;
      float run = 0.f;
#pragma unroll
      for (int x = 0; x < 32; ++x) {
        float e = log_retention(gated_affinity(gram_pow23(__uint_as_float(gr[x])), s3, t3v[x]));
        if (diag && qbase + x <= key) e = 0.f;
        run += e;
        c2[x] = run;
      }
      if (g == 0) sXch[key] = run;
      named_bar_sync(kBarAll, 256);
      const float base = carry + (g == 1 ? sXch[key] : 0.f);
#pragma unroll
      for (int x = 0; x < 32; ++x) {
        float v = base + c2[x];
        if (diag && qbase + x < key) v = mask_value();
        c2[x] = v * kLog2e;
      }
    }

    // ================= heads =================
    float dc[32];
#pragma unroll
    for (int x = 0; x < 32; ++x) dc[x] = 0.f;
    for (int r = 0; r < R; ++r, ++hc) {
      const bool has_next = hc + 1 < total_heads;
      float pre = 0.f;                             // next head's table entry, stored below (its load latency is hidden)
      if (has_next && slotw == 0) pre = fetch_lse(hc + 1) * kLog2e;
      if (has_next && slotw == 1) pre = fetch_cc(hc + 1);
      const int b = u % Cfg::kNB, tb = hc % 3, db = hc % Cfg::kDs;
      if (!c.wait_w(qSFull + b, u / Cfg::kNB)) return;
      tc_fence_after();
      float pv[32];
      uint32_t dp[32];
      {
        uint32_t sr[32];
        tmem_ld32(c.tmem + (b ? Cfg::tS1 : Cfg::tS0) + lane_base + col0, sr);
        tmem_ld32(c.tmem + (b ? Cfg::tP1 : Cfg::tP0) + lane_base + col0, dp);
        tc_wait_ld();
        tc_fence_before();
        c.arrive_w(qLdDone + b);
        ++u;
        const float* l2 = sLse + tb * 64 + col0;
#pragma unroll
        for (int x = 0; x < 32; ++x) pv[x] = ex2(fmaf(__uint_as_float(sr[x]), kLog2e, c2[x] - l2[x]));
      }
      if (kMode == 1) {
        float e[32];
#pragma unroll
        for (int x = 0; x < 32; ++x) e[x] = pv[x] * __uint_as_float(dp[x]);
        const float part = warp_transpose_reduce(e, lane);           // this warp's 32 keys, column col0 + lane
        atomicAdd(sCc + tb * 64 + col0 + lane, -part);
      }
      if (has_next && slotw == 0) sLse[((hc + 1) % 3) * 64 + col0 + lane] = pre;
      if (has_next && slotw == 1) sCc[((hc + 1) % 3) * 64 + col0 + lane] = pre;
      if (!drain()) return;                        // the previous head's dQ (or the previous half tile's dK_j)
      named_bar_sync(kBarGroup + g, 128);
      uint32_t pk[16], dk[16];
      {
        const float* cc = sCc + tb * 64 + col0;
#pragma unroll
        for (int x = 0; x < 16; ++x) {
          const float d0 = pv[2 * x] * (__uint_as_float(dp[2 * x]) + cc[2 * x]);
          const float d1 = pv[2 * x + 1] * (__uint_as_float(dp[2 * x + 1]) + cc[2 * x + 1]);
          dc[2 * x] += d0;
          dc[2 * x + 1] += d1;
          __nv_bfloat162 hp = __floats2bfloat162_rn(pv[2 * x], pv[2 * x + 1]), hd = __floats2bfloat162_rn(d0, d1);
          pk[x] = *reinterpret_cast<uint32_t*>(&hp);
          dk[x] = *reinterpret_cast<uint32_t*>(&hd);
        }
      }
      if (hc >= Cfg::kDs && !c.wait_w(qDsFree + db, hc / Cfg::kDs - 1)) return;
      store_row(c.smem + Cfg::oDs + db * 16384, dk);
      tmem_st16(c.tmem + (b ? Cfg::tS1 : Cfg::tS0) + lane_base + col0, pk);      // P^T over this group's own S columns
      tc_wait_st();
      fence_proxy_async();
      tc_fence_before();
      c.arrive_w(qDsReady + db);
      pending = true;
      pend_map = tmDQ;
      pend_row = (c.bh * R + r) * L + row0;
    }

    // ================= decay gradient =================
    {
      const bool more = ht + 1 < c.nht;
      if (more) carry_next = carry_at(ht + 1);
      float t3pre = 0.f;
      if (more && slotw == 2) t3pre = fetch_t3(ht + 1);
      float run = 0.f;
#pragma unroll
      for (int x = 31; x >= 0; --x) {
        run += dc[x];
        dc[x] = run;                               // sum of dC over this thread's columns x .. 31
      }
      sXch[(1 + g) * 128 + key] = run;
      if (more && slotw == 2) sT3[((ht + 1) & 1) * 64 + col0 + lane] = t3pre;
      if (!drain()) return;                        // the last head's dQ
      named_bar_sync(kBarAll, 256);
      const float other = sXch[(2 - g) * 128 + key];
      const float add = suffix + (g == 0 ? other : 0.f);      // rows after this thread's block
      suffix = suffix + run + other;                          // ... after this half tile (the next one lies below it)

      const int b = u % Cfg::kNB;
      if (!c.wait_w(qSFull + b, u / Cfg::kNB)) return;
      tc_fence_after();
      uint32_t gr[32];
      tmem_ld32(c.tmem + (b ? Cfg::tS1 : Cfg::tS0) + lane_base + col0, gr);
      tc_wait_ld();
      tc_fence_before();
      c.arrive_w(qLdDone + b);
      ++u;
      uint32_t pk[16];
      float dg_hold = 0.f;
#pragma unroll
      for (int x = 31; x >= 0; --x) {
        float dl = dc[x] + add;
        if (diag && qbase + x <= key) dl = 0.f;
        const float gv = __uint_as_float(gr[x]);
        const float t3 = t3v[x];
        const float lg = lg2(gv);                                  // NaN for gv < 0: guarded below
        const float pw = gv > 0.f ? ex2(lg * (2.0f / 3.0f)) : 0.f;
        const float a = gated_affinity(pw, s3, t3);
        float da = __fdividef(dl, fminf(fmaxf(a, clamp_lo_bwd()), clamp_hi()) - 1.0f);
        if (!(a <= clamp_hi())) da = 0.f;
        const float dstat = da * pw;
        ds_acc = fmaf(dstat, t3, ds_acc);
        dc[x] = dstat * s3;                                        // reuse: per-(key, row) term of d static_dest
        float dg = __bfloat162float(__float2bfloat16_rn(da * s3 * t3));
        dg = gv > 0.f ? dg * (2.0f / 3.0f) * ex2(lg * (-1.0f / 3.0f)) : 0.f;
        if (x & 1) {
          dg_hold = dg;
        } else {
          __nv_bfloat162 h = __floats2bfloat162_rn(dg, dg_hold);
          pk[x >> 1] = *reinterpret_cast<uint32_t*>(&h);
        }
      }
      if (ht >= 1 && !c.wait_w(qDgFree, ht - 1)) return;
      store_row(c.smem + Cfg::oDg, pk);
      fence_proxy_async();
      c.arrive_w(qDgReady);
      pending = true;
      pend_map = tmDK;
      pend_row = c.bh * L + row0;
      // d static_dest: sum over the 128 keys of dstat * src^(1/3)
      const float colsum = warp_transpose_reduce(dc, lane);
      const float t3l = t3v[lane];
      if (colsum != 0.f) atomicAdd(p.acc_dt + (size_t)c.bh * L + row0 + col0 + lane, colsum / (3.0f * t3l * t3l));
    }
  }
  if (!drain()) return;                            // the last half tile's dK_j

  // ---- end of the sweep: dV_i, dK_i, d static_src (thread = key, D/2 columns each) ----
  if (!c.wait_w(qFinal, 0)) return;
  tc_fence_after();
  const size_t krow = (size_t)c.bh * L + c.i * 128 + key;
#pragma unroll
  for (int hb = 0; hb < D / 64; ++hb) {
    const int d0 = (D / 2) * g + 32 * hb;
    uint32_t o[32];
    tmem_ld32(c.tmem + Cfg::tDV + lane_base + d0, o);
    tc_wait_ld();
    if (p.acc_dv_in) {
      const float4* extra = reinterpret_cast<const float4*>(p.acc_dv_in + krow * D + d0);
#pragma unroll
      for (int x = 0; x < 8; ++x) {
        const float4 ev = extra[x];
        o[4 * x] = __float_as_uint(__uint_as_float(o[4 * x]) + ev.x);
        o[4 * x + 1] = __float_as_uint(__uint_as_float(o[4 * x + 1]) + ev.y);
        o[4 * x + 2] = __float_as_uint(__uint_as_float(o[4 * x + 2]) + ev.z);
        o[4 * x + 3] = __float_as_uint(__uint_as_float(o[4 * x + 3]) + ev.w);
      }
    }
    uint32_t pk[16];
#pragma unroll
    for (int x = 0; x < 16; ++x) {
      __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(o[2 * x]), __uint_as_float(o[2 * x + 1]));
      pk[x] = *reinterpret_cast<uint32_t*>(&h);
    }
    uint4* dst = reinterpret_cast<uint4*>(p.dvc + krow * D + d0);
#pragma unroll
    for (int x = 0; x < 4; ++x) dst[x] = make_uint4(pk[4 * x], pk[4 * x + 1], pk[4 * x + 2], pk[4 * x + 3]);
    tmem_ld32(c.tmem + Cfg::tDK + lane_base + d0, o);
    tc_wait_ld();
    float* dkp = p.acc_dk + krow * D + d0;
#pragma unroll
    for (int x = 0; x < 8; ++x)
      red_add_v4(dkp + 4 * x, __uint_as_float(o[4 * x]), __uint_as_float(o[4 * x + 1]), __uint_as_float(o[4 * x + 2]),
                 __uint_as_float(o[4 * x + 3]));
  }
  if (g == 1) sXch[key] = ds_acc;
  named_bar_sync(kBarAll, 256);
  if (g == 0) Num<TG>::st(static_cast<TG*>(p.dss) + krow, (ds_acc + sXch[key]) / (3.0f * s3 * s3));
}

template <int D, typename TG, int kMode>
__global__ void __launch_bounds__(320, 1)
bwd2_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
            const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmG,
            const __grid_constant__ CUtensorMap tmDQ, const __grid_constant__ CUtensorMap tmDK, Bwd2Params p) {
  using Cfg = Bwd2Cfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint32_t* misc = reinterpret_cast<uint32_t*>(smem + Cfg::oMisc);      // [0] TMEM base, [1] abort flag, [2] failure note
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int BH = p.s.B * p.s.H;

  Bwd2Ctx c;
  c.smem = smem;
  c.bars = smem_u32(smem + Cfg::oBar);
  c.abort_flag = reinterpret_cast<volatile int*>(misc + 1);
  c.i = blockIdx.x / BH;                       // heavy chunks (small i: most rows) first
  c.bh = blockIdx.x - c.i * BH;
  c.nht = 2 * (p.s.N - c.i);

  if (threadIdx.x == 0) {
    misc[1] = 0;
    misc[2] = 0;
    for (int b = 0; b < qNumBars; ++b) {
      uint32_t count = 1;
      if (b == qLdDone || b == qLdDone + 1 || b == qDsReady || b == qDsReady + 1 || b == qDgReady) count = 8;   // one arrival per worker warp
      if (b == qYFree) count = 4;                                                                            // the four draining warps
      mbar_init(c.bar(b), count);
    }
    mbar_init_fence();
    prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmQ); prefetch_tmap(&tmG);
    prefetch_tmap(&tmDQ); prefetch_tmap(&tmDK);
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(misc), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  c.tmem = misc[0];

  if (warp == 0) {
    if (lane == 0) bwd2_front<D, kMode>(c, p, &tmK, &tmV, &tmQ, &tmG);
  } else if (warp == 1) {
    if (lane == 0) bwd2_back<D>(c, p);
  } else {
    bwd2_worker<D, TG, kMode>(c, p, &tmDQ, &tmDK);
    if (warp == 4 && lane == 0) bulk_wait_all();      // the leader's reduce-adds have landed before the block retires
  }

  tc_fence_before();
  __syncthreads();
  if (*c.abort_flag) {
    if (threadIdx.x == 0) {
      if (atomicExch(p.status, 3) == 0) p.status[1] = (int)misc[2];
    }
    for (int it = 0; it < 64; ++it) __nanosleep(2000);
    __syncthreads();
  }
  if (warp == 0) tmem_dealloc(c.tmem, 512);
}

}  // namespace sm100
}  // namespace ua
