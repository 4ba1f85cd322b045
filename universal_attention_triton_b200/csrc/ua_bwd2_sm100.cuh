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
//        dS = P (dP - sum_k P dP + g_denom) (the sum over the keys is the one cross-lane step: a transpose
//                                             per warp through a shared-memory scratch tile or by shuffles,
//                                             then shared-memory adds across the four warps of a group)
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
// Warps: 0 = "front" MMA issuer (G, S, dP: everything that only needs loaded tiles), 1 and 3 = "back" MMA issuers
// (1: dV, dK_i; 3: dQ, dK_j: everything that needs a tile the workers wrote), 2 = TMA producer, 4.. = workers:
// 64 / CG column groups of 128 threads (thread = key, CG of the 64 columns each, held in registers; CG = 16 or 32).
// dQ_rj / dK_j (64 rows, M = 128 MMAs whose upper 64 lanes compute on whatever the next buffer holds and are
// never read) leave as TMA reduce-adds into fp32 accumulators.  Rows BEFORE the chunk are not handled here.
//
// Every mbarrier wait is bounded; on a timeout the block raises a shared abort flag, every role
// leaves, TMEM is freed and status[0] is set (status[1]: where the first block gave up).
#pragma once
#include <type_traits>

#include "ua_fwd_sm100.cuh"

namespace ua {
namespace sm100 {

struct Bwd2Params {
  Shape s;
  const void* ssrc;
  const void* sdest;
  const float* g_denom;      // (b,h,n,r,L) fp32                             [mode 1]
  const float* lse;          // (b,h,n,r,L) fp32: the forward's log-sum-exp   [mode 1]
  const float* row_lse;      // (b,h,r,L) fp32: log-sum-exp over all keys     [mode 2]
  const float* row_delta;    // (b,h,r,L) fp32: g . merged                    [mode 2]
  const float* carry;        // (b*h*n, n, 2, 128): decay prefix of key k at the start of each 64-row half tile
  float* acc_dk;             // (b*h, L, D) fp32, zeroed (or holding the masked-block part)
  float* acc_dq;             // (b*h, r, L, D) fp32, likewise
  float* acc_dt;             // (b*h, Lr) fp32: d static_dest is ADDED here (by row_side_finish_kernel, after the sweep)
  float* acc_dkr;            // (b*h, L, D) fp32 scratch, zeroed: the row-side dK_j = dG^T K_i of all chunks (see there)
  const float* dv_chunk;     // optional: row dv_chunk[chunk * dv_chunk_stride + d] / 128 is added to every key's dV_i (the
  int dv_chunk_stride;       // masked-block part when it comes from the kernels of the rows before a chunk)
  __nv_bfloat16* dvc;
  void* dss;
  int* status;
  long long* trace;          // profile builds only: per-unit time stamps of block UA_PROFILE_BLOCK (else null)
  // Range of row tiles [j_begin, j_end) (sequence-chunk sharding; whole sequence: 0, N, L, 0).  The row-indexed tensors
  // (xq, g_out, g_denom, lse, static_dest, acc_dq, acc_dt) are slabs of Lr rows that hold the range at row r0; keys,
  // values, static_src and the key-side accumulators always span the whole sequence.
  int j_begin, j_end, Lr, r0;
  int heads;                 // query heads to process: R, or 0 for the correction pass (only what suffix_in induces)
  const float* suffix_in;    // optional (b*h*n, 128): reverse decay carry entering from the rows after the range
  float* dctot_out;          // optional (b*h*n, 128): per key, sum of dC over the rows of the range (what earlier ranges need)
  float* acc_dv;             // optional (b*h, L, D) fp32: dV_i is ADDED here instead of being written to dvc
  float* acc_ds;             // optional (b*h, L) fp32: d static_src is ADDED here instead of being written to dss
  // optional [mode 1, head_dim 64]: the forward's output tiles (b,h,n,r,Lr,D), laid out like g_out.  With them the
  // softmax-gradient row term sum_k P dP is the dot product of a row's output and its upstream gradient (P V = out), which
  // two otherwise idle warps form ahead of the workers; without them the workers sum P dP over the keys themselves.
  const void* out_tiles;
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
  static constexpr int oT3 = oStage + 256 * D;             // float [2][64]: static_dest^(1/3) of a half tile's rows
  // per-row tables that the producer copies next to the tiles (no global load is ever issued by a worker):
  static constexpr int oHeadTab = oT3 + 512;               // kNS x { float lse[64]; float cc[64] }: log-sum-exp and g_denom (or delta) of a head's rows
  static constexpr int kTab = 3;                           // half-tile tables in flight
  static constexpr int kHtTab = 768;                       // { float carry[128]; raw static_dest[64] (<= 256 B) }
  static constexpr int oHtTab = oHeadTab + kNS * 512;
  static constexpr int oXch = oHtTab + kTab * kHtTab;      // float [8][128] totals crossing the column groups
  static constexpr int oBar = oXch + 4096;
  static constexpr int oMisc = oBar + 320;      // (35 barriers of 8 bytes)
  // per-warp scratch tiles for the column sums over the keys ([32 lanes][CG + 4] floats each, at most 40 KB in all);
  // head_dim 128 has no room for them and transposes with shuffles
  static constexpr bool kScratch = (D == 64);
  static constexpr int oScr = oMisc + 256;
  static constexpr int kSmemBytes = oScr + (kScratch ? 40960 : 0) + 1024;     // + slack to align the base to 1024 B
  // builds that take the row term from the forward's output tiles (head_dim 64) keep kNS output half tiles where the
  // scratch tiles would be, and sum the decay gradient's columns with shuffles
  static constexpr bool kOutTiles = kScratch;
  static constexpr int oOut = (oScr + 1023) / 1024 * 1024;
  static_assert(!kOutTiles || oOut + kNS * kHalf <= oScr + 40960, "output tiles fit the scratch area");
  // TMEM columns
  static constexpr uint32_t tDV = 0, tDK = D, tY = 2 * D;
  static constexpr uint32_t tS0 = (D == 64) ? 192 : 384, tP0 = tS0 + 64, tS1 = tS0 + 128, tP1 = tS0 + 192;
  // probabilities (bf16 pairs, 32 columns per head): a buffer pair of their own where TMEM has room, else over S
  static constexpr bool kPtSeparate = (D == 64);
  static constexpr uint32_t tPT = 448;
  static_assert(D == 64 || D == 128, "head_dim 64 or 128");
  static_assert(D == 64 ? (tP1 + 64 <= 512) : (tP0 + 64 <= 512), "TMEM budget");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

enum Bwd2Bar {
  qKvFull = 0,
  qKjFull = 1, qKjFree = 3,        // [2]
  qInFull = 5, qInFree = 9,        // [4]
  qSFull = 13, qLdDone = 15, qPtFree = 17,   // [2] per (S, dP) buffer / per probability buffer
  qDsReady = 19, qDsFree = 21,     // [2] per dS buffer
  qYFull = 23, qYFree = 24, qDgReady = 25, qDgFree = 26, qFinal = 27,
  qTabFull = 28,                   // [3] per half-tile table buffer
  qDelta = 31,                     // [4] per (Q, dO) slot: the row term of the head's table is final (output-tile builds)
  qNumBars = 35
};

struct Bwd2Ctx {
  uint8_t* smem;
  uint32_t bars;
  uint32_t tmem;
  volatile int* abort_flag;
  int i, bh, nht;
  int jtop, jb, r0;          // the sweep starts at row tile jtop - 1; the slabs hold row tile jb at row r0
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
  __device__ __forceinline__ int tile_j(int ht) const { return jtop - 1 - (ht >> 1); }
  __device__ __forceinline__ int half_of(int ht) const { return 1 - (ht & 1); }
  // first row of half tile ht: in the sequence (keys of the same positions, the diagonal), and inside the slabs
  __device__ __forceinline__ int row0_of(int ht) const { return tile_j(ht) * 128 + 64 * half_of(ht); }
  __device__ __forceinline__ int srow0_of(int ht) const { return r0 + (tile_j(ht) - jb) * 128 + 64 * half_of(ht); }
};

// Optional phase timing (compile with -DUA_PROFILE_BWD2): thread 0 of worker warp 4 of block UA_PROFILE_BLOCK accumulates
// clock64() deltas per phase and stores them after the status words.
#ifdef UA_PROFILE_BWD2
#ifndef UA_PROFILE_BLOCK
#define UA_PROFILE_BLOCK 0
#endif
#define UQ_DECL long long uq_t = clock64(), uq_acc[16] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
#define UQ(idx) { long long now_ = clock64(); uq_acc[idx] += now_ - uq_t; uq_t = now_; }
#define UQ_STORE if (blockIdx.x == UA_PROFILE_BLOCK && warp == 8 && lane == 0) { for (int z = 0; z < 16; ++z) reinterpret_cast<long long*>(p.status)[2 + z] = uq_acc[z]; }
#define UQ_STORE_AT(base) if (blockIdx.x == UA_PROFILE_BLOCK) { for (int z = 0; z < 4; ++z) reinterpret_cast<long long*>(p.status)[2 + (base) + z] = uq_acc[z]; }
#define UQ_TRACE(unit, slot) if (p.trace && blockIdx.x == UA_PROFILE_BLOCK && (unit) < 96) p.trace[(unit) * 8 + (slot)] = clock64();
#else
#define UQ_DECL
#define UQ(idx)
#define UQ_STORE
#define UQ_STORE_AT(base)
#define UQ_TRACE(unit, slot)
#endif

// Four tcgen05.mma of one accumulation chain from ONE asm statement: what limits a single issuing thread is the
// instruction count per MMA (descriptor arithmetic, predicate set-up), so the chain shares one predicate set-up and
// advances the 64-bit descriptors by immediate-like steps (in 16-byte units of the descriptor's address field).
__device__ __forceinline__ void mma4_ss(uint32_t d, uint64_t a, uint64_t b, uint64_t sa, uint64_t sb, uint32_t idesc, uint32_t acc_first) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b64 a1, a2, a3, b1, b2, b3;\n\t"
      "setp.ne.b32 p, %6, 0;\n\tsetp.eq.u32 q, 1, 1;\n\t"
      "add.s64 a1, %1, %3;\n\tadd.s64 b1, %2, %4;\n\tadd.s64 a2, a1, %3;\n\tadd.s64 b2, b1, %4;\n\t"
      "add.s64 a3, a2, %3;\n\tadd.s64 b3, b2, %4;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %5, p;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %5, q;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a2, b2, %5, q;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], a3, b3, %5, q;\n\t}" ::"r"(d),
      "l"(a), "l"(b), "l"(sa), "l"(sb), "r"(idesc), "r"(acc_first)
      : "memory");
}
// ... with the A operand in TMEM at four given column addresses
__device__ __forceinline__ void mma4_ts(uint32_t d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint64_t b, uint64_t sb,
                                        uint32_t idesc, uint32_t acc_first) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b64 b1, b2, b3;\n\t"
      "setp.ne.b32 p, %8, 0;\n\tsetp.eq.u32 q, 1, 1;\n\t"
      "add.s64 b1, %5, %6;\n\tadd.s64 b2, b1, %6;\n\tadd.s64 b3, b2, %6;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %5, %7, p;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%2], b1, %7, q;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%3], b2, %7, q;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%4], b3, %7, q;\n\t}" ::"r"(d),
      "r"(a0), "r"(a1), "r"(a2), "r"(a3), "l"(b), "l"(sb), "r"(idesc), "r"(acc_first)
      : "memory");
}

// ------------------------------------------------------------- TMA producer --
template <int D, typename TG, int kMode, bool kOutDelta>
__device__ __forceinline__ void bwd2_producer(const Bwd2Ctx& c, const Bwd2Params& p, const CUtensorMap* tmK, const CUtensorMap* tmV,
                                              const CUtensorMap* tmQ, const CUtensorMap* tmG, const CUtensorMap* tmO) {
  using Cfg = Bwd2Cfg<D>;
  const int L = p.s.L, R = p.s.R, N = p.s.N;
  const uint32_t sb = smem_u32(c.smem);
  const int krow = c.bh * L + c.i * 128;
  const size_t chunk_id = (size_t)c.bh * N + c.i;
  mbar_expect_tx(c.bar(qKvFull), 2 * Cfg::kFull);
#pragma unroll
  for (int b = 0; b < Cfg::kBoxes; ++b)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      tma_load_2d(sb + Cfg::oKi + b * 16384 + h * 8192, tmK, b * 64, krow + h * 64, c.bar(qKvFull));
      tma_load_2d(sb + Cfg::oVi + b * 16384 + h * 8192, tmV, b * 64, krow + h * 64, c.bar(qKvFull));
    }
  // per-half-tile tables: decay prefix of the 128 keys at the start of the half tile, raw static_dest of its 64 rows
  const TG* sd = static_cast<const TG*>(p.sdest) + (size_t)c.bh * p.Lr;
  const int Rh = p.heads;
  auto load_tables = [&](int ht) -> bool {
    const int tb = ht % Cfg::kTab, use = ht / Cfg::kTab;
    if (use >= 1 && !c.wait(qDgReady, ht - Cfg::kTab)) return false;      // the half tile that used the buffer is done with it
    const uint32_t dst = sb + Cfg::oHtTab + tb * Cfg::kHtTab;
    // (the correction pass has no heads and needs no decay prefix: only the gate values travel)
    mbar_expect_tx(c.bar(qTabFull + tb), (Rh > 0 ? 512u : 0u) + 64 * (uint32_t)sizeof(TG));
    if (Rh > 0)
      bulk_load_1d(dst, p.carry + ((chunk_id * N + c.tile_j(ht)) * 2 + c.half_of(ht)) * 128, 512, c.bar(qTabFull + tb));
    bulk_load_1d(dst + 512, sd + c.srow0_of(ht), 64 * (uint32_t)sizeof(TG), c.bar(qTabFull + tb));
    return true;
  };
  if (!load_tables(0)) return;
  // in sweep order: K_j of half tile ht, then the (Q, dO) pairs of its heads (with the log-sum-exp and g_denom rows of
  // the head); a slot is refilled as soon as the MMAs that read it have completed
  int hc = 0;
  for (int ht = 0; ht < c.nht; ++ht) {
    const int row0 = c.row0_of(ht), srow0 = c.srow0_of(ht);
    if (ht + 1 < c.nht && !load_tables(ht + 1)) return;
    {
      const int sl = ht % Cfg::kKj, use = ht / Cfg::kKj;
      if (use >= 1 && !c.wait(qKjFree + sl, use - 1)) return;
      mbar_expect_tx(c.bar(qKjFull + sl), Cfg::kHalf);
#pragma unroll
      for (int b = 0; b < Cfg::kBoxes; ++b)
        tma_load_2d(sb + Cfg::oKj + sl * Cfg::kHalf + b * 8192, tmK, b * 64, c.bh * L + row0, c.bar(qKjFull + sl));
    }
    for (int r = 0; r < Rh; ++r, ++hc) {
      const int sl = hc % Cfg::kNS, use = hc / Cfg::kNS;
      if (use >= 1 && !c.wait(qInFree + sl, use - 1)) return;
      const int qrow = (c.bh * R + r) * p.Lr + srow0;
      const int grow = (kMode == 2) ? qrow : (int)((chunk_id * R + r) * p.Lr + srow0);
      const uint32_t dst = sb + Cfg::oSlot + sl * Cfg::kSlot, tab = sb + Cfg::oHeadTab + sl * 512;
      mbar_expect_tx(c.bar(qInFull + sl), (kOutDelta ? 3 : 2) * Cfg::kHalf + 512);
      if (kOutDelta) tma_load_2d(sb + Cfg::oOut + sl * Cfg::kHalf, tmO, 0, grow, c.bar(qInFull + sl));
#pragma unroll
      for (int b = 0; b < Cfg::kBoxes; ++b) {
        tma_load_2d(dst + b * 8192, tmQ, b * 64, qrow, c.bar(qInFull + sl));
        tma_load_2d(dst + Cfg::kHalf + b * 8192, tmG, b * 64, grow, c.bar(qInFull + sl));
      }
      if (kMode == 2) {
        bulk_load_1d(tab, p.row_lse + qrow, 256, c.bar(qInFull + sl));
        bulk_load_1d(tab + 256, p.row_delta + qrow, 256, c.bar(qInFull + sl));
      } else {
        bulk_load_1d(tab, p.lse + grow, 256, c.bar(qInFull + sl));
        bulk_load_1d(tab + 256, p.g_denom + grow, 256, c.bar(qInFull + sl));
      }
    }
  }
}

// ----------------------------------------------------------- front MMA issuer --
// G, S^T and dP^T: everything that only needs loaded tiles and a free (S, dP) buffer.
template <int D>
__device__ __forceinline__ void bwd2_front(const Bwd2Ctx& c, const Bwd2Params& p) {
  using Cfg = Bwd2Cfg<D>;
  const int R = p.heads;
  const uint32_t sb = smem_u32(c.smem);
  constexpr uint32_t id_g = idesc_bf16(128, 64, 0, 0);
  // D[128 keys x 64 rows] = A[128][D] B[64][D]^T, both K-major; A boxes 16 KB apart, B boxes 8 KB apart
  auto mma_kk = [&](uint32_t d, uint32_t a_lo, uint32_t b_lo) {
    mma4_ss(d, desc_from_lo(a_lo), desc_from_lo(b_lo), 2, 2, id_g, 0);
    if (D == 128) mma4_ss(d, desc_from_lo(a_lo + 1024), desc_from_lo(b_lo + 512), 2, 2, id_g, 1);
  };
  const uint32_t kKi = desc_lo(sb + Cfg::oKi, 16), kVi = desc_lo(sb + Cfg::oVi, 16);

  // (S, dP) buffer b is free again when its previous unit has been consumed: once the workers have loaded it, or -- where
  // the probabilities are written over S (head_dim 128) -- once the dV MMA of a head unit has read them.
  int u = 0, head_uses[2] = {0, 0};
  bool last_was_head[2] = {false, false};
  auto acquire = [&](int b) -> bool {
    const int uses = u / Cfg::kNB;                                // units before u that used buffer b = u % kNB
    if (uses == 0) return true;
    if (!Cfg::kPtSeparate && last_was_head[b]) return c.wait(qPtFree + b, head_uses[b] - 1);
    return c.wait(qLdDone + b, uses - 1);
  };
  auto unit_g = [&](int ht) -> bool {
    const int b = u % Cfg::kNB;
    if (!acquire(b)) return false;
    tc_fence_after();
    mma_kk(c.tmem + (b ? Cfg::tS1 : Cfg::tS0), kKi, desc_lo(sb + Cfg::oKj + (ht % Cfg::kKj) * Cfg::kHalf, 16));
    tc_commit(c.bar(qSFull + b));
    UQ_TRACE(u, 0)
    last_was_head[b] = false;
    ++u;
    return true;
  };

  if (!c.wait(qKvFull, 0)) return;
  int hc = 0;
  UQ_DECL
  for (int ht = 0; ht < c.nht; ++ht) {
    if (!c.wait(qKjFull + ht % Cfg::kKj, ht / Cfg::kKj)) return;
    if (R > 0 && !unit_g(ht)) return;                               // G for the decay recomputation (none without heads)
    UQ(0)
    for (int r = 0; r < R; ++r, ++hc) {
      const int sl = hc % Cfg::kNS, b = u % Cfg::kNB;
      if (!c.wait(qInFull + sl, hc / Cfg::kNS)) return;
      UQ(1)
      if (!acquire(b)) return;
      UQ(2)
      UQ_TRACE(u, 4)
      tc_fence_after();
      const uint32_t slot = sb + Cfg::oSlot + sl * Cfg::kSlot;
      mma_kk(c.tmem + (b ? Cfg::tS1 : Cfg::tS0), kKi, desc_lo(slot, 16));                    // S^T  = K_i Q^T
      mma_kk(c.tmem + (b ? Cfg::tP1 : Cfg::tP0), kVi, desc_lo(slot + Cfg::kHalf, 16));       // dP^T = V_i dO^T
      tc_commit(c.bar(qSFull + b));
      UQ_TRACE(u, 0)
      last_was_head[b] = true;
      ++head_uses[b];
      ++u;
      UQ(3)
    }
    if (!unit_g(ht)) return;                                        // G again for the decay gradient
    UQ(0)
  }
  UQ_STORE_AT(16)
}

// ------------------------------------------------------------ back MMA issuers --
// which = 0: the accumulators that live for the whole sweep (dV_i += P dO, dK_i += dS Q, dK_i += dG K_j);
// which = 1: the row-side results that leave after every unit (Y = dQ_rj = dS^T K_i, Y = dK_j = dG^T K_i).
// MMAs into one accumulator always come from the same thread, so their order is kept.
template <int D, int CG>
__device__ __forceinline__ void bwd2_back(const Bwd2Ctx& c, const Bwd2Params& p, const int which) {
  using Cfg = Bwd2Cfg<D>;
  const int R = p.heads;
  const uint32_t sb = smem_u32(c.smem);
  constexpr uint32_t id_kn = idesc_bf16(128, D, 0, 1);     // A K-major (or TMEM), B MN-major
  constexpr uint32_t id_tn = idesc_bf16(128, D, 1, 1);     // A MN-major, B MN-major
  const uint32_t DV = c.tmem + Cfg::tDV, DK = c.tmem + Cfg::tDK, Y = c.tmem + Cfg::tY;
  const uint64_t mKi = desc_from_lo(desc_lo(sb + Cfg::oKi, 16384));      // K_i as [K = keys][N = D] (MN-major, 64-wide groups 16 KB apart)
  const uint64_t kdG = desc_from_lo(desc_lo(sb + Cfg::oDg, 16)), mdG = desc_from_lo(desc_lo(sb + Cfg::oDg, 16384));
  uint32_t have_dv = 0, have_dk = 0;
  int yc = 0, hc = 0;
  // Y[rows][D] = T^T K_i with T a [128 keys][64 rows] bf16 tile read MN-major; M = 128: lanes 64..127 come from the 16 KB
  // after the tile and are never read
  auto mma_rows_out = [&](uint64_t t_mn) {
    mma4_ss(Y, t_mn, mKi, 128, 128, id_tn, 0);
    mma4_ss(Y, t_mn + 512, mKi + 512, 128, 128, id_tn, 1);
  };
  if (!c.wait(qKvFull, 0)) return;
  UQ_DECL
  for (int ht = 0; ht < c.nht; ++ht) {
    const int u0 = ht * (R + 2);
    for (int r = 0; r < R; ++r, ++hc) {
      const int b = (u0 + 1 + r) % Cfg::kNB, sl = hc % Cfg::kNS, db = hc % Cfg::kDs;
      const uint32_t dsb = sb + Cfg::oDs + db * 16384;
      UQ(0)
      if (!c.wait(qDsReady + db, hc / Cfg::kDs)) return;
      UQ(1)
      if (which == 0) {
        if (!c.wait(qInFull + sl, hc / Cfg::kNS)) return;
        tc_fence_after();
        const uint32_t slot = sb + Cfg::oSlot + sl * Cfg::kSlot;
        const uint64_t mQ = desc_from_lo(desc_lo(slot, 8192)), mGo = desc_from_lo(desc_lo(slot + Cfg::kHalf, 8192));
        // dV_i += P dO: P^T as bf16 pairs in TMEM (its own buffer, or over the S columns of each column group)
        uint32_t pa[4];
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          pa[ks] = Cfg::kPtSeparate ? c.tmem + Cfg::tPT + 32 * (hc & 1) + 8 * ks
                                    : c.tmem + (b ? Cfg::tS1 : Cfg::tS0) + CG * ((16 * ks) / CG) + ((16 * ks) % CG) / 2;
        mma4_ts(DV, pa[0], pa[1], pa[2], pa[3], mGo, 128, id_kn, have_dv);
        have_dv = 1;
        tc_commit(c.bar(qPtFree + (Cfg::kPtSeparate ? (hc & 1) : b)));
        mma4_ss(DK, desc_from_lo(desc_lo(dsb, 16)), mQ, 2, 128, id_kn, have_dk);          // dK_i += dS Q
        have_dk = 1;
        tc_commit(c.bar(qInFree + sl));
        tc_commit(c.bar(qDsFree + db));
      } else {
        if (yc >= 1 && !c.wait(qYFree, yc - 1)) return;
        UQ(2)
        tc_fence_after();
        // (UA_EXP_NO_DQ_MMA / UA_EXP_NO_DRAIN / UA_EXP_NO_COLSUM: builds for timing experiments only -- each leaves one
        // piece of the work out, with wrong results, to show what the kernel time does NOT depend on)
#ifndef UA_EXP_NO_DQ_MMA
        mma_rows_out(desc_from_lo(desc_lo(dsb, 16384)));                                  // dQ_rj = dS^T K_i
#endif
        ++yc;
        tc_commit(c.bar(qYFull));
        tc_commit(c.bar(qDsFree + db));
      }
    }
    UQ(0)
    if (!c.wait(qDgReady, ht)) return;
    UQ(3)
    if (which == 0) {
      tc_fence_after();
      const uint64_t mKj = desc_from_lo(desc_lo(sb + Cfg::oKj + (ht % Cfg::kKj) * Cfg::kHalf, 8192));
      mma4_ss(DK, kdG, mKj, 2, 128, id_kn, have_dk);                                      // dK_i += dG K_j
      have_dk = 1;
      tc_commit(c.bar(qKjFree + ht % Cfg::kKj));
      tc_commit(c.bar(qDgFree));
    } else {
      if (yc >= 1 && !c.wait(qYFree, yc - 1)) return;
      tc_fence_after();
      mma_rows_out(mdG);                                                                  // dK_j = dG^T K_i
      ++yc;
      tc_commit(c.bar(qYFull));
      tc_commit(c.bar(qDgFree));
    }
  }
  tc_commit(c.bar(qFinal));
  UQ_STORE_AT(20 + 4 * which)
}

// --------------------------------------------------------------------- workers --
constexpr int kBarAll = 1, kBarDrain = 2, kBarGroup = 3;     // named barriers (0 is __syncthreads); groups use kBarGroup + g

__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
               "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
template <int N>
__device__ __forceinline__ void tmem_ld_n(uint32_t taddr, uint32_t* r) {
  if (N == 32) tmem_ld32(taddr, r);
  else tmem_ld16(taddr, r);
}

// Sum over the 32 lanes of a warp of v[0..CG): afterwards every lane holds the sum of column (lane % CG).
// With a per-warp shared-memory scratch tile this costs CG/4 vector stores + 32 loads and adds per lane; without one it is
// a shuffle transpose (about 4 instructions per element).
template <int CG>
__device__ __forceinline__ float warp_colsum(float* v, float* scr, int lane) {
  if (scr == nullptr) {
    if (CG == 32) return warp_transpose_reduce(v, lane);
    // 16 columns: halve 8, 4, 2, 1 (the lane keeps the half its bit selects), then the two half warps add up
#pragma unroll
    for (int s = 8; s >= 1; s >>= 1) {
      const bool upper = (lane & s) != 0;
#pragma unroll
      for (int x = 0; x < s; ++x) {
        const float send = upper ? v[x] : v[x + s];
        const float keep = upper ? v[x + s] : v[x];
        v[x] = keep + __shfl_xor_sync(0xffffffffu, send, s);
      }
    }
    return v[0] + __shfl_xor_sync(0xffffffffu, v[0], 16);
  }
  // scratch rows of CG + 4 floats: the 16-byte row writes and the column reads are both conflict free without any
  // address swizzling, so every access is one instruction with an immediate offset
  constexpr int PITCH = CG + 4;
  float4* row = reinterpret_cast<float4*>(scr + lane * PITCH);
#pragma unroll
  for (int cidx = 0; cidx < CG / 4; ++cidx) row[cidx] = make_float4(v[4 * cidx], v[4 * cidx + 1], v[4 * cidx + 2], v[4 * cidx + 3]);
  __syncwarp();
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  if (CG == 32) {
    const float* col = scr + lane;
#pragma unroll
    for (int t = 0; t < 32; t += 4) {
      a0 += col[(t + 0) * PITCH];
      a1 += col[(t + 1) * PITCH];
      a2 += col[(t + 2) * PITCH];
      a3 += col[(t + 3) * PITCH];
    }
  } else {
    // lanes 0..15 read rows 0..15, lanes 16..31 rows 16..31 starting four rows further on (opposite bank halves)
    const int hi = lane >> 4;
    const float* col = scr + (lane & 15) + hi * (16 + 4) * PITCH;
#pragma unroll
    for (int t = 0; t < 16; t += 4) {
      a0 += col[(((t + 0) < 12 || !hi) ? (t + 0) : (t + 0) - 16) * PITCH];
      a1 += col[(((t + 1) < 12 || !hi) ? (t + 1) : (t + 1) - 16) * PITCH];
      a2 += col[(((t + 2) < 12 || !hi) ? (t + 2) : (t + 2) - 16) * PITCH];
      a3 += col[(((t + 3) < 12 || !hi) ? (t + 3) : (t + 3) - 16) * PITCH];
    }
  }
  float acc = (a0 + a1) + (a2 + a3);
  if (CG == 16) acc += __shfl_xor_sync(0xffffffffu, acc, 16);
  __syncwarp();
  return acc;
}

// ----------------------------------------------------------------- drain warps --
// Two warps (TMEM lanes 0..63 = the 64 result rows) take every row-side result out of Y, in sweep order: dQ_rj of each
// head, then dK_j of the half tile.  The 64 x D fp32 tile is staged in shared memory as boxes of [64][32] floats and
// leaves as TMA reduce-adds into the fp32 accumulators (other key chunks add to the same rows), which run behind the
// next unit; the workers never touch it.
//
template <int D>
__device__ __forceinline__ void bwd2_drain(const Bwd2Ctx& c, const Bwd2Params& p, const CUtensorMap* tmDQ, const CUtensorMap* tmDK) {
  using Cfg = Bwd2Cfg<D>;
  const int L = p.s.L, R = p.s.R, Rh = p.heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = (warp & 3) * 32 + lane;               // 0..63
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
  const bool leader = (warp == 4 && lane == 0);
  const uint32_t swz = (uint32_t)(row & 7);
  uint8_t* sStage = c.smem + Cfg::oStage;
  int yc = 0;
  for (int ht = 0; ht < c.nht; ++ht) {
    for (int r = 0; r <= Rh; ++r, ++yc) {
      if (!c.wait_w(qYFull, yc)) return;
      tc_fence_after();
      if (leader) bulk_wait_read_all();                 // the previous reduce-add has read the staging tile
      named_bar_sync(kBarDrain, 64);
#pragma unroll 1
      for (int hb = 0; hb < D / 32; ++hb) {
        uint32_t o[32];
        tmem_ld32(c.tmem + Cfg::tY + lane_base + 32 * hb, o);
        tc_wait_ld();
        if (hb == D / 32 - 1) {
          tc_fence_before();
          c.arrive_w(qYFree);
        }
#ifndef UA_EXP_NO_DRAIN
        uint8_t* box = sStage + hb * 8192 + row * 128;
#pragma unroll
        for (int x = 0; x < 8; ++x)
          *reinterpret_cast<uint4*>(box + ((((uint32_t)x ^ swz) & 7) << 4)) = make_uint4(o[4 * x], o[4 * x + 1], o[4 * x + 2], o[4 * x + 3]);
#endif
      }
      fence_proxy_async();
      named_bar_sync(kBarDrain, 64);
#ifdef UA_EXP_NO_DRAIN
      if (false) {
#else
      if (leader) {
#endif
        const CUtensorMap* tm = (r < Rh) ? tmDQ : tmDK;
        const int y = (r < Rh) ? (c.bh * R + r) * p.Lr + c.srow0_of(ht) : c.bh * L + c.row0_of(ht);
#pragma unroll
        for (int bx = 0; bx < D / 32; ++bx) tma_reduce_add_2d(tm, 32 * bx, y, smem_u32(sStage) + bx * 8192);
        bulk_commit_group();
      }
      __syncwarp();
    }
  }
  if (leader) bulk_wait_all();                          // the reduce-adds have landed before the block retires
}

// --------------------------------------------------------------- row-dot warps --
// Builds that are given the forward's output tiles (head_dim 64): the producer copies the head's output half tile next to
// its dO half tile, and two warps (thread = row of the half tile) turn the g_denom entry of the head's table into
// g_denom - out . dO.  They run ahead of the workers (up to the slot ring), who then need neither the column sums of
// P dP over the keys nor the barrier that completed them.  (Fetching the output rows with plain global loads from these warps
// instead made the kernel slower than the column sums: loads issued inside this kernel queue behind its shared-memory
// traffic.)
__device__ __forceinline__ void dot_bf16x8(const uint4& a, const uint4& b, float& lo, float& hi) {
  const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
  for (int x = 0; x < 4; ++x) {
    lo = fmaf(__uint_as_float(aw[x] << 16), __uint_as_float(bw[x] << 16), lo);
    hi = fmaf(__uint_as_float(aw[x] & 0xffff0000u), __uint_as_float(bw[x] & 0xffff0000u), hi);
  }
}
template <int D>
__device__ __forceinline__ void bwd2_rowdots(const Bwd2Ctx& c, const Bwd2Params& p) {
  using Cfg = Bwd2Cfg<D>;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = (warp - 6) * 32 + lane;               // 0..63
  const uint32_t swz = (uint32_t)(row & 7);
  const int total = c.nht * p.heads;
  for (int hc = 0; hc < total; ++hc) {
    const int sl = hc % Cfg::kNS;
    const uint8_t* go = c.smem + Cfg::oSlot + sl * Cfg::kSlot + Cfg::kHalf + row * 128;
    const uint8_t* oo = c.smem + Cfg::oOut + sl * Cfg::kHalf + row * 128;
    if (!c.wait_w(qInFull + sl, hc / Cfg::kNS)) return;
    float lo = 0.f, hi = 0.f;
#pragma unroll
    for (int x = 0; x < 8; ++x) {
      const uint32_t off = (((uint32_t)x) ^ swz) << 4;
      dot_bf16x8(*reinterpret_cast<const uint4*>(oo + off), *reinterpret_cast<const uint4*>(go + off), lo, hi);
    }
    float* tabC = reinterpret_cast<float*>(c.smem + Cfg::oHeadTab + sl * 512) + 64;
    tabC[row] -= lo + hi;
    c.arrive_w(qDelta + sl);
  }
}

// CG: columns of a half tile per thread (32: two column groups, 8 worker warps; 16: four groups, 16 worker warps)
// kHeads = false: the correction pass (p.heads == 0).  A compile-time switch: as a run-time condition around the decay
// recomputation it cost the whole-sequence kernel 2 % (measured).
// kOutDelta: the row term comes from the delta warps (see bwd2_delta).
template <int D, typename TG, int kMode, int CG, bool kHeads, bool kOutDelta>
__device__ __forceinline__ void bwd2_worker(const Bwd2Ctx& c, const Bwd2Params& p) {
  using Cfg = Bwd2Cfg<D>;
  constexpr int NG = 64 / CG;                    // column groups
  constexpr int H2 = CG / 2;                     // packed pairs per thread
  constexpr int kWorkers = 128 * NG;
  const int L = p.s.L, R = kHeads ? p.heads : 0, N = p.s.N;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = (warp - 8) >> 2;                 // column group: columns [CG g, CG g + CG) of a half tile
  const int quad = warp & 3;                     // TMEM lane quadrant this warp may touch; also its helper duty inside the group
  const int key = quad * 32 + lane;
  const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
  const int col0 = CG * g;
  const bool helper = lane < CG;                 // lanes that fetch table entries (lane = column of the group)
  const float kLog2e = 1.4426950408889634f;
  const float2 kLog2e2 = make_float2(kLog2e, kLog2e), kNegLog2e2 = make_float2(-kLog2e, -kLog2e);
  const TG* ss = static_cast<const TG*>(p.ssrc) + (size_t)c.bh * L;
  const float s3 = cbrtf(Num<TG>::ld(ss + c.i * 128 + key));
  const float2 s32 = make_float2(s3, s3);
  float* sT3 = reinterpret_cast<float*>(c.smem + Cfg::oT3);
  float* sXch = reinterpret_cast<float*>(c.smem + Cfg::oXch);
  // (per-warp scratch tiles for the column sums: only with eight worker warps -- with sixteen the shuffle form is 2.5 %
  // faster, measured, as shared memory is the busier resource then)
  float* scr = (Cfg::kScratch && !kOutDelta && CG == 32) ? reinterpret_cast<float*>(c.smem + Cfg::oScr) + (warp - 8) * (32 * (CG + 4)) : nullptr;
  const uint32_t swz = (uint32_t)(key & 7);
  UQ_DECL

  // Per-row tables arrive in shared memory with the tiles (the TMA producer copies them): the workers issue no global
  // load inside the sweep.  (One coalesced load per head cost every warp ~1000 cycles here: it queues behind the
  // shared-memory traffic of all the other warps.)
  auto ht_table = [&](int ht) -> const uint8_t* { return c.smem + Cfg::oHtTab + (ht % Cfg::kTab) * Cfg::kHtTab; };
  // static_dest^(1/3) of half tile ht's rows, from the raw gate values of its table (lane = column of this group)
  auto t3_from_table = [&](int ht) -> float {
    const TG* raw = reinterpret_cast<const TG*>(ht_table(ht) + 512);
    return cbrtf(Num<TG>::ld(raw + col0 + lane));
  };
  // CG floats of a table row for this group's columns, as pairs
  auto load_pairs = [&](const float* src, float2* dst) {
#pragma unroll
    for (int x = 0; x < CG / 4; ++x) {
      const float4 v = reinterpret_cast<const float4*>(src)[x];
      dst[2 * x] = make_float2(v.x, v.y);
      dst[2 * x + 1] = make_float2(v.z, v.w);
    }
  };

  // this thread's CG columns of row `key` of a [128 keys][64 rows] bf16 tile (128-byte swizzled rows)
  auto store_row = [&](uint8_t* base, const uint32_t* v) {
#pragma unroll
    for (int x = 0; x < CG / 8; ++x) {
      const uint32_t ch = (uint32_t)((CG / 8) * g + x);
      *reinterpret_cast<uint4*>(base + key * 128 + (((ch ^ swz) & 7) << 4)) = make_uint4(v[4 * x], v[4 * x + 1], v[4 * x + 2], v[4 * x + 3]);
    }
  };

  // ---- prologue: static_dest^(1/3) of the first half tile ----
  if (!c.wait_w(qTabFull, 0)) return;
  if (helper && quad == 2) sT3[col0 + lane] = t3_from_table(0);
  float suffix = p.suffix_in ? p.suffix_in[((size_t)c.bh * N + c.i) * 128 + key] : 0.f, ds_acc = 0.f;
  named_bar_sync(kBarAll, kWorkers);

  int u = 0, hc = 0;
  for (int ht = 0; ht < c.nht; ++ht) {
    const int j = p.j_end - 1 - (ht >> 1), half = c.half_of(ht);
    const bool diag = (j == c.i);
    const int qbase = 64 * half + col0;            // row of this thread's first column inside the 128-row tile
    const float* t3v = sT3 + (ht & 1) * 64 + col0;

    // ================= decay recomputation: c2 = log2(e) * decay prefix of (key, CG rows) =================
    float2 c2[H2];
    if (kHeads) {                                  // (the correction pass has no heads: no prefix, no first G unit)
      if (!c.wait_w(qTabFull + ht % Cfg::kTab, ht / Cfg::kTab)) return;
      const float carry = reinterpret_cast<const float*>(ht_table(ht))[key];
      const int b = u % Cfg::kNB;
      if (!c.wait_w(qSFull + b, u / Cfg::kNB)) return;
      tc_fence_after();
      uint32_t gr[CG];
      tmem_ld_n<CG>(c.tmem + (b ? Cfg::tS1 : Cfg::tS0) + lane_base + col0, gr);
      float2 t3p[H2];
      load_pairs(t3v, t3p);
      tc_wait_ld();
      tc_fence_before();
      c.arrive_w(qLdDone + b);
      ++u;
      // log-retention in log2 units: lg2(1 - min(a, hi)), a = relu(g)^(2/3) s^(1/3) t^(1/3); relu through lg2(0) = -inf
      float run = 0.f;
      auto ell_scan = [&](auto on_diag) {
        constexpr bool kDiag = decltype(on_diag)::value;
        const float2 k23 = make_float2(2.0f / 3.0f, 2.0f / 3.0f), one2 = make_float2(1.0f, 1.0f);
#pragma unroll
        for (int x = 0; x < H2; ++x) {
          const float2 lg = make_float2(lg2(fmaxf(__uint_as_float(gr[2 * x]), 0.f)), lg2(fmaxf(__uint_as_float(gr[2 * x + 1]), 0.f)));
          const float2 e23 = fmul2(lg, k23);
          const float2 pw = make_float2(ex2(e23.x), ex2(e23.y));
          const float2 a = fmul2(fmul2(pw, s32), t3p[x]);
          const float2 om = fadd2(one2, make_float2(-fminf(a.x, clamp_hi()), -fminf(a.y, clamp_hi())));
          float e0 = lg2(om.x), e1 = lg2(om.y);
          if (kDiag) {
            if (qbase + 2 * x <= key) e0 = 0.f;
            if (qbase + 2 * x + 1 <= key) e1 = 0.f;
          }
          run += e0;
          c2[x].x = run;
          run += e1;
          c2[x].y = run;
        }
      };
      if (diag) ell_scan(std::true_type{});
      else ell_scan(std::false_type{});
      sXch[g * 128 + key] = run;
      named_bar_sync(kBarAll, kWorkers);
      float base = carry * kLog2e;
#pragma unroll
      for (int q = 0; q < NG - 1; ++q)
        if (q < g) base += sXch[q * 128 + key];
      const float2 base2 = make_float2(base, base);
#pragma unroll
      for (int x = 0; x < H2; ++x) c2[x] = fadd2(c2[x], base2);
      if (diag) {
#pragma unroll
        for (int x = 0; x < H2; ++x) {
          if (qbase + 2 * x < key) c2[x].x = mask_value();
          if (qbase + 2 * x + 1 < key) c2[x].y = mask_value();
        }
      }
    }
    UQ(0)

    // ================= heads =================
    // Software pipelining inside the warp: the tail of a head (storing dS and the probabilities, the hand-over to the MMA
    // issuers) is deferred until the TMEM loads of the NEXT unit have been issued, so that their latency runs under it.
    // (Only where the next unit's MMAs do not wait for that hand-over: with a single (S, dP) buffer whose S columns also
    // hold the probabilities, at head_dim 128, the tail comes first.  And only with eight worker warps and the column sums:
    // sixteen warps do better handing dS over at once (5-6 % against eight that defer, more against sixteen that defer),
    // and so do eight without the group barrier in the middle of a head (4.6 %) -- all measured.)
    constexpr bool kColSums = (kMode == 1 && !kOutDelta);     // the workers sum P dP over the keys themselves
    constexpr bool kDeferTail = Cfg::kPtSeparate && kColSums && (CG == 32);
    float2 dc[H2];
#pragma unroll
    for (int x = 0; x < H2; ++x) dc[x] = make_float2(0.f, 0.f);
    uint32_t pk[H2], dk[H2];                       // the pending tail: packed probabilities and dS of head tail_hc
    int tail_hc = -1, tail_b = 0;
    auto flush_tail = [&]() -> bool {
      if (tail_hc < 0) return true;
      const int thc = tail_hc, db = thc % Cfg::kDs;
      tail_hc = -1;
      if (thc >= Cfg::kDs && !c.wait_w(qDsFree + db, thc / Cfg::kDs - 1)) return false;
      store_row(c.smem + Cfg::oDs + db * 16384, dk);
      // P^T (rows CG g + 2x, 2x + 1 as one 32-bit column): in its own buffer, or over this group's own S columns
      if (Cfg::kPtSeparate && thc >= 2 && !c.wait_w(qPtFree + (thc & 1), (thc >> 1) - 1)) return false;
      const uint32_t pt = Cfg::kPtSeparate ? c.tmem + Cfg::tPT + 32 * (thc & 1) + col0 / 2
                                           : c.tmem + (tail_b ? Cfg::tS1 : Cfg::tS0) + col0;
      if (CG == 32) tmem_st16(pt + lane_base, pk);
      else tmem_st8(pt + lane_base, pk);
      tc_wait_st();
      fence_proxy_async();
      tc_fence_before();
      c.arrive_w(qDsReady + db);
      return true;
    };
    for (int r = 0; r < R; ++r, ++hc) {
      const int b = u % Cfg::kNB, sl = hc % Cfg::kNS;
      float* tabL = reinterpret_cast<float*>(c.smem + Cfg::oHeadTab + sl * 512);      // lse[64] of the head's rows (raw)
      float* tabC = tabL + 64;                                                         // g_denom[64] (or delta[64])
      if (!kDeferTail && !flush_tail()) return;
      if (!c.wait_w(qInFull + sl, hc / Cfg::kNS)) return;                              // (the tables landed with the tiles)
      if (!c.wait_w(qSFull + b, u / Cfg::kNB)) return;
      UQ(1)
      tc_fence_after();
      float2 pv[H2], dp[H2];
      {
        uint32_t sr[CG], dr[CG];
        tmem_ld_n<CG>(c.tmem + (b ? Cfg::tS1 : Cfg::tS0) + lane_base + col0, sr);
        tmem_ld_n<CG>(c.tmem + (b ? Cfg::tP1 : Cfg::tP0) + lane_base + col0, dr);
        if (kDeferTail && !flush_tail()) return;                     // the previous head's tail, under the loads
        UQ(6)
        float2 nl[H2];
        load_pairs(tabL + col0, nl);                                 // lse of the rows
        tc_wait_ld();
        tc_fence_before();
        c.arrive_w(qLdDone + b);
        ++u;
        UQ(15)
#pragma unroll
        for (int x = 0; x < H2; ++x) {
          const float2 sv = make_float2(__uint_as_float(sr[2 * x]), __uint_as_float(sr[2 * x + 1]));
          const float2 arg = ffma2(sv, kLog2e2, ffma2(nl[x], kNegLog2e2, c2[x]));
          pv[x] = make_float2(ex2(arg.x), ex2(arg.y));
          dp[x] = make_float2(__uint_as_float(dr[2 * x]), __uint_as_float(dr[2 * x + 1]));
        }
      }
      if (kColSums) {
        float e[CG];
#pragma unroll
        for (int x = 0; x < H2; ++x) {
          const float2 ev = fmul2(pv[x], dp[x]);
          e[2 * x] = ev.x;
          e[2 * x + 1] = ev.y;
        }
#ifdef UA_EXP_NO_COLSUM
        const float part = e[0] + e[1];
#else
        const float part = warp_colsum<CG>(e, scr, lane);            // this warp's 32 keys, column col0 + lane % CG
#endif
        if (helper) atomicAdd(tabC + col0 + lane, -part);           // g_denom - sum_k P dP, in place
      }
      UQ(2)
      if (kOutDelta) {
        if (!c.wait_w(qDelta + sl, hc / Cfg::kNS)) return;
      } else if (kColSums) {
        named_bar_sync(kBarGroup + g, 128);           // the group's column sums are complete
      }
      UQ(4)
      {
        float2 cc[H2];
        load_pairs(tabC + col0, cc);
#pragma unroll
        for (int x = 0; x < H2; ++x) {
          if (kMode == 2) cc[x] = make_float2(-cc[x].x, -cc[x].y);            // merged mode: dS = P (dP - delta)
          const float2 ds = fmul2(pv[x], fadd2(dp[x], cc[x]));
          dc[x] = fadd2(dc[x], ds);
          __nv_bfloat162 hp = __floats2bfloat162_rn(pv[x].x, pv[x].y), hd = __floats2bfloat162_rn(ds.x, ds.y);
          pk[x] = *reinterpret_cast<uint32_t*>(&hp);
          dk[x] = *reinterpret_cast<uint32_t*>(&hd);
        }
      }
      tail_hc = hc;
      tail_b = b;
      UQ(5)
    }
    if (!kDeferTail && !flush_tail()) return;

    // ================= decay gradient =================
    {
      if (kDeferTail && !flush_tail()) return;     // the last head's tail
      const bool more = ht + 1 < c.nht;
      float run = 0.f;
#pragma unroll
      for (int x = H2 - 1; x >= 0; --x) {
        run += dc[x].y;
        dc[x].y = run;                             // sum of dC over this thread's columns from here to its last one
        run += dc[x].x;
        dc[x].x = run;
      }
      sXch[(NG + g) * 128 + key] = run;
      if (more && quad == 2) {                   // static_dest^(1/3) of the next half tile's rows
        if (!c.wait_w(qTabFull + (ht + 1) % Cfg::kTab, (ht + 1) / Cfg::kTab)) return;
        if (helper) sT3[((ht + 1) & 1) * 64 + col0 + lane] = t3_from_table(ht + 1);
      }
      UQ(7)
      named_bar_sync(kBarAll, kWorkers);
      UQ(8)
      float later = 0.f, others = 0.f;             // totals of the groups to the right / of all other groups
#pragma unroll
      for (int q = 0; q < NG; ++q) {
        if (q == g) continue;
        const float v = sXch[(NG + q) * 128 + key];
        others += v;
        if (q > g) later += v;
      }
      const float add = suffix + later;            // rows after this thread's block
      suffix = suffix + run + others;              // ... after this half tile (the next one lies below it)
      const float2 add2 = make_float2(add, add);

      const int b = u % Cfg::kNB;
      if (!c.wait_w(qSFull + b, u / Cfg::kNB)) return;
      UQ(9)
      tc_fence_after();
      uint32_t gr[CG];
      tmem_ld_n<CG>(c.tmem + (b ? Cfg::tS1 : Cfg::tS0) + lane_base + col0, gr);
      float2 t3p[H2];
      load_pairs(t3v, t3p);
      tc_wait_ld();
      tc_fence_before();
      c.arrive_w(qLdDone + b);
      ++u;
      uint32_t pk[H2];
      float2 dsa = make_float2(0.f, 0.f);
      auto decay_grad = [&](auto on_diag) {
        constexpr bool kDiag = decltype(on_diag)::value;
        const float2 k23 = make_float2(2.0f / 3.0f, 2.0f / 3.0f), km13 = make_float2(-1.0f / 3.0f, -1.0f / 3.0f);
        const float2 mone2 = make_float2(-1.0f, -1.0f), s32k = fmul2(s32, k23);
#pragma unroll
        for (int x = 0; x < H2; ++x) {
          float2 dl = fadd2(dc[x], add2);
          if (kDiag) {
            if (qbase + 2 * x <= key) dl.x = 0.f;
            if (qbase + 2 * x + 1 <= key) dl.y = 0.f;
          }
          const float g0 = __uint_as_float(gr[2 * x]), g1 = __uint_as_float(gr[2 * x + 1]);
          const float2 lg = make_float2(lg2(fmaxf(g0, 0.f)), lg2(fmaxf(g1, 0.f)));      // -inf for g <= 0: pw = 0
          // g^(2/3) = g * g^(-1/3): one exponential serves both powers (relu: zero for g <= 0, where lg = -inf)
          const float2 e13 = fmul2(lg, km13);
          const float2 r13 = make_float2(ex2(e13.x), ex2(e13.y));
          float2 pw = fmul2(make_float2(g0, g1), r13);
          if (!(g0 > 0.f)) pw.x = 0.f;
          if (!(g1 > 0.f)) pw.y = 0.f;
          const float2 st = fmul2(pw, s32);
          const float2 a = fmul2(st, t3p[x]);
          const float2 am = fadd2(make_float2(fminf(fmaxf(a.x, clamp_lo_bwd()), clamp_hi()), fminf(fmaxf(a.y, clamp_lo_bwd()), clamp_hi())), mone2);
          // d affinity = d ell / (clamp(a) - 1), zero above the clamp (the clamp passes no gradient there)
          float2 da = fmul2(dl, make_float2(rcp_approx(am.x), rcp_approx(am.y)));
          if (!(a.x <= clamp_hi())) da.x = 0.f;
          if (!(a.y <= clamp_hi())) da.y = 0.f;
          const float2 dstat = fmul2(da, pw);
          dsa = ffma2(dstat, t3p[x], dsa);
          // dG = dA s^(1/3) t^(1/3) (2/3) g^(-1/3) for g > 0
          float2 dg = fmul2(fmul2(da, t3p[x]), fmul2(s32k, r13));
          if (!(g0 > 0.f)) dg.x = 0.f;
          if (!(g1 > 0.f)) dg.y = 0.f;
          __nv_bfloat162 h = __floats2bfloat162_rn(dg.x, dg.y);
          pk[x] = *reinterpret_cast<uint32_t*>(&h);
        }
      };
      if (diag) decay_grad(std::true_type{});
      else decay_grad(std::false_type{});
      ds_acc += dsa.x + dsa.y;
      if (ht >= 1 && !c.wait_w(qDgFree, ht - 1)) return;
      store_row(c.smem + Cfg::oDg, pk);
      // (d static_dest needs no sum over the keys here: it is taken from dK_j afterwards, see row_side_finish_kernel)
      fence_proxy_async();
      c.arrive_w(qDgReady);
      UQ(10)
    }
  }
  UQ_STORE

  // ---- end of the sweep: dV_i, dK_i, d static_src (thread = key, D / NG columns each) ----
  if (!c.wait_w(qFinal, 0)) return;
  tc_fence_after();
  const size_t krow = (size_t)c.bh * L + c.i * 128 + key;
  if (g == 0 && p.dctot_out) {                     // the range's own dC: what left minus what came in from the rows after it
    const size_t key_id = ((size_t)c.bh * N + c.i) * 128 + key;
    p.dctot_out[key_id] = suffix - (p.suffix_in ? p.suffix_in[key_id] : 0.f);
  }
  constexpr int kPer = D / NG;
#pragma unroll
  for (int pc = 0; pc < kPer / 16; ++pc) {
    const int d0 = kPer * g + 16 * pc;
    uint32_t o[16];
    if (kHeads) {                                  // (the correction pass has no heads: no dV)
    tmem_ld16(c.tmem + Cfg::tDV + lane_base + d0, o);
    tc_wait_ld();
    if (p.dv_chunk) {
      const float4* extra = reinterpret_cast<const float4*>(p.dv_chunk + ((size_t)c.bh * p.s.N + c.i) * p.dv_chunk_stride + d0);
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const float4 ev = extra[x];
        o[4 * x] = __float_as_uint(fmaf(ev.x, 1.0f / 128.0f, __uint_as_float(o[4 * x])));
        o[4 * x + 1] = __float_as_uint(fmaf(ev.y, 1.0f / 128.0f, __uint_as_float(o[4 * x + 1])));
        o[4 * x + 2] = __float_as_uint(fmaf(ev.z, 1.0f / 128.0f, __uint_as_float(o[4 * x + 2])));
        o[4 * x + 3] = __float_as_uint(fmaf(ev.w, 1.0f / 128.0f, __uint_as_float(o[4 * x + 3])));
      }
    }
    if (p.acc_dv) {                                // several row ranges add to the same keys
      float* dvp = p.acc_dv + krow * D + d0;
#pragma unroll
      for (int x = 0; x < 4; ++x)
        red_add_v4(dvp + 4 * x, __uint_as_float(o[4 * x]), __uint_as_float(o[4 * x + 1]), __uint_as_float(o[4 * x + 2]),
                   __uint_as_float(o[4 * x + 3]));
    } else {
      uint32_t pk[8];
#pragma unroll
      for (int x = 0; x < 8; ++x) {
        __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(o[2 * x]), __uint_as_float(o[2 * x + 1]));
        pk[x] = *reinterpret_cast<uint32_t*>(&h);
      }
      uint4* dst = reinterpret_cast<uint4*>(p.dvc + krow * D + d0);
      dst[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      dst[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
    }
    }
    tmem_ld16(c.tmem + Cfg::tDK + lane_base + d0, o);
    tc_wait_ld();
    float* dkp = p.acc_dk + krow * D + d0;
#pragma unroll
    for (int x = 0; x < 4; ++x)
      red_add_v4(dkp + 4 * x, __uint_as_float(o[4 * x]), __uint_as_float(o[4 * x + 1]), __uint_as_float(o[4 * x + 2]),
                 __uint_as_float(o[4 * x + 3]));
  }
  sXch[g * 128 + key] = ds_acc;
  named_bar_sync(kBarAll, kWorkers);
  if (g == 0) {
    float tot = 0.f;
#pragma unroll
    for (int q = 0; q < NG; ++q) tot += sXch[q * 128 + key];
    if (p.acc_ds) atomicAdd(p.acc_ds + krow, tot / (3.0f * s3 * s3));
    else Num<TG>::st(static_cast<TG*>(p.dss) + krow, tot / (3.0f * s3 * s3));
  }
}

template <int D, typename TG, int kMode, int CG, bool kHeads, bool kOutDelta = false>
__global__ void __launch_bounds__(32 * (8 + 4 * (64 / CG)), 1)
bwd2_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
            const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmG,
            const __grid_constant__ CUtensorMap tmDQ, const __grid_constant__ CUtensorMap tmDK,
            const __grid_constant__ CUtensorMap tmO, Bwd2Params p) {
  static_assert(!kOutDelta || (Bwd2Cfg<D>::kOutTiles && kMode == 1 && kHeads), "output-tile builds: head_dim 64, per-chunk form");
  using Cfg = Bwd2Cfg<D>;
  constexpr int NG = 64 / CG;
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
  c.jtop = p.j_end; c.jb = p.j_begin; c.r0 = p.r0;
  c.nht = 2 * (p.j_end - (c.i > p.j_begin ? c.i : p.j_begin));
  if (c.nht <= 0) {
    // no row of the range sees this chunk (sequence sharding only): nothing to add anywhere
    if (p.dctot_out && threadIdx.x < 128) p.dctot_out[((size_t)c.bh * p.s.N + c.i) * 128 + threadIdx.x] = 0.f;
    return;
  }

  if (threadIdx.x == 0) {
    misc[1] = 0;
    misc[2] = 0;
    for (int b = 0; b < qNumBars; ++b) {
      uint32_t count = 1;
      if (b == qLdDone || b == qLdDone + 1 || b == qDsReady || b == qDsReady + 1 || b == qDgReady) count = 4 * NG;   // one arrival per worker warp
      if (b == qYFree || (b >= qDelta && b < qDelta + 4)) count = 2;                                                                                  // the two draining warps
      if (b == qDsFree || b == qDsFree + 1 || b == qDgFree || b == qFinal) count = 2;                               // both back issuers
      mbar_init(c.bar(b), count);
    }
    mbar_init_fence();
    prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmQ); prefetch_tmap(&tmG);
    prefetch_tmap(&tmDQ); prefetch_tmap(&tmDK);
    if (kOutDelta) prefetch_tmap(&tmO);
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(misc), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  c.tmem = misc[0];

  // Register reallocation between the warpgroups: the single-thread roles and the drain warps need few registers, the
  // workers (who keep a half tile's decay prefix, its gradient and a head's probabilities in registers) many.  The block
  // is launched with kLaunchRegs per thread (the most its thread count allows); the first two warpgroups give back what
  // they do not need and every worker warpgroup takes an equal share of it.  (The sums are checked at compile time: a
  // worker request beyond what was given back would never be granted.)
  constexpr int kThreads = 32 * (8 + 4 * NG);
  constexpr int kLaunchRegs = (65536 / kThreads) / 8 * 8;
  // (sixteen worker warps: 80 registers at launch; the tighter split leaves them 96 instead of 88, measured 2.5 % faster)
  constexpr int kRoleRegs = (CG == 16) ? 40 : 48, kDrainRegs = (CG == 16) ? 56 : 64;
  constexpr int kWorkerRegs = kLaunchRegs + ((2 * kLaunchRegs - kRoleRegs - kDrainRegs) * 128 / (128 * NG)) / 8 * 8;
  static_assert(kRoleRegs <= kLaunchRegs && kDrainRegs <= kLaunchRegs, "setmaxnreg.dec must not ask for more");
  static_assert(128 * (kRoleRegs + kDrainRegs) + 128 * NG * kWorkerRegs <= kThreads * kLaunchRegs, "register pool");
  static_assert(kWorkerRegs <= 232, "setmaxnreg range");
  // warps 0-3: the four single-thread roles; warps 4-5: drain warps (6-7 complete their warpgroup); warps 8..: workers
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRoleRegs));
    if (lane == 0) {
      if (warp == 0) bwd2_front<D>(c, p);
      else if (warp == 1) bwd2_back<D, CG>(c, p, 0);
      else if (warp == 2) bwd2_producer<D, TG, kMode, kOutDelta>(c, p, &tmK, &tmV, &tmQ, &tmG, &tmO);
      else bwd2_back<D, CG>(c, p, 1);
    }
  } else if (warp < 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kDrainRegs));
    if (warp < 6) bwd2_drain<D>(c, p, &tmDQ, &tmDK);
    else if (kOutDelta) bwd2_rowdots<D>(c, p);
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kWorkerRegs));
    bwd2_worker<D, TG, kMode, CG, kHeads, kOutDelta>(c, p);
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

// After the sweep: the row-side part of dK joins the accumulator, and d static_dest comes out of it.
// With a = g^(2/3) s^(1/3) t^(1/3):  t dA/dt = a / 3 = g dA/dg / 2, so d t[row] = sum_k dG[k, row] G[k, row] / (2 t[row]),
// summed over the keys k of every chunk; and with G = K K^T that sum is the dot product of K[row] with
// sum_chunks (dG^T K_i)[row] -- the row-side dK_j that the sweep adds up in acc_dkr (with the bf16 dG its MMAs consumed).
// So the sweep needs no column sums over the keys for d static_dest.  One warp per row of the range.
template <int D, typename TG>
__global__ void __launch_bounds__(256)
row_side_finish_kernel(const __nv_bfloat16* __restrict__ kc, const TG* __restrict__ sdest, const float* __restrict__ dkr,
                       float* __restrict__ acc_dk, float* __restrict__ acc_dt, int BH, int L, int Lr, int r0, int row_begin,
                       int row_end) {
  constexpr int E = D / 32;                             // elements per lane
  const int lane = threadIdx.x & 31, nrows = row_end - row_begin;
  const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wid >= (long long)BH * nrows) return;
  const int bh = (int)(wid / nrows), rr = (int)(wid - (long long)bh * nrows);
  const size_t base = ((size_t)bh * L + row_begin + rr) * D + (size_t)lane * E;
  float v[E], kf[E];
  if (E == 2) {
    const float2 t = *reinterpret_cast<const float2*>(dkr + base);
    v[0] = t.x; v[1] = t.y;
    const __nv_bfloat162 kk = *reinterpret_cast<const __nv_bfloat162*>(kc + base);
    kf[0] = __low2float(kk); kf[1] = __high2float(kk);
  } else {
    const float4 t = *reinterpret_cast<const float4*>(dkr + base);
    v[0] = t.x; v[1] = t.y; v[E - 2] = t.z; v[E - 1] = t.w;
    const uint2 kk = *reinterpret_cast<const uint2*>(kc + base);
    kf[0] = __uint_as_float(kk.x << 16); kf[1] = __uint_as_float(kk.x & 0xffff0000u);
    kf[E - 2] = __uint_as_float(kk.y << 16); kf[E - 1] = __uint_as_float(kk.y & 0xffff0000u);
  }
  float dot = 0.f;
#pragma unroll
  for (int x = 0; x < E; ++x) {
    dot = fmaf(v[x], kf[x], dot);
    acc_dk[base + x] += v[x];
  }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
  if (lane == 0 && dot != 0.f) {
    const size_t grow = (size_t)bh * Lr + r0 + rr;
    acc_dt[grow] += 0.5f * dot / Num<TG>::ld(sdest + grow);
  }
}

}  // namespace sm100
}  // namespace ua
