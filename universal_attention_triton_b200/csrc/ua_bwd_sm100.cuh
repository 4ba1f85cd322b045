// Tensor-core backward of the Universal Attention operator for sm_100a
// (bf16, key chunk = 128, head_dim = 64).
//
// One thread block owns one key chunk (b, h, i) and sweeps the row tiles
// DOWNWARDS (j = n-1 .. i), so that the reverse cumulative sum of the decay
// gradient is carried per key in a register (universal_attention_autograd.py:
// 232-259).  The decay prefix at the start of each tile comes from a table that
// a carry-only run of the forward kernel writes (recomputed, never saved by the
// forward).  Rows before the chunk (j < i, uniform softmax) follow when the
// masked-block gradient is requested.
//
// Three ways to form the probabilities (template parameter kMode):
//   0  from the kernel's own row max / sum over the chunk's keys (inputs and upstream gradients only);
//   1  as exp(s - lse) with the per-chunk log-sum-exp that the forward returned;
//   2  "merged": the upstream gradient is that of the MERGED output  sum_n softmax_n(denom) out_n  (SMVecMatMul after
//      the operator, universal_attention_autograd.py:278-297).  Then P = exp(s - L_row) with the log-sum-exp over ALL
//      keys of the row, dO is the same (b,h,r,L,d) tile for every key chunk, dS = P (dP - delta_row) with
//      delta_row = g . merged, nothing crosses the worker groups and the rows before a chunk contribute nothing.
//
// Per tile (q = rows, k = keys of the chunk, all tcgen05.mma with fp32 TMEM accumulators):
//   G    = K_i K_j^T                keys on lanes  -> decay group: C^T to shared memory
//   S_r  = Q_rj K_i^T,  dP_r = dO_rj V_i^T         rows on lanes -> softmax group
//        P = softmax_k(S + C), dS = P (dP - sum_k P dP + g_denom)   (thread-local per row)
//        P and dS go to shared memory as bf16 [row][key] tiles, which serve as
//        K-major and as MN-major operands:
//   dV_i += P^T dO     dK_i += dS^T Q     dQ_rj = dS K_i     dC += dS^T I
//   (the last one transposes dS back to keys-on-lanes through eight N=16 MMAs
//    against a 16x16 identity, accumulating over the R heads in TMEM)
//   G again (recomputed rather than kept, TMEM is full), decay group: reverse scan
//   of dC, d log-retention -> d affinity -> dG (bf16, shared memory), d src, d dest
//   dK_j = dG^T K_i     dK_i += dG K_j
// Rows before the chunk (j < i): every score is -1e12 there, the softmax is uniform (P = 1/128) and
//   dS[k][q] = ( (v_k - vbar) . g_q + gd_q ) / 128      (g = dO row, gd = g_denom, vbar = mean of the chunk's values)
// is of rank <= 65, so nothing is done per (key, row) pair.  With E = a [128][64] tile whose column 0 holds gd:
//   dQ_rj    = [g | E] [ M_i ; ksum_i ] / 128,   M_i = sum_k (v_k - vbar)^T k_k  (64 x 64, once per block)
//   N_i     += [g | E]^T Q_rj                    (64 x 64 plus the row  w = sum_q gd_q q_q ; accumulates in TMEM)
//   dV_i    += (1/128) 1^T g                     (column sums of g on the CUDA cores of the otherwise idle worker groups)
//   dK_i    += [V_i - vbar | 1] [ N_i ; w ] / 128    (once, after the sweep)
//
// dQ_rj and dK_j are added to fp32 global accumulators (other key chunks add to the
// same rows): the tile is staged in shared memory and leaves as a TMA reduce-add, which
// runs behind the next phase; dV_i, dK_i and d src stay in TMEM / registers until the
// sweep ends.
//
// TMEM (512 columns): X0 [0,128) G / S_r | X1 [128,256) dP_r, then dQ_r / dK_j |
//                     XC [256,384) dC | dV [384,448) | dK_i [448,512)
#pragma once
#include "ua_fwd_sm100.cuh"

namespace ua {
namespace sm100 {

struct BwdParams {
  Shape s;
  const void* ssrc;
  const void* sdest;
  const void* g_denom;     // (b,h,n,r,L) fp32 or bf16
  int g_denom_is_f32;
  const float* carry;      // (b*h*n, n, 2, 128) decay prefix at the start of each 64-row half of row tile j (the first half is used)
  float* acc_dk;           // (b*h, L, 64) fp32, zeroed
  float* acc_dq;           // (b*h, r, L, 64) fp32, zeroed
  float* acc_dt;           // (b*h, L) fp32, zeroed
  __nv_bfloat16* dvc;      // written directly
  void* dss;               // gate dtype, written directly
  int* status;
  int skip_masked;
  // Row range (sequence sharding): only the row tiles [j_begin, j_end) are swept; xq, static_dest, g_out, g_denom,
  // acc_dq and acc_dt then hold just those Lr = 128 * (j_end - j_begin) rows.  Keys, values, static_src, acc_dk whole.
  int j_begin, j_end, Lr;  // Lr: rows per slab of the row-indexed tensors
  int r0;                  // row of the slab where the range starts
  const float* suffix_in;  // optional (b*h*n, 128): reverse decay carry entering from the rows after the range
  float* dctot_out;        // optional (b*h*n, 128): per key, sum of dC over the rows of the range (what earlier ranges need)
  float* acc_dv;           // optional (b*h, L, 64) fp32: dV_i is ADDED here instead of written to dvc
  float* acc_ds;           // optional (b*h, L) fp32: d static_src is added here instead of written to dss
  int decay_only;          // correction pass: only the decay gradient that suffix_in induces (no heads, no dV)
  const float* lse;        // optional (b,h,n,r,L) fp32: the forward's log-sum-exp; spares the per-row max / sum (whole-sequence calls)
  // merged mode: g_out is the (b,h,r,L,d) gradient of the merged output (g_denom unused)
  int merged;
  const float* row_lse;    // (b,h,r,L) fp32: log-sum-exp of the row over all keys
  const float* row_delta;  // (b,h,r,L) fp32: g . merged
  const float* gd_f32;     // optional: g_denom as fp32 (16-byte aligned).  The producer then copies each masked step's 128
                           // values next to its tiles and no worker issues a global load for them
  int masked_only;         // only the rows before the chunk (the rows that see it are another kernel's): dV_i and dK_i are
                           // ADDED to acc_dv / acc_dk, d static_src is left alone
};

struct BwdCfg {
  static constexpr int kTileBytes = 16384;    // [128][64] bf16
  static constexpr int oKi = 0, oVi = 16384, oKj = 32768, oQ = 49152, oGo = 65536;
  static constexpr int oCs = 81920;           // 64 KB fp32 C^T[row][key]
  static constexpr int oP = 147456;           // 32 KB bf16 P[row][key]; reused for dG[key][row]
  static constexpr int odS = 180224;          // 32 KB bf16 dS[row][key]
  static constexpr int oI = 212992;           // 2 KB: 16 x 64 bf16, identity in the first 16 columns
  static constexpr int oT3 = 215040;          // 2 x 128 floats
  static constexpr int oXch = 216064;          // 2 slots x 4 groups x 3 x 128 floats mailbox (12 KB)
  static constexpr int oBar = 228352;
  static constexpr int oMisc = oBar + 256;
  static constexpr int kSmemBytes = oMisc + 64 + 1024;
  static constexpr uint32_t tX0 = 0, tX1 = 128, tXC = 256, tDV = 384, tDK = 448;
  // Shared memory of the phase for the rows before the chunk (the decay-prefix tile and dS are idle then):
  // two slots of (Q, dO, E) so that the next step's loads run under the current step's MMAs; step m uses slot m & 1
  static constexpr int oGo1 = oCs + 16384, oE1 = oCs + 32768, oQ1 = oCs + 49152;
  static constexpr int oE = oCs;                // [128][64] bf16, column 0 = g_denom: second 64-wide box after dO
  static constexpr int oBm = oKj;               // [80][64] bf16 rows: M_i / 128 (64 rows), ksum_i / 128, zeros (K_j is idle)
  static_assert(oE == oGo + 16384, "E must follow the dO slot: together they form one two-box operand");
};

enum BwdBar {
  bKvFull = 0, bKjFull, bInFull, bGFull, bX0Free, bSdpFull, bX1Free, bCReady, bCsFree, bPdsReady, bRDone, bG2Full,
  bDgReady, bDkjFull, bXchg, bFinal, bInFree, bStage, bMraw, bMask2, bFinal2, bInFull1, bInFree1, bPdsM0, bPdsM1, bStageFree, bNumBars
};

struct BwdCtx {
  uint8_t* smem;
  uint32_t bars;
  uint32_t tmem;
  volatile int* abort_flag;
  int i, bh, nvalid, ntiles;
  int j_begin, j_end;
  __device__ __forceinline__ uint32_t bar(int idx) const { return bars + 8u * idx; }
  // A wait that gives up leaves (barrier index + 1) | thread << 8 | phase << 20 in the word after the abort flag (first one
  // wins); the kernel copies it to the second status word, so that a host can see where a block stopped.
  __device__ __forceinline__ void note_failure(int idx, uint32_t parity) const {
    atomicCAS(const_cast<int*>(abort_flag) + 1, 0, (idx + 1) | ((int)threadIdx.x << 8) | ((int)(parity & 0x7ff) << 20));
  }
  __device__ __forceinline__ bool wait(int idx, uint32_t parity) const {
    const bool ok = mbar_wait(bar(idx), parity & 1u, abort_flag);
    if (!ok) note_failure(idx, parity);
    return ok;
  }
  // warp-collective forms for the worker groups
  __device__ __forceinline__ bool wait_w(int idx, uint32_t parity) const {
    const bool ok = mbar_wait_warp(bar(idx), parity & 1u, abort_flag);
    if (!ok && (threadIdx.x & 31) == 0) note_failure(idx, parity);
    return ok;
  }
  __device__ __forceinline__ void arrive_w(int idx) const { mbar_arrive_warp(bar(idx)); }
  // row tile index of sweep step T: valid tiles n-1 .. i first, then the masked ones i-1 .. 0
  __device__ __forceinline__ int tile_j(int T, int) const {
    return T < nvalid ? j_end - 1 - T : (i < j_end ? i : j_end) - 1 - (T - nvalid);
  }
};

// Rows before the chunk: step m (counted from the first such (tile, head)) uses slot m & 1.  Slot 0 is the slot of the
// sweep over the valid tiles (its barriers continue their phase sequence, rc0 steps old), slot 1 is fresh.
struct MaskSlot {
  int q, go, e, full_bar, free_bar, phase;
  int ready_bar, ready_phase;   // "operands of the step are complete" (worker groups -> issuers), one barrier per slot:
                                // an issuer that trails by two steps would mistake a phase of a shared barrier
};
__device__ __forceinline__ MaskSlot mask_slot(int m, int rc0) {
  MaskSlot s;
  if ((m & 1) == 0) {
    s.q = BwdCfg::oQ; s.go = BwdCfg::oGo; s.e = BwdCfg::oE; s.full_bar = bInFull; s.free_bar = bInFree; s.phase = rc0 + (m >> 1);
    s.ready_bar = bPdsM0;
  } else {
    s.q = BwdCfg::oQ1; s.go = BwdCfg::oGo1; s.e = BwdCfg::oE1; s.full_bar = bInFull1; s.free_bar = bInFree1; s.phase = m >> 1;
    s.ready_bar = bPdsM1;
  }
  s.ready_phase = m >> 1;
  return s;
}

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// 32 lanes x 32 values: afterwards lane l holds sum over lanes of v[l] in v[0]
__device__ __forceinline__ float warp_transpose_reduce(float* v, int lane) {
#pragma unroll
  for (int s = 16; s >= 1; s >>= 1) {
    const bool upper = (lane & s) != 0;
#pragma unroll
    for (int x = 0; x < s; ++x) {
      const float send = upper ? v[x] : v[x + s];
      const float keep = upper ? v[x + s] : v[x];
      v[x] = keep + __shfl_xor_sync(0xffffffffu, send, s);
    }
  }
  return v[0];
}

// ------------------------------------------------------------------ producer --
__device__ __forceinline__ void bwd_producer(const BwdCtx& c, const BwdParams& p, const CUtensorMap* tmK,
                                             const CUtensorMap* tmV, const CUtensorMap* tmQ, const CUtensorMap* tmG) {
  const int L = p.s.L, R = p.s.R, N = p.s.N;
  const uint32_t sbase = smem_u32(c.smem);
  const int krow = c.bh * L + c.i * 128;
  const size_t chunk_id = (size_t)c.bh * N + c.i;
  mbar_expect_tx(c.bar(bKvFull), 2 * BwdCfg::kTileBytes);
  tma_load_2d(sbase + BwdCfg::oKi, tmK, 0, krow, c.bar(bKvFull));
  tma_load_2d(sbase + BwdCfg::oVi, tmV, 0, krow, c.bar(bKvFull));
  // dO tiles stream from HBM (g_out is far larger than L2): the tiles of the next head / next
  // row tile are prefetched into L2 one phase ahead, so that the load issued when the single
  // shared-memory slot frees up only pays L2 latency.
  auto coords = [&](int T, int r, int& qrow, int& grow) {
    const int j = c.tile_j(T, N);
    qrow = (c.bh * R + r) * p.Lr + p.r0 + (j - p.j_begin) * 128;
    grow = p.merged ? qrow : (int)((chunk_id * R + r) * p.Lr + p.r0 + (size_t)(j - p.j_begin) * 128);
  };
  int rc = 0;
  const int rc0 = c.nvalid * R;                           // steps of the sweep over the valid tiles
  for (int T = 0; T < c.ntiles; ++T) {
    const bool valid = T < c.nvalid;
    const int j = c.tile_j(T, N);
    if (valid) {
      if (T >= 1 && !c.wait(bDkjFull, T - 1)) return;
      mbar_expect_tx(c.bar(bKjFull), BwdCfg::kTileBytes);
      tma_load_2d(sbase + BwdCfg::oKj, tmK, 0, c.bh * L + j * 128, c.bar(bKjFull));
    }
    for (int r = 0; r < (p.decay_only ? 0 : R); ++r, ++rc) {
      int qrow, grow;
      {
        const int nxt = T * R + r + (valid ? 1 : 2);     // two slots before the chunk: look one step further ahead
        const int Tn = nxt / R, rn = nxt - Tn * R;
        if (Tn < c.ntiles) {
          coords(Tn, rn, qrow, grow);
          tma_prefetch_2d(tmG, 0, grow);
          tma_prefetch_2d(tmQ, 0, qrow);
        }
      }
      coords(T, r, qrow, grow);
      MaskSlot ms = mask_slot(0, rc);                     // valid tiles: slot 0, phase rc
      if (!valid) ms = mask_slot(rc - rc0, rc0);
      if (ms.phase >= 1 && !c.wait(ms.free_bar, ms.phase - 1)) return;
      const bool copy_gd = !valid && p.gd_f32 != nullptr;
      mbar_expect_tx(c.bar(ms.full_bar), 2 * BwdCfg::kTileBytes + (copy_gd ? 512 : 0));
      tma_load_2d(sbase + ms.q, tmQ, 0, qrow, c.bar(ms.full_bar));
      tma_load_2d(sbase + ms.go, tmG, 0, grow, c.bar(ms.full_bar));
      if (copy_gd) bulk_load_1d(sbase + BwdCfg::oXch + ((rc - rc0) & 1) * 512, p.gd_f32 + grow, 512, c.bar(ms.full_bar));
    }
  }
}

// --------------------------------------------------------------- MMA issuers --
// tcgen05.mma is issued by single threads, and what limits the tensor pipe here is the
// number of instructions (every one covers only K = 16), not their size: one thread
// sustains one MMA per ~100 cycles, two threads together close to the pipe's ~50.  So
// two issuers (lane 0 of warps 1 and 2) split the accumulators between them:
//   issuer A: X0 (G, S_r, G again), dV_i, dK_i          issuer B: X1 (dP_r, dQ_r, dK_j), dC
// MMAs into one accumulator always come from the same issuer, so their order is kept.
__device__ __forceinline__ void bwd_mma(const BwdCtx& c, const BwdParams& p, const int which) {
  const int R = p.decay_only ? 0 : p.s.R;
  const uint32_t sb = smem_u32(c.smem);
  constexpr uint32_t id_nt = idesc_bf16(128, 128, 0, 0);   // A K-major, B K-major, N = 128
  constexpr uint32_t id_tt = idesc_bf16(128, 64, 1, 1);    // A MN-major, B MN-major, N = 64
  constexpr uint32_t id_nt64 = idesc_bf16(128, 64, 0, 1);  // A K-major,  B MN-major, N = 64
  constexpr uint32_t id_dc = idesc_bf16(128, 16, 1, 0);    // A MN-major, B K-major,  N = 16
  const uint32_t X0 = c.tmem + BwdCfg::tX0, X1 = c.tmem + BwdCfg::tX1, XC = c.tmem + BwdCfg::tXC;
  const uint32_t DV = c.tmem + BwdCfg::tDV, DK = c.tmem + BwdCfg::tDK;

  // Descriptor low words of every operand, built once (shared-memory addresses never change);
  // a k-step is then one 32-bit add per operand.  K-major: +32 B per 16 elements of K (>>4 = 2);
  // MN-major: +2048 B per 16 rows of K (>>4 = 128); second 64-wide box of a K-major tile: +16384 B (>>4 = 1024).
  const uint32_t kKi = desc_lo(sb + BwdCfg::oKi, 16), kKj = desc_lo(sb + BwdCfg::oKj, 16), kQ = desc_lo(sb + BwdCfg::oQ, 16);
  const uint32_t kGo = desc_lo(sb + BwdCfg::oGo, 16), kVi = desc_lo(sb + BwdCfg::oVi, 16), kI = desc_lo(sb + BwdCfg::oI, 16);
  const uint32_t kdS = desc_lo(sb + BwdCfg::odS, 16), kdG = desc_lo(sb + BwdCfg::oP, 16);
  const uint32_t mP = desc_lo(sb + BwdCfg::oP, 16384), mdS = desc_lo(sb + BwdCfg::odS, 16384);
  const uint32_t mGo = desc_lo(sb + BwdCfg::oGo, 16384), mQ = desc_lo(sb + BwdCfg::oQ, 16384);
  const uint32_t mKi = desc_lo(sb + BwdCfg::oKi, 16384), mKj = desc_lo(sb + BwdCfg::oKj, 16384);
  const uint32_t mVi = desc_lo(sb + BwdCfg::oVi, 16384);
  const uint32_t mBm = desc_lo(sb + BwdCfg::oBm, 16384);

  // D[128x128] = A[128][64] B[128][64]^T (both K-major, one 64-element box)
  auto mma_nt = [&](uint32_t d, uint32_t a, uint32_t b) {
    mma_ss_c<false>(d, desc_from_lo(a), desc_from_lo(b), id_nt);
#pragma unroll
    for (int ks = 1; ks < 4; ++ks) mma_ss_c<true>(d, desc_from_lo(a + ks * 2), desc_from_lo(b + ks * 2), id_nt);
  };
  // D[128x64] (+)= A^T B : A stored [K=128 rows][M=128] (two 64-wide boxes), B stored [K=128 rows][N=64]
  auto mma_tt = [&](uint32_t d, uint32_t a, uint32_t b, bool acc) {
    if (acc) mma_ss_c<true>(d, desc_from_lo(a), desc_from_lo(b), id_tt);
    else mma_ss_c<false>(d, desc_from_lo(a), desc_from_lo(b), id_tt);
#pragma unroll
    for (int ks = 1; ks < 8; ++ks) mma_ss_c<true>(d, desc_from_lo(a + ks * 128), desc_from_lo(b + ks * 128), id_tt);
  };
  // D[128x64] (+)= A B : A stored [M=128 rows][K=128] (two boxes), B stored [K=128 rows][N=64]
  auto mma_nn = [&](uint32_t d, uint32_t a, uint32_t b, bool acc) {
    if (acc) mma_ss_c<true>(d, desc_from_lo(a), desc_from_lo(b), id_nt64);
    else mma_ss_c<false>(d, desc_from_lo(a), desc_from_lo(b), id_nt64);
#pragma unroll
    for (int ks = 1; ks < 8; ++ks)
      mma_ss_c<true>(d, desc_from_lo(a + (ks >> 2) * 1024 + (ks & 3) * 2), desc_from_lo(b + ks * 128), id_nt64);
  };

  // D[128x64] (+)= [A0 | A1] Bm with A0 = the dO slot, A1 = the 16 leading columns of the E tile (K = 80), Bm [80][64]
  auto mma_aug = [&](uint32_t d, uint32_t a, bool acc) {
    if (acc) mma_ss_c<true>(d, desc_from_lo(a), desc_from_lo(mBm), id_nt64);
    else mma_ss_c<false>(d, desc_from_lo(a), desc_from_lo(mBm), id_nt64);
#pragma unroll
    for (int ks = 1; ks < 5; ++ks)
      mma_ss_c<true>(d, desc_from_lo(a + (ks >> 2) * 1024 + (ks & 3) * 2), desc_from_lo(mBm + ks * 128), id_nt64);
  };
  const int rc0 = c.nvalid * R;

  if (!c.wait(bKvFull, 0)) return;
  int x_uses = 0, rc = 0;    // writes so far into the issuer's own scratch region (X0 for A, X1 for B)
  bool have_dv = false, have_dk = false, have_n = false;     // dV_i / dK_i / N_i accumulators hold something
  for (int T = 0; T < c.ntiles; ++T) {
    const bool valid = T < c.nvalid;
    if (which == 0) {
      // ------------------------------------------------------------- issuer A
      if (valid) {
        if (!c.wait(bKjFull, T)) return;
        if (!p.decay_only) {
          if (x_uses >= 1 && !c.wait(bX0Free, x_uses - 1)) return;
          tc_fence_after();
          mma_nt(X0, kKi, kKj);                                         // G = K_i K_j^T
          tc_commit(c.bar(bGFull));
          ++x_uses;
        }
      }
      if (!valid && T == c.nvalid) {
        // first tile before the chunk: V_i^T K_i (rows 0..63 of the result; the second box of A is whatever the K_j slot holds)
        if (x_uses >= 1 && !c.wait(bX0Free, x_uses - 1)) return;
        tc_fence_after();
        mma_tt(X0, mVi, mKi, false);
        tc_commit(c.bar(bMraw));
        ++x_uses;
      }
      for (int r = 0; r < R; ++r, ++rc) {
        if (valid) {
          if (!c.wait(bInFull, rc)) return;
          if (!c.wait(bX0Free, x_uses - 1)) return;
          tc_fence_after();
          mma_nt(X0, kQ, kKi);                                          // S = Q K_i^T
          ++x_uses;
          tc_commit(c.bar(bSdpFull));
          if (!c.wait(bPdsReady, rc)) return;
          tc_fence_after();
          mma_tt(DV, mP, mGo, have_dv);                                 // dV_i += P^T dO
          mma_tt(DK, mdS, mQ, have_dk);                                 // dK_i += dS^T Q
          have_dk = true;
          have_dv = true;
          tc_commit(c.bar(bInFree));                                    // Q and dO slots can be refilled (once both issuers say so)
        } else {
          const MaskSlot ms = mask_slot(rc - rc0, rc0);
          if (!c.wait(ms.full_bar, ms.phase) || !c.wait(ms.ready_bar, ms.ready_phase)) return;
          if (!have_n && !c.wait(bX0Free, x_uses - 1)) return;          // M_i has been read out of X0
          tc_fence_after();
          mma_tt(X0, desc_lo(sb + ms.go, 16384), desc_lo(sb + ms.q, 16384), have_n);   // N_i += [g | E]^T Q
          have_n = true;
          tc_commit(c.bar(ms.free_bar));          // (bRDone of these steps belongs to issuer B alone: N_i is not waited for)
          continue;
        }
        tc_commit(c.bar(bRDone));
      }
      if (valid) {
        if (x_uses >= 1 && !c.wait(bX0Free, x_uses - 1)) return;
        tc_fence_after();
        mma_nt(X0, kKi, kKj);                                           // G again for the decay backward
        tc_commit(c.bar(bG2Full));
        ++x_uses;
        if (!c.wait(bDgReady, T)) return;
        tc_fence_after();
        mma_nn(DK, kdG, mKj, have_dk);                                  // dK_i += dG K_j
        have_dk = true;
        tc_commit(c.bar(bDkjFull));
      }
    } else {
      // ------------------------------------------------------------- issuer B
      for (int r = 0; r < R; ++r, ++rc) {
        if (valid) {
          if (!c.wait(bInFull, rc)) return;
          if (x_uses >= 1 && !c.wait(bX1Free, x_uses - 1)) return;
          tc_fence_after();
          mma_nt(X1, kGo, kVi);                                         // dP = dO V_i^T
          ++x_uses;
          tc_commit(c.bar(bSdpFull));
          tc_commit(c.bar(bInFree));                                    // this issuer's last read of the Q / dO slot
          if (!c.wait(bPdsReady, rc)) return;
          tc_fence_after();
          mma_nn(X1, kdS, mKi, false);                                  // dQ = dS K_i  (dP has been consumed)
#pragma unroll
          for (int nb = 0; nb < 8; ++nb) {                              // dC[key][row] (+)= dS^T I
            if (r > 0) mma_ss_c<true>(XC + nb * 16, desc_from_lo(mdS + nb * 128), desc_from_lo(kI), id_dc);
            else mma_ss_c<false>(XC + nb * 16, desc_from_lo(mdS + nb * 128), desc_from_lo(kI), id_dc);
          }
        } else {
          const MaskSlot ms = mask_slot(rc - rc0, rc0);
          if (!c.wait(ms.full_bar, ms.phase) || !c.wait(ms.ready_bar, ms.ready_phase)) return;
          if (x_uses >= 1 && !c.wait(bX1Free, x_uses - 1)) return;
          tc_fence_after();
          mma_aug(X1, desc_lo(sb + ms.go, 16), false);                  // dQ = [g | E] [M_i ; ksum_i] / 128
          ++x_uses;
          tc_commit(c.bar(ms.free_bar));
          tc_commit(c.bar(bRDone));               // both arrivals: the workers wait for dQ only, N_i trails behind
        }
        tc_commit(c.bar(bRDone));
      }
      if (valid) {
        if (!c.wait(bDgReady, T)) return;
        if (x_uses >= 1 && !c.wait(bX1Free, x_uses - 1)) return;
        tc_fence_after();
        mma_tt(X1, mP, mKi, false);                                     // dK_j = dG^T K_i
        ++x_uses;
        tc_commit(c.bar(bDkjFull));
      }
    }
  }
  tc_commit(c.bar(bFinal));
  if (which == 0 && c.ntiles > c.nvalid) {
    if (!c.wait(bMask2, 0)) return;
    tc_fence_after();
    mma_aug(DK, kGo, have_dk);                                          // dK_i += [V_i - vbar | 1] [N_i ; w] / 128
    tc_commit(c.bar(bFinal2));
  }
}

// ------------------------------------------------------------ worker groups --
// Four groups of 128 threads share every elementwise phase: thread t of group
// `part` owns row/key t and the 32 tile columns [32*part, 32*part+32), which it
// keeps in registers across the passes of a phase.  Partial row/key statistics
// cross between the groups through a shared-memory mailbox and an mbarrier
// rendezvous in which all 512 threads take part, in the same order, every time.
constexpr int kParts = 4;

struct Mailbox {
  const BwdCtx* c;
  float* box;       // [2 slots][kParts][3][128]
  int part, tid, n;
  bool ok;
  // publish (x, y, z), wait for everybody, return all four triples (index = part; w unused)
  __device__ __forceinline__ void gather(float4 mine, float4* all) {
    float* slot = box + (n & 1) * kParts * 3 * 128;
    slot[(part * 3 + 0) * 128 + tid] = mine.x;
    slot[(part * 3 + 1) * 128 + tid] = mine.y;
    slot[(part * 3 + 2) * 128 + tid] = mine.z;
    if (part == 0 && tid == 0) bulk_wait_read_all();   // see drain_x1: the staging buffer is rewritten after a rendezvous
    c->arrive_w(bXchg);
    if (!c->wait_w(bXchg, n)) ok = false;
#pragma unroll
    for (int q = 0; q < kParts; ++q)
      all[q] = make_float4(slot[(q * 3 + 0) * 128 + tid], slot[(q * 3 + 1) * 128 + tid], slot[(q * 3 + 2) * 128 + tid], 0.f);
    ++n;
  }
  __device__ __forceinline__ void sync() {
    if (part == 0 && tid == 0) bulk_wait_read_all();
    c->arrive_w(bXchg);
    if (!c->wait_w(bXchg, n)) ok = false;
    ++n;
  }
};

// Optional phase timing (compile with -DUA_PROFILE_PHASES): thread 0 of worker group 0 of block 0
// accumulates clock64() deltas per phase and stores them after the status word.
#ifdef UA_PROFILE_PHASES
#ifndef UA_PROFILE_BLOCK
#define UA_PROFILE_BLOCK 0
#endif
#define UA_PH_DECL long long ph_t = clock64(), ph_acc[20] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
#define UA_PH(idx) { long long now_ = clock64(); ph_acc[idx] += now_ - ph_t; ph_t = now_; }
#define UA_PH_STORE if (blockIdx.x == UA_PROFILE_BLOCK && part == 0 && tid == 0) { for (int z = 0; z < 20; ++z) reinterpret_cast<long long*>(p.status)[2 + z] = ph_acc[z]; }
#else
#define UA_PH_DECL
#define UA_PH(idx)
#define UA_PH_STORE
#endif

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

template <typename TG, int kMode>
__device__ __forceinline__ void bwd_worker(const BwdCtx& c, const BwdParams& p, const int part, const CUtensorMap* tmDQ,
                                           const CUtensorMap* tmDK) {
  const int L = p.s.L, R = p.decay_only ? 0 : p.s.R, N = p.s.N, Rq = p.s.R;
  const int tid = threadIdx.x & 127, lane = threadIdx.x & 31;
  const uint32_t lane_base = (uint32_t)((threadIdx.x >> 5) & 3) * 32u << 16;
  const TG* ss = static_cast<const TG*>(p.ssrc) + (size_t)c.bh * L;
  const TG* sd = static_cast<const TG*>(p.sdest) + (size_t)c.bh * p.Lr;
  const float s3 = cbrtf(Num<TG>::ld(ss + c.i * 128 + tid));
  float* sT3 = reinterpret_cast<float*>(c.smem + BwdCfg::oT3);
  uint8_t* sCs = c.smem + BwdCfg::oCs;
  uint8_t* sP = c.smem + BwdCfg::oP;
  uint8_t* sdS = c.smem + BwdCfg::odS;
  const size_t chunk_id = (size_t)c.bh * N + c.i;
  const int col0 = 32 * part;
  const uint32_t X0 = c.tmem + BwdCfg::tX0 + lane_base + col0;
  const uint32_t X1 = c.tmem + BwdCfg::tX1 + lane_base;
  const uint32_t XC = c.tmem + BwdCfg::tXC + lane_base + col0;
  const float kLog2e = 1.4426950408889634f;
  const uint32_t swz = (uint32_t)(tid & 7);
  Mailbox mb{&c, reinterpret_cast<float*>(c.smem + BwdCfg::oXch), part, tid, 0, true};
  UA_PH_DECL
  const size_t key_id = chunk_id * 128 + tid;
  float suffix = p.suffix_in ? p.suffix_in[key_id] : 0.f, ds_acc = 0.f, dct = 0.f;

  // this thread's 32 columns of row `tid` of a [row][key] bf16 tile: 4 chunks of box part/2
  auto store_row = [&](uint8_t* base, const uint32_t* v) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint32_t ch = (uint32_t)((part & 1) * 4 + u);
      *reinterpret_cast<uint4*>(base + (part >> 1) * 16384 + tid * 128 + (((ch ^ swz) & 7) << 4)) =
          make_uint4(v[u * 4], v[u * 4 + 1], v[u * 4 + 2], v[u * 4 + 3]);
    }
  };
  // The 128 x 64 fp32 tile in X1 (dQ_rj or dK_j) is added to rows [y, y+128) of a global accumulator: every thread
  // moves 16 columns of row `tid` into the (idle) P buffer as two 128-byte-swizzled [128][32] boxes, and once all 16
  // warps have arrived the group leader issues two TMA reduce-adds.  The buffer is rewritten only after a mailbox
  // rendezvous, before which the leader waits until the reduce has read it.  (The rows before the chunk alternate
  // between two staging buffers, see there.)
  int nstage = 0;
  // release_late: X1 is released only after the arrival at bStage.  Needed where no rendezvous separates two drains (the
  // rows before the chunk): the next write into X1, and with it the next tile to stage, must not overtake a warp that has
  // not arrived at bStage yet, or its arrival would be counted for the wrong tile.
  auto drain_x1 = [&](const CUtensorMap* tm, int y, uint8_t* stage, bool release_late) -> bool {
    uint32_t o[16];
    tmem_ld16(X1 + 16 * part, o);
    tc_wait_ld();
    tc_fence_before();
    if (!release_late) c.arrive_w(bX1Free);
    store_row(stage, o);
    fence_proxy_async();
    c.arrive_w(bStage);
    if (release_late) c.arrive_w(bX1Free);
    bool ok = true;
    if (part == 0 && tid == 0) {
      UA_PH(17)
      ok = c.wait(bStage, nstage);
      UA_PH(18)
      if (ok) {
        tma_reduce_add_2d(tm, 0, y, smem_u32(stage));
        tma_reduce_add_2d(tm, 32, y, smem_u32(stage) + 16384);
        bulk_commit_group();
      }
      UA_PH(19)
    }
    __syncwarp();
    ++nstage;
    return ok;
  };

  int rc = 0;
  // ================================ row tiles that see the chunk (j >= i), swept downwards ================================
  for (int T = 0; T < c.nvalid; ++T) {
    constexpr bool valid = true;
    const int j = c.tile_j(T, N);
    const bool diag = (j == c.i);
    const int rl = p.r0 + (j - p.j_begin) * 128;  // first row of the tile inside the slab
    float* t3buf = sT3 + (T & 1) * 128;

    if (valid && p.decay_only) {
      if (part == 0) t3buf[tid] = cbrtf(Num<TG>::ld(sd + rl + tid));
      mb.sync();
      if (!mb.ok) return;
    }
    if (valid && !p.decay_only) {
      // ---- decay prefix (forward recomputation): thread = key, C^T[row][key] to shared memory ----
      if (part == 0) t3buf[tid] = cbrtf(Num<TG>::ld(sd + rl + tid));
      const float carry = p.carry[(chunk_id * N + j) * 256 + tid];
      mb.sync();                                  // t3 visible; every reader of the previous tile's C^T is done
      UA_PH(0)
      if (!mb.ok || !c.wait_w(bGFull, T)) return;
      UA_PH(1)
      tc_fence_after();
      float ell[32];
      {
        uint32_t g[32];
        tmem_ld32(X0, g);
        tc_wait_ld();
        tc_fence_before();
        c.arrive_w(bX0Free);
#pragma unroll
        for (int x = 0; x < 32; ++x) {
          const int q = col0 + x;
          float e = log_retention(gated_affinity(gram_pow23(__uint_as_float(g[x])), s3, t3buf[q]));
          if (diag && q <= tid) e = 0.f;
          ell[x] = e;
        }
      }
      // block-local scan; the totals of the earlier blocks are added in the forward kernel's order
      float local = 0.f;
#pragma unroll
      for (int x = 0; x < 32; ++x) {
        local += ell[x];
        ell[x] = local;
      }
      float4 tots[kParts];
      mb.gather(make_float4(local, 0.f, 0.f, 0.f), tots);
      if (!mb.ok) return;
      float tprev = 0.f;
#pragma unroll
      for (int q = 0; q < kParts; ++q)
        if (q < part) tprev += tots[q].x;
#pragma unroll
      for (int x = 0; x < 32; ++x) {
        const int q = col0 + x;
        const float v = (diag && q < tid) ? mask_value() : (carry + (tprev + ell[x]));
        *reinterpret_cast<float*>(sCs + q * 512 + ((((tid >> 2) ^ (q & 7)) & 31) << 4) + (tid & 3) * 4) = v;
      }
      mb.sync();                                  // C^T complete
      if (!mb.ok) return;
      UA_PH(2)
    }

    for (int r = 0; r < R; ++r, ++rc) {
      const size_t grow = (chunk_id * Rq + r) * p.Lr + (size_t)rl + tid;
      const size_t qrow = ((size_t)c.bh * Rq + r) * p.Lr + (size_t)rl + tid;
      float gd = 0.f, lse2 = 0.f;
      if (kMode == 2) {
        gd = -p.row_delta[qrow];
        lse2 = p.row_lse[qrow] * kLog2e;
      } else {
        gd = p.g_denom_is_f32 ? static_cast<const float*>(p.g_denom)[grow]
                              : __bfloat162float(static_cast<const __nv_bfloat16*>(p.g_denom)[grow]);
        if (kMode == 1) lse2 = p.lse[grow] * kLog2e;
      }
      if (!c.wait_w(bSdpFull, rc)) return;
      UA_PH(3)
      tc_fence_after();
      uint32_t pp[16], dd[16];
      {
        // ---- thread = row: s = S + C on 32 columns held in registers ------------------------
        float sv[32];
        uint32_t dp[32];
        {
          uint32_t t[32];
          tmem_ld32(X0, t);
          tc_wait_ld();
          tc_fence_before();
          c.arrive_w(bX0Free);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const uint32_t chunk = (uint32_t)(8 * part + u);
            const float4 cv = *reinterpret_cast<const float4*>(sCs + tid * 512 + (((chunk ^ swz) & 31) << 4));
            sv[4 * u + 0] = __uint_as_float(t[4 * u + 0]) + cv.x;
            sv[4 * u + 1] = __uint_as_float(t[4 * u + 1]) + cv.y;
            sv[4 * u + 2] = __uint_as_float(t[4 * u + 2]) + cv.z;
            sv[4 * u + 3] = __uint_as_float(t[4 * u + 3]) + cv.w;
          }
        }
        float corr, linv;
        if (kMode == 2) {
          // merged upstream gradient: P = exp(s - L_row), dS = P (dP - g.merged); nothing crosses the groups
          tmem_ld32(X1 + col0, dp);
          tc_wait_ld();
#pragma unroll
          for (int x = 0; x < 32; ++x) sv[x] = ex2(fmaf(sv[x], kLog2e, -lse2));
          corr = gd;
          linv = 1.0f;
        } else if (kMode == 1) {
          // the forward's log-sum-exp makes P = exp(s - lse) directly; only sum_k P dP crosses the groups
          tmem_ld32(X1 + col0, dp);
          tc_wait_ld();
          float edp = 0.f;
#pragma unroll
          for (int x = 0; x < 32; ++x) {
            const float e = ex2(fmaf(sv[x], kLog2e, -lse2));
            sv[x] = e;
            edp = fmaf(e, __uint_as_float(dp[x]), edp);
          }
          UA_PH(13)
          float4 all[kParts];
          mb.gather(make_float4(edp, 0.f, 0.f, 0.f), all);
          if (!mb.ok) return;
          UA_PH(14)
          corr = gd - ((all[0].x + all[1].x) + (all[2].x + all[3].x));       // g_denom - sum_k P dP
          linv = 1.0f;
        } else {
          // every group stabilises its 32 columns with its own maximum; one rendezvous then
          // combines (max, sum e, sum e dP) of the four groups
          float m = sv[0];
#pragma unroll
          for (int x = 1; x < 32; ++x) m = fmaxf(m, sv[x]);
          UA_PH(11)
          const float mbias = m * kLog2e;
          tmem_ld32(X1 + col0, dp);
          tc_wait_ld();
          float l = 0.f, edp = 0.f;
#pragma unroll
          for (int x = 0; x < 32; ++x) {
            const float e = ex2(fmaf(sv[x], kLog2e, -mbias));
            sv[x] = e;
            l += e;
            edp = fmaf(e, __uint_as_float(dp[x]), edp);
          }
          UA_PH(13)
          float4 all[kParts];
          mb.gather(make_float4(m, l, edp, 0.f), all);
          if (!mb.ok) return;
          UA_PH(14)
          const float mrow = fmaxf(fmaxf(all[0].x, all[1].x), fmaxf(all[2].x, all[3].x));
          float lrow = 0.f, edprow = 0.f;
#pragma unroll
          for (int q = 0; q < kParts; ++q) {
            const float f = ex2((all[q].x - mrow) * kLog2e);
            lrow = fmaf(all[q].y, f, lrow);
            edprow = fmaf(all[q].z, f, edprow);
          }
          linv = ex2((m - mrow) * kLog2e) / lrow;                      // own rescale folded into 1/l
          corr = gd - edprow / lrow;                                   // g_denom - sum_k P dP
        }
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const float p0 = kMode ? sv[2 * u] : sv[2 * u] * linv, p1 = kMode ? sv[2 * u + 1] : sv[2 * u + 1] * linv;
          const float d0 = p0 * (__uint_as_float(dp[2 * u]) + corr), d1 = p1 * (__uint_as_float(dp[2 * u + 1]) + corr);
          __nv_bfloat162 hp = __floats2bfloat162_rn(p0, p1), hd = __floats2bfloat162_rn(d0, d1);
          pp[u] = *reinterpret_cast<uint32_t*>(&hp);
          dd[u] = *reinterpret_cast<uint32_t*>(&hd);
        }
      }
      UA_PH(15)
      if (kMode == 2) {
        // No rendezvous has happened since the previous head's dQ tile was staged in the P buffer: the leader tells
        // everybody when the reduce-add has read it.
        if (part == 0 && tid == 0) {
          bulk_wait_read_all();
          mbar_arrive(c.bar(bStageFree));
        }
        if (!c.wait_w(bStageFree, rc)) return;
      }
      store_row(sP, pp);
      store_row(sdS, dd);
      UA_PH(16)
      fence_proxy_async();
      tc_fence_before();
      c.arrive_w(bPdsReady);
      UA_PH(4)
      // dQ_rj leaves through fp32 atomics: other key chunks add to the same rows
      if (!c.wait_w(bRDone, rc)) return;
      UA_PH(5)
      tc_fence_after();
      drain_x1(tmDQ, (c.bh * Rq + r) * p.Lr + rl, sP, false);
      UA_PH(6)
    }

    if (valid) {
      // ---- decay backward: thread = key; reverse scan of dC, then d affinity -> dG, d src, d dest ----
      if (!c.wait_w(bG2Full, T)) return;
      UA_PH(7)
      tc_fence_after();
      float dcs[32];
      if (p.decay_only) {
        // correction pass: no dC of its own; d ell = suffix_in on every unmasked (key, row) pair
#pragma unroll
        for (int x = 0; x < 32; ++x) dcs[x] = 0.f;
      } else {
        uint32_t t[32];
        tmem_ld32(XC, t);
        tc_wait_ld();
        float run = 0.f;
#pragma unroll
        for (int x = 31; x >= 0; --x) {
          run += __uint_as_float(t[x]);
          dcs[x] = run;
        }
        float4 tots[kParts];
        mb.gather(make_float4(run, 0.f, 0.f, 0.f), tots);
        if (!mb.ok) return;
        dct += (tots[0].x + tots[1].x) + (tots[2].x + tots[3].x);
        // rows after this thread's block: the carried suffix plus the totals of the later blocks
#pragma unroll
        for (int q = kParts - 1; q >= 0; --q)
          if (q > part) suffix += tots[q].x;
      }
      float first = 0.f;
      {
        uint32_t g[32];
        tmem_ld32(X0, g);
        tc_wait_ld();
        tc_fence_before();
        c.arrive_w(bX0Free);
        uint32_t pk[16];
        float dg_hold = 0.f;
#pragma unroll
        for (int x = 31; x >= 0; --x) {
          const int q = col0 + x;
          float dl = dcs[x] + suffix;
          if (diag && q <= tid) dl = 0.f;
          if (q == 0) first = dl;
          const float gv = __uint_as_float(g[x]);
          const float t3 = t3buf[q];
          const float lg = lg2(gv);                                  // NaN for gv < 0: guarded below
          const float pw = gv > 0.f ? ex2(lg * (2.0f / 3.0f)) : 0.f;
          const float a = gated_affinity(pw, s3, t3);
          float da = __fdividef(dl, fminf(fmaxf(a, clamp_lo_bwd()), clamp_hi()) - 1.0f);
          if (!(a <= clamp_hi())) da = 0.f;
          const float dstat = da * pw;
          ds_acc = fmaf(dstat, t3, ds_acc);
          dcs[x] = dstat * s3;                                       // reuse: per-(key,row) term of d static_dest
          float dg = __bfloat162float(__float2bfloat16_rn(da * s3 * t3));
          dg = gv > 0.f ? dg * (2.0f / 3.0f) * ex2(lg * (-1.0f / 3.0f)) : 0.f;
          if (x & 1) {
            dg_hold = dg;
          } else {
            __nv_bfloat162 h = __floats2bfloat162_rn(dg, dg_hold);
            pk[x >> 1] = *reinterpret_cast<uint32_t*>(&h);
          }
        }
        store_row(sP, pk);                     // dG[key][row] reuses the P buffer (rows = keys here)
      }
      fence_proxy_async();
      tc_fence_before();
      c.arrive_w(bDgReady);
      // d static_dest: sum over the 128 keys of dstat * src^(1/3)
      {
        const float colsum = warp_transpose_reduce(dcs, lane);
        const float t3l = t3buf[col0 + lane];
        if (colsum != 0.f) atomicAdd(p.acc_dt + (size_t)c.bh * p.Lr + rl + col0 + lane, colsum / (3.0f * t3l * t3l));
      }
      // the suffix carried to the next (lower) tile is d ell at the tile's first row
      if (!p.decay_only) {
        float4 f[kParts];
        mb.gather(make_float4(first, 0.f, 0.f, 0.f), f);
        if (!mb.ok) return;
        suffix = f[0].x;
      }
      UA_PH(8)
      if (!c.wait_w(bDkjFull, T)) return;
      UA_PH(9)
      tc_fence_after();
      drain_x1(tmDK, c.bh * L + j * 128, sP, false);      // dK_j
      UA_PH(10)
    }
  }
  // ================================ rows before the chunk (j < i): uniform softmax ================================
  if (c.ntiles > c.nvalid) {
    {
      // ---- first tile before the chunk: constants of the rank-65 form of dS (see the head of this file) ----
      const int wt = part * 128 + tid;
      mb.sync();                                  // every reader of C^T / dS / staged tiles is done (and the reduce has read them)
      if (!mb.ok || !c.wait_w(bKvFull, 0)) return;   // K_i, V_i are read from shared memory below
      {
        uint4* e4 = reinterpret_cast<uint4*>(c.smem + BwdCfg::oE);
        uint4* e41 = reinterpret_cast<uint4*>(c.smem + BwdCfg::oE1);
        e4[wt] = make_uint4(0u, 0u, 0u, 0u);
        e4[wt + 512] = make_uint4(0u, 0u, 0u, 0u);
        e41[wt] = make_uint4(0u, 0u, 0u, 0u);
        e41[wt + 512] = make_uint4(0u, 0u, 0u, 0u);
        if (wt < 64) sT3[128 + wt] = 0.f;         // column sums of g, reduced after the sweep
        if (wt >= 256 && wt < 384) reinterpret_cast<uint4*>(c.smem + BwdCfg::oBm + 64 * 128)[wt - 256] = make_uint4(0u, 0u, 0u, 0u);
      }
      if (part == 0) {                            // column sums: sT3[0..63] = sum_k K_i, sT3[64..127] = sum_k V_i
        const uint8_t* tile = c.smem + (tid < 64 ? BwdCfg::oKi : BwdCfg::oVi);
        const int col = tid & 63;
        float acc = 0.f;
#pragma unroll 8
        for (int k = 0; k < 128; ++k)
          acc += __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(tile + k * 128 + ((((col >> 3) ^ k) & 7) << 4) + (col & 7) * 2));
        sT3[tid] = acc;
      }
      mb.sync();
      if (!mb.ok || !c.wait_w(bMraw, 0)) return;
      tc_fence_after();
      if (part == 0 && tid < 64) {                // warps of lanes 0..63: row e = tid of M_i = V_i^T K_i - vsum_e ksum / 128
        const float vb = sT3[64 + tid] * (1.0f / 128.0f);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t m[32];
          tmem_ld32(c.tmem + BwdCfg::tX0 + lane_base + 32 * half, m);
          tc_wait_ld();
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint32_t w4[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) {
              const int d0 = 32 * half + 8 * u + 2 * x;
              const float a0 = (__uint_as_float(m[8 * u + 2 * x]) - vb * sT3[d0]) * (1.0f / 128.0f);
              const float a1 = (__uint_as_float(m[8 * u + 2 * x + 1]) - vb * sT3[d0 + 1]) * (1.0f / 128.0f);
              __nv_bfloat162 hh = __floats2bfloat162_rn(a0, a1);
              w4[x] = *reinterpret_cast<uint32_t*>(&hh);
            }
            *reinterpret_cast<uint4*>(c.smem + BwdCfg::oBm + tid * 128 + ((((4 * half + u) ^ tid) & 7) << 4)) =
                make_uint4(w4[0], w4[1], w4[2], w4[3]);
          }
        }
      }
      if (part == 0 && tid >= 64) {               // row 64 of the operand: ksum / 128 (64 threads x 1 element)
        const int d0 = tid - 64;
        *reinterpret_cast<__nv_bfloat16*>(c.smem + BwdCfg::oBm + 64 * 128 + (((d0 >> 3) & 7) << 4) + (d0 & 7) * 2) =
            __float2bfloat16_rn(sT3[d0] * (1.0f / 128.0f));
      }
      tc_fence_before();
      c.arrive_w(bX0Free);
    }

    const int rc0 = rc;
    float gsum[16];                               // this thread's share of the column sums of g (for dV_i)
#pragma unroll
    for (int x = 0; x < 16; ++x) gsum[x] = 0.f;
    // Steps m = 0 .. M-1 over (tile, head).  prepare(m) -- this thread's part of the operands of step m -- runs BEFORE the
    // wait for the MMAs of step m-1, so that issuer B can start step m as soon as X1 has been read out.
    const int M = (c.ntiles - c.nvalid) * R;
    auto step_row0 = [&](int m) -> int {            // first row (inside the slab) of step m's tile
      return p.r0 + (c.tile_j(c.nvalid + m / R, N) - p.j_begin) * 128;
    };
    // g_denom of row `tid`, fetched two steps ahead: its latency would otherwise sit in every step's chain
    auto load_gd = [&](int m) -> float {
      if (m >= M || part != 0 || p.gd_f32) return 0.f;
      const size_t grow = (chunk_id * Rq + (m % R)) * p.Lr + (size_t)step_row0(m) + tid;
      return p.g_denom_is_f32 ? static_cast<const float*>(p.g_denom)[grow]
                              : __bfloat162float(static_cast<const __nv_bfloat16*>(p.g_denom)[grow]);
    };
    auto prepare = [&](int m, float gd) -> bool {
      const MaskSlot ms = mask_slot(m, rc0);
      if (!c.wait_w(ms.full_bar, ms.phase)) return false;   // the dO tile has landed ...
      // ... which also means that the slot was free: the MMAs of two steps ago, the readers of this slot's E, are complete
      if (p.gd_f32) gd = reinterpret_cast<const float*>(c.smem + BwdCfg::oXch)[(m & 1) * 128 + tid];      // (came with the tiles)
      if (part == 0) *reinterpret_cast<__nv_bfloat16*>(c.smem + ms.e + tid * 128 + ((tid & 7) << 4)) = __float2bfloat16_rn(gd);
#pragma unroll
      for (int u = 0; u < 2; ++u) {                 // 16 columns of row `tid` of dO into the column sums
        const uint4 raw = *reinterpret_cast<const uint4*>(c.smem + ms.go + tid * 128 + ((((uint32_t)(2 * part + u) ^ swz) & 7) << 4));
        const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const __nv_bfloat162 hv = *reinterpret_cast<const __nv_bfloat162*>(&rw[x]);
          gsum[8 * u + 2 * x] += __bfloat162float(hv.x);
          gsum[8 * u + 2 * x + 1] += __bfloat162float(hv.y);
        }
      }
      fence_proxy_async();
      // step m stages its dQ tile in buffer m & 1, last used by step m-2, whose reduce-add has been issued by now: it must
      // have read the buffer before anybody passes bRDone of step m, which follows the completion of this bPdsReady
      if (part == 0 && tid == 0) bulk_wait_read_all();
      c.arrive_w(ms.ready_bar);
      return true;
    };
    float gd0 = load_gd(0), gd1 = load_gd(1);
    if (!prepare(0, gd0)) return;
    for (int m = 0; m < M; ++m, ++rc) {
      const float gd2 = load_gd(m + 2);
      if (m + 1 < M && !prepare(m + 1, gd1)) return;
      gd1 = gd2;
      if (!c.wait_w(bRDone, rc)) return;
      tc_fence_after();
      drain_x1(tmDQ, (c.bh * Rq + (m % R)) * p.Lr + step_row0(m), (m & 1) ? sdS : sP, true);
    }
#pragma unroll
    for (int x = 0; x < 16; ++x) {
      float v = gsum[x];
#pragma unroll
      for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) atomicAdd(sT3 + 128 + 16 * part + x, v);
    }
  }
  UA_PH_STORE

  // ---- end of the sweep: dV_i, dK_i, d static_src (thread = key, 16 of the 64 columns each) ----
  if (!c.wait_w(bFinal, 0)) return;
  tc_fence_after();
  if (c.ntiles > c.nvalid) {
    // rows before the chunk: dK_i += [V_i - vbar | 1] [N_i ; w] / 128 through one more MMA
    if (part == 0 && tid < 96) {                  // lanes 0..63 hold N_i, lane 64 holds w (warps of lanes 0..95 load)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t m[32];
        tmem_ld32(c.tmem + BwdCfg::tX0 + lane_base + 32 * half, m);
        tc_wait_ld();
        if (tid <= 64) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint32_t w4[4];
#pragma unroll
            for (int x = 0; x < 4; ++x) {
              __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(m[8 * u + 2 * x]) * (1.0f / 128.0f),
                                                        __uint_as_float(m[8 * u + 2 * x + 1]) * (1.0f / 128.0f));
              w4[x] = *reinterpret_cast<uint32_t*>(&hh);
            }
            *reinterpret_cast<uint4*>(c.smem + BwdCfg::oBm + tid * 128 + ((((4 * half + u) ^ tid) & 7) << 4)) =
                make_uint4(w4[0], w4[1], w4[2], w4[3]);
          }
        }
      }
    }
    {                                             // V_i - vbar into the dO slot, 16 columns of key `tid` per thread
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const uint32_t off = (uint32_t)tid * 128 + ((((uint32_t)(2 * part + u) ^ swz) & 7) << 4);
        const uint4 raw = *reinterpret_cast<const uint4*>(c.smem + BwdCfg::oVi + off);
        const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
        uint32_t w4[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const __nv_bfloat162 hv = *reinterpret_cast<const __nv_bfloat162*>(&rw[x]);
          const int d0 = 16 * part + 8 * u + 2 * x;
          __nv_bfloat162 hh = __floats2bfloat162_rn(__bfloat162float(hv.x) - sT3[64 + d0] * (1.0f / 128.0f),
                                                    __bfloat162float(hv.y) - sT3[64 + d0 + 1] * (1.0f / 128.0f));
          w4[x] = *reinterpret_cast<uint32_t*>(&hh);
        }
        *reinterpret_cast<uint4*>(c.smem + BwdCfg::oGo + off) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
      }
      if (part == 0) *reinterpret_cast<__nv_bfloat16*>(c.smem + BwdCfg::oE + tid * 128 + ((tid & 7) << 4)) = __float2bfloat16_rn(1.0f);
    }
    fence_proxy_async();
    tc_fence_before();
    c.arrive_w(bMask2);
    mb.sync();                                    // the column sums of g are complete
    if (!mb.ok || !c.wait_w(bFinal2, 0)) return;
    tc_fence_after();
  }
  const size_t krow = (size_t)c.bh * L + c.i * 128 + tid;
  {
    uint32_t o[16];
    if (!p.decay_only) {
      if (c.nvalid > 0) {
        tmem_ld16(c.tmem + BwdCfg::tDV + lane_base + 16 * part, o);
        tc_wait_ld();
      } else {
#pragma unroll
        for (int u = 0; u < 16; ++u) o[u] = 0u;
      }
      if (c.ntiles > c.nvalid) {                  // rows before the chunk: dV_i += (1/128) 1^T g for every key
#pragma unroll
        for (int u = 0; u < 16; ++u) o[u] = __float_as_uint(__uint_as_float(o[u]) + sT3[128 + 16 * part + u] * (1.0f / 128.0f));
      }
      if (p.acc_dv) {
        float* dst = p.acc_dv + krow * 64 + 16 * part;          // several row ranges may add to the same keys
#pragma unroll
        for (int u = 0; u < 4; ++u)
          red_add_v4(dst + u * 4, __uint_as_float(o[u * 4]), __uint_as_float(o[u * 4 + 1]), __uint_as_float(o[u * 4 + 2]),
                     __uint_as_float(o[u * 4 + 3]));
      } else {
        uint32_t pk[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(o[2 * u]), __uint_as_float(o[2 * u + 1]));
          pk[u] = *reinterpret_cast<uint32_t*>(&h);
        }
        uint4* dst = reinterpret_cast<uint4*>(p.dvc + krow * 64 + 16 * part);
        dst[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        dst[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
      }
    }
    tmem_ld16(c.tmem + BwdCfg::tDK + lane_base + 16 * part, o);
    tc_wait_ld();
    float* dk = p.acc_dk + krow * 64 + 16 * part;
#pragma unroll
    for (int u = 0; u < 4; ++u)
      red_add_v4(dk + u * 4, __uint_as_float(o[u * 4]), __uint_as_float(o[u * 4 + 1]), __uint_as_float(o[u * 4 + 2]),
                 __uint_as_float(o[u * 4 + 3]));
  }
  float4 od[kParts];
  mb.gather(make_float4(ds_acc, 0.f, 0.f, 0.f), od);
  if (mb.ok && part == 0 && !p.masked_only) {
    const float dsv = ((od[0].x + od[1].x) + (od[2].x + od[3].x)) / (3.0f * s3 * s3);
    if (p.acc_ds) atomicAdd(p.acc_ds + krow, dsv);
    else Num<TG>::st(static_cast<TG*>(p.dss) + krow, dsv);
    if (p.dctot_out) p.dctot_out[key_id] = dct;
  }
}

template <typename TG, int kMode>
__global__ void __launch_bounds__(640, 1)
bwd_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
           const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmG,
           const __grid_constant__ CUtensorMap tmDQ, const __grid_constant__ CUtensorMap tmDK, BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint32_t* misc = reinterpret_cast<uint32_t*>(smem + BwdCfg::oMisc);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int BH = p.s.B * p.s.H;

  BwdCtx c;
  c.smem = smem;
  c.bars = smem_u32(smem + BwdCfg::oBar);
  c.abort_flag = reinterpret_cast<volatile int*>(misc + 1);
  c.i = blockIdx.x / BH;
  c.bh = blockIdx.x - c.i * BH;
  c.j_begin = p.j_begin;
  c.j_end = p.j_end;
  {
    const int lo = c.i > p.j_begin ? c.i : p.j_begin;               // first row tile of the range that sees the chunk
    const int top = c.i < p.j_end ? c.i : p.j_end;                  // rows below this tile index lie before the chunk
    c.nvalid = (p.j_end > lo && !p.masked_only) ? p.j_end - lo : 0;
    const int nmask = (p.skip_masked || p.decay_only || p.merged || top <= p.j_begin) ? 0 : top - p.j_begin;
    c.ntiles = c.nvalid + nmask;
  }

  if (threadIdx.x == 0) {
    misc[1] = 0;
    misc[2] = 0;
    for (int b = 0; b < bNumBars; ++b) {
      uint32_t count = 1;
      if (b == bX0Free || b == bX1Free || b == bPdsReady || b == bDgReady || b == bXchg || b == bStage || b == bMask2 || b == bPdsM0 || b == bPdsM1) count = 16;   // one arrival per worker warp
      if (b == bSdpFull || b == bRDone || b == bDkjFull || b == bFinal || b == bInFree || b == bInFree1) count = 2;                       // one commit per MMA issuer
      mbar_init(c.bar(b), count);
    }
    mbar_init_fence();
    prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmQ); prefetch_tmap(&tmG);
    prefetch_tmap(&tmDQ); prefetch_tmap(&tmDK);
  }
  // identity tile: 16 rows x 64 bf16 (128-byte swizzled rows), ones on the diagonal of the first 16 columns
  for (int e = threadIdx.x; e < 512; e += blockDim.x) reinterpret_cast<uint32_t*>(smem + BwdCfg::oI)[e] = 0u;
  __syncthreads();
  if (threadIdx.x < 16) {
    const int n = threadIdx.x;
    *reinterpret_cast<__nv_bfloat16*>(smem + BwdCfg::oI + (n >> 3) * 1024 + (n & 7) * 128 + ((((n >> 3) ^ (n & 7)) & 7) << 4) +
                                      (n & 7) * 2) = __float2bfloat16_rn(1.0f);
  }
  fence_proxy_async();
  if (warp == 0) {
    tmem_alloc(smem_u32(misc), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  c.tmem = misc[0];

  if (c.ntiles == 0) {
    // no row of the range touches this chunk (sequence sharding only): nothing to add anywhere
    if (warp >= 4 && warp < 8 && p.dctot_out) p.dctot_out[((size_t)c.bh * p.s.N + c.i) * 128 + (threadIdx.x & 127)] = 0.f;
  } else if (warp == 0) {
    if (lane == 0) bwd_producer(c, p, &tmK, &tmV, &tmQ, &tmG);
  } else if (warp == 1 || warp == 2) {
    if (lane == 0) bwd_mma(c, p, warp - 1);
  } else if (warp >= 4) {
    bwd_worker<TG, kMode>(c, p, (warp - 4) >> 2, &tmDQ, &tmDK);
    if (threadIdx.x == 128) bulk_wait_all();      // the leader's reduce-adds have landed before the block retires
  }

  tc_fence_before();
  __syncthreads();
  if (*c.abort_flag) {
    if (threadIdx.x == 0) {
      if (atomicExch(p.status, 2) == 0) p.status[1] = (int)misc[2];   // where the first block to give up stopped
    }
    for (int it = 0; it < 64; ++it) __nanosleep(2000);
    __syncthreads();
  }
  if (warp == 0) tmem_dealloc(c.tmem, 512);
}

}  // namespace sm100
}  // namespace ua
