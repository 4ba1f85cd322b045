// Tensor-core forward of the Universal Attention operator for sm_100a.
//
// bf16 inputs, key chunk = 128, head_dim D in {64, 128}.  One thread block owns
// one key chunk (b, h, i) and sweeps the row tiles j = i .. n-1 (128 rows each)
// upwards, so the per-key decay prefix is carried in registers.
//
//   G    = K_i  K_j^T    tcgen05.mma  M = keys, N = rows   (keys on TMEM lanes)
//   S_r  = Q_rj K_i^T    tcgen05.mma  M = rows, N = keys   (rows on TMEM lanes)
//   O_r  = P_r  V_i      tcgen05.mma  A = P (bf16, TMEM), B = V_i (MN-major smem)
//
// Warp roles (512 threads):
//   warp 0      TMA producer: K_i, V_i once; K_j and Q_rj tiles through mbarrier rings
//   warp 1      MMA issuer (one elected thread issues every tcgen05.mma / commit)
//   warps 4-7   decay group: thread = key.  Reads G from TMEM, computes the
//               log-retention, scans it along the rows in registers (carry kept
//               across tiles), writes the prefix C^T[row][key] to shared memory.
//   warps 8-15  two softmax groups alternating over (tile, r): thread = row.
//               S + C, row max / sum in registers (no shuffles), P -> TMEM as
//               bf16, then the epilogue O / l -> out and m + log l -> lse.
//
// The two reductions of the operator run along perpendicular axes of the tile
// (scan along rows per key, softmax along keys per row); putting keys on lanes
// for G and rows on lanes for S makes both of them thread-local, at the price
// of one 64 KB shared-memory transpose of C per tile, shared by the R heads.
//
// Every mbarrier wait is bounded; on a timeout the block raises a shared abort
// flag, every role leaves its loop, TMEM is freed and status[0] is set.
#pragma once
#include <type_traits>
#include "ua_common.cuh"
#include "ua_ptx.cuh"

namespace ua {
namespace sm100 {

using namespace ua::ptx;

#ifdef UA_PROFILE_FWD
#define UF_DECL long long uf_t = clock64(), uf_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#define UF(idx) { long long now_ = clock64(); uf_acc[idx] += now_ - uf_t; uf_t = now_; }
#define UF_STORE(cond, base) if (blockIdx.x == 0 && (cond)) { for (int z = 0; z < 8; ++z) reinterpret_cast<long long*>(p.status)[2 + (base) + z] = uf_acc[z]; }
#else
#define UF_DECL
#define UF(idx)
#define UF_STORE(cond, base)
#endif

struct FwdParams {
  Shape s;
  const void* ssrc;
  const void* sdest;
  const void* vc;        // values, for the masked-row fill
  __nv_bfloat16* out;    // chunk-major (b,h,n,r,L,d); null: only lse / denom are produced
  float* lse;            // (b,h,n,r,L)
  __nv_bfloat16* denom;  // (b,h,n,r,L) or null
  int* status;           // device word: 0 = ok, otherwise a role-specific timeout code
  int fill_masked;       // write the rows before the key chunk (uniform softmax) from the two otherwise idle warps
  // Row range (sequence sharding): this call computes row tiles [j_begin, j_end) only.  xq, static_dest, out,
  // lse and denom then hold just those Lr = (j_end - j_begin) * 128 rows; keys, values and static_src are whole.
  int j_begin, j_end, Lr;  // Lr: rows per (chunk, head) slab of the row-indexed tensors
  int r0;                  // row of the slab where the range starts (several ranges can share one slab)
  const float* carry_in;   // optional (b*h*n, 128): decay prefix of key k at its first row tile of the range
  float* total_out;        // optional (b*h*n, 128): decay prefix after the last row tile of the range
  float* carry;          // optional (required in carry-only mode): (b*h*n, n, 2, 128) decay prefix of key k at the start of each 64-row half of row tile j
  // merged-output mode (fwd_kernel<..., kMerge = true>): instead of writing `out`, every (chunk, row tile, head) adds its
  // share of the row's softmax over ALL keys, exp(m - row_lse) * (P~ V) with P~ = exp(s - m) unnormalised, to merged_acc
  float* merged_acc;     // (b,h,r,L,d) fp32, zeroed by the caller
  const float* row_lse;  // (b,h,r,L) fp32: log-sum-exp of every row over all key chunks (from a statistics-only run)
};

// Gated affinity and log-retention of one (key, row) pair from the Gram value
// (universal_attention_autograd.py:148-150), with hardware ex2/lg2.  Shared by
// the forward, the carry pre-pass and the backward so that recomputation is
// bit-identical.
__device__ __forceinline__ float gram_pow23(float gv) { return gv > 0.f ? ex2(lg2(gv) * (2.0f / 3.0f)) : 0.f; }
__device__ __forceinline__ float gated_affinity(float pw, float s3, float t3) { return pw * s3 * t3; }
__device__ __forceinline__ float log_retention(float a) {
  return lg2(1.0f - fminf(a, clamp_hi())) * 0.6931471805599453f;
}

// packed fp32 pairs (one instruction for two lanes of work: the element-wise phases are bound by instruction issue)
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  float2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(reinterpret_cast<unsigned long long&>(d))
      : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)));
  return d;
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
  float2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(reinterpret_cast<unsigned long long&>(d))
      : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)));
  return d;
}
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(reinterpret_cast<unsigned long long&>(d))
      : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)),
        "l"(reinterpret_cast<unsigned long long&>(c)));
  return d;
}

// What the softmax groups produce: the per-chunk output tiles (and log-sum-exp), the merged-output contribution, or the
// log-sum-exp alone (then no probabilities are written, no PV product is issued, nothing is drained).
enum FwdOut { kOutTiles = 0, kOutMerged = 1, kOutStats = 2 };

// three-input maximum (one instruction on sm_100)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

template <int D>
struct FwdCfg {
  static constexpr int kTileBytes = 128 * D * 2;   // one [128][D] bf16 tile
  static constexpr int kBoxBytes = 128 * 128;      // one TMA box: 128 rows x 64 elements
  static constexpr int kBoxes = D / 64;
  static constexpr int kKjStages = (D == 64) ? 2 : 1;
  static constexpr int kQStages = 2;
  static constexpr int kOBufs = (D == 64) ? 2 : 1;
  static constexpr int oKi = 0;
  static constexpr int oVi = oKi + kTileBytes;
  static constexpr int oKj = oVi + kTileBytes;
  static constexpr int oQ = oKj + kKjStages * kTileBytes;
  // The decay prefix crosses from keys-on-lanes to rows-on-lanes through a 64 KB fp32 tile C^T[row][key].  With two
  // of them (head_dim 64: they fit) the decay group computes tile T+1 while the softmax groups consume tile T;
  // with one, the two alternate (measured at head_dim 64: 18.7k cycles per tile = decay 9.8k + softmax 14k, minus overlap).
  static constexpr int kCBufs = (D == 64) ? 2 : 1;
  static constexpr int oCs = oQ + kQStages * kTileBytes;
  static constexpr int oT3 = oCs + kCBufs * 65536;
  static constexpr int oBar = oT3 + 1024;
  static constexpr int oMisc = oBar + 256;
  static constexpr int oFill = oMisc + 64;                // bf16[D]: value of a fully masked output row
  static constexpr int kSmemBytes = oFill + 256 + 1024;  // + slack to align the base to 1024 B
  static constexpr uint32_t tG = 0, tS0 = 128, tS1 = 256, tO0 = 384, tO1 = 384 + D;
};

enum FwdBar {
  // (kCReady / kCFree: one barrier per C^T buffer, so that no waiter can fall two phases behind on a shared one)
  kKvFull = 0, kKjFull = 1, kKjEmpty = 3, kQFull = 5, kQEmpty = 7, kGFull = 9, kGFree = 10, kCReady = 11, kCFree = 13,
  kSFull = 15, kPReady = 17, kOFull = 19, kOFree = 21, kT3Ready = 23, kNumBars = 24
};

template <int D>
struct FwdCtx {
  uint8_t* smem;
  uint32_t bars;      // shared address of barrier 0
  uint32_t tmem;
  volatile int* abort_flag;
  int i, bh, ntiles;
  int j0;             // first row tile this block computes: max(i, j_begin)
  __device__ __forceinline__ uint32_t bar(int idx) const { return bars + 8u * idx; }
  __device__ __forceinline__ bool wait(int idx, uint32_t parity) const { return mbar_wait(bar(idx), parity & 1u, abort_flag); }
  // warp-collective forms for the decay and softmax groups
  __device__ __forceinline__ bool wait_w(int idx, uint32_t parity) const { return mbar_wait_warp(bar(idx), parity & 1u, abort_flag); }
  __device__ __forceinline__ void arrive_w(int idx) const { mbar_arrive_warp(bar(idx)); }
};

// ------------------------------------------------------------------ producer --
template <int D, bool kCarryOnly>
__device__ __forceinline__ void fwd_producer(const FwdCtx<D>& c, const FwdParams& p, const CUtensorMap* tmK,
                                             const CUtensorMap* tmV, const CUtensorMap* tmQ) {
  using Cfg = FwdCfg<D>;
  const int L = p.s.L, R = p.s.R;
  const uint32_t sbase = smem_u32(c.smem);
  const int krow = c.bh * L + c.i * 128;
  mbar_expect_tx(c.bar(kKvFull), (kCarryOnly ? 1 : 2) * Cfg::kTileBytes);
  for (int b = 0; b < Cfg::kBoxes; ++b) {
    tma_load_2d(sbase + Cfg::oKi + b * Cfg::kBoxBytes, tmK, b * 64, krow, c.bar(kKvFull));
    if (!kCarryOnly) tma_load_2d(sbase + Cfg::oVi + b * Cfg::kBoxBytes, tmV, b * 64, krow, c.bar(kKvFull));
  }
  auto load_kj = [&](int T) -> bool {
    const int ks = T % Cfg::kKjStages, u = T / Cfg::kKjStages;
    if (u >= 1 && !c.wait(kKjEmpty + ks, u - 1)) return false;
    mbar_expect_tx(c.bar(kKjFull + ks), Cfg::kTileBytes);
    for (int b = 0; b < Cfg::kBoxes; ++b)
      tma_load_2d(sbase + Cfg::oKj + ks * Cfg::kTileBytes + b * Cfg::kBoxBytes, tmK, b * 64, c.bh * L + (c.j0 + T) * 128,
                  c.bar(kKjFull + ks));
    return true;
  };
  if (!load_kj(0)) return;
  if (kCarryOnly) {
    for (int T = 1; T < c.ntiles; ++T)
      if (!load_kj(T)) return;
    return;
  }
  int t = 0;
  for (int T = 0; T < c.ntiles; ++T) {
    for (int r = 0; r < R; ++r, ++t) {
      const int qs = t & 1, u = t >> 1;
      if (u >= 1 && !c.wait(kQEmpty + qs, u - 1)) return;
      mbar_expect_tx(c.bar(kQFull + qs), Cfg::kTileBytes);
      for (int b = 0; b < Cfg::kBoxes; ++b)
        tma_load_2d(sbase + Cfg::oQ + qs * Cfg::kTileBytes + b * Cfg::kBoxBytes, tmQ, b * 64,
                    (c.bh * R + r) * p.Lr + p.r0 + (c.j0 + T - p.j_begin) * 128, c.bar(kQFull + qs));
      if (r == 0 && T + 1 < c.ntiles && !load_kj(T + 1)) return;
    }
  }
}

// ---------------------------------------------------------------- MMA issuer --
template <int D, bool kCarryOnly, int kOut>
__device__ __forceinline__ void fwd_mma(const FwdCtx<D>& c, const FwdParams& p) {
  using Cfg = FwdCfg<D>;
  const int R = p.s.R;
  const uint32_t sbase = smem_u32(c.smem);
  constexpr uint32_t idesc_sq = idesc_bf16(128, 128, 0, 0);
  constexpr uint32_t idesc_pv = idesc_bf16(128, D, 0, 1);
  const uint32_t tS[2] = {c.tmem + Cfg::tS0, c.tmem + Cfg::tS1};
  const uint32_t tO[2] = {c.tmem + Cfg::tO0, c.tmem + (Cfg::kOBufs == 2 ? Cfg::tO1 : Cfg::tO0)};

  // D[128 x 128] = A[128][D] * B[128][D]^T, both K-major.  Operands are passed as descriptor low words
  // (built once: shared-memory addresses never change); a k-step of 16 elements is +32 B (>>4 = 2), the
  // second 64-element box of a tile +16384 B (>>4 = 1024).
  auto issue_kmajor = [&](uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo) {
    mma_ss_c<false>(d_tmem, desc_from_lo(a_lo), desc_from_lo(b_lo), idesc_sq);
#pragma unroll
    for (int ks = 1; ks < D / 16; ++ks) {
      const uint32_t off = (ks >> 2) * 1024 + (ks & 3) * 2;
      mma_ss_c<true>(d_tmem, desc_from_lo(a_lo + off), desc_from_lo(b_lo + off), idesc_sq);
    }
  };
  const uint32_t kKi = desc_lo(sbase + Cfg::oKi, 16);
  const uint32_t mVi = desc_lo(sbase + Cfg::oVi, Cfg::kBoxBytes);
  auto issue_g = [&](int T) -> bool {
    const int ks = T % Cfg::kKjStages, u = T / Cfg::kKjStages;
    if (!c.wait(kKjFull + ks, u)) return false;
    if (T >= 1 && !c.wait(kGFree, T - 1)) return false;
    tc_fence_after();
    issue_kmajor(c.tmem + Cfg::tG, kKi, desc_lo(sbase + Cfg::oKj + ks * Cfg::kTileBytes, 16));
    tc_commit(c.bar(kGFull));
    tc_commit(c.bar(kKjEmpty + ks));
    return true;
  };
  auto issue_pv = [&](int tt) -> bool {
    const int sb = tt & 1, ob = tt % Cfg::kOBufs;
    if (!c.wait(kPReady + sb, tt >> 1)) return false;       // (statistics only: the group is done with the S buffer)
    if (kOut == kOutStats) return true;
    // the O buffer must have been drained by the epilogue that used it last
    // (barriers are per softmax group so that each waiter sees consecutive phases)
    if (Cfg::kOBufs == 2) {
      if (tt >= 2 && !c.wait(kOFree + sb, (tt >> 1) - 1)) return false;
    } else {
      if (tt >= 1 && !c.wait(kOFree + ((tt - 1) & 1), (tt - 1) >> 1)) return false;
    }
    tc_fence_after();
    mma_ts_c<false>(tO[ob], tS[sb], desc_from_lo(mVi), idesc_pv);
#pragma unroll
    for (int ks = 1; ks < 8; ++ks) mma_ts_c<true>(tO[ob], tS[sb] + ks * 8, desc_from_lo(mVi + ks * 128), idesc_pv);
    tc_commit(c.bar(kOFull + sb));
    return true;
  };

  if (!c.wait(kKvFull, 0)) return;
  if (!issue_g(0)) return;
  if (kCarryOnly) {
    for (int T = 1; T < c.ntiles; ++T)
      if (!issue_g(T)) return;
    return;
  }
  int t = 0;
  for (int T = 0; T < c.ntiles; ++T) {
    for (int r = 0; r < R; ++r, ++t) {
      const int qs = t & 1;
      if (!c.wait(kQFull + qs, t >> 1)) return;
      tc_fence_after();
      issue_kmajor(tS[t & 1], desc_lo(sbase + Cfg::oQ + qs * Cfg::kTileBytes, 16), kKi);
      tc_commit(c.bar(kSFull + (t & 1)));
      tc_commit(c.bar(kQEmpty + qs));
      if (t >= 1 && !issue_pv(t - 1)) return;
      if (r == 0 && T + 1 < c.ntiles && !issue_g(T + 1)) return;
    }
  }
  if (t >= 1) issue_pv(t - 1);
}

// --------------------------------------------------------------- decay group --
template <int D, typename TG, bool kCarryOnly>
__device__ __forceinline__ void fwd_decay(const FwdCtx<D>& c, const FwdParams& p) {
  using Cfg = FwdCfg<D>;
  const int L = p.s.L;
  const int k = threadIdx.x & 127;
  const uint32_t lane_base = (uint32_t)((threadIdx.x >> 5) & 3) * 32u << 16;
  const TG* ss = static_cast<const TG*>(p.ssrc) + (size_t)c.bh * L;
  const TG* sd = static_cast<const TG*>(p.sdest) + (size_t)c.bh * p.Lr + p.r0 + (c.j0 - p.j_begin) * 128 + k;
  const float s3 = cbrtf(Num<TG>::ld(ss + c.i * 128 + k));
  float raw_next = Num<TG>::ld(sd);      // the gate value of the next tile is fetched one pass ahead: its latency hides behind the pass
  float* sT3 = reinterpret_cast<float*>(c.smem + Cfg::oT3);
  uint8_t* sCs = c.smem + Cfg::oCs;
  const size_t key_id = ((size_t)c.bh * p.s.N + c.i) * 128 + k;
  // The prefix carried from tile to tile reaches -2e4 at L = 4096, where fp32 spacing is 2e-3: it is kept as an
  // unevaluated sum carry + carry_lo (the rounding error of every tile's addition is carried along), so that what a
  // row sees is one rounding away from the exact sum however many tiles came before it.
  float carry = p.carry_in ? p.carry_in[key_id] : 0.f, carry_lo = 0.f;
  UF_DECL
  for (int T = 0; T < c.ntiles; ++T) {
    const int j = c.j0 + T;
    float* t3buf = sT3 + (T & 1) * 128;
    t3buf[k] = cbrtf(raw_next);
    if (T + 1 < c.ntiles) raw_next = Num<TG>::ld(sd + (T + 1) * 128);
    c.arrive_w(kT3Ready);
    if (!c.wait_w(kT3Ready, T)) return;
    UF(0)
    if (!c.wait_w(kGFull, T)) return;
    UF(1)
    tc_fence_after();
    const bool diag = (j == c.i);
    float* carry_row = p.carry ? p.carry + (((size_t)c.bh * p.s.N + c.i) * p.s.N + j) * 256 + k : nullptr;
    if (carry_row) carry_row[0] = carry;
    // The prefix inside a tile is  carry + (carry_lo + sum of the totals of earlier 32-row blocks + scan inside the block).
    float tprev = carry_lo, cval = carry;
#pragma unroll 1
    for (int cb = 0; cb < 4; ++cb) {
      uint32_t g[32];
      tmem_ld32(c.tmem + Cfg::tG + lane_base + cb * 32, g);
      tc_wait_ld();
      if (cb == 3) {
        tc_fence_before();
        c.arrive_w(kGFree);
      }
      if (cb == 2 && carry_row) carry_row[128] = cval;      // prefix after the first 64 rows of the tile
      float v[32], t3r[32];
#pragma unroll
      for (int x = 0; x < 8; ++x) {
        const float4 t4 = reinterpret_cast<const float4*>(t3buf + cb * 32)[x];
        t3r[4 * x] = t4.x; t3r[4 * x + 1] = t4.y; t3r[4 * x + 2] = t4.z; t3r[4 * x + 3] = t4.w;
      }
      float local = 0.f;
      // (the diagonal tile is the only one with masked pairs: its tests are compiled into a path of its own)
      auto scan32 = [&](auto on_diag) {
        constexpr bool kDiag = decltype(on_diag)::value;
        const float2 k23 = make_float2(2.0f / 3.0f, 2.0f / 3.0f), s32 = make_float2(s3, s3), one2 = make_float2(1.0f, 1.0f),
                     mone2 = make_float2(-1.0f, -1.0f), ln2 = make_float2(0.6931471805599453f, 0.6931471805599453f);
#pragma unroll
        for (int x = 0; x < 32; x += 2) {
          // two rows at a time with packed fp32 arithmetic: relu(g)^(2/3) through lg2(max(g, 0)) = -inf for g <= 0
          const float2 lg = make_float2(lg2(fmaxf(__uint_as_float(g[x]), 0.f)), lg2(fmaxf(__uint_as_float(g[x + 1]), 0.f)));
          const float2 e23 = fmul2(lg, k23);
          const float2 pw = make_float2(ex2(e23.x), ex2(e23.y));
          const float2 a = fmul2(fmul2(pw, s32), make_float2(t3r[x], t3r[x + 1]));
          const float2 om = ffma2(make_float2(fminf(a.x, clamp_hi()), fminf(a.y, clamp_hi())), mone2, one2);
          const float2 el = fmul2(make_float2(lg2(om.x), lg2(om.y)), ln2);
#pragma unroll
          for (int y = 0; y < 2; ++y) {
            const int q = cb * 32 + x + y;
            float ell = y ? el.y : el.x;
            if (kDiag && q <= k) ell = 0.f;
            local += ell;
            cval = carry + (tprev + local);
            v[x + y] = (kDiag && q < k) ? mask_value() : cval;
          }
        }
      };
      if (diag) scan32(std::true_type{});
      else scan32(std::false_type{});
      tprev += local;
      if (!kCarryOnly) {
        UF(2)
        if (cb == 0 && T >= Cfg::kCBufs && !c.wait_w(kCFree + T % Cfg::kCBufs, T / Cfg::kCBufs - 1)) return;
        UF(3)
#pragma unroll
        for (int x = 0; x < 32; ++x) {
          const int q = cb * 32 + x;
          *reinterpret_cast<float*>(sCs + (T % Cfg::kCBufs) * 65536 + q * 512 + ((((k >> 2) ^ (q & 7)) & 31) << 4) + (k & 3) * 4) = v[x];
        }
      }
    }
    {
      // carry + tprev (tprev = carry_lo + the tile's total) as an exact two-term sum
      const float sum = carry + tprev, bb = sum - carry;
      carry_lo = (carry - (sum - bb)) + (tprev - bb);
      carry = sum;
    }
    if (!kCarryOnly) c.arrive_w(kCReady + T % Cfg::kCBufs);
    UF(2)
  }
  UF_STORE(k == 0, 0)
  if (p.total_out) p.total_out[key_id] = carry;
}

// ------------------------------------------------------------ softmax groups --
template <int D, int kOut>
__device__ __forceinline__ void fwd_softmax(const FwdCtx<D>& c, const FwdParams& p, int me) {
  constexpr bool kMerge = (kOut == kOutMerged);
  using Cfg = FwdCfg<D>;
  const int R = p.s.R, N = p.s.N;
  const int row = threadIdx.x & 127;
  const uint32_t lane_base = (uint32_t)((threadIdx.x >> 5) & 3) * 32u << 16;
  const uint8_t* sCrow0 = c.smem + Cfg::oCs + row * 512;
  const size_t chunk_id = (size_t)c.bh * N + c.i;
  const float kLog2e = 1.4426950408889634f, kLn2 = 0.6931471805599453f;
  int t = 0;
  UF_DECL
  for (int T = 0; T < c.ntiles; ++T) {
    // Every softmax thread observes every phase of c_ready and arrives on c_free exactly
    // once per tile (after its last read of C in that tile), whether or not its group has
    // a head to process in this tile; parity waits stay within one phase of the barrier.
    UF(0)
    const int cbuf = T % Cfg::kCBufs;
    const uint8_t* sCrow = sCrow0 + cbuf * 65536;
    if (!c.wait_w(kCReady + cbuf, T / Cfg::kCBufs)) return;
    UF(1)
    int last_r = -1;
    for (int r = R - 1; r >= 0; --r)
      if (((T * R + r) & 1) == me) { last_r = r; break; }
    if (last_r < 0) c.arrive_w(kCFree + cbuf);
    for (int r = 0; r < R; ++r, ++t) {
      if ((t & 1) != me) continue;
      const int sb = t & 1, ob = t % Cfg::kOBufs;
      const uint32_t tS = c.tmem + (sb ? Cfg::tS1 : Cfg::tS0) + lane_base;
      const uint32_t tO = c.tmem + ((Cfg::kOBufs == 2 && ob) ? Cfg::tO1 : Cfg::tO0) + lane_base;
      UF(0)
      if (!c.wait_w(kSFull + sb, t >> 1)) return;
      UF(2)
      tc_fence_after();
      // pass 1: s = S + C (written back to TMEM), row max.  64 columns per round trip: the two loads are in flight together.
      float m = -INFINITY;
#pragma unroll 1
      for (int cb = 0; cb < 2; ++cb) {
        uint32_t s[64];
        tmem_ld32(tS + cb * 64, s);
        tmem_ld32(tS + cb * 64 + 32, s + 32);
        tc_wait_ld();
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const int chunk = cb * 16 + u;
          const float4 cv = *reinterpret_cast<const float4*>(sCrow + (((chunk ^ (row & 7)) & 31) << 4));
          const float2 a01 = fadd2(make_float2(__uint_as_float(s[u * 4 + 0]), __uint_as_float(s[u * 4 + 1])), make_float2(cv.x, cv.y));
          const float2 a23 = fadd2(make_float2(__uint_as_float(s[u * 4 + 2]), __uint_as_float(s[u * 4 + 3])), make_float2(cv.z, cv.w));
          m = fmax3(m, fmax3(a01.x, a01.y, a23.x), a23.y);
          s[u * 4 + 0] = __float_as_uint(a01.x); s[u * 4 + 1] = __float_as_uint(a01.y);
          s[u * 4 + 2] = __float_as_uint(a23.x); s[u * 4 + 3] = __float_as_uint(a23.y);
        }
        tmem_st32(tS + cb * 64, s);
        tmem_st32(tS + cb * 64 + 32, s + 32);
      }
      tc_wait_st();
      UF(3)
      if (r == last_r) c.arrive_w(kCFree + cbuf);
      // pass 2: P = exp(s - m) as bf16 into the first 64 columns of the S buffer
      const float mb = m * kLog2e;
      const float2 kL2 = make_float2(kLog2e, kLog2e), nmb2 = make_float2(-mb, -mb);
      float2 l2 = make_float2(0.f, 0.f);
#pragma unroll 1
      for (int cb = 0; cb < 2; ++cb) {
        uint32_t s[64];
        tmem_ld32(tS + cb * 64, s);
        tmem_ld32(tS + cb * 64 + 32, s + 32);
        tc_wait_ld();
        uint32_t pk[32];
#pragma unroll
        for (int u = 0; u < 32; ++u) {
          const float2 arg = ffma2(make_float2(__uint_as_float(s[2 * u]), __uint_as_float(s[2 * u + 1])), kL2, nmb2);
          const float2 pe = make_float2(ex2(arg.x), ex2(arg.y));
          __nv_bfloat162 h = __floats2bfloat162_rn(pe.x, pe.y);
          // the row sum uses the unrounded probabilities: the reference normalises in fp32 and rounds P afterwards
          // (universal_attention_autograd.py:158-159)
          l2 = fadd2(l2, pe);
          pk[u] = *reinterpret_cast<uint32_t*>(&h);
        }
        if (kOut != kOutStats) tmem_st32(tS + cb * 32, pk);
      }
      if (kOut != kOutStats) tc_wait_st();
      tc_fence_before();
      c.arrive_w(kPReady + sb);
      UF(4)
      const int qg = p.r0 + (c.j0 + T - p.j_begin) * 128 + row;      // row index inside the slab
      const float l = l2.x + l2.y;
      const float lse = m + lg2(l) * kLn2;
      const size_t orow = (chunk_id * R + r) * p.Lr + qg;
      const size_t mrow = ((size_t)c.bh * R + r) * p.Lr + qg;       // the row in (b,h,r,L) order (merged-output mode)
      float linv;
      if (kMerge) {
        // exp(lse - row_lse) / l = exp(m - row_lse): weight of this chunk in the row's softmax over all keys, applied
        // to the unnormalised P~ V (the load's latency runs under the wait for the PV product)
        linv = ex2((m - p.row_lse[mrow]) * kLog2e);
      } else {
        p.lse[orow] = lse;
        if (p.denom) p.denom[orow] = __float2bfloat16_rn(lse);
        linv = 1.0f / l;
      }
      UF(5)
      if (kOut == kOutStats) continue;
      if (!c.wait_w(kOFull + sb, t >> 1)) return;
      UF(6)
      tc_fence_after();
      __nv_bfloat16* orow_ptr = p.out + orow * D;
#pragma unroll 1
      for (int cb = 0; cb < D / 32; ++cb) {
        uint32_t o[32];
        tmem_ld32(tO + cb * 32, o);
        tc_wait_ld();
        if (cb == D / 32 - 1) {
          tc_fence_before();
          c.arrive_w(kOFree + sb);
        }
        if (kMerge) {
          float* dst = p.merged_acc + mrow * D + cb * 32;
#pragma unroll
          for (int u = 0; u < 8; ++u)
            red_add_v4(dst + 4 * u, __uint_as_float(o[4 * u]) * linv, __uint_as_float(o[4 * u + 1]) * linv,
                       __uint_as_float(o[4 * u + 2]) * linv, __uint_as_float(o[4 * u + 3]) * linv);
          continue;
        }
        if (!p.out) continue;                 // statistics-only run (the log-sum-exp for a backward that was not given one)
#ifdef UA_EXPERIMENT_NO_OUT_STORE
        if (cb >= 0) continue;
#endif
        uint32_t pk[16];
        const float2 linv2 = make_float2(linv, linv);
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const float2 ov = fmul2(make_float2(__uint_as_float(o[2 * u]), __uint_as_float(o[2 * u + 1])), linv2);
          __nv_bfloat162 h = __floats2bfloat162_rn(ov.x, ov.y);
          pk[u] = *reinterpret_cast<uint32_t*>(&h);
        }
        uint4* dst = reinterpret_cast<uint4*>(orow_ptr + cb * 32);
        dst[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        dst[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        dst[2] = make_uint4(pk[8], pk[9], pk[10], pk[11]);
        dst[3] = make_uint4(pk[12], pk[13], pk[14], pk[15]);
      }
      UF(7)
    }
  }
  UF_STORE(row == 0 && me == 0, 8)
}

// Rows before the key chunk (j < i): every score is -1e12 (fp32 absorbs k.q), the softmax is
// uniform, so out = sum_k bf16(1/128) V_k and lse = -1e12 (universal_attention_autograd.py:28,
// :154).  Pure HBM writes (i * 128 * R rows), done by warps 2-3 while the others compute the
// n - i valid tiles: chunks with many masked rows have few tiles to compute.
template <int D>
__device__ __forceinline__ void fwd_fill_rows(const FwdCtx<D>& c, const FwdParams& p, __nv_bfloat16* vmean) {
  const int t = threadIdx.x - 64;                      // 0..63
  const int L = p.s.L, R = p.s.R, N = p.s.N;
  const __nv_bfloat16* v = static_cast<const __nv_bfloat16*>(p.vc) + ((size_t)c.bh * L + (size_t)c.i * 128) * D;
  const float w = 1.0f / 128.0f;
  for (int d = t; d < D; d += 64) {
    float acc = 0.f;
    for (int k = 0; k < 128; ++k) acc = fmaf(w, __bfloat162float(v[(size_t)k * D + d]), acc);
    vmean[d] = __float2bfloat16_rn(acc);
  }
  named_bar_sync(2, 64);
  const size_t chunk_id = (size_t)c.bh * N + c.i;
  const int rows = ((c.i < p.j_end ? c.i : p.j_end) - p.j_begin) * 128;    // rows of the range that lie before the chunk
  constexpr int kVecPerRow = D / 8;                    // 16-byte vectors
  const uint4 mine = reinterpret_cast<const uint4*>(vmean)[t % kVecPerRow];   // 64 % kVecPerRow == 0: fixed per thread
  for (int r = 0; r < R; ++r) {
    uint4* o = reinterpret_cast<uint4*>(p.out + ((chunk_id * R + r) * p.Lr + p.r0) * D);
    const size_t nvec = (size_t)rows * kVecPerRow;
    for (size_t e = t; e < nvec; e += 64) o[e] = mine;
    float* lr = p.lse + (chunk_id * R + r) * p.Lr + p.r0;
    for (int q = t; q < rows; q += 64) {
      lr[q] = mask_value();
      if (p.denom) p.denom[(chunk_id * R + r) * p.Lr + p.r0 + q] = __float2bfloat16_rn(mask_value());
    }
  }
}

template <int D, typename TG, bool kCarryOnly, int kOut = kOutTiles>
__global__ void __launch_bounds__(512, 1)
fwd_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
           const __grid_constant__ CUtensorMap tmQ, FwdParams p) {
  using Cfg = FwdCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint32_t* misc = reinterpret_cast<uint32_t*>(smem + Cfg::oMisc);   // [0] tmem base, [1] abort flag
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int BH = p.s.B * p.s.H;

  FwdCtx<D> c;
  c.smem = smem;
  c.bars = smem_u32(smem + Cfg::oBar);
  c.abort_flag = reinterpret_cast<volatile int*>(misc + 1);
  c.i = blockIdx.x / BH;                 // heavy chunks (small i: most row tiles) first
  c.bh = blockIdx.x - c.i * BH;
  c.j0 = c.i > p.j_begin ? c.i : p.j_begin;
  c.ntiles = p.j_end - c.j0;            // <= 0: nothing to compute for this chunk in the row range (only the fill)

  if (threadIdx.x == 0) {
    misc[1] = 0;
    for (int b = 0; b < kNumBars; ++b) {
      uint32_t count = 1;
      // one arrival per warp of the group that signals
      if (b == kGFree || b == kCReady || b == kCReady + 1 || b == kT3Ready) count = 4;
      if (b == kCFree || b == kCFree + 1) count = 8;
      if (b == kPReady || b == kPReady + 1 || b == kOFree || b == kOFree + 1) count = 4;
      mbar_init(c.bar(b), count);
    }
    mbar_init_fence();
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    prefetch_tmap(&tmQ);
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
    if (lane == 0 && c.ntiles > 0) fwd_producer<D, kCarryOnly>(c, p, &tmK, &tmV, &tmQ);
  } else if (warp == 1) {
    if (lane == 0 && c.ntiles > 0) fwd_mma<D, kCarryOnly, kOut>(c, p);
  } else if (warp >= 4 && warp < 8) {
    if (c.ntiles > 0) fwd_decay<D, TG, kCarryOnly>(c, p);
    else if (p.total_out)      // no row of the range sees this chunk: its prefix does not move
      p.total_out[((size_t)c.bh * p.s.N + c.i) * 128 + (threadIdx.x & 127)] =
          p.carry_in ? p.carry_in[((size_t)c.bh * p.s.N + c.i) * 128 + (threadIdx.x & 127)] : 0.f;
  } else if (warp >= 8 && !kCarryOnly) {
    if (c.ntiles > 0) fwd_softmax<D, kOut>(c, p, (warp - 8) >> 2);
  } else if ((warp == 2 || warp == 3) && !kCarryOnly && p.fill_masked && c.i > p.j_begin) {
    fwd_fill_rows<D>(c, p, reinterpret_cast<__nv_bfloat16*>(smem + Cfg::oFill));
  }

  tc_fence_before();
  __syncthreads();
  if (*c.abort_flag) {
    if (threadIdx.x == 0) atomicExch(p.status, 1);
    // let copies and MMAs that are still in flight drain before shared memory and TMEM are released
    for (int it = 0; it < 64; ++it) __nanosleep(2000);
    __syncthreads();
  }
  if (warp == 0) tmem_dealloc(c.tmem, 512);
}

}  // namespace sm100
}  // namespace ua
