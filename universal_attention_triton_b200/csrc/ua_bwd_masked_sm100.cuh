// Backward through the rows BEFORE a key chunk (row tile j < chunk i), sm_100a.
//
// Every score of such a block is the mask value (universal_attention_autograd.py:26-28: the affinity mask replaces the
// decay and the k.q term is absorbed by -1e12 in fp32), so the softmax over the chunk's 128 keys is uniform, P = 1/128,
// and with g = a row of the upstream gradient of `out`, gd = the upstream gradient of `denom`:
//   dS[k][q] = ( (v_k - vbar) . g_q + gd_q ) / 128           vbar = mean of the chunk's values
// which has rank <= D + 1.  Nothing is therefore done per (key, row) pair:
//   dQ_rj  += g M_i + gd (x) ksum_i / 128     M_i = sum_k (v_k - vbar)^T k_k / 128   (D x D, once per chunk: prep kernel)
//   N_i    += g^T Q_rj,  w_i += gd^T Q_rj,  u_i += 1^T g            (accumulated over all rows before the chunk)
//   dK_i   += ( (V_i - vbar) N_i + 1 (x) w_i ) / 128,   dV_i += 1 (x) u_i / 128             (once per chunk: finish kernel)
// The sweep kernel in the middle is a stream over the upstream gradient, read exactly once from HBM: per row tile and
// head it loads Q_rj, and for each of the G chunks of its group the gradient tile g (the only large operand), and issues
//   Y    (+)= g Mt_c^T                 [128 rows][64]   summed over the group's chunks in TMEM, then ONE reduce-add into dQ
//   Nt_c (+)= [Q | E]^T g              [64 + 16][D]     lanes 0..63: N_c^T, lane 72: u_c   (E: see below)
//   Wt   (+)= [Q | E]^T E              [64 + 16][16]    column c of lanes 0..63: w_c
//   Y      = E Ks                      the rank-1 terms gd_c (x) ksum_c / 128 of all chunks in one K = 16 MMA
// E is a [128 rows][64] bf16 tile beside each Q tile: column c < G holds gd of chunk c for this (row tile, head), column 8
// holds ones, the rest zeros; it is written by four warps from rows of g_denom that arrive with the producer's copies.
// head_dim 128 runs as two blocks per work item, one per 64-wide half of the output columns of Y / lanes of Nt.
// A work item is (batch*head, group of G chunks, range of row tiles); partial N / w / u leave as fp32 global adds.
#pragma once
#include "ua_bwd_sm100.cuh"

namespace ua {
namespace sm100 {

struct MaskedParams {
  Shape s;
  const float* g_denom;          // (b*h*n, r, L) fp32, 16-byte aligned
  uint8_t* mt;                   // (b*h*n) images of M_i^T / 128 as bf16: [D/64 halves of d'][D/64 boxes of d][64][64], 128-byte swizzled
  __nv_bfloat16* ksum;           // (b*h*n, D): column sums of K_i / 128
  float* nacc;                   // (b*h*n, D + 3, D) fp32: rows 0..D-1 = N^T[d'][d], row D = w[d'], row D + 1 = u[d], row D + 2 = vbar[d]
  float* acc_dk;                 // (b*h*L, D) fp32, added to
  float* acc_dv;                 // (b*h*L, D) fp32, written (rows of chunk 0 untouched)
  int* status;
  int jp;                        // row tiles per work item
  int items_per_bh;              // sum over groups of ceil(row tiles before the group's last chunk / jp)
};

template <int D> __host__ __device__ constexpr int kNaccRows() { return D + 3; }

template <int D>
struct MkCfg {
  static constexpr int kKB = D / 64;
  static constexpr int kG = 256 / D;                       // chunks per group: their N^T accumulators fill 256 TMEM columns
  static constexpr int kStages = (D == 64) ? 3 : 2;        // ring of upstream-gradient tiles
  static constexpr int kDoBytes = kKB * 16384;
  static constexpr int kStageBufs = (D == 64) ? 2 : 1;     // staging tiles of the dQ reduce-add
  static constexpr int kMtBytes = kKB * 8192;              // one half (64 rows d') of a chunk's M^T image
  static constexpr int oDo = 0;
  static constexpr int oQE = oDo + kStages * kDoBytes;     // 2 x { Q [128][64] | E [128][64] }
  static constexpr int oMt = oQE + 2 * 32768;
  static constexpr int oKs = oMt + kG * kMtBytes;          // [64 d'][64] bf16, column c = ksum_c / 128
  static constexpr int oStage = oKs + 8192;                // kStageBufs x two [128][32] fp32 boxes
  static constexpr int oGd = oStage + kStageBufs * 32768;  // 2 x kG x float[128]: g_denom rows of a step
  static constexpr int oBar = oGd + 2 * kG * 512;
  static constexpr int oMisc = oBar + 256;
  static constexpr int kSmemBytes = oMisc + 64 + 1024;     // + slack to align the base to 1024 B
  static constexpr uint32_t tY0 = 0, tY1 = 64, tN = 128, tW = 128 + kG * D;
  static_assert(tW + 16 <= 512, "TMEM budget");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

enum MkBar {
  mMtFull = 0, mQFull = 1, mQEFree = 3, mEReady = 5, mYFull = 7, mYFree = 9, mDone = 11, mDoFull = 12, mDoFree = 15, mNumBars = 18
};

struct MkCtx {
  uint8_t* smem;
  uint32_t bars, tmem;
  volatile int* abort_flag;
  int bh, i0, jlo, jhi, chi, h;        // chunks i0 + c, c < chi; row tiles [jlo, jhi); output half h
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
  // first chunk of the group that has row tile j before it
  __device__ __forceinline__ int clo(int j) const { return max(0, j + 1 - i0); }
};

// ------------------------------------------------------------------ prep kernel --
// One block per chunk: ksum / 128 (bf16), M^T / 128 (bf16, in the swizzled layout the sweep kernel's MMAs read), and the
// chunk's N / w / u accumulators set to zero.
template <int D>
__global__ void __launch_bounds__(256) masked_prep_kernel(const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc,
                                                          MaskedParams p) {
  extern __shared__ __align__(16) uint8_t prep_smem[];
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(prep_smem);
  __nv_bfloat16* sV = sK + 128 * D;
  float* sSum = reinterpret_cast<float*>(sV + 128 * D);
  const size_t chunk = blockIdx.x;
  const int t = threadIdx.x;
  float* nacc = p.nacc + chunk * (size_t)kNaccRows<D>() * D;
  for (int x = t; x < (D + 2) * D / 4; x += 256) reinterpret_cast<float4*>(nacc)[x] = make_float4(0.f, 0.f, 0.f, 0.f);
  const uint4* gk = reinterpret_cast<const uint4*>(kc + chunk * 128 * D);
  const uint4* gv = reinterpret_cast<const uint4*>(vc + chunk * 128 * D);
  for (int x = t; x < 128 * D / 8; x += 256) {
    reinterpret_cast<uint4*>(sK)[x] = gk[x];
    reinterpret_cast<uint4*>(sV)[x] = gv[x];
  }
  __syncthreads();
  if (t < 2 * D) {
    const __nv_bfloat16* src = (t < D) ? sK + t : sV + (t - D);
    float acc = 0.f;
#pragma unroll 8
    for (int k = 0; k < 128; ++k) acc += __bfloat162float(src[k * D]);
    sSum[t] = acc;
    if (t < D) p.ksum[chunk * D + t] = __float2bfloat16_rn(acc * (1.0f / 128.0f));
    else nacc[(size_t)(D + 2) * D + (t - D)] = acc * (1.0f / 128.0f);
  }
  __syncthreads();
  uint8_t* img = p.mt + chunk * (size_t)(D * D * 2);
  for (int o = t; o < D * D / 8; o += 256) {
    const int dp = o / (D / 8), d0 = (o % (D / 8)) * 8;      // row d' of M^T, eight columns d0..d0+7
    float acc[8];
#pragma unroll
    for (int x = 0; x < 8; ++x) acc[x] = 0.f;
#pragma unroll 4
    for (int k = 0; k < 128; ++k) {
      const float kv = __bfloat162float(sK[k * D + dp]);
      const uint4 raw = *reinterpret_cast<const uint4*>(sV + k * D + d0);
      const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const __nv_bfloat162 hv = *reinterpret_cast<const __nv_bfloat162*>(&rw[x]);
        acc[2 * x] = fmaf(kv, __bfloat162float(hv.x), acc[2 * x]);
        acc[2 * x + 1] = fmaf(kv, __bfloat162float(hv.y), acc[2 * x + 1]);
      }
    }
    const float ks = sSum[dp] * (1.0f / 128.0f);
    uint32_t w4[4];
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      __nv_bfloat162 hh = __floats2bfloat162_rn((acc[2 * x] - ks * sSum[D + d0 + 2 * x]) * (1.0f / 128.0f),
                                                (acc[2 * x + 1] - ks * sSum[D + d0 + 2 * x + 1]) * (1.0f / 128.0f));
      w4[x] = *reinterpret_cast<uint32_t*>(&hh);
    }
    const int half = dp >> 6, row = dp & 63, box = d0 >> 6, chunk16 = (d0 & 63) >> 3;
    *reinterpret_cast<uint4*>(img + ((size_t)(half * (D / 64) + box) * 64 + row) * 128 + (((chunk16 ^ row) & 7) << 4)) =
        make_uint4(w4[0], w4[1], w4[2], w4[3]);
  }
}

// ---------------------------------------------------------------- finish kernel --
// One block per chunk i >= 1 (thread = key): dK_i += ((V_i - vbar) N_i + 1 (x) w_i) / 128,  dV_i = 1 (x) u_i / 128.
template <int D>
__global__ void __launch_bounds__(128) masked_finish_kernel(const __nv_bfloat16* __restrict__ vc, MaskedParams p) {
  __shared__ __align__(16) float sN[32 * D];          // 32 rows d' of N^T at a time
  __shared__ float sW[D];
  const int N = p.s.N;
  const size_t chunk = blockIdx.x;
  if (chunk % N == 0) return;           // no rows before the first chunk
  const int key = threadIdx.x;
  const float* nacc = p.nacc + chunk * (size_t)kNaccRows<D>() * D;
  const float* u = nacc + (size_t)(D + 1) * D;
  const float* vbar = nacc + (size_t)(D + 2) * D;
  float vcen[D];
  {
    const uint4* gv = reinterpret_cast<const uint4*>(vc + (chunk * 128 + key) * D);
#pragma unroll
    for (int x = 0; x < D / 8; ++x) {
      const uint4 raw = gv[x];
      const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int y = 0; y < 4; ++y) {
        const __nv_bfloat162 hv = *reinterpret_cast<const __nv_bfloat162*>(&rw[y]);
        vcen[8 * x + 2 * y] = __bfloat162float(hv.x) - vbar[8 * x + 2 * y];
        vcen[8 * x + 2 * y + 1] = __bfloat162float(hv.y) - vbar[8 * x + 2 * y + 1];
      }
    }
  }
  for (int x = key; x < D; x += 128) sW[x] = nacc[(size_t)D * D + x];
  float* dk = p.acc_dk + (chunk * 128 + key) * D;
  float* dv = p.acc_dv + (chunk * 128 + key) * D;
#pragma unroll 4
  for (int x = 0; x < D; x += 4)
    *reinterpret_cast<float4*>(dv + x) = make_float4(u[x] * (1.0f / 128.0f), u[x + 1] * (1.0f / 128.0f), u[x + 2] * (1.0f / 128.0f),
                                                     u[x + 3] * (1.0f / 128.0f));
#pragma unroll 1
  for (int blk = 0; blk < D / 32; ++blk) {
    __syncthreads();
    for (int x = key; x < 32 * D / 4; x += 128) reinterpret_cast<float4*>(sN)[x] = reinterpret_cast<const float4*>(nacc + (size_t)blk * 32 * D)[x];
    __syncthreads();
#pragma unroll 1
    for (int q = 0; q < 32; q += 4) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int d = 0; d < D; ++d) {
#pragma unroll
        for (int x = 0; x < 4; ++x) acc[x] = fmaf(vcen[d], sN[(q + x) * D + d], acc[x]);
      }
      float4* dst = reinterpret_cast<float4*>(dk + blk * 32 + q);
      float4 cur = *dst;
      cur.x += (acc[0] + sW[blk * 32 + q]) * (1.0f / 128.0f);
      cur.y += (acc[1] + sW[blk * 32 + q + 1]) * (1.0f / 128.0f);
      cur.z += (acc[2] + sW[blk * 32 + q + 2]) * (1.0f / 128.0f);
      cur.w += (acc[3] + sW[blk * 32 + q + 3]) * (1.0f / 128.0f);
      *dst = cur;
    }
  }
}

// ----------------------------------------------------------------- sweep kernel --
template <int D>
__device__ __forceinline__ void mk_producer(const MkCtx& c, const MaskedParams& p, const CUtensorMap* tmQ, const CUtensorMap* tmG) {
  using Cfg = MkCfg<D>;
  const int L = p.s.L, R = p.s.R, N = p.s.N;
  const uint32_t sb = smem_u32(c.smem);
  {
    const int c0 = c.clo(c.jlo);
    mbar_expect_tx(c.bar(mMtFull), (uint32_t)(c.chi - c0) * Cfg::kMtBytes);
    for (int cc = c0; cc < c.chi; ++cc)
      bulk_load_1d(sb + Cfg::oMt + cc * Cfg::kMtBytes,
                   p.mt + ((size_t)c.bh * N + c.i0 + cc) * (size_t)(D * D * 2) + (size_t)c.h * Cfg::kMtBytes, Cfg::kMtBytes,
                   c.bar(mMtFull));
  }
  int s = 0, dc = 0;
  for (int j = c.jlo; j < c.jhi; ++j) {
    const int c0 = c.clo(j);
    for (int r = 0; r < R; ++r, ++s) {
      const int qs = s & 1;
      if (s >= 2 && !c.wait(mQEFree + qs, s / 2 - 1)) return;
      mbar_expect_tx(c.bar(mQFull + qs), 16384u + (uint32_t)(c.chi - c0) * 512u);
      tma_load_2d(sb + Cfg::oQE + qs * 32768, tmQ, 64 * c.h, (c.bh * R + r) * L + j * 128, c.bar(mQFull + qs));
      for (int cc = c0; cc < c.chi; ++cc)
        bulk_load_1d(sb + Cfg::oGd + (qs * Cfg::kG + cc) * 512,
                     p.g_denom + (((size_t)c.bh * N + c.i0 + cc) * R + r) * L + (size_t)j * 128, 512, c.bar(mQFull + qs));
      for (int cc = c0; cc < c.chi; ++cc, ++dc) {
        const int st = dc % Cfg::kStages;
        if (dc >= Cfg::kStages && !c.wait(mDoFree + st, dc / Cfg::kStages - 1)) return;
        mbar_expect_tx(c.bar(mDoFull + st), Cfg::kDoBytes);
#pragma unroll
        for (int b = 0; b < Cfg::kKB; ++b)
          tma_load_2d(sb + Cfg::oDo + st * Cfg::kDoBytes + b * 16384, tmG, 64 * b,
                      (int)((((size_t)c.bh * N + c.i0 + cc) * R + r) * L + (size_t)j * 128), c.bar(mDoFull + st));
      }
    }
  }
}

template <int D>
__device__ __forceinline__ void mk_issuer(const MkCtx& c, const MaskedParams& p) {
  using Cfg = MkCfg<D>;
  const int R = p.s.R;
  const uint32_t sb = smem_u32(c.smem);
  constexpr uint32_t id_y = idesc_bf16(128, 64, 0, 0);       // rows x 64: A K-major, B K-major
  constexpr uint32_t id_n = idesc_bf16(128, D, 1, 1);        // [Q | E]^T g: both MN-major
  constexpr uint32_t id_w = idesc_bf16(128, 16, 1, 1);       // [Q | E]^T E
  const uint64_t kKs = desc_from_lo(desc_lo(sb + Cfg::oKs, 16));
  if (!c.wait(mMtFull, 0)) return;
  int s = 0, dc = 0;
  for (int j = c.jlo; j < c.jhi; ++j) {
    const int c0 = c.clo(j);
    for (int r = 0; r < R; ++r, ++s) {
      const int qs = s & 1;
      const uint32_t q_addr = sb + Cfg::oQE + qs * 32768, e_addr = q_addr + 16384;
      if (!c.wait(mQFull + qs, s / 2) || !c.wait(mEReady + qs, s / 2)) return;
      if (s >= 2 && !c.wait(mYFree + qs, s / 2 - 1)) return;
      tc_fence_after();
      const uint32_t Y = c.tmem + (qs ? Cfg::tY1 : Cfg::tY0);
      const uint64_t mQE = desc_from_lo(desc_lo(q_addr, 16384));     // [K = rows][M = 64 of Q, then 64 of E]
      const uint64_t mE = desc_from_lo(desc_lo(e_addr, 16384)), kE = desc_from_lo(desc_lo(e_addr, 16));
      mma_ss(Y, kE, kKs, id_y, 0);                                   // Y = sum_c gd_c (x) ksum_c / 128
      mma4_ss(c.tmem + Cfg::tW, mQE, mE, 128, 128, id_w, s > 0);     // Wt += [Q | E]^T E
      mma4_ss(c.tmem + Cfg::tW, mQE + 512, mE + 512, 128, 128, id_w, 1);
      for (int cc = c0; cc < c.chi; ++cc, ++dc) {
        const int st = dc % Cfg::kStages;
        if (!c.wait(mDoFull + st, dc / Cfg::kStages)) return;
        tc_fence_after();
        const uint32_t g_addr = sb + Cfg::oDo + st * Cfg::kDoBytes;
#pragma unroll
        for (int b = 0; b < Cfg::kKB; ++b)                           // Y += g Mt_c^T
          mma4_ss(Y, desc_from_lo(desc_lo(g_addr + b * 16384, 16)), desc_from_lo(desc_lo(sb + Cfg::oMt + cc * Cfg::kMtBytes + b * 8192, 16)),
                  2, 2, id_y, 1);
        const uint64_t mG = desc_from_lo(desc_lo(g_addr, 16384));
        const uint32_t Nt = c.tmem + Cfg::tN + cc * D;
        mma4_ss(Nt, mQE, mG, 128, 128, id_n, s > 0);                 // Nt_c += [Q | E]^T g
        mma4_ss(Nt, mQE + 512, mG + 512, 128, 128, id_n, 1);
        tc_commit(c.bar(mDoFree + st));
      }
      tc_commit(c.bar(mYFull + qs));
      tc_commit(c.bar(mQEFree + qs));
    }
  }
  tc_commit(c.bar(mDone));
}

// Four warps, thread = row: column c of E <- g_denom of chunk c (bf16), for the chunks that have this row tile before them.
template <int D>
__device__ __forceinline__ void mk_gate_writer(const MkCtx& c, const MaskedParams& p) {
  using Cfg = MkCfg<D>;
  const int R = p.s.R;
  const int row = threadIdx.x & 127;
  int s = 0;
  for (int j = c.jlo; j < c.jhi; ++j) {
    const int c0 = c.clo(j);
    for (int r = 0; r < R; ++r, ++s) {
      const int qs = s & 1;
      if (!c.wait_w(mQFull + qs, s / 2)) return;
      const float* gd = reinterpret_cast<const float*>(c.smem + Cfg::oGd + qs * Cfg::kG * 512) + row;
      uint32_t w[Cfg::kG / 2];
#pragma unroll
      for (int x = 0; x < Cfg::kG / 2; ++x) {
        const float a = (2 * x >= c0 && 2 * x < c.chi) ? gd[(2 * x) * 128] : 0.f;
        const float b = (2 * x + 1 >= c0 && 2 * x + 1 < c.chi) ? gd[(2 * x + 1) * 128] : 0.f;
        __nv_bfloat162 hh = __floats2bfloat162_rn(a, b);
        w[x] = *reinterpret_cast<uint32_t*>(&hh);
      }
      uint8_t* dst = c.smem + Cfg::oQE + qs * 32768 + 16384 + row * 128 + ((row & 7) << 4);
      if (Cfg::kG == 4) *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[Cfg::kG / 2 - 1]);
      else *reinterpret_cast<uint32_t*>(dst) = w[0];
      fence_proxy_async();
      c.arrive_w(mEReady + qs);
    }
  }
}

// Four warps (TMEM lane quadrant = warp % 4): Y of each step -> staging tile -> TMA reduce-add into the dQ accumulator;
// after the last step the group's N^T / w / u partial sums -> global adds.
template <int D>
__device__ __forceinline__ void mk_drain(const MkCtx& c, const MaskedParams& p, const CUtensorMap* tmDQ) {
  using Cfg = MkCfg<D>;
  const int L = p.s.L, R = p.s.R, N = p.s.N;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = (warp & 3) * 32 + lane;
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
  const bool leader = (warp == 4 && lane == 0);
  const uint32_t swz = (uint32_t)(row & 7);
  int s = 0;
  for (int j = c.jlo; j < c.jhi; ++j) {
    for (int r = 0; r < R; ++r, ++s) {
      const int qs = s & 1;
      uint8_t* stage = c.smem + Cfg::oStage + (s % Cfg::kStageBufs) * 32768;
      if (!c.wait_w(mYFull + qs, s / 2)) return;
      tc_fence_after();
      // the reduce-add that last used this staging tile has read it
      if (leader) {
        if (Cfg::kStageBufs == 2) bulk_wait_read_but_last();
        else bulk_wait_read_all();
      }
      named_bar_sync(2, 128);
#pragma unroll 1
      for (int hb = 0; hb < 2; ++hb) {
        uint32_t o[32];
        tmem_ld32(c.tmem + (qs ? Cfg::tY1 : Cfg::tY0) + lane_base + 32 * hb, o);
        tc_wait_ld();
        if (hb == 1) {
          tc_fence_before();
          c.arrive_w(mYFree + qs);
        }
        uint8_t* box = stage + hb * 16384 + row * 128;
#pragma unroll
        for (int x = 0; x < 8; ++x)
          *reinterpret_cast<uint4*>(box + ((((uint32_t)x ^ swz) & 7) << 4)) = make_uint4(o[4 * x], o[4 * x + 1], o[4 * x + 2], o[4 * x + 3]);
      }
      fence_proxy_async();
      named_bar_sync(2, 128);
      if (leader) {
        const int y = (c.bh * R + r) * L + j * 128;
        tma_reduce_add_2d(tmDQ, 64 * c.h, y, smem_u32(stage));
        tma_reduce_add_2d(tmDQ, 64 * c.h + 32, y, smem_u32(stage) + 16384);
        bulk_commit_group();
      }
    }
  }
  if (!c.wait_w(mDone, 0)) {
    if (leader) bulk_wait_all();
    return;
  }
  tc_fence_after();
  const int c0 = c.clo(c.jlo);
  if ((warp & 3) < 2) {                    // lanes 0..63: rows d' = 64 h + row of N^T, and w
    uint32_t wv[16];
    tmem_ld16(c.tmem + Cfg::tW + lane_base, wv);
    tc_wait_ld();
    for (int cc = c0; cc < c.chi; ++cc) {
      float* nacc = p.nacc + ((size_t)c.bh * N + c.i0 + cc) * (size_t)kNaccRows<D>() * D;
#pragma unroll 1
      for (int hb = 0; hb < D / 32; ++hb) {
        uint32_t o[32];
        tmem_ld32(c.tmem + Cfg::tN + cc * D + lane_base + 32 * hb, o);
        tc_wait_ld();
        float* dst = nacc + (size_t)(64 * c.h + row) * D + 32 * hb;
#pragma unroll
        for (int x = 0; x < 8; ++x)
          red_add_v4(dst + 4 * x, __uint_as_float(o[4 * x]), __uint_as_float(o[4 * x + 1]), __uint_as_float(o[4 * x + 2]),
                     __uint_as_float(o[4 * x + 3]));
      }
      float wsel = 0.f;
#pragma unroll
      for (int x = 0; x < Cfg::kG; ++x) wsel = (x == cc) ? __uint_as_float(wv[x]) : wsel;
      atomicAdd(nacc + (size_t)D * D + 64 * c.h + row, wsel);
    }
  } else if ((warp & 3) == 2 && c.h == 0) {    // lane 72 (column 8 of E holds ones): u_c = column sums of g
    for (int cc = c0; cc < c.chi; ++cc) {
      float* nacc = p.nacc + ((size_t)c.bh * N + c.i0 + cc) * (size_t)kNaccRows<D>() * D + (size_t)(D + 1) * D;
#pragma unroll 1
      for (int hb = 0; hb < D / 32; ++hb) {
        uint32_t o[32];
        tmem_ld32(c.tmem + Cfg::tN + cc * D + lane_base + 32 * hb, o);
        tc_wait_ld();
        if (lane == 8) {
#pragma unroll
          for (int x = 0; x < 8; ++x)
            red_add_v4(nacc + 32 * hb + 4 * x, __uint_as_float(o[4 * x]), __uint_as_float(o[4 * x + 1]), __uint_as_float(o[4 * x + 2]),
                       __uint_as_float(o[4 * x + 3]));
        }
      }
    }
  }
  if (leader) bulk_wait_all();
}

template <int D>
__global__ void __launch_bounds__(384, 1)
masked_sweep_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmG,
                    const __grid_constant__ CUtensorMap tmDQ, MaskedParams p) {
  using Cfg = MkCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint32_t* misc = reinterpret_cast<uint32_t*>(smem + Cfg::oMisc);      // [0] TMEM base, [1] abort flag, [2] failure note
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int N = p.s.N;

  MkCtx c;
  c.smem = smem;
  c.bars = smem_u32(smem + Cfg::oBar);
  c.abort_flag = reinterpret_cast<volatile int*>(misc + 1);
  {
    // work item -> (batch*head, group, piece of the group's row tiles); the two halves of head_dim 128 are neighbours
    const int item = blockIdx.x / Cfg::kKB;
    c.h = blockIdx.x % Cfg::kKB;
    c.bh = item / p.items_per_bh;
    int rem = item % p.items_per_bh;
    int g = 0;
    bool found = false;
    for (; g * Cfg::kG < N; ++g) {
      const int jmax = min((g + 1) * Cfg::kG, N) - 1;                    // row tiles before the group's last chunk
      const int pieces = (jmax + p.jp - 1) / p.jp;
      if (rem < pieces) {
        c.jlo = rem * p.jp;
        c.jhi = min(c.jlo + p.jp, jmax);
        found = true;
        break;
      }
      rem -= pieces;
    }
    if (!found) return;                                                  // (a grid larger than the item count)
    c.i0 = g * Cfg::kG;
    c.chi = min(Cfg::kG, N - c.i0);
  }

  if (threadIdx.x == 0) {
    misc[1] = 0;
    misc[2] = 0;
    for (int b = 0; b < mNumBars; ++b) {
      uint32_t count = 1;
      if (b == mEReady || b == mEReady + 1 || b == mYFree || b == mYFree + 1) count = 4;     // one arrival per warp
      mbar_init(c.bar(b), count);
    }
    mbar_init_fence();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmG); prefetch_tmap(&tmDQ);
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(misc), 512);
    tmem_relinquish();
  }
  if (warp >= 8) {
    // E tiles: zeros, ones in column 8; Ks: column c = ksum_c / 128 of this block's 64 output columns
    const int t = threadIdx.x - 256;
    for (int x = t; x < 4096; x += 128) {
      const int buf = x >> 11, off = (x & 2047) << 4;
      *reinterpret_cast<uint4*>(smem + Cfg::oQE + buf * 32768 + 16384 + off) = make_uint4(0u, 0u, 0u, 0u);
    }
    for (int x = t; x < 512; x += 128) *reinterpret_cast<uint4*>(smem + Cfg::oKs + (x << 4)) = make_uint4(0u, 0u, 0u, 0u);
    named_bar_sync(3, 128);
    for (int buf = 0; buf < 2; ++buf)
      *reinterpret_cast<__nv_bfloat16*>(smem + Cfg::oQE + buf * 32768 + 16384 + t * 128 + (((1 ^ t) & 7) << 4)) = __float2bfloat16_rn(1.0f);
    if (t < 64) {
      const int c0 = c.clo(c.jlo);
      for (int cc = c0; cc < c.chi; ++cc)
        *reinterpret_cast<__nv_bfloat16*>(smem + Cfg::oKs + t * 128 + ((t & 7) << 4) + 2 * cc) =
            p.ksum[((size_t)c.bh * N + c.i0 + cc) * D + 64 * c.h + t];
    }
    fence_proxy_async();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  c.tmem = misc[0];

  if (warp == 0) {
    if (lane == 0) mk_producer<D>(c, p, &tmQ, &tmG);
  } else if (warp == 1) {
    if (lane == 0) mk_issuer<D>(c, p);
  } else if (warp >= 4 && warp < 8) {
    mk_drain<D>(c, p, &tmDQ);
  } else if (warp >= 8) {
    mk_gate_writer<D>(c, p);
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
