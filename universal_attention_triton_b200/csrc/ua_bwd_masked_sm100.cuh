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
//   Nt_c (+)= [Q | O]^T g              [64 + 64][D]     lanes 0..63: N_c^T, lane 64: u_c  (O: a constant tile, column 0 = ones)
// A tcgen05.mma of M = 128, K = 16 takes about 60 cycles at N = 64 and at N = 128 alike (measured), so the N^T products
// of neighbouring chunks share one instruction: their gradient tiles sit side by side in a 32 KB slot and form one
// MN-major B operand of N = 128.  The terms in gd stay on the CUDA cores, in fp32: four warps accumulate
// w_c += gd_c^T Q_rj from the Q tile in shared memory, and the drain warps add gd_c (x) ksum_c / 128 to Y on its way out.
// head_dim 128 runs as two blocks per work item, one per 64-wide half of the output columns of Y / lanes of Nt.
// A work item is (batch*head, group of G chunks, range of row tiles); partial N / w / u leave as fp32 global adds.
#pragma once
#include "ua_fwd_sm100.cuh"

namespace ua {
namespace sm100 {

struct MaskedParams {
  Shape s;
  const float* g_denom;          // (b*h*n, r, L) fp32, 16-byte aligned
  uint8_t* mt;                   // (b*h*n) images of M_i^T / 128 as bf16: [D/64 halves of d'][D/64 boxes of d][64][64], 128-byte swizzled
  __nv_bfloat16* ksum;           // (b*h*n, D): column sums of K_i / 128
  float* nacc;                   // (b*h*n, D + 3, D) fp32: rows 0..D-1 = N^T[d'][d], row D = w[d'], row D + 1 = u[d], row D + 2 = vbar[d]
  float* acc_dk;                 // (b*h*L, D) fp32, added to
  int* status;
  int jp;                        // row tiles per work item
  int items_per_bh;              // number of (group, piece of row tiles) items per batch*head (set by the launcher)
  // Range of row tiles [j_begin, j_end) (sequence-chunk sharding; whole sequence: 0, N, L, 0): xq, g_out, g_denom and
  // the dQ accumulator are slabs of Lr rows that hold the range at row r0.
  int j_begin, j_end, Lr, r0;
  float* acc_dv;                 // row ranges only: (b*h, L, D) fp32, dV_i = 1 (x) u_i / 128 is ADDED here by the finish kernel
};

template <int D> __host__ __device__ constexpr int kNaccRows() { return D + 3; }

template <int D>
struct MkCfg {
  static constexpr int kKB = D / 64;
  static constexpr int kG = 256 / D;                       // chunks per group: their N^T accumulators fill 256 TMEM columns
  static constexpr int kPer = 128 / D;                     // gradient tiles per 32 KB slot (one N = 128 operand)
  static constexpr int kUnits = kG / kPer;                 // slots per step when every chunk of the group is active
  static constexpr int kSlots = 3;
  static constexpr int kDoBytes = kKB * 16384;
  static constexpr int kAhead = (D == 64) ? 12 : 6;        // gradient tiles requested into L2 ahead of the ring
  static constexpr int kMtBytes = kKB * 8192;              // one half (64 rows d') of a chunk's M^T image
  static constexpr int oSlot = 0;
  static constexpr int oQ = oSlot + kSlots * 32768;        // 2 x Q [128][64]
  static constexpr int oOnes = oQ + 2 * 16384;             // [128][64] bf16: column 0 = 1, the rest 0 (after the Q tiles: the
                                                           // second 64 lanes of the [Q | O] operand, reached through LBO)
  static constexpr int oMt = oOnes + 16384;
  static constexpr int oStage = oMt + kG * kMtBytes;       // two [128][32] fp32 boxes
  static constexpr int oGd = oStage + 32768;               // 2 x kG x float[128]: g_denom rows of a step
  static constexpr int oKs = oGd + 2 * kG * 512;           // float [64][kG]: ksum_c / 128 of this block's 64 output columns
  static constexpr int oBar = oKs + 64 * kG * 4;
  static constexpr int oMisc = oBar + 256;
  static constexpr int kSmemBytes = oMisc + 64 + 1024;     // + slack to align the base to 1024 B
  static constexpr uint32_t tY0 = 0, tY1 = 64, tN = 128;
  static_assert(tN + kG * D <= 512, "TMEM budget");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

enum MkBar {
  mMtFull = 0, mQFull = 1, mQFree = 3, mYFull = 5, mYFree = 7, mDone = 9, mSlotFull = 10, mSlotFree = 13, mNumBars = 16
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
  int jb, r0;                          // the slabs hold row tile jb at row r0
  __device__ __forceinline__ int srow(int j) const { return r0 + (j - jb) * 128; }
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
  // each thread: four rows d' (dp0 .. dp0 + 3) x eight columns d0 .. d0 + 7 of M^T, so that a value tile row is converted once per four rows
  for (int o = t; o < D * D / 32; o += 256) {
    const int dp0 = (o / (D / 8)) * 4, d0 = (o % (D / 8)) * 8;
    float acc[4][8];
#pragma unroll
    for (int y = 0; y < 4; ++y)
#pragma unroll
      for (int x = 0; x < 8; ++x) acc[y][x] = 0.f;
#pragma unroll 2
    for (int k = 0; k < 128; ++k) {
      const uint2 kraw = *reinterpret_cast<const uint2*>(sK + k * D + dp0);
      const float kv[4] = {__uint_as_float(kraw.x << 16), __uint_as_float(kraw.x & 0xffff0000u), __uint_as_float(kraw.y << 16),
                           __uint_as_float(kraw.y & 0xffff0000u)};
      const uint4 raw = *reinterpret_cast<const uint4*>(sV + k * D + d0);
      const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
      float vv[8];
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        vv[2 * x] = __uint_as_float(rw[x] << 16);
        vv[2 * x + 1] = __uint_as_float(rw[x] & 0xffff0000u);
      }
#pragma unroll
      for (int y = 0; y < 4; ++y)
#pragma unroll
        for (int x = 0; x < 8; ++x) acc[y][x] = fmaf(kv[y], vv[x], acc[y][x]);
    }
#pragma unroll
    for (int y = 0; y < 4; ++y) {
      const int dp = dp0 + y;
      const float ks = sSum[dp] * (1.0f / 128.0f);
      uint32_t w4[4];
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        __nv_bfloat162 hh = __floats2bfloat162_rn((acc[y][2 * x] - ks * sSum[D + d0 + 2 * x]) * (1.0f / 128.0f),
                                                  (acc[y][2 * x + 1] - ks * sSum[D + d0 + 2 * x + 1]) * (1.0f / 128.0f));
        w4[x] = *reinterpret_cast<uint32_t*>(&hh);
      }
      const int half = dp >> 6, row = dp & 63, box = d0 >> 6, chunk16 = (d0 & 63) >> 3;
      *reinterpret_cast<uint4*>(img + ((size_t)(half * (D / 64) + box) * 64 + row) * 128 + (((chunk16 ^ row) & 7) << 4)) =
          make_uint4(w4[0], w4[1], w4[2], w4[3]);
    }
  }
}

// ---------------------------------------------------------------- finish kernel --
// One block per chunk i >= 1 (thread = key): dK_i += ((V_i - vbar) N_i + 1 (x) w_i) / 128.  (dV_i = 1 (x) u_i / 128 is the same row
// for every key: the main backward kernel adds it from the chunk's u row when it writes dV_i.)
template <int D>
__global__ void __launch_bounds__(128) masked_finish_kernel(const __nv_bfloat16* __restrict__ vc, MaskedParams p) {
  __shared__ __align__(16) float sN[32 * D];          // 32 rows d' of N^T at a time
  __shared__ float sW[D];
  const int N = p.s.N;
  const size_t chunk = blockIdx.x;
  if (chunk % N == 0) return;           // no rows before the first chunk
  const int key = threadIdx.x;
  const float* nacc = p.nacc + chunk * (size_t)kNaccRows<D>() * D;
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
  if (p.acc_dv) {                       // row ranges: the same row u / 128 for every key, added to the shared fp32 buffer
    const float* u = nacc + (size_t)(D + 1) * D;
    float4* dv = reinterpret_cast<float4*>(p.acc_dv + (chunk * 128 + key) * D);
#pragma unroll 4
    for (int x = 0; x < D / 4; ++x) {
      float4 cur = dv[x];
      cur.x += u[4 * x] * (1.0f / 128.0f); cur.y += u[4 * x + 1] * (1.0f / 128.0f);
      cur.z += u[4 * x + 2] * (1.0f / 128.0f); cur.w += u[4 * x + 3] * (1.0f / 128.0f);
      dv[x] = cur;
    }
  }
#pragma unroll 1
  for (int blk = 0; blk < D / 32; ++blk) {
    __syncthreads();
    for (int x = key; x < 32 * D / 4; x += 128) reinterpret_cast<float4*>(sN)[x] = reinterpret_cast<const float4*>(nacc + (size_t)blk * 32 * D)[x];
    __syncthreads();
#pragma unroll 1
    for (int q = 0; q < 32; q += 4) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int d = 0; d < D; d += 4) {
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const float4 nv = *reinterpret_cast<const float4*>(sN + (q + x) * D + d);
          acc[x] = fmaf(vcen[d], nv.x, fmaf(vcen[d + 1], nv.y, fmaf(vcen[d + 2], nv.z, fmaf(vcen[d + 3], nv.w, acc[x]))));
        }
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
// Optional phase timing (compile with -DUA_PROFILE_MK=<block>): each role of that block accumulates clock64() deltas per
// phase and stores them after the status words.
#ifdef UA_PROFILE_MK
#define MQ_DECL long long mq_t = clock64(), mq_acc[4] = {0, 0, 0, 0};
#define MQ(idx) { long long now_ = clock64(); mq_acc[idx] += now_ - mq_t; mq_t = now_; }
#define MQ_STORE(base) if (blockIdx.x == UA_PROFILE_MK) { for (int z = 0; z < 4; ++z) reinterpret_cast<long long*>(p.status)[2 + (base) + z] = mq_acc[z]; }
#else
#define MQ_DECL
#define MQ(idx)
#define MQ_STORE(base)
#endif

// Slot unit u of a step: the chunks [u kPer, (u + 1) kPer) of the group that have the step's row tile before them.
template <int D>
struct MkUnit {
  int lo, hi;
  __device__ __forceinline__ MkUnit(int u, int c0, int chi) {
    lo = max(u * MkCfg<D>::kPer, c0);
    hi = min((u + 1) * MkCfg<D>::kPer, chi);
  }
  __device__ __forceinline__ bool active() const { return lo < hi; }
};

template <int D>
__device__ __forceinline__ void mk_producer(const MkCtx& c, const MaskedParams& p, const CUtensorMap* tmQ, const CUtensorMap* tmG) {
  using Cfg = MkCfg<D>;
  const int L = p.Lr, R = p.s.R, N = p.s.N;      // (L: rows per slab of the row-indexed tensors)
  const uint32_t sb = smem_u32(c.smem);
  {
    const int c0 = c.clo(c.jlo);
    mbar_expect_tx(c.bar(mMtFull), (uint32_t)(c.chi - c0) * Cfg::kMtBytes);
    for (int cc = c0; cc < c.chi; ++cc)
      bulk_load_1d(sb + Cfg::oMt + cc * Cfg::kMtBytes,
                   p.mt + ((size_t)c.bh * N + c.i0 + cc) * (size_t)(D * D * 2) + (size_t)c.h * Cfg::kMtBytes, Cfg::kMtBytes,
                   c.bar(mMtFull));
  }
  // The gradient tiles are asked into L2 kAhead tiles before their turn in the shared-memory ring: the ring alone (a few
  // tiles per SM) does not cover the latency of HBM at full bandwidth.
  int pj = c.jlo, pr = 0, pc = c.clo(c.jlo);
  auto prefetch_next = [&]() {
    if (pj >= c.jhi) return;
#pragma unroll
    for (int b = 0; b < Cfg::kKB; ++b)
      tma_prefetch_2d(tmG, 64 * b, (int)((((size_t)c.bh * N + c.i0 + pc) * R + pr) * L + (size_t)c.srow(pj)));
    if (++pc >= c.chi) {
      if (++pr >= R) { pr = 0; ++pj; }
      pc = c.clo(pj);
    }
  };
  for (int x = 0; x < Cfg::kAhead; ++x) prefetch_next();
  int s = 0, uc = 0;
  MQ_DECL
  for (int j = c.jlo; j < c.jhi; ++j) {
    const int c0 = c.clo(j);
    for (int r = 0; r < R; ++r, ++s) {
      const int qs = s & 1;
      MQ(0)
      if (s >= 2 && !c.wait(mQFree + qs, s / 2 - 1)) return;
      MQ(1)
      mbar_expect_tx(c.bar(mQFull + qs), 16384u + (uint32_t)(c.chi - c0) * 512u);
      tma_load_2d(sb + Cfg::oQ + qs * 16384, tmQ, 64 * c.h, (c.bh * R + r) * L + c.srow(j), c.bar(mQFull + qs));
      for (int cc = c0; cc < c.chi; ++cc)
        bulk_load_1d(sb + Cfg::oGd + (qs * Cfg::kG + cc) * 512,
                     p.g_denom + (((size_t)c.bh * N + c.i0 + cc) * R + r) * L + (size_t)c.srow(j), 512, c.bar(mQFull + qs));
      for (int u = 0; u < Cfg::kUnits; ++u) {
        const MkUnit<D> un(u, c0, c.chi);
        if (!un.active()) continue;
        const int sl = uc % Cfg::kSlots;
        MQ(0)
        if (uc >= Cfg::kSlots && !c.wait(mSlotFree + sl, uc / Cfg::kSlots - 1)) return;
        MQ(2)
        ++uc;
        mbar_expect_tx(c.bar(mSlotFull + sl), (uint32_t)(un.hi - un.lo) * Cfg::kDoBytes);
        for (int cc = un.lo; cc < un.hi; ++cc) {
#pragma unroll
          for (int b = 0; b < Cfg::kKB; ++b)
            tma_load_2d(sb + Cfg::oSlot + sl * 32768 + (cc - u * Cfg::kPer) * Cfg::kDoBytes + b * 16384, tmG, 64 * b,
                        (int)((((size_t)c.bh * N + c.i0 + cc) * R + r) * L + (size_t)c.srow(j)), c.bar(mSlotFull + sl));
          prefetch_next();
        }
      }
    }
  }
  MQ_STORE(8)
}

template <int D>
__device__ __forceinline__ void mk_issuer(const MkCtx& c, const MaskedParams& p) {
  using Cfg = MkCfg<D>;
  const int R = p.s.R;
  const uint32_t sb = smem_u32(c.smem);
  constexpr uint32_t id_y = idesc_bf16(128, 64, 0, 0);       // rows x 64: A K-major, B K-major
  if (!c.wait(mMtFull, 0)) return;
  int s = 0, uc = 0;
  MQ_DECL
  for (int j = c.jlo; j < c.jhi; ++j) {
    const int c0 = c.clo(j);
    for (int r = 0; r < R; ++r, ++s) {
      const int qs = s & 1;
      const uint32_t q_addr = sb + Cfg::oQ + qs * 16384;
      MQ(3)
      if (!c.wait(mQFull + qs, s / 2)) return;
      MQ(0)
      if (s >= 2 && !c.wait(mYFree + qs, s / 2 - 1)) return;
      MQ(1)
      tc_fence_after();
      const uint32_t Y = c.tmem + (qs ? Cfg::tY1 : Cfg::tY0);
      // [K = rows][M = the 64 columns of Q, then the 64 columns of the ones tile]
      const uint64_t mQO = desc_from_lo(desc_lo(q_addr, (sb + Cfg::oOnes) - q_addr));
      uint32_t have_y = 0;
      for (int u = 0; u < Cfg::kUnits; ++u) {
        const MkUnit<D> un(u, c0, c.chi);
        if (!un.active()) continue;
        const int sl = uc % Cfg::kSlots;
        MQ(3)
        if (!c.wait(mSlotFull + sl, uc / Cfg::kSlots)) return;
        MQ(2)
        ++uc;
        tc_fence_after();
        const uint32_t slot = sb + Cfg::oSlot + sl * 32768;
        for (int cc = un.lo; cc < un.hi; ++cc) {                     // Y += g Mt_c^T
          const uint32_t g_addr = slot + (cc - u * Cfg::kPer) * Cfg::kDoBytes;
#pragma unroll
          for (int b = 0; b < Cfg::kKB; ++b) {
            mma4_ss(Y, desc_from_lo(desc_lo(g_addr + b * 16384, 16)), desc_from_lo(desc_lo(sb + Cfg::oMt + cc * Cfg::kMtBytes + b * 8192, 16)),
                    2, 2, id_y, have_y);
            have_y = 1;
          }
        }
        // Nt_lo.. += [Q | O]^T [g_lo | ..]: the unit's tiles as one MN-major operand, 64-column groups 16 KB apart
        const uint64_t mG = desc_from_lo(desc_lo(slot + (un.lo - u * Cfg::kPer) * Cfg::kDoBytes, 16384));
        const uint32_t id_n = idesc_bf16(128, (un.hi - un.lo) * D, 1, 1);
        const uint32_t Nt = c.tmem + Cfg::tN + un.lo * D;
        mma4_ss(Nt, mQO, mG, 128, 128, id_n, s > 0);
        mma4_ss(Nt, mQO + 512, mG + 512, 128, 128, id_n, 1);
        tc_commit(c.bar(mSlotFree + sl));
      }
      tc_commit(c.bar(mYFull + qs));
      tc_commit(c.bar(mQFree + qs));
    }
  }
  tc_commit(c.bar(mDone));
  MQ(3)
  MQ_STORE(0)
}

// Four warps on the CUDA cores: w_c[d'] += sum_rows gd_c[row] Q[row][d'] for the group's chunks, from the Q tile in shared
// memory.  Warp = 16 of the 64 columns, lane = row (four passes of 32 rows): every shared-memory access is conflict free
// and nothing is broadcast, so the warps take little of the bandwidth that the MMA operands need.  The sums stay in
// registers over the whole work item and are added up over the lanes once, at its end.
template <int D>
__device__ __forceinline__ void mk_gate_sums(const MkCtx& c, const MaskedParams& p) {
  using Cfg = MkCfg<D>;
  const int R = p.s.R, N = p.s.N;
  const int t = threadIdx.x & 127, lane = t & 31, w = t >> 5;
  float acc[Cfg::kG * 16];
#pragma unroll
  for (int x = 0; x < Cfg::kG * 16; ++x) acc[x] = 0.f;
  int s = 0;
  MQ_DECL
  for (int j = c.jlo; j < c.jhi; ++j) {
    const int c0 = c.clo(j);
    for (int r = 0; r < R; ++r, ++s) {
      const int qs = s & 1;
      MQ(1)
      if (!c.wait_w(mQFull + qs, s / 2)) return;
      MQ(0)
      const uint8_t* q = c.smem + Cfg::oQ + qs * 16384;
      const float* gd = reinterpret_cast<const float*>(c.smem + Cfg::oGd + qs * Cfg::kG * 512);
#pragma unroll 1
      for (int pass = 0; pass < 4; ++pass) {
        const int row = pass * 32 + lane;
        float g[Cfg::kG];
#pragma unroll
        for (int cc = 0; cc < Cfg::kG; ++cc)      // (chunks that do not have this row tile before them: their rows of the table are stale)
          g[cc] = (cc >= c0 && cc < c.chi) ? gd[cc * 128 + row] : 0.f;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const uint4 raw = *reinterpret_cast<const uint4*>(q + row * 128 + ((((2 * w + k) ^ row) & 7) << 4));
          const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const float q0 = __uint_as_float(rw[x] << 16), q1 = __uint_as_float(rw[x] & 0xffff0000u);
#pragma unroll
            for (int cc = 0; cc < Cfg::kG; ++cc) {
              acc[cc * 16 + 8 * k + 2 * x] = fmaf(g[cc], q0, acc[cc * 16 + 8 * k + 2 * x]);
              acc[cc * 16 + 8 * k + 2 * x + 1] = fmaf(g[cc], q1, acc[cc * 16 + 8 * k + 2 * x + 1]);
            }
          }
        }
      }
      c.arrive_w(mQFree + qs);
    }
  }
#ifdef UA_PROFILE_MK
  if (t == 0) { MQ(1) MQ_STORE(12) }
#endif
  const int c0 = c.clo(c.jlo);
#pragma unroll
  for (int grp = 0; grp < Cfg::kG / 2; ++grp) {
    const float tot = warp_transpose_reduce(acc + 32 * grp, lane);      // lane l: sum over the lanes of value 32 grp + l
    const int cc = 2 * grp + (lane >> 4);
    if (cc >= c0 && cc < c.chi)
      atomicAdd(p.nacc + ((size_t)c.bh * N + c.i0 + cc) * (size_t)kNaccRows<D>() * D + (size_t)D * D + 64 * c.h + 16 * w + (lane & 15), tot);
  }
}

// Four warps (TMEM lane quadrant = warp % 4): Y of each step, plus sum_c gd_c (x) ksum_c / 128 -> staging tile -> TMA
// reduce-add into the dQ accumulator; after the last step the group's N^T / u partial sums -> global adds.
template <int D>
__device__ __forceinline__ void mk_drain(const MkCtx& c, const MaskedParams& p, const CUtensorMap* tmDQ) {
  using Cfg = MkCfg<D>;
  const int L = p.Lr, R = p.s.R, N = p.s.N;      // (L: rows per slab of the row-indexed tensors)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = (warp & 3) * 32 + lane;
  const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
  const bool leader = (warp == 4 && lane == 0);
  const uint32_t swz = (uint32_t)(row & 7);
  uint8_t* stage = c.smem + Cfg::oStage;
  const float* ks = reinterpret_cast<const float*>(c.smem + Cfg::oKs);
  int s = 0;
  MQ_DECL
  for (int j = c.jlo; j < c.jhi; ++j) {
    const int c0 = c.clo(j);
    for (int r = 0; r < R; ++r, ++s) {
      const int qs = s & 1;
      MQ(3)
      if (!c.wait_w(mYFull + qs, s / 2)) return;
      MQ(0)
      tc_fence_after();
      float gd[Cfg::kG];
#pragma unroll
      for (int cc = 0; cc < Cfg::kG; ++cc)
        gd[cc] = (cc >= c0 && cc < c.chi) ? reinterpret_cast<const float*>(c.smem + Cfg::oGd + (qs * Cfg::kG + cc) * 512)[row] : 0.f;
      c.arrive_w(mQFree + qs);                     // the step's g_denom rows have been read
      if (leader) bulk_wait_read_all();            // the previous reduce-add has read the staging tile
      named_bar_sync(2, 128);
      MQ(1)
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
        for (int x = 0; x < 8; ++x) {
          float v[4];
#pragma unroll
          for (int y = 0; y < 4; ++y) {
            v[y] = __uint_as_float(o[4 * x + y]);
            if constexpr (Cfg::kG == 4) {
              const float4 k4 = *reinterpret_cast<const float4*>(ks + (32 * hb + 4 * x + y) * 4);
              v[y] = fmaf(gd[0], k4.x, fmaf(gd[1], k4.y, fmaf(gd[2], k4.z, fmaf(gd[3], k4.w, v[y]))));
            } else {
              const float2 k2 = *reinterpret_cast<const float2*>(ks + (32 * hb + 4 * x + y) * 2);
              v[y] = fmaf(gd[0], k2.x, fmaf(gd[1], k2.y, v[y]));
            }
          }
          *reinterpret_cast<float4*>(box + ((((uint32_t)x ^ swz) & 7) << 4)) = make_float4(v[0], v[1], v[2], v[3]);
        }
      }
      MQ(2)
      fence_proxy_async();
      named_bar_sync(2, 128);
      if (leader) {
        const int y = (c.bh * R + r) * L + c.srow(j);
        tma_reduce_add_2d(tmDQ, 64 * c.h, y, smem_u32(stage));
        tma_reduce_add_2d(tmDQ, 64 * c.h + 32, y, smem_u32(stage) + 16384);
        bulk_commit_group();
      }
    }
  }
#ifdef UA_PROFILE_MK
  if (leader) { MQ(3) MQ_STORE(4) }
#endif
  if (!c.wait_w(mDone, 0)) {
    if (leader) bulk_wait_all();
    return;
  }
  tc_fence_after();
  const int c0 = c.clo(c.jlo);
  if ((warp & 3) < 2) {                    // lanes 0..63: rows d' = 64 h + row of N^T
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
    }
  } else if ((warp & 3) == 2 && c.h == 0) {    // lane 64 (column 0 of the ones tile): u_c = column sums of g
    for (int cc = c0; cc < c.chi; ++cc) {
      float* nacc = p.nacc + ((size_t)c.bh * N + c.i0 + cc) * (size_t)kNaccRows<D>() * D + (size_t)(D + 1) * D;
#pragma unroll 1
      for (int hb = 0; hb < D / 32; ++hb) {
        uint32_t o[32];
        tmem_ld32(c.tmem + Cfg::tN + cc * D + lane_base + 32 * hb, o);
        tc_wait_ld();
        if (lane == 0) {
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
    // Items in launch order: by range of row tiles, then batch*head, then group.  The groups that add to the same rows of
    // dQ (and read the same Q tiles) therefore run at about the same time, and the fp32 dQ accumulator -- larger than L2
    // as a whole -- sees each of its tiles come from HBM and go back once instead of once per group.
    int idx = blockIdx.x / Cfg::kKB;
    const int BH = p.s.B * p.s.H, groups = (N + Cfg::kG - 1) / Cfg::kG;
    c.h = blockIdx.x % Cfg::kKB;
    int g = 0;
    bool found = false;
    c.jb = p.j_begin; c.r0 = p.r0;
    // row tiles of the range that lie before the last chunk of group gg: [j_begin, min(j_end, last chunk of gg))
    auto jmax_of = [&](int gg) { return min(min((gg + 1) * Cfg::kG, N) - 1, p.j_end); };
    for (int piece = 0; p.j_begin + piece * p.jp < min(N - 1, p.j_end); ++piece) {
      const int jlo = p.j_begin + piece * p.jp;
      int cnt = 0;                                                       // groups that have row tiles of this piece before a chunk
      for (int gg = 0; gg < groups; ++gg) cnt += (jmax_of(gg) > jlo) ? 1 : 0;
      if (idx < BH * cnt) {
        c.bh = idx / cnt;
        g = groups - 1 - idx % cnt;
        c.jlo = jlo;
        c.jhi = min(c.jlo + p.jp, jmax_of(g));
        found = true;
        break;
      }
      idx -= BH * cnt;
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
      if (b == mYFree || b == mYFree + 1) count = 4;     // one arrival per draining warp
      if (b == mQFree || b == mQFree + 1) count = 9;     // the issuer's commit, the four gate-sum warps, the four draining warps
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
    // ones tile: zeros, ones in column 0; ksum table of this block's 64 output columns
    const int t = threadIdx.x - 256;
    for (int x = t; x < 1024; x += 128) *reinterpret_cast<uint4*>(smem + Cfg::oOnes + (x << 4)) = make_uint4(0u, 0u, 0u, 0u);
    named_bar_sync(3, 128);
    *reinterpret_cast<__nv_bfloat16*>(smem + Cfg::oOnes + t * 128 + ((t & 7) << 4)) = __float2bfloat16_rn(1.0f);
    if (t < 64) {
      const int c0 = c.clo(c.jlo);
      float* ks = reinterpret_cast<float*>(smem + Cfg::oKs) + t * Cfg::kG;
      for (int cc = 0; cc < Cfg::kG; ++cc)
        ks[cc] = (cc >= c0 && cc < c.chi) ? __bfloat162float(p.ksum[((size_t)c.bh * N + c.i0 + cc) * D + 64 * c.h + t]) : 0.f;
    }
    fence_proxy_async();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  c.tmem = misc[0];

#ifdef UA_PROFILE_MK
  const long long mk_t0 = clock64();
#endif
  if (warp == 0) {
    if (lane == 0) mk_producer<D>(c, p, &tmQ, &tmG);
  } else if (warp == 1) {
    if (lane == 0) mk_issuer<D>(c, p);
  } else if (warp >= 4 && warp < 8) {
    mk_drain<D>(c, p, &tmDQ);
  } else if (warp >= 8) {
    mk_gate_sums<D>(c, p);
  }

  tc_fence_before();
  __syncthreads();
#ifdef UA_PROFILE_MK
  if (blockIdx.x == UA_PROFILE_MK && threadIdx.x == 0) reinterpret_cast<long long*>(p.status)[2 + 16] = clock64() - mk_t0;
#endif
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
