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
// dQ_rj and dK_j leave through fp32 red.global (other key chunks add to the same
// rows); dV_i, dK_i and d src stay in TMEM / registers until the sweep ends.
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
  const float* carry;      // (b*h*n, n, 128) decay prefix at the start of row tile j
  float* acc_dk;           // (b*h, L, 64) fp32, zeroed
  float* acc_dq;           // (b*h, r, L, 64) fp32, zeroed
  float* acc_dt;           // (b*h, L) fp32, zeroed
  __nv_bfloat16* dvc;      // written directly
  void* dss;               // gate dtype, written directly
  int* status;
  int skip_masked;
};

struct BwdCfg {
  static constexpr int kTileBytes = 16384;    // [128][64] bf16
  static constexpr int oKi = 0, oVi = 16384, oKj = 32768, oQ = 49152, oGo = 65536;
  static constexpr int oCs = 81920;           // 64 KB fp32 C^T[row][key]
  static constexpr int oP = 147456;           // 32 KB bf16 P[row][key]; reused for dG[key][row]
  static constexpr int odS = 180224;          // 32 KB bf16 dS[row][key]
  static constexpr int oI = 212992;           // 2 KB: 16 x 64 bf16, identity in the first 16 columns
  static constexpr int oT3 = 215040;          // 2 x 128 floats
  static constexpr int oBar = 216064;
  static constexpr int oMisc = oBar + 256;
  static constexpr int kSmemBytes = oMisc + 64 + 1024;
  static constexpr uint32_t tX0 = 0, tX1 = 128, tXC = 256, tDV = 384, tDK = 448;
};

enum BwdBar {
  bKvFull = 0, bKjFull, bInFull, bGFull, bX0Free, bSdpFull, bX1Free, bCReady, bCsFree, bPdsReady, bRDone, bG2Full,
  bDgReady, bDkjFull, bT3Ready, bFinal, bNumBars
};

struct BwdCtx {
  uint8_t* smem;
  uint32_t bars;
  uint32_t tmem;
  volatile int* abort_flag;
  int i, bh, nvalid, ntiles;
  __device__ __forceinline__ uint32_t bar(int idx) const { return bars + 8u * idx; }
  __device__ __forceinline__ bool wait(int idx, uint32_t parity) const { return mbar_wait(bar(idx), parity & 1u, abort_flag); }
  // row tile index of sweep step T: valid tiles n-1 .. i first, then the masked ones i-1 .. 0
  __device__ __forceinline__ int tile_j(int T, int N) const { return T < nvalid ? N - 1 - T : i - 1 - (T - nvalid); }
};

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
  int rc = 0;
  for (int T = 0; T < c.ntiles; ++T) {
    const bool valid = T < c.nvalid;
    const int j = c.tile_j(T, N);
    if (valid) {
      if (T >= 1 && !c.wait(bDkjFull, T - 1)) return;
      mbar_expect_tx(c.bar(bKjFull), BwdCfg::kTileBytes);
      tma_load_2d(sbase + BwdCfg::oKj, tmK, 0, c.bh * L + j * 128, c.bar(bKjFull));
    }
    for (int r = 0; r < R; ++r, ++rc) {
      if (rc >= 1 && !c.wait(bRDone, rc - 1)) return;
      mbar_expect_tx(c.bar(bInFull), 2 * BwdCfg::kTileBytes);
      tma_load_2d(sbase + BwdCfg::oQ, tmQ, 0, (c.bh * R + r) * L + j * 128, c.bar(bInFull));
      tma_load_2d(sbase + BwdCfg::oGo, tmG, 0, (int)((chunk_id * R + r) * L + (size_t)j * 128), c.bar(bInFull));
    }
  }
}

// ---------------------------------------------------------------- MMA issuer --
__device__ __forceinline__ void bwd_mma(const BwdCtx& c, const BwdParams& p) {
  const int R = p.s.R, N = p.s.N;
  (void)N;
  const uint32_t sb = smem_u32(c.smem);
  constexpr uint32_t id_nt = idesc_bf16(128, 128, 0, 0);   // A K-major, B K-major, N = 128
  constexpr uint32_t id_tt = idesc_bf16(128, 64, 1, 1);    // A MN-major, B MN-major, N = 64
  constexpr uint32_t id_nt64 = idesc_bf16(128, 64, 0, 1);  // A K-major,  B MN-major, N = 64
  constexpr uint32_t id_dc = idesc_bf16(128, 16, 1, 0);    // A MN-major, B K-major,  N = 16
  const uint32_t X0 = c.tmem + BwdCfg::tX0, X1 = c.tmem + BwdCfg::tX1, XC = c.tmem + BwdCfg::tXC;
  const uint32_t DV = c.tmem + BwdCfg::tDV, DK = c.tmem + BwdCfg::tDK;

  // D[128x128] = A[128][64] B[128][64]^T (both K-major, one 64-element box)
  auto mma_nt = [&](uint32_t d, uint32_t a, uint32_t b) {
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
      mma_ss(d, smem_desc_sw128(a + ks * 32, 16, 1024), smem_desc_sw128(b + ks * 32, 16, 1024), id_nt, ks > 0);
  };
  // D[128x64] (+)= A^T B : A stored [K=128 rows][M=128] (two 64-wide boxes), B stored [K=128 rows][N=64]
  auto mma_tt = [&](uint32_t d, uint32_t a, uint32_t b, bool acc) {
#pragma unroll
    for (int ks = 0; ks < 8; ++ks)
      mma_ss(d, smem_desc_sw128(a + ks * 2048, 16384, 1024), smem_desc_sw128(b + ks * 2048, 16384, 1024), id_tt,
             (acc || ks > 0) ? 1u : 0u);
  };
  // D[128x64] (+)= A B : A stored [M=128 rows][K=128] (two boxes), B stored [K=128 rows][N=64]
  auto mma_nn = [&](uint32_t d, uint32_t a, uint32_t b, bool acc) {
#pragma unroll
    for (int ks = 0; ks < 8; ++ks)
      mma_ss(d, smem_desc_sw128(a + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024), smem_desc_sw128(b + ks * 2048, 16384, 1024),
             id_nt64, (acc || ks > 0) ? 1u : 0u);
  };

  if (!c.wait(bKvFull, 0)) return;
  int x0_uses = 0, x1_uses = 0, rc = 0;
  bool have_acc = false;     // dV / dK_i accumulators hold something
  for (int T = 0; T < c.ntiles; ++T) {
    const bool valid = T < c.nvalid;
    if (valid) {
      if (!c.wait(bKjFull, T)) return;
      if (x0_uses >= 1 && !c.wait(bX0Free, x0_uses - 1)) return;
      tc_fence_after();
      mma_nt(X0, sb + BwdCfg::oKi, sb + BwdCfg::oKj);                 // G = K_i K_j^T
      tc_commit(c.bar(bGFull));
      ++x0_uses;
    }
    for (int r = 0; r < R; ++r, ++rc) {
      if (!c.wait(bInFull, rc)) return;
      if (valid) {
        if (!c.wait(bX0Free, x0_uses - 1)) return;
        tc_fence_after();
        mma_nt(X0, sb + BwdCfg::oQ, sb + BwdCfg::oKi);                // S = Q K_i^T
        ++x0_uses;
      }
      if (x1_uses >= 1 && !c.wait(bX1Free, x1_uses - 1)) return;
      tc_fence_after();
      mma_nt(X1, sb + BwdCfg::oGo, sb + BwdCfg::oVi);                 // dP = dO V_i^T
      ++x1_uses;
      tc_commit(c.bar(bSdpFull));
      if (!c.wait(bPdsReady, rc)) return;
      tc_fence_after();
      mma_tt(DV, sb + BwdCfg::oP, sb + BwdCfg::oGo, have_acc);        // dV_i += P^T dO
      mma_tt(DK, sb + BwdCfg::odS, sb + BwdCfg::oQ, have_acc);        // dK_i += dS^T Q
      have_acc = true;
      mma_nn(X1, sb + BwdCfg::odS, sb + BwdCfg::oKi, false);          // dQ = dS K_i  (dP has been consumed)
      if (valid) {
#pragma unroll
        for (int nb = 0; nb < 8; ++nb)                                 // dC[key][row] (+)= dS^T I
          mma_ss(XC + nb * 16, smem_desc_sw128(sb + BwdCfg::odS + nb * 2048, 16384, 1024),
                 smem_desc_sw128(sb + BwdCfg::oI, 16, 1024), id_dc, r > 0 ? 1u : 0u);
      }
      tc_commit(c.bar(bRDone));
    }
    if (valid) {
      if (!c.wait(bX0Free, x0_uses - 1)) return;
      tc_fence_after();
      mma_nt(X0, sb + BwdCfg::oKi, sb + BwdCfg::oKj);                 // G again for the decay backward
      tc_commit(c.bar(bG2Full));
      ++x0_uses;
      if (!c.wait(bDgReady, T)) return;
      if (!c.wait(bX1Free, x1_uses - 1)) return;
      tc_fence_after();
      mma_tt(X1, sb + BwdCfg::oP, sb + BwdCfg::oKi, false);           // dK_j = dG^T K_i
      ++x1_uses;
      mma_nn(DK, sb + BwdCfg::oP, sb + BwdCfg::oKj, true);            // dK_i += dG K_j
      tc_commit(c.bar(bDkjFull));
    }
  }
  tc_commit(c.bar(bFinal));
}

// --------------------------------------------------------------- decay group --
template <typename TG>
__device__ __forceinline__ void bwd_decay(const BwdCtx& c, const BwdParams& p) {
  const int L = p.s.L, N = p.s.N;
  const int k = threadIdx.x & 127, lane = threadIdx.x & 31;
  const uint32_t lane_base = (uint32_t)((threadIdx.x >> 5) & 3) * 32u << 16;
  const TG* ss = static_cast<const TG*>(p.ssrc) + (size_t)c.bh * L;
  const TG* sd = static_cast<const TG*>(p.sdest) + (size_t)c.bh * L;
  const float s3 = cbrtf(Num<TG>::ld(ss + c.i * 128 + k));
  float* sT3 = reinterpret_cast<float*>(c.smem + BwdCfg::oT3);
  uint8_t* sCs = c.smem + BwdCfg::oCs;
  uint8_t* sdG = c.smem + BwdCfg::oP;
  const size_t chunk_id = (size_t)c.bh * N + c.i;
  const uint32_t X0 = c.tmem + BwdCfg::tX0 + lane_base, XC = c.tmem + BwdCfg::tXC + lane_base;
  float suffix = 0.f, ds_acc = 0.f;

  for (int T = 0; T < c.nvalid; ++T) {
    const int j = N - 1 - T;
    const bool diag = (j == c.i);
    float* t3buf = sT3 + (T & 1) * 128;
    t3buf[k] = cbrtf(Num<TG>::ld(sd + j * 128 + k));
    mbar_arrive(c.bar(bT3Ready));
    if (!c.wait(bT3Ready, T)) return;
    const float carry = p.carry[(chunk_id * N + j) * 128 + k];
    if (!c.wait(bGFull, T)) return;
    tc_fence_after();
    if (T >= 1 && !c.wait(bCsFree, T - 1)) return;
    // ---- forward recomputation: decay prefix C^T[row][key] ------------------
    float local = 0.f;
#pragma unroll 1
    for (int cb = 0; cb < 4; ++cb) {
      uint32_t g[32];
      tmem_ld32(X0 + cb * 32, g);
      tc_wait_ld();
#pragma unroll
      for (int x = 0; x < 32; ++x) {
        const int q = cb * 32 + x;
        float ell = log_retention(gated_affinity(gram_pow23(__uint_as_float(g[x])), s3, t3buf[q]));
        if (diag && q <= k) ell = 0.f;
        local += ell;
        const float v = (diag && q < k) ? mask_value() : (local + carry);
        *reinterpret_cast<float*>(sCs + q * 512 + ((((k >> 2) ^ (q & 7)) & 31) << 4) + (k & 3) * 4) = v;
      }
    }
    tc_fence_before();
    mbar_arrive(c.bar(bX0Free));
    mbar_arrive(c.bar(bCReady));

    // ---- backward: reverse scan of dC, gradients of the decay term -----------
    if (!c.wait(bG2Full, T)) return;
    tc_fence_after();
    float run = 0.f, first = 0.f;
#pragma unroll 1
    for (int cb = 3; cb >= 0; --cb) {
      uint32_t g[32], dc[32];
      tmem_ld32(X0 + cb * 32, g);
      tmem_ld32(XC + cb * 32, dc);
      tc_wait_ld();
      float xs[32];
      uint32_t pk[16];
      float dg_hold = 0.f;
#pragma unroll
      for (int x = 31; x >= 0; --x) {
        const int q = cb * 32 + x;
        run += __uint_as_float(dc[x]);
        float dl = run + suffix;
        if (diag && q <= k) dl = 0.f;
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
        xs[x] = dstat * s3;
        float dg = __bfloat162float(__float2bfloat16_rn(da * s3 * t3));
        dg = gv > 0.f ? dg * (2.0f / 3.0f) * ex2(lg * (-1.0f / 3.0f)) : 0.f;
        if (x & 1) {
          dg_hold = dg;
        } else {
          __nv_bfloat162 h = __floats2bfloat162_rn(dg, dg_hold);
          pk[x >> 1] = *reinterpret_cast<uint32_t*>(&h);
        }
      }
      // dG[key][row] bf16, 128-byte swizzled, rows = keys, two boxes of 64 rows-of-the-tile
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int ch = cb * 4 + u;
        *reinterpret_cast<uint4*>(sdG + (ch >> 3) * 16384 + k * 128 + ((((ch & 7) ^ (k & 7)) & 7) << 4)) =
            make_uint4(pk[u * 4 + 0], pk[u * 4 + 1], pk[u * 4 + 2], pk[u * 4 + 3]);
      }
      // d static_dest: sum over the 128 keys of dstat * src^(1/3)
      const float colsum = warp_transpose_reduce(xs, lane);
      const float t3l = t3buf[cb * 32 + lane];
      if (colsum != 0.f) atomicAdd(p.acc_dt + (size_t)c.bh * L + j * 128 + cb * 32 + lane, colsum / (3.0f * t3l * t3l));
    }
    suffix = first;
    fence_proxy_async();
    tc_fence_before();
    mbar_arrive(c.bar(bX0Free));
    mbar_arrive(c.bar(bDgReady));
  }

  // ---- end of the sweep: dV_i, dK_i, d static_src ----------------------------
  if (!c.wait(bFinal, 0)) return;
  tc_fence_after();
  const size_t krow = (size_t)c.bh * L + c.i * 128 + k;
#pragma unroll 1
  for (int cb = 0; cb < 2; ++cb) {
    uint32_t o[32];
    tmem_ld32(c.tmem + BwdCfg::tDV + lane_base + cb * 32, o);
    tc_wait_ld();
    uint32_t pk[16];
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(o[2 * u]), __uint_as_float(o[2 * u + 1]));
      pk[u] = *reinterpret_cast<uint32_t*>(&h);
    }
    uint4* dst = reinterpret_cast<uint4*>(p.dvc + krow * 64 + cb * 32);
    dst[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    dst[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
    dst[2] = make_uint4(pk[8], pk[9], pk[10], pk[11]);
    dst[3] = make_uint4(pk[12], pk[13], pk[14], pk[15]);
    tmem_ld32(c.tmem + BwdCfg::tDK + lane_base + cb * 32, o);
    tc_wait_ld();
    float* dk = p.acc_dk + krow * 64 + cb * 32;
#pragma unroll
    for (int u = 0; u < 8; ++u)
      red_add_v4(dk + u * 4, __uint_as_float(o[u * 4]), __uint_as_float(o[u * 4 + 1]), __uint_as_float(o[u * 4 + 2]),
                 __uint_as_float(o[u * 4 + 3]));
  }
  Num<TG>::st(static_cast<TG*>(p.dss) + krow, ds_acc / (3.0f * s3 * s3));
}

// ------------------------------------------------------------- softmax group --
__device__ __forceinline__ void bwd_softmax(const BwdCtx& c, const BwdParams& p) {
  const int L = p.s.L, R = p.s.R, N = p.s.N;
  const int row = threadIdx.x & 127;
  const uint32_t lane_base = (uint32_t)((threadIdx.x >> 5) & 3) * 32u << 16;
  const uint8_t* sCrow = c.smem + BwdCfg::oCs + row * 512;
  uint8_t* sP = c.smem + BwdCfg::oP;
  uint8_t* sdS = c.smem + BwdCfg::odS;
  const size_t chunk_id = (size_t)c.bh * N + c.i;
  const uint32_t X0 = c.tmem + BwdCfg::tX0 + lane_base, X1 = c.tmem + BwdCfg::tX1 + lane_base;
  const float kLog2e = 1.4426950408889634f;
  const uint32_t swz = (uint32_t)(row & 7);

  auto store_rows = [&](int cb, const uint32_t* pp, const uint32_t* dd) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int ch = cb * 4 + u;
      const uint32_t off = (ch >> 3) * 16384 + row * 128 + ((((uint32_t)(ch & 7) ^ swz) & 7) << 4);
      *reinterpret_cast<uint4*>(sP + off) = make_uint4(pp[u * 4], pp[u * 4 + 1], pp[u * 4 + 2], pp[u * 4 + 3]);
      *reinterpret_cast<uint4*>(sdS + off) = make_uint4(dd[u * 4], dd[u * 4 + 1], dd[u * 4 + 2], dd[u * 4 + 3]);
    }
  };
  auto drain_x1 = [&](float* dst_row) {
#pragma unroll 1
    for (int cb = 0; cb < 2; ++cb) {
      uint32_t o[32];
      tmem_ld32(X1 + cb * 32, o);
      tc_wait_ld();
#pragma unroll
      for (int u = 0; u < 8; ++u)
        red_add_v4(dst_row + cb * 32 + u * 4, __uint_as_float(o[u * 4]), __uint_as_float(o[u * 4 + 1]),
                   __uint_as_float(o[u * 4 + 2]), __uint_as_float(o[u * 4 + 3]));
    }
    tc_fence_before();
    mbar_arrive(c.bar(bX1Free));
  };

  int rc = 0;
  for (int T = 0; T < c.ntiles; ++T) {
    const bool valid = T < c.nvalid;
    const int j = c.tile_j(T, N);
    for (int r = 0; r < R; ++r, ++rc) {
      const size_t grow = (chunk_id * R + r) * L + (size_t)j * 128 + row;
      const float gd = p.g_denom_is_f32 ? static_cast<const float*>(p.g_denom)[grow]
                                        : __bfloat162float(static_cast<const __nv_bfloat16*>(p.g_denom)[grow]);
      if (!c.wait(bSdpFull, rc)) return;
      tc_fence_after();
      if (valid) {
        if (r == 0 && !c.wait(bCReady, T)) return;
        // pass 1: s = S + C, row max
        float m = -INFINITY;
#pragma unroll 1
        for (int cb = 0; cb < 4; ++cb) {
          uint32_t s[32];
          tmem_ld32(X0 + cb * 32, s);
          tc_wait_ld();
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int chunk = cb * 8 + u;
            const float4 cv = *reinterpret_cast<const float4*>(sCrow + ((((uint32_t)chunk ^ swz) & 31) << 4));
            const float a0 = __uint_as_float(s[u * 4 + 0]) + cv.x, a1 = __uint_as_float(s[u * 4 + 1]) + cv.y;
            const float a2 = __uint_as_float(s[u * 4 + 2]) + cv.z, a3 = __uint_as_float(s[u * 4 + 3]) + cv.w;
            m = fmaxf(m, fmaxf(fmaxf(a0, a1), fmaxf(a2, a3)));
            s[u * 4 + 0] = __float_as_uint(a0); s[u * 4 + 1] = __float_as_uint(a1);
            s[u * 4 + 2] = __float_as_uint(a2); s[u * 4 + 3] = __float_as_uint(a3);
          }
          tmem_st32(X0 + cb * 32, s);
        }
        tc_wait_st();
        if (r == R - 1) mbar_arrive(c.bar(bCsFree));
        // pass 2: e = exp(s - m), l = sum e, sum e dP
        const float mb = m * kLog2e;
        float l = 0.f, edp = 0.f;
#pragma unroll 1
        for (int cb = 0; cb < 4; ++cb) {
          uint32_t s[32], dp[32];
          tmem_ld32(X0 + cb * 32, s);
          tmem_ld32(X1 + cb * 32, dp);
          tc_wait_ld();
#pragma unroll
          for (int x = 0; x < 32; ++x) {
            const float e = ex2(fmaf(__uint_as_float(s[x]), kLog2e, -mb));
            l += e;
            edp = fmaf(e, __uint_as_float(dp[x]), edp);
            s[x] = __float_as_uint(e);
          }
          tmem_st32(X0 + cb * 32, s);
        }
        tc_wait_st();
        const float linv = 1.0f / l;
        const float corr = gd - edp * linv;          // g_denom - sum_k P dP
        // pass 3: P = e / l, dS = P (dP + corr)
#pragma unroll 1
        for (int cb = 0; cb < 4; ++cb) {
          uint32_t s[32], dp[32];
          tmem_ld32(X0 + cb * 32, s);
          tmem_ld32(X1 + cb * 32, dp);
          tc_wait_ld();
          uint32_t pp[16], dd[16];
#pragma unroll
          for (int u = 0; u < 16; ++u) {
            const float p0 = __uint_as_float(s[2 * u]) * linv, p1 = __uint_as_float(s[2 * u + 1]) * linv;
            const float d0 = p0 * (__uint_as_float(dp[2 * u]) + corr), d1 = p1 * (__uint_as_float(dp[2 * u + 1]) + corr);
            __nv_bfloat162 hp = __floats2bfloat162_rn(p0, p1), hd = __floats2bfloat162_rn(d0, d1);
            pp[u] = *reinterpret_cast<uint32_t*>(&hp);
            dd[u] = *reinterpret_cast<uint32_t*>(&hd);
          }
          store_rows(cb, pp, dd);
        }
        tc_fence_before();
        mbar_arrive(c.bar(bX0Free));
      } else {
        // rows before the chunk: uniform softmax P = 1/128 (universal_attention_autograd.py:154)
        float sum = 0.f;
#pragma unroll 1
        for (int cb = 0; cb < 4; ++cb) {
          uint32_t dp[32];
          tmem_ld32(X1 + cb * 32, dp);
          tc_wait_ld();
#pragma unroll
          for (int x = 0; x < 32; ++x) sum += __uint_as_float(dp[x]);
        }
        const float pu = 1.0f / 128.0f;
        const float corr = gd - sum * pu;
        __nv_bfloat162 hp = __floats2bfloat162_rn(pu, pu);
        const uint32_t pconst = *reinterpret_cast<uint32_t*>(&hp);
#pragma unroll 1
        for (int cb = 0; cb < 4; ++cb) {
          uint32_t dp[32];
          tmem_ld32(X1 + cb * 32, dp);
          tc_wait_ld();
          uint32_t pp[16], dd[16];
#pragma unroll
          for (int u = 0; u < 16; ++u) {
            __nv_bfloat162 hd = __floats2bfloat162_rn(pu * (__uint_as_float(dp[2 * u]) + corr),
                                                      pu * (__uint_as_float(dp[2 * u + 1]) + corr));
            pp[u] = pconst;
            dd[u] = *reinterpret_cast<uint32_t*>(&hd);
          }
          store_rows(cb, pp, dd);
        }
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(c.bar(bPdsReady));
      // dQ_rj leaves through fp32 atomics: other key chunks add to the same rows
      if (!c.wait(bRDone, rc)) return;
      tc_fence_after();
      drain_x1(p.acc_dq + (((size_t)c.bh * R + r) * L + (size_t)j * 128 + row) * 64);
    }
    if (valid) {
      if (!c.wait(bDkjFull, T)) return;
      tc_fence_after();
      drain_x1(p.acc_dk + ((size_t)c.bh * L + (size_t)j * 128 + row) * 64);      // dK_j
    }
  }
}

template <typename TG>
__global__ void __launch_bounds__(384, 1)
bwd_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
           const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmG, BwdParams p) {
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
  c.nvalid = p.s.N - c.i;
  c.ntiles = c.nvalid + (p.skip_masked ? 0 : c.i);

  if (threadIdx.x == 0) {
    misc[1] = 0;
    for (int b = 0; b < bNumBars; ++b) {
      uint32_t count = 1;
      if (b == bX0Free || b == bX1Free || b == bCReady || b == bCsFree || b == bPdsReady || b == bDgReady || b == bT3Ready)
        count = 128;
      mbar_init(c.bar(b), count);
    }
    mbar_init_fence();
    prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmQ); prefetch_tmap(&tmG);
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

  if (warp == 0) {
    if (lane == 0) bwd_producer(c, p, &tmK, &tmV, &tmQ, &tmG);
  } else if (warp == 1) {
    if (lane == 0) bwd_mma(c, p);
  } else if (warp >= 4 && warp < 8) {
    bwd_decay<TG>(c, p);
  } else if (warp >= 8) {
    bwd_softmax(c, p);
  }

  tc_fence_before();
  __syncthreads();
  if (*c.abort_flag) {
    if (threadIdx.x == 0) atomicExch(p.status, 2);
    for (int it = 0; it < 64; ++it) __nanosleep(2000);
    __syncthreads();
  }
  if (warp == 0) tmem_dealloc(c.tmem, 512);
}

}  // namespace sm100
}  // namespace ua
