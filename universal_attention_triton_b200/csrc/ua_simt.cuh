// Generic fp32 SIMT kernels for the Universal Attention operator.
//
// One thread block owns one key chunk (b, h, i) and sweeps the rows of the
// sequence in tiles of RT rows.  All arithmetic is fp32 on CUDA cores; bf16
// inputs are widened on load and the probabilities / score gradients are
// rounded to the input dtype before the contractions that the reference
// performs in that dtype (universal_attention_autograd.py:159, :245, :251).
// These kernels serve the fp32 mode, odd shapes, and as a device-side
// cross-check of the tensor-core kernels; they are not the fast path.
//
// Mathematics per (key k, row q) of chunk i  (universal_attention_autograd.py:148-159):
//   g   = K_k . K_q
//   a   = relu(g)^(2/3) * src_k^(1/3) * dest_q^(1/3)
//   ell = log1p(-clamp(a, 0, 1-1e-6))            for q > k, else 0
//   C   = running sum of ell over q               (carry kept per key across row tiles)
//   S_r = K_k . Q_rq + (q < k ? -1e12 : C)
//   lse = logsumexp_k S_r ;  P = softmax_k S_r ;  out = sum_k P * V_k
#pragma once
#include "ua_common.cuh"

namespace ua {
namespace simt {

constexpr int kThreads = 128;

struct FwdParams {
  Shape s;
  const void *kc, *vc, *xq, *ssrc, *sdest;
  void* out;      // chunk-major (b,h,n,r,L,d)
  float* lse;     // (b,h,n,r,L)
  void* denom;    // (b,h,n,r,L) in T, may be null
  int rt;         // rows per tile
  int skip_masked_fill;
};

struct BwdParams {
  Shape s;
  const void *kc, *vc, *xq, *ssrc, *sdest;
  const void* g_out;    // chunk-major (b,h,n,r,L,d), T
  const void* g_denom;  // (b,h,n,r,L), fp32 or T
  int g_denom_is_f32;
  float *acc_dk, *acc_dv, *acc_dq, *acc_ds, *acc_dt;  // fp32 accumulators (zeroed by the host)
  float* carry;   // (b*h*n, L/rt, c) decay prefix at the start of each row tile
  int rt;
  int skip_masked;
  int masked_only;   // only the row tiles that lie wholly before the chunk (the others are another kernel's)
};

__device__ __forceinline__ float dot4(const float* a, const float* b, int D) {
  float acc = 0.f;
  for (int d = 0; d < D; d += 4) {
    float4 x = *reinterpret_cast<const float4*>(a + d);
    float4 y = *reinterpret_cast<const float4*>(b + d);
    acc = fmaf(x.x, y.x, acc);
    acc = fmaf(x.y, y.y, acc);
    acc = fmaf(x.z, y.z, acc);
    acc = fmaf(x.w, y.w, acc);
  }
  return acc;
}

// Storage of the chunk's own K_i / V_i tiles in shared memory: fp32 (default) or, for shapes whose
// fp32 tiles would not fit (chunk 256 x head_dim 128), the input's bf16.
template <typename S> struct KVS;
template <> struct KVS<float> {
  static constexpr int kPad = 4;
  static __device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ float ld1(const float* p) { return *p; }
  static __device__ __forceinline__ void st(float* p, float v) { *p = v; }
};
template <> struct KVS<__nv_bfloat16> {
  static constexpr int kPad = 8;
  static __device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
    const uint2 x = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&x.x), b = *reinterpret_cast<const __nv_bfloat162*>(&x.y);
    return make_float4(__bfloat162float(a.x), __bfloat162float(a.y), __bfloat162float(b.x), __bfloat162float(b.y));
  }
  static __device__ __forceinline__ float ld1(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

template <typename S>
__device__ __forceinline__ float dotk(const S* a, const float* b, int D) {
  float acc = 0.f;
  for (int d = 0; d < D; d += 4) {
    const float4 x = KVS<S>::ld4(a + d);
    const float4 y = *reinterpret_cast<const float4*>(b + d);
    acc = fmaf(x.x, y.x, acc);
    acc = fmaf(x.y, y.y, acc);
    acc = fmaf(x.z, y.z, acc);
    acc = fmaf(x.w, y.w, acc);
  }
  return acc;
}

template <typename T, typename S>
__device__ __forceinline__ void load_tile_k(S* dst, const T* src, int rows, int D, int DPK) {
  for (int e = threadIdx.x; e < rows * D; e += kThreads) {
    int rr = e / D, dd = e - rr * D;
    KVS<S>::st(dst + rr * DPK + dd, Num<T>::ld(src + e));
  }
}

__device__ __forceinline__ float pow23(float g) { return g > 0.f ? powf(g, 2.0f / 3.0f) : 0.f; }

__device__ __forceinline__ float log_retention(float a) {
  return log1pf(-fminf(fmaxf(a, 0.f), clamp_hi()));
}

// Copy a [rows][D] tile of T from global into padded fp32 shared memory.
template <typename T>
__device__ __forceinline__ void load_tile(float* dst, const T* src, int rows, int D, int DP) {
  for (int e = threadIdx.x; e < rows * D; e += kThreads) {
    int rr = e / D, dd = e - rr * D;
    dst[rr * DP + dd] = Num<T>::ld(src + e);
  }
}

// Column softmax over the C keys of sS[k][q] (stride RTP); one warp per column.
// Writes max to sM and sum(exp) to sL.
__device__ __forceinline__ void column_stats(const float* sS, float* sM, float* sL, int C, int RT, int RTP) {
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int q = warp; q < RT; q += kThreads / 32) {
    float m = -INFINITY;
    for (int k = lane; k < C; k += 32) m = fmaxf(m, sS[k * RTP + q]);
    for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float l = 0.f;
    for (int k = lane; k < C; k += 32) l += expf(sS[k * RTP + q] - m);
    for (int o = 16; o; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0) { sM[q] = m; sL[q] = l; }
  }
}

inline size_t kv_bytes(int C, int D, int elem) {      // the two [C][D + pad] tiles K_i, V_i, 16-byte aligned
  size_t b = (size_t)2 * C * (D + 16 / elem) * elem;
  return (b + 15) / 16 * 16;
}
inline size_t fwd_smem_bytes(int C, int D, int RT, int kv_elem = 4) {
  size_t DP = D + 4, RTP = RT + 1;
  return kv_bytes(C, D, kv_elem) + sizeof(float) * (2 * RT * DP + 2 * C * RTP + 2 * C + 3 * RT + D);
}

template <typename T, typename TG, typename S>
__global__ void __launch_bounds__(kThreads) fwd_kernel(FwdParams p) {
  extern __shared__ __align__(16) float smem[];
  const int C = p.s.C, D = p.s.D, L = p.s.L, N = p.s.N, R = p.s.R, RT = p.rt;
  const int DP = D + 4, RTP = RT + 1, DPK = D + KVS<S>::kPad;
  S* sKi = reinterpret_cast<S*>(smem);
  S* sVi = sKi + C * DPK;
  float* sKj = smem + ((size_t)2 * C * DPK * sizeof(S) + 15) / 16 * 4;
  float* sQ = sKj + RT * DP;
  float* sC = sQ + RT * DP;
  float* sS = sC + C * RTP;
  float* sS3 = sS + C * RTP;
  float* sCarry = sS3 + C;
  float* sT3 = sCarry + C;
  float* sM = sT3 + RT;
  float* sL = sM + RT;
  float* sVmean = sL + RT;

  const int BH = p.s.B * p.s.H;
  const int i = blockIdx.x / BH;            // heavy chunks (small i) are scheduled first
  const int bh = blockIdx.x - i * BH;
  const int tid = threadIdx.x;

  const T* kc = static_cast<const T*>(p.kc) + (size_t)bh * L * D;
  const T* vc = static_cast<const T*>(p.vc) + (size_t)bh * L * D;
  const T* xq = static_cast<const T*>(p.xq) + (size_t)bh * R * L * D;
  const TG* ss = static_cast<const TG*>(p.ssrc) + (size_t)bh * L;
  const TG* sd = static_cast<const TG*>(p.sdest) + (size_t)bh * L;
  const size_t chunk_id = (size_t)bh * N + i;
  T* out = static_cast<T*>(p.out) + chunk_id * R * L * D;
  float* lse = p.lse + chunk_id * R * L;
  T* denom = p.denom ? static_cast<T*>(p.denom) + chunk_id * R * L : nullptr;

  load_tile_k<T, S>(sKi, kc + (size_t)i * C * D, C, D, DPK);
  load_tile_k<T, S>(sVi, vc + (size_t)i * C * D, C, D, DPK);
  for (int k = tid; k < C; k += kThreads) {
    sS3[k] = cbrtf(Num<TG>::ld(ss + i * C + k));
    sCarry[k] = 0.f;
  }
  __syncthreads();
  // Value a fully masked row takes: softmax over C equal scores is 1/C per key
  // (rounded to T, as the reference rounds P), so out = sum_k rnd(1/C) * V_k.
  {
    const float w = Num<T>::rnd(1.0f / (float)C);
    for (int d = tid; d < D; d += kThreads) {
      float acc = 0.f;
      for (int k = 0; k < C; ++k) acc = fmaf(w, KVS<S>::ld1(sVi + k * DPK + d), acc);
      sVmean[d] = acc;
    }
  }
  __syncthreads();

  for (int j0 = 0; j0 < L; j0 += RT) {
    if (j0 + RT <= i * C) {
      // rows entirely before the chunk: every score is -1e12 (k.q is absorbed in fp32)
      if (!p.skip_masked_fill) {
        for (int r = 0; r < R; ++r) {
          for (int e = tid; e < RT * D; e += kThreads) {
            int q = e / D, d = e - q * D;
            Num<T>::st(out + ((size_t)r * L + j0 + q) * D + d, sVmean[d]);
          }
          for (int q = tid; q < RT; q += kThreads) {
            lse[(size_t)r * L + j0 + q] = mask_value();
            if (denom) Num<T>::st(denom + (size_t)r * L + j0 + q, mask_value());
          }
        }
      }
      continue;
    }
    load_tile<T>(sKj, kc + (size_t)j0 * D, RT, D, DP);
    for (int q = tid; q < RT; q += kThreads) sT3[q] = cbrtf(Num<TG>::ld(sd + j0 + q));
    __syncthreads();
    // decay prefix for this tile: thread <-> key, sequential over rows
    for (int k = tid; k < C; k += kThreads) {
      const int kg = i * C + k;
      const float carry = sCarry[k], s3 = sS3[k];
      float local = 0.f, c = carry;
      for (int q = 0; q < RT; ++q) {
        const int qg = j0 + q;
        float g = dotk<S>(sKi + k * DPK, sKj + q * DP, D);
        float ell = log_retention(pow23(g) * s3 * sT3[q]);
        if (qg <= kg) ell = 0.f;
        local += ell;
        c = local + carry;
        sC[k * RTP + q] = (qg < kg) ? mask_value() : c;
      }
      sCarry[k] = c;
    }
    __syncthreads();
    for (int r = 0; r < R; ++r) {
      load_tile<T>(sQ, xq + ((size_t)r * L + j0) * D, RT, D, DP);
      __syncthreads();
      for (int k = tid; k < C; k += kThreads)
        for (int q = 0; q < RT; ++q)
          sS[k * RTP + q] = dotk<S>(sKi + k * DPK, sQ + q * DP, D) + sC[k * RTP + q];
      __syncthreads();
      column_stats(sS, sM, sL, C, RT, RTP);
      __syncthreads();
      for (int k = tid; k < C; k += kThreads)
        for (int q = 0; q < RT; ++q)
          sS[k * RTP + q] = Num<T>::rnd(expf(sS[k * RTP + q] - sM[q]) / sL[q]);
      for (int q = tid; q < RT; q += kThreads) {
        float v = sM[q] + logf(sL[q]);
        lse[(size_t)r * L + j0 + q] = v;
        if (denom) Num<T>::st(denom + (size_t)r * L + j0 + q, v);
      }
      __syncthreads();
      // out[q][d] = sum_k P[k][q] V[k][d]
      const int D4 = D >> 2;
      for (int e = tid; e < RT * D4; e += kThreads) {
        const int d4 = e / RT, q = e - d4 * RT;     // lanes run over q: conflict-free P reads, broadcast V reads
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < C; ++k) {
          const float pk = sS[k * RTP + q];
          const float4 v = KVS<S>::ld4(sVi + k * DPK + d4 * 4);
          acc.x = fmaf(pk, v.x, acc.x); acc.y = fmaf(pk, v.y, acc.y);
          acc.z = fmaf(pk, v.z, acc.z); acc.w = fmaf(pk, v.w, acc.w);
        }
        T* o = out + ((size_t)r * L + j0 + q) * D + d4 * 4;
        Num<T>::st(o + 0, acc.x); Num<T>::st(o + 1, acc.y); Num<T>::st(o + 2, acc.z); Num<T>::st(o + 3, acc.w);
      }
      __syncthreads();
    }
  }
}

inline size_t bwd_smem_bytes(int C, int D, int RT, int kv_elem = 4) {
  size_t DP = D + 4, RTP = RT + 1;
  return kv_bytes(C, D, kv_elem) + sizeof(float) * (3 * RT * DP + 5 * C * RTP + 3 * C + 5 * RT);
}

// out[k][d4] (+)= sum_q A[k][q] * Bm[q][d]   for k < C; result added to global fp32 rows with atomics.
__device__ __forceinline__ void acc_rows_atomic(const float* sA, const float* sB, float* gdst, int C, int RT,
                                                int RTP, int D, int DP) {
  const int D4 = D >> 2;
  for (int e = threadIdx.x; e < C * D4; e += kThreads) {
    const int k = e / D4, d4 = e - k * D4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int q = 0; q < RT; ++q) {
      const float a = sA[k * RTP + q];
      const float4 b = *reinterpret_cast<const float4*>(sB + q * DP + d4 * 4);
      acc.x = fmaf(a, b.x, acc.x); acc.y = fmaf(a, b.y, acc.y);
      acc.z = fmaf(a, b.z, acc.z); acc.w = fmaf(a, b.w, acc.w);
    }
    float* o = gdst + (size_t)k * D + d4 * 4;
    atomicAdd(o + 0, acc.x); atomicAdd(o + 1, acc.y); atomicAdd(o + 2, acc.z); atomicAdd(o + 3, acc.w);
  }
}

// out[q][d4] += sum_k A[k][q] * Bm[k][d]   for q < RT
template <typename S>
__device__ __forceinline__ void acc_cols_atomic(const float* sA, const S* sB, float* gdst, int C, int RT,
                                                int RTP, int D, int DP) {
  const int D4 = D >> 2;
  for (int e = threadIdx.x; e < RT * D4; e += kThreads) {
    const int d4 = e / RT, q = e - d4 * RT;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < C; ++k) {
      const float a = sA[k * RTP + q];
      const float4 b = KVS<S>::ld4(sB + k * DP + d4 * 4);
      acc.x = fmaf(a, b.x, acc.x); acc.y = fmaf(a, b.y, acc.y);
      acc.z = fmaf(a, b.z, acc.z); acc.w = fmaf(a, b.w, acc.w);
    }
    float* o = gdst + (size_t)q * D + d4 * 4;
    atomicAdd(o + 0, acc.x); atomicAdd(o + 1, acc.y); atomicAdd(o + 2, acc.z); atomicAdd(o + 3, acc.w);
  }
}

// Backward.  Pass 1 walks the row tiles upwards and records the decay prefix at
// the start of every tile (recomputed, not saved by the forward); pass 2 walks
// them downwards so that the reverse cumulative sum of the decay gradient can
// be carried per key (universal_attention_autograd.py:232-259).
template <typename T, typename TG, typename S>
__global__ void __launch_bounds__(kThreads) bwd_kernel(BwdParams p) {
  extern __shared__ __align__(16) float smem[];
  const int C = p.s.C, D = p.s.D, L = p.s.L, N = p.s.N, R = p.s.R, RT = p.rt;
  const int DP = D + 4, RTP = RT + 1, NT = L / RT, DPK = D + KVS<S>::kPad;
  S* sKi = reinterpret_cast<S*>(smem);
  S* sVi = sKi + C * DPK;
  float* sKj = smem + ((size_t)2 * C * DPK * sizeof(S) + 15) / 16 * 4;
  float* sQ = sKj + RT * DP;
  float* sGo = sQ + RT * DP;
  float* sG = sGo + RT * DP;      // [C][RTP] key-key Gram tile
  float* sC = sG + C * RTP;       // decay prefix (masked)
  float* sP = sC + C * RTP;       // scores -> probabilities
  float* sdS = sP + C * RTP;      // dP -> dS -> dG
  float* sDC = sdS + C * RTP;     // sum over r of dS (fp32)
  float* sS3 = sDC + C * RTP;
  float* sCarry = sS3 + C;
  float* sSuf = sCarry + C;
  float* sT3 = sSuf + C;
  float* sM = sT3 + RT;
  float* sL = sM + RT;
  float* sGd = sL + RT;
  float* sDt = sGd + RT;

  const int BH = p.s.B * p.s.H;
  const int i = blockIdx.x / BH;
  const int bh = blockIdx.x - i * BH;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  const T* kc = static_cast<const T*>(p.kc) + (size_t)bh * L * D;
  const T* vc = static_cast<const T*>(p.vc) + (size_t)bh * L * D;
  const T* xq = static_cast<const T*>(p.xq) + (size_t)bh * R * L * D;
  const TG* ss = static_cast<const TG*>(p.ssrc) + (size_t)bh * L;
  const TG* sd = static_cast<const TG*>(p.sdest) + (size_t)bh * L;
  const size_t chunk_id = (size_t)bh * N + i;
  const T* g_out = static_cast<const T*>(p.g_out) + chunk_id * R * L * D;
  const size_t gd_off = chunk_id * R * L;
  float* carry_tab = p.carry + chunk_id * NT * C;
  float* acc_dk = p.acc_dk + (size_t)bh * L * D;
  float* acc_dv = p.acc_dv + (size_t)bh * L * D;
  float* acc_dq = p.acc_dq + (size_t)bh * R * L * D;
  float* acc_ds = p.acc_ds + (size_t)bh * L;
  float* acc_dt = p.acc_dt + (size_t)bh * L;

  load_tile_k<T, S>(sKi, kc + (size_t)i * C * D, C, D, DPK);
  load_tile_k<T, S>(sVi, vc + (size_t)i * C * D, C, D, DPK);
  for (int k = tid; k < C; k += kThreads) {
    sS3[k] = cbrtf(Num<TG>::ld(ss + i * C + k));
    sCarry[k] = 0.f;
    sSuf[k] = 0.f;
  }
  __syncthreads();

  // ---- pass 1: decay prefix at the start of every row tile --------------------
  for (int jt = 0; jt < NT && !p.masked_only; ++jt) {
    const int j0 = jt * RT;
    if (j0 + RT <= i * C) {
      for (int k = tid; k < C; k += kThreads) carry_tab[(size_t)jt * C + k] = 0.f;
      continue;
    }
    load_tile<T>(sKj, kc + (size_t)j0 * D, RT, D, DP);
    for (int q = tid; q < RT; q += kThreads) sT3[q] = cbrtf(Num<TG>::ld(sd + j0 + q));
    __syncthreads();
    for (int k = tid; k < C; k += kThreads) {
      const int kg = i * C + k;
      const float carry = sCarry[k], s3 = sS3[k];
      carry_tab[(size_t)jt * C + k] = carry;
      float local = 0.f;
      for (int q = 0; q < RT; ++q) {
        float g = dotk<S>(sKi + k * DPK, sKj + q * DP, D);
        float ell = log_retention(pow23(g) * s3 * sT3[q]);
        if (j0 + q <= kg) ell = 0.f;
        local += ell;
      }
      sCarry[k] = local + carry;
    }
    __syncthreads();
  }

  // ---- pass 2: gradients, row tiles in descending order -----------------------
  for (int jt = NT - 1; jt >= 0; --jt) {
    const int j0 = jt * RT;
    const bool fully_masked = (j0 + RT <= i * C);
    if (fully_masked && p.skip_masked) break;     // every remaining tile is masked too
    if (!fully_masked && p.masked_only) continue;
    load_tile<T>(sKj, kc + (size_t)j0 * D, RT, D, DP);
    for (int q = tid; q < RT; q += kThreads) {
      sT3[q] = cbrtf(Num<TG>::ld(sd + j0 + q));
      sDt[q] = 0.f;
    }
    __syncthreads();
    // recompute Gram tile and decay prefix
    for (int k = tid; k < C; k += kThreads) {
      const int kg = i * C + k;
      const float carry = fully_masked ? 0.f : carry_tab[(size_t)jt * C + k], s3 = sS3[k];
      float local = 0.f;
      for (int q = 0; q < RT; ++q) {
        const int qg = j0 + q;
        float g = dotk<S>(sKi + k * DPK, sKj + q * DP, D);
        sG[k * RTP + q] = g;
        float ell = log_retention(pow23(g) * s3 * sT3[q]);
        if (qg <= kg) ell = 0.f;
        local += ell;
        sC[k * RTP + q] = (qg < kg) ? mask_value() : (local + carry);
        sDC[k * RTP + q] = 0.f;
      }
    }
    __syncthreads();

    for (int r = 0; r < R; ++r) {
      load_tile<T>(sQ, xq + ((size_t)r * L + j0) * D, RT, D, DP);
      load_tile<T>(sGo, g_out + ((size_t)r * L + j0) * D, RT, D, DP);
      for (int q = tid; q < RT; q += kThreads) {
        size_t o = gd_off + (size_t)r * L + j0 + q;
        sGd[q] = p.g_denom_is_f32 ? static_cast<const float*>(p.g_denom)[o]
                                  : Num<T>::ld(static_cast<const T*>(p.g_denom) + o);
      }
      __syncthreads();
      for (int k = tid; k < C; k += kThreads)
        for (int q = 0; q < RT; ++q) {
          sP[k * RTP + q] = dotk<S>(sKi + k * DPK, sQ + q * DP, D) + sC[k * RTP + q];
          sdS[k * RTP + q] = dotk<S>(sVi + k * DPK, sGo + q * DP, D);        // dP
        }
      __syncthreads();
      column_stats(sP, sM, sL, C, RT, RTP);
      __syncthreads();
      // per column: P, delta = sum_k P dP, dS = P (dP - delta + g_denom)
      for (int q = warp; q < RT; q += kThreads / 32) {
        const float m = sM[q], linv = 1.0f / sL[q];
        float delta = 0.f;
        for (int k = lane; k < C; k += 32) {
          float pr = expf(sP[k * RTP + q] - m) * linv;
          sP[k * RTP + q] = pr;
          delta = fmaf(pr, sdS[k * RTP + q], delta);
        }
        for (int o = 16; o; o >>= 1) delta += __shfl_xor_sync(0xffffffffu, delta, o);
        const float gd = sGd[q];
        for (int k = lane; k < C; k += 32) {
          float pr = sP[k * RTP + q];
          float ds = pr * (sdS[k * RTP + q] - delta) + pr * gd;
          sDC[k * RTP + q] += ds;
          sdS[k * RTP + q] = Num<T>::rnd(ds);
          sP[k * RTP + q] = Num<T>::rnd(pr);
        }
      }
      __syncthreads();
      acc_rows_atomic(sP, sGo, acc_dv + (size_t)i * C * D, C, RT, RTP, D, DP);                 // dV_i += P  . g_out
      acc_rows_atomic(sdS, sQ, acc_dk + (size_t)i * C * D, C, RT, RTP, D, DP);                 // dK_i += dS . Q
      acc_cols_atomic<S>(sdS, sKi, acc_dq + ((size_t)r * L + j0) * D, C, RT, RTP, D, DPK);         // dQ_j += dS^T . K_i
      __syncthreads();
    }

    // decay path: reverse running sum over rows with a per-key suffix carry
    for (int k = tid; k < C; k += kThreads) {
      const int kg = i * C + k;
      const float suffix = sSuf[k], s3 = sS3[k];
      float run = 0.f, dsrc = 0.f, first = 0.f;
      for (int q = RT - 1; q >= 0; --q) {
        const int qg = j0 + q;
        run += sDC[k * RTP + q];
        float dl = run + suffix;
        if (qg <= kg) dl = 0.f;
        if (q == 0) first = dl;
        const float g = sG[k * RTP + q];
        const float pw = pow23(g);
        const float t3 = sT3[q];
        const float a = pw * s3 * t3;
        float da = dl / (fminf(fmaxf(a, clamp_lo_bwd()), clamp_hi()) - 1.0f);
        if (!(a <= clamp_hi())) da = 0.f;
        const float dstat = da * pw;
        dsrc = fmaf(dstat, t3, dsrc);
        sP[k * RTP + q] = dstat * s3;                                    // summed over keys below -> d dest
        float dg = Num<T>::rnd(da * s3 * t3);
        dg = (g > 0.f) ? dg * (2.0f / 3.0f) * powf(fabsf(g) + 1e-9f, -1.0f / 3.0f) : 0.f;
        sdS[k * RTP + q] = Num<T>::rnd(dg);
      }
      sSuf[k] = first;
      if (dsrc != 0.f) atomicAdd(acc_ds + kg, dsrc / (3.0f * s3 * s3));
    }
    __syncthreads();
    for (int q = warp; q < RT; q += kThreads / 32) {
      float acc = 0.f;
      for (int k = lane; k < C; k += 32) acc += sP[k * RTP + q];
      for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lane == 0 && acc != 0.f) atomicAdd(acc_dt + j0 + q, acc / (3.0f * sT3[q] * sT3[q]));
    }
    acc_cols_atomic<S>(sdS, sKi, acc_dk + (size_t)j0 * D, C, RT, RTP, D, DPK);                     // dK_j += dG^T . K_i
    acc_rows_atomic(sdS, sKj, acc_dk + (size_t)i * C * D, C, RT, RTP, D, DP);                  // dK_i += dG . K_j
    __syncthreads();
  }
}

// fp32 accumulator -> output dtype
template <typename T>
__global__ void convert_kernel(const float* __restrict__ src, T* __restrict__ dst, size_t n) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; idx < n; idx += stride) Num<T>::st(dst + idx, src[idx]);
}

// ... eight elements per thread and step (two 16-byte loads, one 16- or 32-byte store); n8 = n / 8, both pointers 16-byte aligned
template <typename T>
__global__ void convert8_kernel(const float4* __restrict__ src, T* __restrict__ dst, size_t n8) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; idx < n8; idx += stride) {
    const float4 a = src[2 * idx], b = src[2 * idx + 1];
    if (sizeof(T) == 2) {
      __nv_bfloat162 h0 = __floats2bfloat162_rn(a.x, a.y), h1 = __floats2bfloat162_rn(a.z, a.w);
      __nv_bfloat162 h2 = __floats2bfloat162_rn(b.x, b.y), h3 = __floats2bfloat162_rn(b.z, b.w);
      reinterpret_cast<uint4*>(dst)[idx] = make_uint4(*reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1),
                                                      *reinterpret_cast<uint32_t*>(&h2), *reinterpret_cast<uint32_t*>(&h3));
    } else {
      reinterpret_cast<float4*>(dst)[2 * idx] = a;
      reinterpret_cast<float4*>(dst)[2 * idx + 1] = b;
    }
  }
}

}  // namespace simt
}  // namespace ua
