// HBM-bound helper kernels: layout conversion between chunk-major storage and
// the reference's key-chunk-innermost tensors, and the merge over key chunks
// (SMVecMatMul, universal_attention_autograd.py:278-297).
#pragma once
#include "ua_common.cuh"

namespace ua {
namespace aux {

// Batched transpose.  For every batch index g (= (bh, r)):
//   to_reference:  dst[(g*X + x)*N + n] = src[((bh*N + n)*R + r)*X + x]
//   else        :  dst[((bh*N + n)*R + r)*X + x] = src[(g*X + x)*N + n]
// with X = L*inner.  32x32 shared-memory tiles keep both sides coalesced.
template <typename E>
__global__ void __launch_bounds__(256) relayout_kernel(const E* __restrict__ src, E* __restrict__ dst, int N, int R,
                                                       long long X, int to_reference) {
  __shared__ E tile[32][33];
  const int g = blockIdx.z;
  const int bh = g / R, r = g - bh * R;
  const long long x0 = (long long)blockIdx.x * 32;
  const int n0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
  if (to_reference) {
    for (int yy = ty; yy < 32; yy += 8) {
      int n = n0 + yy;
      long long x = x0 + tx;
      if (n < N && x < X) tile[yy][tx] = src[(((long long)bh * N + n) * R + r) * X + x];
    }
    __syncthreads();
    for (int yy = ty; yy < 32; yy += 8) {
      long long x = x0 + yy;
      int n = n0 + tx;
      if (n < N && x < X) dst[((long long)g * X + x) * N + n] = tile[tx][yy];
    }
  } else {
    for (int yy = ty; yy < 32; yy += 8) {
      long long x = x0 + yy;
      int n = n0 + tx;
      if (n < N && x < X) tile[yy][tx] = src[((long long)g * X + x) * N + n];
    }
    __syncthreads();
    for (int yy = ty; yy < 32; yy += 8) {
      int n = n0 + yy;
      long long x = x0 + tx;
      if (n < N && x < X) dst[(((long long)bh * N + n) * R + r) * X + x] = tile[tx][yy];
    }
  }
}

// ---- merge over key chunks (SMVecMatMul) -----------------------------------------
// One group of TPR = D * sizeof(T) / 16 threads per output row (b,h,r,l); every thread owns
// one 16-byte slice of the row (8 bf16 or 4 floats), so a warp reads whole contiguous rows of
// out_cm.  Chunks whose softmax weight is exactly zero (rows before a key chunk have
// lse = -1e12) are never read; on B4 H8 L4096 that halves the traffic.
constexpr int kMergeThreads = 256;

template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int kN = 4;
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int kN = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    const uint4 x = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
      v[2 * i] = __bfloat162float(h.x);
      v[2 * i + 1] = __bfloat162float(h.y);
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

template <int TPR>
__device__ __forceinline__ float group_max(float v) {
#pragma unroll
  for (int o = TPR / 2; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
template <int TPR>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = TPR / 2; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// row statistics of the softmax over chunks: max and 1 / sum exp
template <int TPR>
__device__ __forceinline__ void merge_row_stats(const float* lse_row, size_t nstride, int N, int sub, float& m, float& zinv) {
  float mm = -INFINITY;
  for (int n = sub; n < N; n += TPR) mm = fmaxf(mm, lse_row[(size_t)n * nstride]);
  m = group_max<TPR>(mm);
  float z = 0.f;
  for (int n = sub; n < N; n += TPR) z += expf(lse_row[(size_t)n * nstride] - m);
  zinv = 1.0f / group_sum<TPR>(z);
}

// merged[row][d] = sum_n softmax_n(lse[n][row]) * out_cm[n][row][d]
template <typename T, int TPR>
__global__ void __launch_bounds__(kMergeThreads) merge_fwd_kernel(const T* __restrict__ out_cm, const float* __restrict__ lse_cm,
                                                                  T* __restrict__ merged, float* __restrict__ row_lse,
                                                                  long long rows, int N, int R, int L) {
  constexpr int kN = Vec16<T>::kN;
  constexpr int D = TPR * kN;
  const long long row = (long long)blockIdx.x * (kMergeThreads / TPR) + threadIdx.x / TPR;
  const int sub = threadIdx.x % TPR;
  const bool live = row < rows;
  const long long rr = live ? row : rows - 1;          // keep whole warps in the shuffles
  const int l = (int)(rr % L);
  const long long gr = rr / L;
  const int r = (int)(gr % R);
  const long long bh = gr / R;
  const size_t nstride = (size_t)R * L;
  const size_t base = ((size_t)bh * N * R + r) * L + l;
  float m, zinv;
  merge_row_stats<TPR>(lse_cm + base, nstride, N, sub, m, zinv);
  float acc[kN];
#pragma unroll
  for (int i = 0; i < kN; ++i) acc[i] = 0.f;
  for (int n = 0; n < N; ++n) {
    const float w = expf(lse_cm[base + (size_t)n * nstride] - m) * zinv;
    if (w != 0.f) {
      float v[kN];
      Vec16<T>::load(out_cm + (base + (size_t)n * nstride) * D + sub * kN, v);
#pragma unroll
      for (int i = 0; i < kN; ++i) acc[i] = fmaf(w, v[i], acc[i]);
    }
  }
  if (live) Vec16<T>::store(merged + (size_t)row * D + sub * kN, acc);
  if (live && sub == 0 && row_lse) row_lse[row] = m - logf(zinv);      // log-sum-exp of the row over all key chunks
}

// out[row] = a[row] . b[row] over D = TPR * kN elements (the delta = g . merged of the merged backward)
template <typename T, int TPR>
__global__ void __launch_bounds__(kMergeThreads) row_dot_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                                                float* __restrict__ out, long long rows) {
  constexpr int kN = Vec16<T>::kN;
  constexpr int D = TPR * kN;
  const long long row = (long long)blockIdx.x * (kMergeThreads / TPR) + threadIdx.x / TPR;
  const int sub = threadIdx.x % TPR;
  const bool live = row < rows;
  const long long rr = live ? row : rows - 1;
  float x[kN], y[kN];
  Vec16<T>::load(a + (size_t)rr * D + sub * kN, x);
  Vec16<T>::load(b + (size_t)rr * D + sub * kN, y);
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < kN; ++i) acc = fmaf(x[i], y[i], acc);
  acc = group_sum<TPR>(acc);
  if (live && sub == 0) out[row] = acc;
}

// Backward of the merge: g_out_cm[n][row][:] = g[row][:] w_n ; g_lse[n][row] = (s_n - sum_m s_m w_m) w_n,
// s_n = g[row] . out_cm[n][row].  With skip_masked, the (row, chunk) blocks with row < n * chunk (rows before
// the key chunk, whose weight is exactly zero) are not written: the caller promises not to read them.
template <typename T, int TPR>
__global__ void __launch_bounds__(kMergeThreads) merge_bwd_kernel(const T* __restrict__ out_cm, const float* __restrict__ lse_cm,
                                                                  const T* __restrict__ g_merged, T* __restrict__ g_out_cm,
                                                                  float* __restrict__ g_lse_cm, long long rows, int N, int R,
                                                                  int L, int skip_masked) {
  constexpr int kN = Vec16<T>::kN;
  constexpr int D = TPR * kN;
  const long long row = (long long)blockIdx.x * (kMergeThreads / TPR) + threadIdx.x / TPR;
  const int sub = threadIdx.x % TPR;
  const bool live = row < rows;
  const long long rr = live ? row : rows - 1;
  const int l = (int)(rr % L);
  const long long gr = rr / L;
  const int r = (int)(gr % R);
  const long long bh = gr / R;
  const size_t nstride = (size_t)R * L;
  const size_t base = ((size_t)bh * N * R + r) * L + l;
  const int chunk = L / N;
  float m, zinv;
  merge_row_stats<TPR>(lse_cm + base, nstride, N, sub, m, zinv);
  float g[kN];
  Vec16<T>::load(g_merged + (size_t)rr * D + sub * kN, g);
  float t = 0.f;
  for (int n = 0; n < N; ++n) {
    const size_t idx = base + (size_t)n * nstride;
    const float w = expf(lse_cm[idx] - m) * zinv;
    float s = 0.f;
    if (w != 0.f) {
      float v[kN], o[kN];
      Vec16<T>::load(out_cm + idx * D + sub * kN, v);
#pragma unroll
      for (int i = 0; i < kN; ++i) {
        s = fmaf(g[i], v[i], s);
        o[i] = g[i] * w;
      }
      if (live) Vec16<T>::store(g_out_cm + idx * D + sub * kN, o);
    } else if (!(skip_masked && l < n * chunk) && live) {
      float o[kN];
#pragma unroll
      for (int i = 0; i < kN; ++i) o[i] = 0.f;
      Vec16<T>::store(g_out_cm + idx * D + sub * kN, o);
    }
    s = group_sum<TPR>(s);
    t = fmaf(s, w, t);
    if (live && sub == 0 && !(skip_masked && l < n * chunk)) g_lse_cm[idx] = s;     // parked; finished below by the same thread
  }
  if (live && sub == 0) {
    for (int n = 0; n < N; ++n) {
      const size_t idx = base + (size_t)n * nstride;
      const float w = expf(lse_cm[idx] - m) * zinv;
      if (!(skip_masked && l < n * chunk)) g_lse_cm[idx] = (g_lse_cm[idx] - t) * w;
    }
  }
}

// ---- input prologue -----------------------------------------------------------------
// The model hands over projections in token-major order: query_state (b,s,n,d), key_state / value_state (b,s,n_kv,d)
// and gate logits (b,s,2,n_kv).  The operator wants head-major tensors: xq (b,n_kv,rep,s,d) (query head kv*rep + r),
// kc / vc (b,n_kv,s,d), static_src / static_dest (b,n_kv,s) (the reference's driver does this with transposes and
// views, main.py:24-31).  One pass does the transposes and, on request, the two things a model applies on the way
// (Universal_Attention/triton/_debug.py:470-475): keys divided by (|k| + 1e-6) and gates through a sigmoid.
// One group of TPR threads per row of d elements; rows = b * s * (n + 2 n_kv).
struct PrepDims {
  int b, s, n, n_kv, normalize_keys, sigmoid_gates;
};

template <typename T, int TPR>
__global__ void __launch_bounds__(kMergeThreads) prepare_fwd_kernel(PrepDims pd, const T* __restrict__ qs, const T* __restrict__ ks,
                                                                    const T* __restrict__ vs, T* __restrict__ xq, T* __restrict__ kc,
                                                                    T* __restrict__ vc, float* __restrict__ key_norm) {
  constexpr int kN = Vec16<T>::kN;
  constexpr int D = TPR * kN;
  const int heads = pd.n + 2 * pd.n_kv;
  const long long rows = (long long)pd.b * pd.s * heads;
  const long long row = (long long)blockIdx.x * (kMergeThreads / TPR) + threadIdx.x / TPR;
  const int sub = threadIdx.x % TPR;
  const bool live = row < rows;
  const long long rr = live ? row : rows - 1;
  const int hh = (int)(rr % heads);
  const long long tok = rr / heads;                 // bb * s + ss
  const int ss = (int)(tok % pd.s);
  const long long bb = tok / pd.s;
  const bool is_q = hh < pd.n, is_k = !is_q && hh < pd.n + pd.n_kv;
  const int kv = is_q ? 0 : (is_k ? hh - pd.n : hh - pd.n - pd.n_kv);
  const size_t hm = ((size_t)bb * pd.n_kv + kv) * pd.s + ss;          // head-major row of a key / value
  float v[kN];
  if (is_q) Vec16<T>::load(qs + ((size_t)tok * pd.n + hh) * D + sub * kN, v);
  else Vec16<T>::load((is_k ? ks : vs) + ((size_t)tok * pd.n_kv + kv) * D + sub * kN, v);
  float ssq = 0.f;
#pragma unroll
  for (int i = 0; i < kN; ++i) ssq = fmaf(v[i], v[i], ssq);
  ssq = group_sum<TPR>(ssq);                        // every lane takes part, whatever kind of row its group holds
  const float nrm = sqrtf(ssq);
  if (is_k && pd.normalize_keys) {
    const float inv = 1.0f / (nrm + 1e-6f);
#pragma unroll
    for (int i = 0; i < kN; ++i) v[i] *= inv;
  }
  if (!live) return;
  if (is_q) {
    Vec16<T>::store(xq + (((size_t)bb * pd.n + hh) * pd.s + ss) * D + sub * kN, v);
  } else {
    Vec16<T>::store((is_k ? kc : vc) + hm * D + sub * kN, v);
    if (is_k && sub == 0 && key_norm) key_norm[hm] = nrm;
  }
}

// gates: one thread per (b, s, which, kv)
template <typename T>
__global__ void prepare_gates_kernel(PrepDims pd, const T* __restrict__ gs, T* __restrict__ ssrc, T* __restrict__ sdest, int backward,
                                     const T* __restrict__ g_src, const T* __restrict__ g_dest, T* __restrict__ d_gs) {
  const long long total = (long long)pd.b * pd.s * 2 * pd.n_kv;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    const int kv = (int)(e % pd.n_kv);
    const int which = (int)((e / pd.n_kv) % 2);
    const long long tok = e / (2 * pd.n_kv);
    const int ss = (int)(tok % pd.s);
    const long long bb = tok / pd.s;
    const size_t dst = ((size_t)bb * pd.n_kv + kv) * pd.s + ss;
    if (!backward) {
      float x = Num<T>::ld(gs + e);
      if (pd.sigmoid_gates) x = 1.0f / (1.0f + __expf(-x));
      Num<T>::st((which ? sdest : ssrc) + dst, x);
    } else {
      // ssrc / sdest hold the forward's outputs (the gate values), g_* their gradients
      const float gate = Num<T>::ld((which ? sdest : ssrc) + dst);
      float g = Num<T>::ld((which ? g_dest : g_src) + dst);
      if (pd.sigmoid_gates) g *= gate * (1.0f - gate);
      Num<T>::st(d_gs + e, g);
    }
  }
}

// backward of prepare_fwd_kernel: gradients flow back along the same row mapping; key rows pass through the
// derivative of k / (|k| + eps):  dk = g / (|k| + eps) - khat (g . khat) / |k|
template <typename T, int TPR>
__global__ void __launch_bounds__(kMergeThreads) prepare_bwd_kernel(PrepDims pd, const T* __restrict__ g_xq, const T* __restrict__ g_kc,
                                                                    const T* __restrict__ g_vc, const T* __restrict__ kc,
                                                                    const float* __restrict__ key_norm, T* __restrict__ d_qs,
                                                                    T* __restrict__ d_ks, T* __restrict__ d_vs) {
  constexpr int kN = Vec16<T>::kN;
  constexpr int D = TPR * kN;
  const int heads = pd.n + 2 * pd.n_kv;
  const long long rows = (long long)pd.b * pd.s * heads;
  const long long row = (long long)blockIdx.x * (kMergeThreads / TPR) + threadIdx.x / TPR;
  const int sub = threadIdx.x % TPR;
  const bool live = row < rows;
  const long long rr = live ? row : rows - 1;
  const int hh = (int)(rr % heads);
  const long long tok = rr / heads;
  const int ss = (int)(tok % pd.s);
  const long long bb = tok / pd.s;
  const bool is_q = hh < pd.n, is_k = !is_q && hh < pd.n + pd.n_kv;
  const int kv = is_q ? 0 : (is_k ? hh - pd.n : hh - pd.n - pd.n_kv);
  const size_t hm = ((size_t)bb * pd.n_kv + kv) * pd.s + ss;
  float g[kN], kh[kN];
  if (is_q) Vec16<T>::load(g_xq + (((size_t)bb * pd.n + hh) * pd.s + ss) * D + sub * kN, g);
  else Vec16<T>::load((is_k ? g_kc : g_vc) + hm * D + sub * kN, g);
  float dot = 0.f;
  const bool norm = is_k && pd.normalize_keys;
  if (norm) {
    Vec16<T>::load(kc + hm * D + sub * kN, kh);
#pragma unroll
    for (int i = 0; i < kN; ++i) dot = fmaf(g[i], kh[i], dot);
  }
  dot = group_sum<TPR>(dot);
  if (norm) {
    const float nrm = key_norm[hm];
    const float a = 1.0f / (nrm + 1e-6f), c = nrm > 0.f ? dot / nrm : 0.f;
#pragma unroll
    for (int i = 0; i < kN; ++i) g[i] = g[i] * a - kh[i] * c;
  }
  if (!live) return;
  if (is_q) Vec16<T>::store(d_qs + ((size_t)tok * pd.n + hh) * D + sub * kN, g);
  else Vec16<T>::store((is_k ? d_ks : d_vs) + ((size_t)tok * pd.n_kv + kv) * D + sub * kN, g);
}

}  // namespace aux
}  // namespace ua
