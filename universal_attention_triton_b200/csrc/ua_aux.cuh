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

}  // namespace aux
}  // namespace ua
