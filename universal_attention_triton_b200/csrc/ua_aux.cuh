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

constexpr int kMergeWarps = 4;

// merged[row][d] = sum_n softmax_n(lse[n][row]) * out_cm[n][row][d]; one warp per row.
template <typename T>
__global__ void __launch_bounds__(kMergeWarps * 32) merge_fwd_kernel(const T* __restrict__ out_cm,
                                                                     const float* __restrict__ lse_cm,
                                                                     T* __restrict__ merged, int BH, int N, int R,
                                                                     int L, int D) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long rows = (long long)BH * R * L;
  for (long long row = (long long)blockIdx.x * kMergeWarps + warp; row < rows; row += (long long)gridDim.x * kMergeWarps) {
    const int l = (int)(row % L);
    const long long gr = row / L;
    const int r = (int)(gr % R);
    const long long bh = gr / R;
    const size_t base = ((size_t)bh * N * R + r) * L + l;      // + n*R*L
    float m = -INFINITY;
    for (int n = 0; n < N; ++n) m = fmaxf(m, lse_cm[base + (size_t)n * R * L]);
    float z = 0.f;
    for (int n = 0; n < N; ++n) z += expf(lse_cm[base + (size_t)n * R * L] - m);
    const float zinv = 1.0f / z;
    for (int d = lane; d < D; d += 32) {
      float acc = 0.f;
      for (int n = 0; n < N; ++n) {
        const float w = expf(lse_cm[base + (size_t)n * R * L] - m) * zinv;
        if (w != 0.f) acc = fmaf(w, Num<T>::ld(out_cm + (base + (size_t)n * R * L) * D + d), acc);
      }
      Num<T>::st(merged + (size_t)row * D + d, acc);
    }
  }
}

// Backward of the merge; one warp per row.  Dynamic shared memory: kMergeWarps * 2 * N floats.
template <typename T>
__global__ void __launch_bounds__(kMergeWarps * 32) merge_bwd_kernel(const T* __restrict__ out_cm,
                                                                     const float* __restrict__ lse_cm,
                                                                     const T* __restrict__ g_merged,
                                                                     T* __restrict__ g_out_cm,
                                                                     float* __restrict__ g_lse_cm, int BH, int N,
                                                                     int R, int L, int D) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* w = sm + (size_t)warp * 2 * N;
  float* s = w + N;
  const long long rows = (long long)BH * R * L;
  for (long long row = (long long)blockIdx.x * kMergeWarps + warp; row < rows; row += (long long)gridDim.x * kMergeWarps) {
    const int l = (int)(row % L);
    const long long gr = row / L;
    const int r = (int)(gr % R);
    const long long bh = gr / R;
    const size_t base = ((size_t)bh * N * R + r) * L + l;
    float m = -INFINITY;
    for (int n = lane; n < N; n += 32) m = fmaxf(m, lse_cm[base + (size_t)n * R * L]);
    for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float z = 0.f;
    for (int n = lane; n < N; n += 32) {
      float e = expf(lse_cm[base + (size_t)n * R * L] - m);
      w[n] = e;
      z += e;
    }
    for (int o = 16; o; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
    __syncwarp();
    const float zinv = 1.0f / z;
    float t = 0.f;                                            // sum_n s_n w_n
    for (int n = 0; n < N; ++n) {
      const float wn = w[n] * zinv;
      float part = 0.f;
      const size_t o = (base + (size_t)n * R * L) * D;
      for (int d = lane; d < D; d += 32) {
        const float g = Num<T>::ld(g_merged + (size_t)row * D + d);
        Num<T>::st(g_out_cm + o + d, g * wn);
        if (wn != 0.f) part = fmaf(g, Num<T>::ld(out_cm + o + d), part);
      }
      for (int oo = 16; oo; oo >>= 1) part += __shfl_xor_sync(0xffffffffu, part, oo);
      if (lane == 0) s[n] = part;
      t = fmaf(part, wn, t);
    }
    __syncwarp();
    for (int n = lane; n < N; n += 32) {
      const float wn = w[n] * zinv;
      g_lse_cm[base + (size_t)n * R * L] = (s[n] - t) * wn;
    }
    __syncwarp();
  }
}

}  // namespace aux
}  // namespace ua
