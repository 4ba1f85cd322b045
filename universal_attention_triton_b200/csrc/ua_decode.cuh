// Incremental (decode) step of the Universal Attention operator: ONE new row against cached keys and values.
//
// The operator's forward (universal_attention_autograd.py:9-38, row-chunked form :104-163) needs, for a new row t and
// every earlier key k, the decay prefix  C[k, t] = sum_{k < q <= t} log1p(-affinity(k, q)).  That prefix is a running
// sum per key, so a serving loop keeps it as state next to the key / value caches:
//     state[k] <- state[k] + log1p(-clamp(relu(k_k . k_t)^(2/3) src_k^(1/3) dest_t^(1/3)))     for k < t
//     state[t]  = 0
// and the new row's outputs are, per key chunk i of `chunk` keys (only the chunks that hold keys <= t exist),
//     lse[r][i] = logsumexp_k (k_k . q_r + state[k]),     out[r][i][:] = sum_k softmax_k(...) v_k
// exactly row t of the full forward.  O(t * d) work and cache reads per step: HBM-bound, one block per (b, h, chunk),
// one thread per key of the chunk, fp32 CUDA-core arithmetic (no tile is large enough for the tensor cores).
#pragma once
#include "ua_aux.cuh"
#include "ua_common.cuh"

namespace ua {
namespace decode {

struct Params {
  int BH, R, D, C;        // (batch * kv heads), query heads per kv head, head_dim, keys per chunk (= threads per block)
  int Lcap;               // rows of the caches per (b, h)
  int t;                  // position of the new row; keys 0..t are in the caches
  const void* kcache;     // (BH, Lcap, D)
  const void* vcache;     // (BH, Lcap, D)
  const void* src;        // (BH, Lcap) gate of the keys
  const void* q;          // (BH, R, D) queries of the new row
  const void* dest;       // (BH) gate of the new row
  float* state;           // (BH, Lcap) decay prefix, updated in place
  void* out;              // (BH, nt, R, D), nt = t / C + 1
  float* lse;             // (BH, nt, R)
};

constexpr int kMaxR = 8;

template <typename T, typename TG>
__global__ void step_kernel(Params p) {
  extern __shared__ float sm[];
  const int D = p.D, R = p.R, C = p.C;
  float* s_kt = sm;                    // [D]   key of the new row
  float* s_q = s_kt + D;               // [R][D]
  float* s_p = s_q + R * D;            // [R][C] probabilities
  float* s_red = s_p + R * C;          // [2][kMaxR][32] warp partials
  const int bh = blockIdx.x, i = blockIdx.y, tid = threadIdx.x;
  const int nt = p.t / C + 1;
  const T* kc = static_cast<const T*>(p.kcache) + (size_t)bh * p.Lcap * D;
  const T* vc = static_cast<const T*>(p.vcache) + (size_t)bh * p.Lcap * D;
  for (int e = tid; e < D; e += C) s_kt[e] = Num<T>::ld(kc + (size_t)p.t * D + e);
  for (int e = tid; e < R * D; e += C) s_q[e] = Num<T>::ld(static_cast<const T*>(p.q) + (size_t)bh * R * D + e);
  __syncthreads();

  const int kk = i * C + tid;          // this thread's key
  const bool live = kk <= p.t;
  float g = 0.f, s[kMaxR];
#pragma unroll
  for (int r = 0; r < kMaxR; ++r) s[r] = 0.f;
  if (live) {
    // the thread's key row, 16 bytes at a time (head_dim is a multiple of 16 bytes: checked by the host)
    constexpr int kN = aux::Vec16<T>::kN;
    const T* krow = kc + (size_t)kk * D;
    for (int e0 = 0; e0 < D; e0 += kN) {
      float kv[kN];
      aux::Vec16<T>::load(krow + e0, kv);
#pragma unroll
      for (int u = 0; u < kN; ++u) {
        g = fmaf(kv[u], s_kt[e0 + u], g);
#pragma unroll
        for (int r = 0; r < kMaxR; ++r)
          if (r < R) s[r] = fmaf(kv[u], s_q[r * D + e0 + u], s[r]);
      }
    }
  }
  // decay state of this key after row t
  float cstate = 0.f;
  if (live && kk < p.t) {
    const float s3 = cbrtf(Num<TG>::ld(static_cast<const TG*>(p.src) + (size_t)bh * p.Lcap + kk));
    const float t3 = cbrtf(Num<TG>::ld(static_cast<const TG*>(p.dest) + bh));
    const float pw = g > 0.f ? powf(g, 2.0f / 3.0f) : 0.f;
    const float a = pw * s3 * t3;
    cstate = p.state[(size_t)bh * p.Lcap + kk] + log1pf(-fminf(fmaxf(a, 0.f), clamp_hi()));
  }
  if (live) p.state[(size_t)bh * p.Lcap + kk] = cstate;

  // softmax over the chunk's keys, per head: block-wide max and sum through warp shuffles and shared memory
  const int warp = tid >> 5, lane = tid & 31, nwarps = (C + 31) >> 5;
  float m[kMaxR];
#pragma unroll
  for (int r = 0; r < kMaxR; ++r) {
    float v = (live && r < R) ? s[r] + cstate : -INFINITY;
    s[r] = v;
#pragma unroll
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if (lane == 0) s_red[r * 32 + warp] = v;
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < kMaxR; ++r) {
    float v = -INFINITY;
    for (int w = 0; w < nwarps; ++w) v = fmaxf(v, s_red[r * 32 + w]);
    m[r] = v;
  }
#pragma unroll
  for (int r = 0; r < kMaxR; ++r) {
    const float e = (live && r < R) ? __expf(s[r] - m[r]) : 0.f;
    s[r] = e;
    float v = e;
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) s_red[(kMaxR + r) * 32 + warp] = v;
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < kMaxR; ++r) {
    float v = 0.f;
    for (int w = 0; w < nwarps; ++w) v += s_red[(kMaxR + r) * 32 + w];
    // the reference rounds the normalised probabilities to the input dtype before the product with V (:159)
    if (r < R) {
      s_p[r * C + tid] = Num<T>::rnd(s[r] / v);
      if (tid == 0) p.lse[((size_t)bh * nt + i) * R + r] = m[r] + logf(v);
    }
  }
  __syncthreads();

  // out[r][d] = sum_k P[r][k] v_k[d]: thread = (d, r modulo), keys in the loop; V rows are read coalesced along d
  const int nkeys = min(C, p.t - i * C + 1);
  for (int o = tid; o < R * D; o += C) {
    const int r = o / D, d = o - r * D;
    float acc = 0.f;
    for (int k = 0; k < nkeys; ++k) acc = fmaf(s_p[r * C + k], Num<T>::ld(vc + (size_t)(i * C + k) * D + d), acc);
    Num<T>::st(static_cast<T*>(p.out) + (((size_t)bh * nt + i) * R + r) * D + d, acc);
  }
}

inline size_t smem_bytes(const Params& p) {
  return sizeof(float) * ((size_t)p.D + (size_t)p.R * p.D + (size_t)p.R * p.C + 2 * kMaxR * 32);
}

}  // namespace decode
}  // namespace ua
