// C ABI of libua_b200.so: argument checking and kernel dispatch.
// Declarations and the reference interfaces they replace: include/ua_b200.h.
#include "../../include/ua_b200.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <mutex>

#include <algorithm>

#include "ua_aux.cuh"
#include "ua_decode.cuh"
#include "ua_simt.cuh"
#include "ua_sm100_host.cuh"

namespace {

using bf16 = __nv_bfloat16;
constexpr size_t kMaxDynSmem = 227 * 1024;

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

int check_dims(const UaDims* d) {
  if (!d) return UA_ERR_NULL_POINTER;
  if (d->batch <= 0 || d->kv_heads <= 0 || d->q_per_kv <= 0 || d->n_chunks <= 0 || d->chunk <= 0 || d->head_dim <= 0)
    return UA_ERR_BAD_DIMS;
  if (d->chunk % 16 != 0 || d->head_dim % 4 != 0) return UA_ERR_BAD_DIMS;
  return UA_OK;
}

ua::Shape to_shape(const UaDims* d) {
  ua::Shape s;
  s.B = d->batch; s.H = d->kv_heads; s.R = d->q_per_kv; s.N = d->n_chunks; s.C = d->chunk; s.D = d->head_dim;
  s.L = s.N * s.C;
  return s;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Tiling of the SIMT kernels: rows per tile and whether K_i / V_i sit in shared memory as fp32 or (bf16 inputs only)
// as bf16; the first choice that divides the chunk and fits shared memory.
struct SimtCfg {
  int rt;        // 0: nothing fits
  bool compact;  // K_i, V_i kept as bf16
};

SimtCfg simt_cfg(int C, int D, int dtype, bool bwd) {
  const int rts[4] = {32, 16, 16, 8};
  const bool compact[4] = {false, false, true, true};
  for (int t = 0; t < 4; ++t) {
    if (C % rts[t]) continue;
    if (compact[t] && dtype != UA_BF16) continue;
    const int elem = compact[t] ? 2 : 4;
    size_t need = bwd ? ua::simt::bwd_smem_bytes(C, D, rts[t], elem) : ua::simt::fwd_smem_bytes(C, D, rts[t], elem);
    if (need <= kMaxDynSmem) return SimtCfg{rts[t], compact[t]};
  }
  return SimtCfg{0, false};
}

struct BwdWorkspace {
  size_t off_dk, off_dv, off_dq, off_ds, off_dt, off_carry, acc_bytes, total;
};

BwdWorkspace bwd_layout(const ua::Shape& s, int rt) {
  BwdWorkspace w;
  const size_t BH = (size_t)s.B * s.H, f = sizeof(float);
  size_t o = 256;   // [0, 256): status word
  w.off_dk = o; o = align_up(o + BH * s.L * s.D * f, 256);
  w.off_dv = o; o = align_up(o + BH * s.L * s.D * f, 256);
  w.off_dq = o; o = align_up(o + BH * s.R * s.L * s.D * f, 256);
  w.off_ds = o; o = align_up(o + BH * s.L * f, 256);
  w.off_dt = o; o = align_up(o + BH * s.L * f, 256);
  w.acc_bytes = o;
  w.off_carry = o; o = align_up(o + BH * s.N * (size_t)(s.L / rt) * s.C * f, 256);
  w.total = o;
  return w;
}

struct BwdWorkspaceTc {
  size_t off_dk, off_dq, off_dt, off_dkr, off_carry, off_lse, off_gd, off_mt, off_ksum, off_nacc, acc_bytes, total;
};

// Scratch of the tensor-core backward: status | fp32 accumulators dK, dQ, d dest, row-side dK | decay-prefix table (two entries per
// 128-row tile) | log-sum-exp (only written when the caller has none) | fp32 copy of g_denom (only written when the
// caller's is bf16) | per-chunk data of the kernels for the rows before a chunk.
BwdWorkspaceTc bwd_layout_tc(const ua::Shape& s) {
  BwdWorkspaceTc w;
  const size_t BH = (size_t)s.B * s.H, f = sizeof(float);
  size_t o = 256;   // [0, 256): status word
  w.off_dk = o; o = align_up(o + BH * s.L * s.D * f, 256);
  w.off_dq = o; o = align_up(o + BH * s.R * s.L * s.D * f, 256);
  w.off_dt = o; o = align_up(o + BH * s.L * f, 256);
  w.off_dkr = o; o = align_up(o + BH * s.L * s.D * f, 256);
  w.acc_bytes = o;
  w.off_carry = o; o = align_up(o + BH * s.N * (size_t)s.N * 256 * f, 256);
  w.off_lse = o; o = align_up(o + BH * s.N * (size_t)s.R * s.L * f, 256);
  w.off_gd = o; o = align_up(o + BH * s.N * (size_t)s.R * s.L * f, 256);
  // per-chunk constants and partial sums of the rows-before-the-chunk kernels: M^T images, ksum, N / w / u / vbar
  w.off_mt = o; o = align_up(o + BH * s.N * (size_t)s.D * s.D * 2, 256);
  w.off_ksum = o; o = align_up(o + BH * s.N * (size_t)s.D * 2, 256);
  w.off_nacc = o; o = align_up(o + BH * s.N * (size_t)(s.D + 3) * s.D * f, 256);
  w.total = o;
  return w;
}

template <typename T, typename TG, typename S>
int launch_simt_fwd(const ua::simt::FwdParams& p, cudaStream_t st) {
  size_t smem = ua::simt::fwd_smem_bytes(p.s.C, p.s.D, p.rt, (int)sizeof(S));
  auto kern = ua::simt::fwd_kernel<T, TG, S>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return UA_ERR_CUDA;
  kern<<<p.s.B * p.s.H * p.s.N, ua::simt::kThreads, smem, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? UA_OK : UA_ERR_CUDA;
}

template <typename T, typename TG, typename S>
int launch_simt_bwd(const ua::simt::BwdParams& p, cudaStream_t st) {
  size_t smem = ua::simt::bwd_smem_bytes(p.s.C, p.s.D, p.rt, (int)sizeof(S));
  auto kern = ua::simt::bwd_kernel<T, TG, S>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return UA_ERR_CUDA;
  kern<<<p.s.B * p.s.H * p.s.N, ua::simt::kThreads, smem, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? UA_OK : UA_ERR_CUDA;
}

__global__ void widen_bf16_kernel(const bf16* __restrict__ src, float* __restrict__ dst, size_t n) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; idx < n; idx += stride) dst[idx] = __bfloat162float(src[idx]);
}

template <typename T>
int launch_convert(const float* src, void* dst, size_t n, cudaStream_t st) {
  if (n % 8 == 0 && n >= 8 && aligned16(src) && aligned16(dst)) {
    const size_t n8 = n / 8;
    int blocks = (int)((n8 + 255) / 256);
    if (blocks > 148 * 8) blocks = 148 * 8;
    ua::simt::convert8_kernel<T><<<blocks, 256, 0, st>>>(reinterpret_cast<const float4*>(src), static_cast<T*>(dst), n8);
    return cudaGetLastError() == cudaSuccess ? UA_OK : UA_ERR_CUDA;
  }
  int blocks = (int)((n + 1023) / 1024);
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  ua::simt::convert_kernel<T><<<blocks, 256, 0, st>>>(src, static_cast<T*>(dst), n);
  return cudaGetLastError() == cudaSuccess ? UA_OK : UA_ERR_CUDA;
}

int convert_any(int dtype, const float* src, void* dst, size_t n, cudaStream_t st) {
  return dtype == UA_F32 ? launch_convert<float>(src, dst, n, st) : launch_convert<bf16>(src, dst, n, st);
}

// ---- chunks of 256, 384, ... keys on the tensor-core kernels ---------------------------------------------------
// The softmax of the operator runs over the keys of one chunk (universal_attention_autograd.py:85-93); everything else --
// affinity, decay prefix along the rows, mask -- is per key.  A chunk of m * 128 keys is therefore swept as m sub-chunks
// of 128 keys by the kernels above, and the m (out, log-sum-exp) pairs of each chunk are merged with softmax weights
// exp(lse_sub - lse_chunk): the same merge as SMVecMatMul's, over groups of m neighbouring sub-chunks.  The backward
// runs the sub-chunk forward again (the merge backward needs its outputs), the merge backward, and the sub-chunk backward.
int sub_chunks(const ua::Shape& s, int dtype, int flags) {
  if ((flags & UA_FLAG_FORCE_SIMT) || dtype != UA_BF16 || s.C <= 128 || s.C % 128 != 0 || s.C / 128 > 8) return 0;
  ua::Shape t = s;
  t.C = 128; t.N = s.N * (s.C / 128);
  return (ua::sm100::fwd_supported(t, dtype) && ua::sm100::bwd2_supported(t, dtype)) ? s.C / 128 : 0;
}
UaDims sub_dims(const UaDims* d, int m) {
  UaDims t = *d;
  t.n_chunks = d->n_chunks * m; t.chunk = 128;
  return t;
}
// the merge kernels' view of the sub-chunk tensors: (batch, kv head, chunk) as the batch, the m sub-chunks as the merged axis
UaDims group_dims(const UaDims* d, int m) {
  UaDims t = *d;
  t.batch = d->batch * d->kv_heads * d->n_chunks; t.kv_heads = 1; t.n_chunks = m; t.chunk = d->n_chunks * d->chunk / m;
  return t;
}
struct SubWorkspace {
  size_t off_inner, off_out, off_gout, off_lse, off_glse, off_carry, off_status, total;
};
SubWorkspace sub_layout(const ua::Shape& s, int m, bool backward, size_t inner_bytes) {
  SubWorkspace w{};
  const size_t rows = (size_t)s.B * s.H * s.N * m * s.R * s.L;
  size_t o = align_up(inner_bytes < 256 ? 256 : inner_bytes, 256);     // the inner call's workspace comes first: its status word is the caller's
  w.off_out = o; o = align_up(o + rows * s.D * 2, 256);
  w.off_lse = o; o = align_up(o + rows * sizeof(float), 256);
  if (backward) {
    w.off_gout = o; o = align_up(o + rows * s.D * 2, 256);
    w.off_glse = o; o = align_up(o + rows * sizeof(float), 256);
    w.off_carry = o; o = align_up(o + (size_t)s.B * s.H * s.N * m * s.N * m * 256 * sizeof(float), 256);
    w.off_status = o; o += 256;
  }
  w.total = o;
  return w;
}

// g_lse_sub += g_denom_chunk * exp(lse_sub - lse_chunk): the chunk's denom is the log-sum-exp over its sub-chunks
template <typename TD>
__global__ void group_denom_grad_kernel(const float* __restrict__ lse_sub, const TD* __restrict__ g_denom, float* __restrict__ g_lse_sub,
                                        size_t groups, size_t rl, int m) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < groups * rl; idx += stride) {
    const size_t grp = idx / rl, x = idx - grp * rl;
    const float* l = lse_sub + grp * m * rl + x;
    float mx = l[0];
    for (int q = 1; q < m; ++q) mx = fmaxf(mx, l[q * rl]);
    float z = 0.f;
    for (int q = 0; q < m; ++q) z += expf(l[q * rl] - mx);
    const float g = ua::Num<TD>::ld(g_denom + idx) / z;
    float* gl = g_lse_sub + grp * m * rl + x;
    for (int q = 0; q < m; ++q) gl[q * rl] += g * expf(l[q * rl] - mx);
  }
}
// One block, two waiters on an mbarrier that nothing completes: thread 0 with the single-thread wait, warp 1 with the
// warp-collective one, both with a short wall-time limit.  Both give up, and the block reports it as the kernels do.
__global__ void wait_selftest_kernel(int* status, unsigned long long limit_ns) {
  __shared__ __align__(8) unsigned long long bar_mem;
  __shared__ int flags[2];      // [0] abort flag, [1] note of the first waiter to give up
  const uint32_t bar = ua::ptx::smem_u32(&bar_mem);
  if (threadIdx.x == 0) {
    flags[0] = 0; flags[1] = 0;
    ua::ptx::mbar_init(bar, 1);
    ua::ptx::mbar_init_fence();
  }
  __syncthreads();
  volatile int* abort_flag = flags;
  bool ok = true;
  if (threadIdx.x == 0) ok = ua::ptx::mbar_wait(bar, 0, abort_flag, limit_ns);
  else if (threadIdx.x >= 32) ok = ua::ptx::mbar_wait_warp(bar, 0, abort_flag, limit_ns);
  if (!ok && (threadIdx.x & 31) == 0) atomicCAS(flags + 1, 0, 1 | ((int)threadIdx.x << 8));
  __syncthreads();
  if (threadIdx.x == 0 && flags[0]) {
    if (atomicExch(status, 3) == 0) status[1] = flags[1];
  }
}

// log-sum-exp of every row over the key chunks that hold keys at or before it (the later chunks are fully masked for the
// row; their entries of lse_cm need not have been written)
__global__ void row_lse_kernel(const float* __restrict__ lse_cm, float* __restrict__ row_lse, size_t bh_count, int N, int R, int L) {
  const size_t total = bh_count * R * L, stride = (size_t)gridDim.x * blockDim.x;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const int l = (int)(idx % L);
    const size_t br = idx / L;                  // bh * R + r
    const size_t bh = br / R, r = br % R;
    const float* src = lse_cm + ((bh * N) * R + r) * (size_t)L + l;
    const size_t nstride = (size_t)R * L;
    const int last = l / 128;
    float mx = src[0];
    for (int i = 1; i <= last; ++i) mx = fmaxf(mx, src[i * nstride]);
    float z = 0.f;
    for (int i = 0; i <= last; ++i) z += expf(src[i * nstride] - mx);
    row_lse[idx] = mx + logf(z);
  }
}

// a status word raised by an inner call on its own buffer is carried over to the caller's
__global__ void carry_status_kernel(const int* __restrict__ from, int* __restrict__ to) {
  if (from[0] != 0 && atomicCAS(to, 0, from[0]) == 0) to[1] = from[1];
}

bool dtype_ok(int dtype, int gate_dtype) {
  if (dtype != UA_F32 && dtype != UA_BF16) return false;
  if (gate_dtype != UA_F32 && gate_dtype != UA_BF16) return false;
  if (dtype == UA_F32 && gate_dtype == UA_BF16) return false;
  return true;
}

// ---- scratch for ua_bwd_static -------------------------------------------------
// Lives in every CUDA context that loads this library, from load to exit.
constexpr size_t kStaticScratchBytes = UA_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not an address a
// kernel can use; the device address has to be asked for, with that device current.
int static_scratch_for_current_device(void** out) {
  // Asked for on every call rather than remembered: after a cudaDeviceReset the module is loaded again into the new
  // context and a remembered address would belong to the context that is gone.  (The runtime keeps its own table; the
  // query neither allocates nor synchronises once the module is loaded.)
  void* ptr = nullptr;
  if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || !ptr) return UA_ERR_CUDA;
  *out = ptr;
  return UA_OK;
}

}  // namespace

namespace {
template <typename T, int TPR>
int launch_prepare(const ua::aux::PrepDims& pd, int backward, const void* a0, const void* a1, const void* a2, const void* a3,
                   const float* key_norm_in, void* o0, void* o1, void* o2, float* key_norm_out, cudaStream_t st) {
  const long long rows = (long long)pd.b * pd.s * (pd.n + 2 * pd.n_kv);
  const unsigned blocks = (unsigned)((rows * TPR + ua::aux::kMergeThreads - 1) / ua::aux::kMergeThreads);
  if (!backward)
    ua::aux::prepare_fwd_kernel<T, TPR><<<blocks, ua::aux::kMergeThreads, 0, st>>>(
        pd, static_cast<const T*>(a0), static_cast<const T*>(a1), static_cast<const T*>(a2), static_cast<T*>(o0), static_cast<T*>(o1),
        static_cast<T*>(o2), key_norm_out);
  else
    ua::aux::prepare_bwd_kernel<T, TPR><<<blocks, ua::aux::kMergeThreads, 0, st>>>(
        pd, static_cast<const T*>(a0), static_cast<const T*>(a1), static_cast<const T*>(a2), static_cast<const T*>(a3), key_norm_in,
        static_cast<T*>(o0), static_cast<T*>(o1), static_cast<T*>(o2));
  return cudaGetLastError() == cudaSuccess ? UA_OK : UA_ERR_CUDA;
}
template <typename T>
int dispatch_prepare(int tpr, const ua::aux::PrepDims& pd, int backward, const void* a0, const void* a1, const void* a2,
                     const void* a3, const float* kn_in, void* o0, void* o1, void* o2, float* kn_out, cudaStream_t st) {
  switch (tpr) {
    case 1: return launch_prepare<T, 1>(pd, backward, a0, a1, a2, a3, kn_in, o0, o1, o2, kn_out, st);
    case 2: return launch_prepare<T, 2>(pd, backward, a0, a1, a2, a3, kn_in, o0, o1, o2, kn_out, st);
    case 4: return launch_prepare<T, 4>(pd, backward, a0, a1, a2, a3, kn_in, o0, o1, o2, kn_out, st);
    case 8: return launch_prepare<T, 8>(pd, backward, a0, a1, a2, a3, kn_in, o0, o1, o2, kn_out, st);
    case 16: return launch_prepare<T, 16>(pd, backward, a0, a1, a2, a3, kn_in, o0, o1, o2, kn_out, st);
    case 32: return launch_prepare<T, 32>(pd, backward, a0, a1, a2, a3, kn_in, o0, o1, o2, kn_out, st);
    default: return UA_ERR_UNSUPPORTED;
  }
}
int prepare_common(int b, int s, int n_heads, int n_kv, int head_dim, int dtype, int flags, ua::aux::PrepDims* pd, int* tpr) {
  if (b <= 0 || s <= 0 || n_heads <= 0 || n_kv <= 0 || head_dim <= 0 || n_heads % n_kv) return UA_ERR_BAD_DIMS;
  if (dtype != UA_F32 && dtype != UA_BF16) return UA_ERR_BAD_DTYPE;
  const int bytes = head_dim * (dtype == UA_F32 ? 4 : 2);
  if (bytes % 16) return UA_ERR_UNSUPPORTED;
  *tpr = bytes / 16;
  pd->b = b; pd->s = s; pd->n = n_heads; pd->n_kv = n_kv;
  pd->normalize_keys = (flags & UA_PREP_NORMALIZE_KEYS) ? 1 : 0;
  pd->sigmoid_gates = (flags & UA_PREP_SIGMOID_GATES) ? 1 : 0;
  return UA_OK;
}
}  // namespace

extern "C" {

int ua_version(void) { return 1; }

const char* ua_error_string(int code) {
  switch (code) {
    case UA_OK: return "ok";
    case UA_ERR_BAD_DIMS: return "bad dims (all > 0, chunk a multiple of 16, head_dim a multiple of 4)";
    case UA_ERR_BAD_DTYPE: return "unsupported dtype combination";
    case UA_ERR_NULL_POINTER: return "null pointer argument";
    case UA_ERR_WORKSPACE: return "workspace missing, too small or not 256-byte aligned";
    case UA_ERR_UNSUPPORTED: return "no kernel for this shape";
    case UA_ERR_CUDA: return "CUDA runtime error";
    case UA_ERR_ALIGNMENT: return "tensor pointer not 16-byte aligned";
    case UA_ERR_DEVICE: return "device is not compute capability 10.x";
    case UA_ERR_STATIC_LIMIT: return "problem needs more scratch than the built-in static buffer of ua_bwd_static holds";
    case UA_ERR_TIMEOUT: return "a kernel gave up on a bounded device-side wait (results are invalid)";
    default: return "unknown error code";
  }
}

size_t ua_fwd_workspace_bytes(const UaDims* dims, int dtype, int flags) {
  if (check_dims(dims) == UA_OK) {
    ua::Shape s = to_shape(dims);
    if (const int m = sub_chunks(s, dtype, flags)) return sub_layout(s, m, false, 256).total;
  }
  return 256;   // status word
}

size_t ua_bwd_workspace_bytes(const UaDims* dims, int dtype, int flags) {
  if (check_dims(dims) != UA_OK) return 0;
  ua::Shape s = to_shape(dims);
  if (const int m = sub_chunks(s, dtype, flags)) {
    const UaDims sd = sub_dims(dims, m);
    return sub_layout(s, m, true, bwd_layout_tc(to_shape(&sd)).total).total;
  }
  if (!(flags & UA_FLAG_FORCE_SIMT) && ua::sm100::bwd2_supported(s, dtype)) return bwd_layout_tc(s).total;
  const SimtCfg cfg = simt_cfg(s.C, s.D, dtype, true);
  if (!cfg.rt) return 0;
  return bwd_layout(s, cfg.rt).total;
}

size_t ua_carry_bytes(const UaDims* dims, int dtype, int flags) {
  if (check_dims(dims) != UA_OK) return 0;
  ua::Shape s = to_shape(dims);
  if (const int m = sub_chunks(s, dtype, flags)) return (size_t)s.B * s.H * s.N * m * s.N * m * 256 * sizeof(float);
  if ((flags & UA_FLAG_FORCE_SIMT) || !ua::sm100::bwd2_supported(s, dtype)) return 0;
  return (size_t)s.B * s.H * s.N * s.N * 256 * sizeof(float);
}

int ua_fwd(const UaDims* dims, int dtype, int gate_dtype, const void* kc, const void* vc, const void* xq,
           const void* static_src, const void* static_dest, void* out_cm, float* lse_cm, void* denom_cm,
           void* workspace, size_t workspace_bytes, int flags, void* stream) {
  return ua_fwd_keep(dims, dtype, gate_dtype, kc, vc, xq, static_src, static_dest, out_cm, lse_cm, denom_cm, nullptr,
                     workspace, workspace_bytes, flags, stream);
}

int ua_fwd_keep(const UaDims* dims, int dtype, int gate_dtype, const void* kc, const void* vc, const void* xq,
                const void* static_src, const void* static_dest, void* out_cm, float* lse_cm, void* denom_cm,
                void* carry_out, void* workspace, size_t workspace_bytes, int flags, void* stream) {
  int e = check_dims(dims);
  if (e) return e;
  if (!dtype_ok(dtype, gate_dtype)) return UA_ERR_BAD_DTYPE;
  if (!kc || !vc || !xq || !static_src || !static_dest || !out_cm || !lse_cm) return UA_ERR_NULL_POINTER;
  if (!aligned16(kc) || !aligned16(vc) || !aligned16(xq) || !aligned16(out_cm)) return UA_ERR_ALIGNMENT;
  if (!workspace || workspace_bytes < 256 || (reinterpret_cast<uintptr_t>(workspace) & 255u)) return UA_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ua::Shape s = to_shape(dims);
  if (const int m = sub_chunks(s, dtype, flags)) {
    // sub-chunks of 128 keys, then the merge inside each chunk (see sub_chunks)
    const SubWorkspace w = sub_layout(s, m, false, 256);
    if (workspace_bytes < w.total) return UA_ERR_WORKSPACE;
    char* ws = static_cast<char*>(workspace);
    const UaDims sd = sub_dims(dims, m), gd = group_dims(dims, m);
    void* out_sub = ws + w.off_out;
    float* lse_sub = reinterpret_cast<float*>(ws + w.off_lse);
    if ((e = ua_fwd_keep(&sd, dtype, gate_dtype, kc, vc, xq, static_src, static_dest, out_sub, lse_sub, nullptr, carry_out, workspace,
                         256, flags & ~UA_FLAG_SKIP_MASKED_FILL, stream)))
      return e;
    if ((e = ua_merge_fwd_stats(&gd, dtype, out_sub, lse_sub, out_cm, lse_cm, stream))) return e;
    if (denom_cm) e = convert_any(dtype, lse_cm, denom_cm, (size_t)s.B * s.H * s.N * s.R * s.L, st);
    return e;
  }
  if (cudaMemsetAsync(workspace, 0, 256, st) != cudaSuccess) return UA_ERR_CUDA;

  if (!(flags & UA_FLAG_FORCE_SIMT) && ua::sm100::fwd_supported(s, dtype)) {
    ua::sm100::FwdParams fp{};
    fp.s = s; fp.ssrc = static_src; fp.sdest = static_dest;
    fp.out = static_cast<bf16*>(out_cm); fp.lse = lse_cm; fp.denom = static_cast<bf16*>(denom_cm);
    fp.status = static_cast<int*>(workspace);
    fp.carry = ua_carry_bytes(dims, dtype, flags) ? static_cast<float*>(carry_out) : nullptr;
    ua::sm100::whole_sequence(fp);
    return ua::sm100::launch_fwd<false>(s, gate_dtype, kc, vc, xq, fp, !(flags & UA_FLAG_SKIP_MASKED_FILL), st);
  }

  ua::simt::FwdParams p;
  p.s = s; p.kc = kc; p.vc = vc; p.xq = xq; p.ssrc = static_src; p.sdest = static_dest;
  p.out = out_cm; p.lse = lse_cm; p.denom = denom_cm;
  p.skip_masked_fill = (flags & UA_FLAG_SKIP_MASKED_FILL) ? 1 : 0;
  const SimtCfg cfg = simt_cfg(s.C, s.D, dtype, false);
  p.rt = cfg.rt;
  if (!p.rt) return UA_ERR_UNSUPPORTED;
  if (dtype == UA_F32) return launch_simt_fwd<float, float, float>(p, st);
  if (cfg.compact) return gate_dtype == UA_F32 ? launch_simt_fwd<bf16, float, bf16>(p, st) : launch_simt_fwd<bf16, bf16, bf16>(p, st);
  if (gate_dtype == UA_F32) return launch_simt_fwd<bf16, float, float>(p, st);
  return launch_simt_fwd<bf16, bf16, float>(p, st);
}

namespace {
// Row range [tile_begin, tile_end) placed at row `row_offset` of slabs of `rows_total` rows.
int check_rows(const ua::Shape& s, bool ok_shape, const UaRows* rows) {
  if (!rows) return UA_ERR_NULL_POINTER;
  if (!ok_shape) return UA_ERR_UNSUPPORTED;
  if (rows->tile_begin < 0 || rows->tile_end > s.N || rows->tile_begin >= rows->tile_end) return UA_ERR_BAD_DIMS;
  const int len = (rows->tile_end - rows->tile_begin) * 128;
  if (rows->row_offset < 0 || rows->row_offset % 128 != 0 || rows->rows_total < rows->row_offset + len) return UA_ERR_BAD_DIMS;
  return UA_OK;
}
}  // namespace

int ua_fwd_rows(const UaDims* dims, int dtype, int gate_dtype, const UaRows* rows, const void* kc, const void* vc,
                const void* xq_rows, const void* static_src, const void* static_dest_rows, const float* carry_in,
                void* out_cm_rows, float* lse_cm_rows, void* denom_cm_rows, void* workspace, size_t workspace_bytes,
                int flags, void* stream) {
  return ua_fwd_rows_keep(dims, dtype, gate_dtype, rows, kc, vc, xq_rows, static_src, static_dest_rows, carry_in, out_cm_rows,
                          lse_cm_rows, denom_cm_rows, nullptr, workspace, workspace_bytes, flags, stream);
}

int ua_fwd_rows_keep(const UaDims* dims, int dtype, int gate_dtype, const UaRows* rows, const void* kc, const void* vc,
                     const void* xq_rows, const void* static_src, const void* static_dest_rows, const float* carry_in,
                     void* out_cm_rows, float* lse_cm_rows, void* denom_cm_rows, float* carry_table_out, void* workspace,
                     size_t workspace_bytes, int flags, void* stream) {
  int e = check_dims(dims);
  if (e) return e;
  if (!dtype_ok(dtype, gate_dtype)) return UA_ERR_BAD_DTYPE;
  if (!kc || !vc || !xq_rows || !static_src || !static_dest_rows || !out_cm_rows || !lse_cm_rows) return UA_ERR_NULL_POINTER;
  if (!aligned16(kc) || !aligned16(vc) || !aligned16(xq_rows) || !aligned16(out_cm_rows)) return UA_ERR_ALIGNMENT;
  if (!workspace || workspace_bytes < 256 || (reinterpret_cast<uintptr_t>(workspace) & 255u)) return UA_ERR_WORKSPACE;
  ua::Shape s = to_shape(dims);
  if ((e = check_rows(s, ua::sm100::fwd_supported(s, dtype), rows))) return e;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(workspace, 0, 256, st) != cudaSuccess) return UA_ERR_CUDA;
  ua::sm100::FwdParams fp{};
  fp.s = s; fp.ssrc = static_src; fp.sdest = static_dest_rows;
  fp.out = static_cast<bf16*>(out_cm_rows); fp.lse = lse_cm_rows; fp.denom = static_cast<bf16*>(denom_cm_rows);
  fp.status = static_cast<int*>(workspace); fp.carry = carry_table_out;
  fp.j_begin = rows->tile_begin; fp.j_end = rows->tile_end; fp.Lr = rows->rows_total; fp.r0 = rows->row_offset;
  fp.carry_in = carry_in; fp.total_out = nullptr;
  return ua::sm100::launch_fwd<false>(s, gate_dtype, kc, vc, xq_rows, fp, !(flags & UA_FLAG_SKIP_MASKED_FILL), st);
}

int ua_decay_totals_rows(const UaDims* dims, int dtype, int gate_dtype, const UaRows* rows, const void* kc,
                         const void* static_src, const void* static_dest_rows, const float* carry_in, float* total_out,
                         void* workspace, size_t workspace_bytes, void* stream) {
  int e = check_dims(dims);
  if (e) return e;
  if (!dtype_ok(dtype, gate_dtype)) return UA_ERR_BAD_DTYPE;
  if (!kc || !static_src || !static_dest_rows || !total_out) return UA_ERR_NULL_POINTER;
  if (!aligned16(kc)) return UA_ERR_ALIGNMENT;
  if (!workspace || workspace_bytes < 256 || (reinterpret_cast<uintptr_t>(workspace) & 255u)) return UA_ERR_WORKSPACE;
  ua::Shape s = to_shape(dims);
  if ((e = check_rows(s, ua::sm100::fwd_supported(s, dtype), rows))) return e;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(workspace, 0, 256, st) != cudaSuccess) return UA_ERR_CUDA;
  ua::sm100::FwdParams fp{};
  fp.s = s; fp.ssrc = static_src; fp.sdest = static_dest_rows; fp.out = nullptr; fp.lse = nullptr; fp.denom = nullptr;
  fp.status = static_cast<int*>(workspace); fp.carry = nullptr;
  fp.j_begin = rows->tile_begin; fp.j_end = rows->tile_end; fp.Lr = rows->rows_total; fp.r0 = rows->row_offset;
  fp.carry_in = carry_in; fp.total_out = total_out;
  return ua::sm100::launch_fwd<true>(s, gate_dtype, kc, nullptr, nullptr, fp, false, st);
}

size_t ua_bwd_rows_workspace_bytes(const UaDims* dims, int dtype) {
  if (check_dims(dims) != UA_OK) return 0;
  ua::Shape s = to_shape(dims);
  if (!ua::sm100::bwd2_supported(s, dtype)) return 0;
  // status | row-side dK scratch (as for ua_bwd_rows_suffix) | decay-prefix table | log-sum-exp of the range's rows | fp32
  // copy of a bf16 g_denom (both sized for Ls = L) | per-chunk data of the kernels for the rows before a chunk (M^T images,
  // ksum, N / w / u / vbar)
  const size_t rows = (size_t)s.B * s.H * s.N * s.R * s.L, chunks = (size_t)s.B * s.H * s.N;
  return ua_bwd_rows_suffix_workspace_bytes(dims, dtype) + align_up(chunks * (size_t)s.N * 256 * sizeof(float), 256) +
         2 * align_up(rows * sizeof(float), 256) + align_up(chunks * s.D * s.D * 2, 256) + align_up(chunks * s.D * 2, 256) +
         align_up(chunks * (s.D + 3) * s.D * sizeof(float), 256);
}

size_t ua_bwd_rows_suffix_workspace_bytes(const UaDims* dims, int dtype) {
  if (check_dims(dims) != UA_OK) return 0;
  ua::Shape s = to_shape(dims);
  if (!ua::sm100::bwd2_supported(s, dtype)) return 0;
  // status | fp32 (b*h, L, d) scratch for the row-side dK, from which d static_dest is taken
  return 256 + align_up((size_t)s.B * s.H * s.L * s.D * sizeof(float), 256);
}

int ua_bwd_rows(const UaDims* dims, int dtype, int gate_dtype, const UaRows* rows, const void* kc, const void* vc,
                const void* xq_rows, const void* static_src, const void* static_dest_rows, const void* g_out_cm_rows,
                const void* g_denom_cm_rows, int g_denom_dtype, const float* carry_in, const float* suffix_in,
                float* dk_f32, float* dv_f32, float* dxq_rows_f32, float* dsrc_f32, float* ddest_rows_f32,
                float* dctot_out, void* workspace, size_t workspace_bytes, int flags, void* stream) {
  return ua_bwd_rows_kept(dims, dtype, gate_dtype, rows, kc, vc, xq_rows, static_src, static_dest_rows, g_out_cm_rows,
                          g_denom_cm_rows, g_denom_dtype, carry_in, suffix_in, nullptr, nullptr, dk_f32, dv_f32, dxq_rows_f32,
                          dsrc_f32, ddest_rows_f32, dctot_out, workspace, workspace_bytes, flags, stream);
}

int ua_bwd_rows_kept(const UaDims* dims, int dtype, int gate_dtype, const UaRows* rows, const void* kc, const void* vc,
                     const void* xq_rows, const void* static_src, const void* static_dest_rows, const void* g_out_cm_rows,
                     const void* g_denom_cm_rows, int g_denom_dtype, const float* carry_in, const float* suffix_in,
                     const float* carry_table, const float* lse_cm_rows, float* dk_f32, float* dv_f32, float* dxq_rows_f32,
                     float* dsrc_f32, float* ddest_rows_f32, float* dctot_out, void* workspace, size_t workspace_bytes,
                     int flags, void* stream) {
  int e = check_dims(dims);
  if (e) return e;
  if (!dtype_ok(dtype, gate_dtype)) return UA_ERR_BAD_DTYPE;
  if (g_denom_dtype != UA_F32 && g_denom_dtype != dtype) return UA_ERR_BAD_DTYPE;
  if (!kc || !vc || !xq_rows || !static_src || !static_dest_rows || !g_out_cm_rows || !g_denom_cm_rows || !dk_f32 || !dv_f32 ||
      !dxq_rows_f32 || !dsrc_f32 || !ddest_rows_f32)
    return UA_ERR_NULL_POINTER;
  if (!aligned16(kc) || !aligned16(vc) || !aligned16(xq_rows) || !aligned16(g_out_cm_rows) || !aligned16(dk_f32) ||
      !aligned16(dv_f32) || !aligned16(dxq_rows_f32))
    return UA_ERR_ALIGNMENT;
  ua::Shape s = to_shape(dims);
  if ((e = check_rows(s, ua::sm100::bwd2_supported(s, dtype), rows))) return e;
  const bool skip_masked = (flags & UA_FLAG_SKIP_MASKED_GRADS) != 0;
  const size_t need = ua_bwd_rows_workspace_bytes(dims, dtype);
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u)) return UA_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t head = ua_bwd_rows_suffix_workspace_bytes(dims, dtype);       // status word + row-side dK scratch, both zeroed
  if (cudaMemsetAsync(workspace, 0, head, st) != cudaSuccess) return UA_ERR_CUDA;
  float* acc_dkr = reinterpret_cast<float*>(static_cast<char*>(workspace) + 256);
  int* status = static_cast<int*>(workspace);
  char* ws = static_cast<char*>(workspace) + head - 256;                    // (the offsets below count from a 256-byte header)
  const size_t BHs = (size_t)s.B * s.H;
  const size_t tab_bytes = align_up(BHs * s.N * (size_t)s.N * 256 * sizeof(float), 256);
  const size_t row_elems = BHs * s.N * (size_t)s.R * rows->rows_total;
  const float* carry_tab = carry_table;
  const float* lse_rows = lse_cm_rows;
  float* gd_tmp = reinterpret_cast<float*>(ws + 256 + tab_bytes + align_up(BHs * s.N * (size_t)s.R * s.L * sizeof(float), 256));
  // (1) log-sum-exp and decay-prefix table of the range, unless the forward handed them over: the forward kernel without
  // its output (carry_in enters here)
  if (!carry_table || !lse_cm_rows) {
    float* tab = reinterpret_cast<float*>(ws + 256);
    float* lse_ws = reinterpret_cast<float*>(ws + 256 + tab_bytes);
    carry_tab = tab; lse_rows = lse_ws;
    ua::sm100::FwdParams fp{};
    fp.s = s; fp.ssrc = static_src; fp.sdest = static_dest_rows; fp.out = nullptr; fp.denom = nullptr; fp.lse = lse_ws;
    fp.status = status; fp.carry = tab;
    fp.j_begin = rows->tile_begin; fp.j_end = rows->tile_end; fp.Lr = rows->rows_total; fp.r0 = rows->row_offset;
    fp.carry_in = carry_in; fp.total_out = nullptr;
    if ((e = ua::sm100::launch_fwd<false>(s, gate_dtype, kc, vc, xq_rows, fp, false, st))) return e;
  }
  const float* gd32 = static_cast<const float*>(g_denom_cm_rows);
  if (g_denom_dtype != UA_F32) {
    widen_bf16_kernel<<<148 * 8, 256, 0, st>>>(static_cast<const bf16*>(g_denom_cm_rows), gd_tmp, row_elems);
    if (cudaGetLastError() != cudaSuccess) return UA_ERR_CUDA;
    gd32 = gd_tmp;
  }
  if (!aligned16(gd32) || !aligned16(static_dest_rows) || !aligned16(carry_tab) || !aligned16(lse_rows)) return UA_ERR_ALIGNMENT;
  // (2) rows of the range that lie before a chunk (uniform softmax): their own three kernels, over the range
  if (!skip_masked && s.N > 1) {
    const size_t chunks = BHs * s.N;
    char* q = ws + 256 + tab_bytes + 2 * align_up(BHs * s.N * (size_t)s.R * s.L * sizeof(float), 256);
    ua::sm100::MaskedParams mp{};
    mp.s = s; mp.g_denom = gd32;
    mp.mt = reinterpret_cast<uint8_t*>(q); q += align_up(chunks * s.D * s.D * 2, 256);
    mp.ksum = reinterpret_cast<__nv_bfloat16*>(q); q += align_up(chunks * s.D * 2, 256);
    mp.nacc = reinterpret_cast<float*>(q);
    mp.acc_dk = dk_f32; mp.status = status;
    mp.j_begin = rows->tile_begin; mp.j_end = rows->tile_end; mp.Lr = rows->rows_total; mp.r0 = rows->row_offset;
    mp.acc_dv = dv_f32;
    if ((e = ua::sm100::launch_masked(s, kc, vc, xq_rows, g_out_cm_rows, dxq_rows_f32, mp, st))) return e;
  }
  // (3) the rows that see their chunk: the keys-on-lanes kernel over the range
  ua::sm100::Bwd2Params qp{};
  qp.s = s; qp.ssrc = static_src; qp.sdest = static_dest_rows; qp.g_denom = gd32; qp.lse = lse_rows; qp.carry = carry_tab;
  qp.acc_dk = dk_f32; qp.acc_dq = dxq_rows_f32; qp.acc_dt = ddest_rows_f32; qp.dv_chunk = nullptr;
  qp.dvc = nullptr; qp.dss = nullptr; qp.status = status; qp.trace = nullptr;
  qp.j_begin = rows->tile_begin; qp.j_end = rows->tile_end; qp.Lr = rows->rows_total; qp.r0 = rows->row_offset;
  qp.heads = s.R; qp.suffix_in = suffix_in; qp.dctot_out = dctot_out; qp.acc_dv = dv_f32; qp.acc_ds = dsrc_f32;
  qp.acc_dkr = acc_dkr;
  return ua::sm100::launch_bwd2(s, gate_dtype, false, kc, vc, xq_rows, g_out_cm_rows, qp, st);
}

int ua_bwd_rows_suffix(const UaDims* dims, int dtype, int gate_dtype, const UaRows* rows, const void* kc, const void* vc,
                       const void* static_src, const void* static_dest_rows, const float* suffix, float* dk_f32,
                       float* dsrc_f32, float* ddest_rows_f32, void* workspace, size_t workspace_bytes, void* stream) {
  int e = check_dims(dims);
  if (e) return e;
  if (!dtype_ok(dtype, gate_dtype)) return UA_ERR_BAD_DTYPE;
  if (!kc || !vc || !static_src || !static_dest_rows || !suffix || !dk_f32 || !dsrc_f32 || !ddest_rows_f32) return UA_ERR_NULL_POINTER;
  if (!aligned16(kc) || !aligned16(vc) || !aligned16(dk_f32)) return UA_ERR_ALIGNMENT;
  ua::Shape s = to_shape(dims);
  if ((e = check_rows(s, ua::sm100::bwd2_supported(s, dtype), rows))) return e;
  const size_t need = ua_bwd_rows_suffix_workspace_bytes(dims, dtype);
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u)) return UA_ERR_WORKSPACE;
  if (!aligned16(static_dest_rows)) return UA_ERR_ALIGNMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(workspace, 0, need, st) != cudaSuccess) return UA_ERR_CUDA;
  // the keys-on-lanes kernel without heads: recomputed G, the decay gradient that `suffix` induces, the two dK products
  ua::sm100::Bwd2Params qp{};
  qp.s = s; qp.ssrc = static_src; qp.sdest = static_dest_rows; qp.g_denom = nullptr; qp.lse = nullptr; qp.carry = nullptr;
  qp.acc_dk = dk_f32; qp.acc_dq = nullptr; qp.acc_dt = ddest_rows_f32; qp.dv_chunk = nullptr;
  qp.dvc = nullptr; qp.dss = nullptr; qp.status = static_cast<int*>(workspace); qp.trace = nullptr;
  qp.j_begin = rows->tile_begin; qp.j_end = rows->tile_end; qp.Lr = rows->rows_total; qp.r0 = rows->row_offset;
  qp.acc_dkr = reinterpret_cast<float*>(static_cast<char*>(workspace) + 256);
  qp.heads = 0; qp.suffix_in = suffix; qp.dctot_out = nullptr; qp.acc_dv = nullptr; qp.acc_ds = dsrc_f32;
  return ua::sm100::launch_bwd2(s, gate_dtype, false, kc, vc, nullptr, nullptr, qp, st);
}

int ua_bwd(const UaDims* dims, int dtype, int gate_dtype, const void* kc, const void* vc, const void* xq,
           const void* static_src, const void* static_dest, const void* g_out_cm, const void* g_denom_cm,
           int g_denom_dtype, void* dkc, void* dvc, void* dxq, void* dstatic_src, void* dstatic_dest,
           void* workspace, size_t workspace_bytes, int flags, void* stream) {
  return ua_bwd_kept(dims, dtype, gate_dtype, kc, vc, xq, static_src, static_dest, g_out_cm, g_denom_cm, g_denom_dtype,
                     nullptr, nullptr, dkc, dvc, dxq, dstatic_src, dstatic_dest, workspace, workspace_bytes, flags, stream);
}

int ua_bwd_kept(const UaDims* dims, int dtype, int gate_dtype, const void* kc, const void* vc, const void* xq,
                const void* static_src, const void* static_dest, const void* g_out_cm, const void* g_denom_cm,
                int g_denom_dtype, const void* carry_in, const float* lse_cm, void* dkc, void* dvc, void* dxq,
                void* dstatic_src, void* dstatic_dest, void* workspace, size_t workspace_bytes, int flags, void* stream) {
  return ua_bwd_saved(dims, dtype, gate_dtype, kc, vc, xq, static_src, static_dest, g_out_cm, g_denom_cm, g_denom_dtype,
                      carry_in, lse_cm, nullptr, dkc, dvc, dxq, dstatic_src, dstatic_dest, workspace, workspace_bytes, flags, stream);
}

int ua_bwd_saved(const UaDims* dims, int dtype, int gate_dtype, const void* kc, const void* vc, const void* xq,
                 const void* static_src, const void* static_dest, const void* g_out_cm, const void* g_denom_cm,
                 int g_denom_dtype, const void* carry_in, const float* lse_cm, const void* out_cm, void* dkc, void* dvc,
                 void* dxq, void* dstatic_src, void* dstatic_dest, void* workspace, size_t workspace_bytes, int flags,
                 void* stream) {
  int e = check_dims(dims);
  if (e) return e;
  if (!dtype_ok(dtype, gate_dtype)) return UA_ERR_BAD_DTYPE;
  if (g_denom_dtype != UA_F32 && g_denom_dtype != dtype) return UA_ERR_BAD_DTYPE;
  if (!kc || !vc || !xq || !static_src || !static_dest || !g_out_cm || !g_denom_cm || !dkc || !dvc || !dxq ||
      !dstatic_src || !dstatic_dest)
    return UA_ERR_NULL_POINTER;
  if (!aligned16(kc) || !aligned16(vc) || !aligned16(xq) || !aligned16(g_out_cm)) return UA_ERR_ALIGNMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ua::Shape s = to_shape(dims);

  if (const int m = sub_chunks(s, dtype, flags)) {
    // chunks of m * 128 keys (see sub_chunks): sub-chunk forward again, merge backward inside each chunk, sub-chunk backward.
    // (lse_cm, the chunks' log-sum-exp, is not what the sub-chunk kernels need; carry_in is already per sub-chunk.)
    const UaDims sd = sub_dims(dims, m), gd = group_dims(dims, m);
    const size_t inner = bwd_layout_tc(to_shape(&sd)).total;
    const SubWorkspace w = sub_layout(s, m, true, inner);
    if (!workspace || workspace_bytes < w.total || (reinterpret_cast<uintptr_t>(workspace) & 255u)) return UA_ERR_WORKSPACE;
    char* ws = static_cast<char*>(workspace);
    void* out_sub = ws + w.off_out;
    void* g_out_sub = ws + w.off_gout;
    float* lse_sub = reinterpret_cast<float*>(ws + w.off_lse);
    float* g_lse_sub = reinterpret_cast<float*>(ws + w.off_glse);
    void* carry_sub = carry_in ? nullptr : static_cast<void*>(ws + w.off_carry);
    if ((e = ua_fwd_keep(&sd, dtype, gate_dtype, kc, vc, xq, static_src, static_dest, out_sub, lse_sub, nullptr, carry_sub,
                         ws + w.off_status, 256, flags & ~UA_FLAG_SKIP_MASKED_FILL, stream)))
      return e;
    if ((e = ua_merge_bwd(&gd, dtype, out_sub, lse_sub, g_out_cm, g_out_sub, g_lse_sub, 0, stream))) return e;
    {
      const size_t groups = (size_t)s.B * s.H * s.N, rl = (size_t)s.R * s.L;
      if (g_denom_dtype == UA_F32)
        group_denom_grad_kernel<float><<<148 * 8, 256, 0, st>>>(lse_sub, static_cast<const float*>(g_denom_cm), g_lse_sub, groups, rl, m);
      else
        group_denom_grad_kernel<bf16><<<148 * 8, 256, 0, st>>>(lse_sub, static_cast<const bf16*>(g_denom_cm), g_lse_sub, groups, rl, m);
      if (cudaGetLastError() != cudaSuccess) return UA_ERR_CUDA;
    }
    // (the sub-chunk output tiles were just recomputed: the inner call takes its row term from them)
    if ((e = ua_bwd_saved(&sd, dtype, gate_dtype, kc, vc, xq, static_src, static_dest, g_out_sub, g_lse_sub, UA_F32,
                          carry_in ? carry_in : carry_sub, lse_sub, out_sub, dkc, dvc, dxq, dstatic_src, dstatic_dest, workspace,
                          inner, flags, stream)))
      return e;
    carry_status_kernel<<<1, 1, 0, st>>>(reinterpret_cast<const int*>(ws + w.off_status), reinterpret_cast<int*>(ws));
    return cudaGetLastError() == cudaSuccess ? UA_OK : UA_ERR_CUDA;
  }

  if (!(flags & UA_FLAG_FORCE_SIMT) && ua::sm100::bwd2_supported(s, dtype)) {
    if (!aligned16(dvc) || !aligned16(dkc) || !aligned16(dxq)) return UA_ERR_ALIGNMENT;
    BwdWorkspaceTc w = bwd_layout_tc(s);
    if (!workspace || workspace_bytes < w.total || (reinterpret_cast<uintptr_t>(workspace) & 255u)) return UA_ERR_WORKSPACE;
    char* ws = static_cast<char*>(workspace);
    if (cudaMemsetAsync(ws, 0, w.acc_bytes, st) != cudaSuccess) return UA_ERR_CUDA;
    float* carry_tab = carry_in ? const_cast<float*>(static_cast<const float*>(carry_in)) : reinterpret_cast<float*>(ws + w.off_carry);
    float* acc_dk = reinterpret_cast<float*>(ws + w.off_dk);
    float* acc_dq = reinterpret_cast<float*>(ws + w.off_dq);
    float* acc_dt = reinterpret_cast<float*>(ws + w.off_dt);
    const bool skip_masked = (flags & UA_FLAG_SKIP_MASKED_GRADS) != 0;
    const size_t BHs = (size_t)s.B * s.H;
    // What the keys-on-lanes kernel needs besides the inputs: the decay-prefix table and the forward's log-sum-exp.  A
    // caller that has neither gets both from one statistics-only run of the forward kernel (no output tile is written).
    const float* lse = lse_cm;
    if (!lse || !carry_in) {
      ua::sm100::FwdParams fp{};
      fp.s = s; fp.ssrc = static_src; fp.sdest = static_dest; fp.out = nullptr; fp.denom = nullptr;
      fp.lse = lse ? nullptr : reinterpret_cast<float*>(ws + w.off_lse);
      fp.status = reinterpret_cast<int*>(ws);
      fp.carry = carry_in ? nullptr : carry_tab;
      ua::sm100::whole_sequence(fp);
      if (lse) e = ua::sm100::launch_fwd<true>(s, gate_dtype, kc, nullptr, nullptr, fp, false, st);      // decay-only pass
      else e = ua::sm100::launch_fwd<false>(s, gate_dtype, kc, vc, xq, fp, false, st);
      if (e) return e;
      if (!lse) lse = fp.lse;
    }
    // the kernel's producer copies rows of lse / g_denom with 16-byte bulk copies: fp32, 16-byte aligned
    const float* gd32 = static_cast<const float*>(g_denom_cm);
    if (g_denom_dtype != UA_F32) {
      float* tmp = reinterpret_cast<float*>(ws + w.off_gd);
      const size_t n_gd = BHs * s.N * (size_t)s.R * s.L;
      widen_bf16_kernel<<<148 * 8, 256, 0, st>>>(static_cast<const bf16*>(g_denom_cm), tmp, n_gd);
      if (cudaGetLastError() != cudaSuccess) return UA_ERR_CUDA;
      gd32 = tmp;
    }
    if (!aligned16(gd32) || !aligned16(lse) || !aligned16(static_dest) || !aligned16(carry_tab)) return UA_ERR_ALIGNMENT;
    // Rows before a chunk (uniform softmax): their gradient is added to the accumulators by a kernel of its own.
    const float* dv_chunk = nullptr;
    if (!skip_masked && s.N > 1) {
      ua::sm100::MaskedParams mp{};
      mp.s = s; ua::sm100::whole_sequence(mp); mp.g_denom = gd32;
      mp.mt = reinterpret_cast<uint8_t*>(ws + w.off_mt);
      mp.ksum = reinterpret_cast<__nv_bfloat16*>(ws + w.off_ksum);
      mp.nacc = reinterpret_cast<float*>(ws + w.off_nacc);
      mp.acc_dk = acc_dk; mp.status = reinterpret_cast<int*>(ws);
      dv_chunk = mp.nacc + (size_t)(s.D + 1) * s.D;
      e = ua::sm100::launch_masked(s, kc, vc, xq, g_out_cm, acc_dq, mp, st);
      if (e) return e;
    }
    ua::sm100::Bwd2Params qp{};
    qp.s = s; ua::sm100::whole_sequence(qp); qp.ssrc = static_src; qp.sdest = static_dest;
    qp.g_denom = gd32;
    qp.lse = lse; qp.row_lse = nullptr; qp.row_delta = nullptr; qp.carry = carry_tab;
    qp.acc_dk = acc_dk; qp.acc_dq = acc_dq; qp.acc_dt = acc_dt;
    qp.acc_dkr = reinterpret_cast<float*>(ws + w.off_dkr);
    qp.dv_chunk = dv_chunk; qp.dv_chunk_stride = (s.D + 3) * s.D;
    qp.dvc = static_cast<bf16*>(dvc); qp.dss = dstatic_src; qp.status = reinterpret_cast<int*>(ws);
    qp.trace = nullptr;
    qp.out_tiles = (out_cm && aligned16(out_cm)) ? out_cm : nullptr;
#ifdef UA_PROFILE_BWD2
    if (const char* tp = getenv("UA_TRACE_PTR")) qp.trace = reinterpret_cast<long long*>(strtoull(tp, nullptr, 0));
#endif
    e = ua::sm100::launch_bwd2(s, gate_dtype, false, kc, vc, xq, g_out_cm, qp, st);
    if (e) return e;
    if ((e = convert_any(dtype, acc_dk, dkc, BHs * s.L * s.D, st))) return e;
    if ((e = convert_any(dtype, acc_dq, dxq, BHs * s.R * s.L * s.D, st))) return e;
    if ((e = convert_any(gate_dtype, acc_dt, dstatic_dest, BHs * s.L, st))) return e;
    return UA_OK;
  }

  const SimtCfg cfg = simt_cfg(s.C, s.D, dtype, true);
  const int rt = cfg.rt;
  if (!rt) return UA_ERR_UNSUPPORTED;
  BwdWorkspace w = bwd_layout(s, rt);
  if (!workspace || workspace_bytes < w.total || (reinterpret_cast<uintptr_t>(workspace) & 255u)) return UA_ERR_WORKSPACE;
  char* ws = static_cast<char*>(workspace);
  if (cudaMemsetAsync(ws, 0, w.acc_bytes, st) != cudaSuccess) return UA_ERR_CUDA;

  ua::simt::BwdParams p;
  p.s = s; p.kc = kc; p.vc = vc; p.xq = xq; p.ssrc = static_src; p.sdest = static_dest;
  p.g_out = g_out_cm; p.g_denom = g_denom_cm; p.g_denom_is_f32 = (g_denom_dtype == UA_F32);
  p.acc_dk = reinterpret_cast<float*>(ws + w.off_dk);
  p.acc_dv = reinterpret_cast<float*>(ws + w.off_dv);
  p.acc_dq = reinterpret_cast<float*>(ws + w.off_dq);
  p.acc_ds = reinterpret_cast<float*>(ws + w.off_ds);
  p.acc_dt = reinterpret_cast<float*>(ws + w.off_dt);
  p.carry = reinterpret_cast<float*>(ws + w.off_carry);
  p.rt = rt;
  p.skip_masked = (flags & UA_FLAG_SKIP_MASKED_GRADS) ? 1 : 0;
  p.masked_only = 0;
  if (dtype == UA_F32) e = launch_simt_bwd<float, float, float>(p, st);
  else if (cfg.compact) e = gate_dtype == UA_F32 ? launch_simt_bwd<bf16, float, bf16>(p, st) : launch_simt_bwd<bf16, bf16, bf16>(p, st);
  else if (gate_dtype == UA_F32) e = launch_simt_bwd<bf16, float, float>(p, st);
  else e = launch_simt_bwd<bf16, bf16, float>(p, st);
  if (e) return e;

  const size_t BH = (size_t)s.B * s.H;
  if ((e = convert_any(dtype, p.acc_dk, dkc, BH * s.L * s.D, st))) return e;
  if ((e = convert_any(dtype, p.acc_dv, dvc, BH * s.L * s.D, st))) return e;
  if ((e = convert_any(dtype, p.acc_dq, dxq, BH * s.R * s.L * s.D, st))) return e;
  if ((e = convert_any(gate_dtype, p.acc_ds, dstatic_src, BH * s.L, st))) return e;
  if ((e = convert_any(gate_dtype, p.acc_dt, dstatic_dest, BH * s.L, st))) return e;
  return UA_OK;
}

size_t ua_static_scratch_bytes(void) { return kStaticScratchBytes; }

int ua_bwd_static(const UaDims* dims, int dtype, int gate_dtype, const void* kc, const void* vc, const void* xq,
                  const void* static_src, const void* static_dest, const void* g_out_cm, const void* g_denom_cm,
                  int g_denom_dtype, void* dkc, void* dvc, void* dxq, void* dstatic_src, void* dstatic_dest, int flags,
                  void* stream) {
  int e = check_dims(dims);
  if (e) return e;
  const size_t need = ua_bwd_workspace_bytes(dims, dtype, flags);
  if (need == 0) return UA_ERR_UNSUPPORTED;
  if (need > kStaticScratchBytes) return UA_ERR_STATIC_LIMIT;
  void* scratch = nullptr;
  if ((e = static_scratch_for_current_device(&scratch))) return e;
  // ua_bwd clears the part of the scratch that must start at zero (accumulators, status word)
  return ua_bwd(dims, dtype, gate_dtype, kc, vc, xq, static_src, static_dest, g_out_cm, g_denom_cm, g_denom_dtype, dkc, dvc,
                dxq, dstatic_src, dstatic_dest, scratch, kStaticScratchBytes, flags, stream);
}

int ua_static_status(void* stream) {
  void* scratch = nullptr;
  int e = static_scratch_for_current_device(&scratch);
  if (e) return e;
  return ua_workspace_status(scratch, stream);
}

int ua_selftest_wait_timeout(void* workspace, size_t workspace_bytes, unsigned limit_us, void* stream) {
  if (!workspace) return UA_ERR_NULL_POINTER;
  if (workspace_bytes < 256 || (reinterpret_cast<uintptr_t>(workspace) & 255u)) return UA_ERR_WORKSPACE;
  if (limit_us < 1 || limit_us > 100000) return UA_ERR_BAD_DIMS;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(workspace, 0, 256, st) != cudaSuccess) return UA_ERR_CUDA;
  wait_selftest_kernel<<<1, 64, 0, st>>>(static_cast<int*>(workspace), (unsigned long long)limit_us * 1000ull);
  return cudaGetLastError() == cudaSuccess ? UA_OK : UA_ERR_CUDA;
}

int ua_workspace_status(const void* workspace, void* stream) {
  if (!workspace) return UA_ERR_NULL_POINTER;
  int host = 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(&host, workspace, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess) return UA_ERR_CUDA;
  if (cudaStreamSynchronize(st) != cudaSuccess) return UA_ERR_CUDA;
  return host == 0 ? UA_OK : UA_ERR_TIMEOUT;
}

int ua_relayout(const UaDims* dims, int inner, int elem_bytes, int to_reference, const void* src, void* dst,
                void* stream) {
  int e = check_dims(dims);
  if (e) return e;
  if (!src || !dst) return UA_ERR_NULL_POINTER;
  if (inner <= 0) return UA_ERR_BAD_DIMS;
  if (elem_bytes != 2 && elem_bytes != 4) return UA_ERR_BAD_DTYPE;
  ua::Shape s = to_shape(dims);
  const long long X = (long long)s.L * inner;
  const long long G = (long long)s.B * s.H * s.R;
  if (G > 65535) return UA_ERR_UNSUPPORTED;
  dim3 grid((unsigned)((X + 31) / 32), (unsigned)((s.N + 31) / 32), (unsigned)G);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (elem_bytes == 2)
    ua::aux::relayout_kernel<uint16_t><<<grid, 256, 0, st>>>(static_cast<const uint16_t*>(src),
                                                             static_cast<uint16_t*>(dst), s.N, s.R, X, to_reference);
  else
    ua::aux::relayout_kernel<uint32_t><<<grid, 256, 0, st>>>(static_cast<const uint32_t*>(src),
                                                             static_cast<uint32_t*>(dst), s.N, s.R, X, to_reference);
  return cudaGetLastError() == cudaSuccess ? UA_OK : UA_ERR_CUDA;
}

int ua_prepare_inputs(int batch, int seq, int n_heads, int n_kv_heads, int head_dim, int dtype, int flags,
                      const void* query_state, const void* key_state, const void* value_state, const void* gate_state,
                      void* xq, void* kc, void* vc, void* static_src, void* static_dest, float* key_norm, void* stream) {
  ua::aux::PrepDims pd;
  int tpr = 0;
  int e = prepare_common(batch, seq, n_heads, n_kv_heads, head_dim, dtype, flags, &pd, &tpr);
  if (e) return e;
  if (!query_state || !key_state || !value_state || !gate_state || !xq || !kc || !vc || !static_src || !static_dest) return UA_ERR_NULL_POINTER;
  if (pd.normalize_keys && !key_norm) return UA_ERR_NULL_POINTER;
  if (!aligned16(query_state) || !aligned16(key_state) || !aligned16(value_state) || !aligned16(xq) || !aligned16(kc) || !aligned16(vc))
    return UA_ERR_ALIGNMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  e = dtype == UA_F32 ? dispatch_prepare<float>(tpr, pd, 0, query_state, key_state, value_state, nullptr, nullptr, xq, kc, vc, key_norm, st)
                      : dispatch_prepare<bf16>(tpr, pd, 0, query_state, key_state, value_state, nullptr, nullptr, xq, kc, vc, key_norm, st);
  if (e) return e;
  const long long total = (long long)batch * seq * 2 * n_kv_heads;
  const unsigned gblocks = (unsigned)std::min<long long>((total + 255) / 256, 4096);
  if (dtype == UA_F32)
    ua::aux::prepare_gates_kernel<float><<<gblocks, 256, 0, st>>>(pd, static_cast<const float*>(gate_state), static_cast<float*>(static_src),
                                                                 static_cast<float*>(static_dest), 0, nullptr, nullptr, nullptr);
  else
    ua::aux::prepare_gates_kernel<bf16><<<gblocks, 256, 0, st>>>(pd, static_cast<const bf16*>(gate_state), static_cast<bf16*>(static_src),
                                                                static_cast<bf16*>(static_dest), 0, nullptr, nullptr, nullptr);
  return cudaGetLastError() == cudaSuccess ? UA_OK : UA_ERR_CUDA;
}

int ua_prepare_inputs_bwd(int batch, int seq, int n_heads, int n_kv_heads, int head_dim, int dtype, int flags,
                          const void* g_xq, const void* g_kc, const void* g_vc, const void* g_static_src, const void* g_static_dest,
                          const void* kc, const float* key_norm, const void* static_src, const void* static_dest,
                          void* d_query_state, void* d_key_state, void* d_value_state, void* d_gate_state, void* stream) {
  ua::aux::PrepDims pd;
  int tpr = 0;
  int e = prepare_common(batch, seq, n_heads, n_kv_heads, head_dim, dtype, flags, &pd, &tpr);
  if (e) return e;
  if (!g_xq || !g_kc || !g_vc || !g_static_src || !g_static_dest || !static_src || !static_dest || !d_query_state || !d_key_state ||
      !d_value_state || !d_gate_state)
    return UA_ERR_NULL_POINTER;
  if (pd.normalize_keys && (!kc || !key_norm)) return UA_ERR_NULL_POINTER;
  if (!aligned16(g_xq) || !aligned16(g_kc) || !aligned16(g_vc) || !aligned16(d_query_state) || !aligned16(d_key_state) ||
      !aligned16(d_value_state) || (kc && !aligned16(kc)))
    return UA_ERR_ALIGNMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  e = dtype == UA_F32 ? dispatch_prepare<float>(tpr, pd, 1, g_xq, g_kc, g_vc, kc, key_norm, d_query_state, d_key_state, d_value_state, nullptr, st)
                      : dispatch_prepare<bf16>(tpr, pd, 1, g_xq, g_kc, g_vc, kc, key_norm, d_query_state, d_key_state, d_value_state, nullptr, st);
  if (e) return e;
  const long long total = (long long)batch * seq * 2 * n_kv_heads;
  const unsigned gblocks = (unsigned)std::min<long long>((total + 255) / 256, 4096);
  if (dtype == UA_F32)
    ua::aux::prepare_gates_kernel<float><<<gblocks, 256, 0, st>>>(
        pd, nullptr, const_cast<float*>(static_cast<const float*>(static_src)), const_cast<float*>(static_cast<const float*>(static_dest)), 1,
        static_cast<const float*>(g_static_src), static_cast<const float*>(g_static_dest), static_cast<float*>(d_gate_state));
  else
    ua::aux::prepare_gates_kernel<bf16><<<gblocks, 256, 0, st>>>(
        pd, nullptr, const_cast<bf16*>(static_cast<const bf16*>(static_src)), const_cast<bf16*>(static_cast<const bf16*>(static_dest)), 1,
        static_cast<const bf16*>(g_static_src), static_cast<const bf16*>(g_static_dest), static_cast<bf16*>(d_gate_state));
  return cudaGetLastError() == cudaSuccess ? UA_OK : UA_ERR_CUDA;
}

int ua_decode_step(const UaDims* dims, int dtype, int gate_dtype, int t, const void* k_cache, const void* v_cache,
                   const void* src_cache, const void* q_t, const void* dest_t, float* decay_state, void* out_t, float* lse_t,
                   void* stream) {
  int e = check_dims(dims);
  if (e) return e;
  if (!dtype_ok(dtype, gate_dtype)) return UA_ERR_BAD_DTYPE;
  if (!k_cache || !v_cache || !src_cache || !q_t || !dest_t || !decay_state || !out_t || !lse_t) return UA_ERR_NULL_POINTER;
  ua::Shape s = to_shape(dims);
  if (t < 0 || t >= s.L) return UA_ERR_BAD_DIMS;
  if (s.R > ua::decode::kMaxR || s.C > 1024 || (s.C & 31)) return UA_ERR_UNSUPPORTED;
  if ((s.D * (dtype == UA_F32 ? 4 : 2)) % 16 != 0) return UA_ERR_UNSUPPORTED;
  if (!aligned16(k_cache) || !aligned16(v_cache)) return UA_ERR_ALIGNMENT;
  ua::decode::Params p;
  p.BH = s.B * s.H; p.R = s.R; p.D = s.D; p.C = s.C; p.Lcap = s.L; p.t = t;
  p.kcache = k_cache; p.vcache = v_cache; p.src = src_cache; p.q = q_t; p.dest = dest_t; p.state = decay_state;
  p.out = out_t; p.lse = lse_t;
  const size_t smem = ua::decode::smem_bytes(p);
  if (smem > 48 * 1024) return UA_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid((unsigned)p.BH, (unsigned)(t / s.C + 1));
  if (dtype == UA_F32) ua::decode::step_kernel<float, float><<<grid, s.C, smem, st>>>(p);
  else if (gate_dtype == UA_F32) ua::decode::step_kernel<bf16, float><<<grid, s.C, smem, st>>>(p);
  else ua::decode::step_kernel<bf16, bf16><<<grid, s.C, smem, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? UA_OK : UA_ERR_CUDA;
}

int ua_merge_fwd(const UaDims* dims, int dtype, const void* out_cm, const float* lse_cm, void* merged, void* stream) {
  return ua_merge_fwd_stats(dims, dtype, out_cm, lse_cm, merged, nullptr, stream);
}

int ua_merge_fwd_stats(const UaDims* dims, int dtype, const void* out_cm, const float* lse_cm, void* merged, float* row_lse,
                       void* stream) {
  int e = check_dims(dims);
  if (e) return e;
  if (dtype != UA_F32 && dtype != UA_BF16) return UA_ERR_BAD_DTYPE;
  if (!out_cm || !lse_cm || !merged) return UA_ERR_NULL_POINTER;
  if (!aligned16(out_cm) || !aligned16(merged)) return UA_ERR_ALIGNMENT;
  ua::Shape s = to_shape(dims);
  const long long rows = (long long)s.B * s.H * s.R * s.L;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int tpr = s.D * (dtype == UA_F32 ? 4 : 2) / 16;
  const unsigned blocks = (unsigned)((rows * tpr + ua::aux::kMergeThreads - 1) / ua::aux::kMergeThreads);
#define UA_MERGE_FWD(T, TPR)                                                                                         \
  ua::aux::merge_fwd_kernel<T, TPR><<<blocks, ua::aux::kMergeThreads, 0, st>>>(static_cast<const T*>(out_cm), lse_cm, \
                                                                                static_cast<T*>(merged), row_lse, rows, s.N, s.R, s.L)
  if (dtype == UA_BF16 && s.D == 64) UA_MERGE_FWD(bf16, 8);
  else if (dtype == UA_BF16 && s.D == 128) UA_MERGE_FWD(bf16, 16);
  else if (dtype == UA_BF16 && s.D == 32) UA_MERGE_FWD(bf16, 4);
  else if (dtype == UA_BF16 && s.D == 16) UA_MERGE_FWD(bf16, 2);
  else if (dtype == UA_BF16 && s.D == 8) UA_MERGE_FWD(bf16, 1);
  else if (dtype == UA_F32 && s.D == 128) UA_MERGE_FWD(float, 32);
  else if (dtype == UA_F32 && s.D == 64) UA_MERGE_FWD(float, 16);
  else if (dtype == UA_F32 && s.D == 32) UA_MERGE_FWD(float, 8);
  else if (dtype == UA_F32 && s.D == 16) UA_MERGE_FWD(float, 4);
  else if (dtype == UA_F32 && s.D == 8) UA_MERGE_FWD(float, 2);
  else if (dtype == UA_F32 && s.D == 4) UA_MERGE_FWD(float, 1);
  else return UA_ERR_UNSUPPORTED;
#undef UA_MERGE_FWD
  return cudaGetLastError() == cudaSuccess ? UA_OK : UA_ERR_CUDA;
}

size_t ua_fwd_merged_workspace_bytes(const UaDims* dims, int dtype) {
  if (check_dims(dims) != UA_OK) return 0;
  ua::Shape s = to_shape(dims);
  if (!ua::sm100::fwd_supported(s, dtype)) return 0;
  const size_t BH = (size_t)s.B * s.H;
  return 256 + align_up(BH * s.N * (size_t)s.R * s.L * sizeof(float), 256) + align_up(BH * s.R * (size_t)s.L * s.D * sizeof(float), 256);
}

int ua_fwd_merged(const UaDims* dims, int dtype, int gate_dtype, const void* kc, const void* vc, const void* xq,
                  const void* static_src, const void* static_dest, void* merged, float* row_lse, void* carry_out,
                  void* workspace, size_t workspace_bytes, void* stream) {
  int e = check_dims(dims);
  if (e) return e;
  if (!dtype_ok(dtype, gate_dtype)) return UA_ERR_BAD_DTYPE;
  if (!kc || !vc || !xq || !static_src || !static_dest || !merged || !row_lse) return UA_ERR_NULL_POINTER;
  if (!aligned16(kc) || !aligned16(vc) || !aligned16(xq) || !aligned16(merged)) return UA_ERR_ALIGNMENT;
  ua::Shape s = to_shape(dims);
  if (!ua::sm100::fwd_supported(s, dtype)) return UA_ERR_UNSUPPORTED;
  const size_t need = ua_fwd_merged_workspace_bytes(dims, dtype);
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u)) return UA_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  char* ws = static_cast<char*>(workspace);
  const size_t BH = (size_t)s.B * s.H;
  float* lse_cm = reinterpret_cast<float*>(ws + 256);
  float* acc = reinterpret_cast<float*>(ws + 256 + align_up(BH * s.N * (size_t)s.R * s.L * sizeof(float), 256));
  if (cudaMemsetAsync(ws, 0, 256, st) != cudaSuccess) return UA_ERR_CUDA;
  if (cudaMemsetAsync(acc, 0, BH * s.R * (size_t)s.L * s.D * sizeof(float), st) != cudaSuccess) return UA_ERR_CUDA;
  // pass 1: the per-chunk log-sum-exp of every row (no output tile is written) and, on request, the decay-prefix table
  ua::sm100::FwdParams fp{};
  fp.s = s; fp.ssrc = static_src; fp.sdest = static_dest; fp.out = nullptr; fp.denom = nullptr; fp.lse = lse_cm;
  fp.status = reinterpret_cast<int*>(ws);
  fp.carry = ua_carry_bytes(dims, dtype, 0) ? static_cast<float*>(carry_out) : nullptr;
  ua::sm100::whole_sequence(fp);
  if ((e = ua::sm100::launch_fwd<false>(s, gate_dtype, kc, vc, xq, fp, false, st))) return e;
  // the row's log-sum-exp over all key chunks
  row_lse_kernel<<<148 * 8, 256, 0, st>>>(lse_cm, row_lse, BH, s.N, s.R, s.L);
  if (cudaGetLastError() != cudaSuccess) return UA_ERR_CUDA;
  // pass 2: every (chunk, row tile, head) adds exp(m - row_lse) P~ V to the fp32 merged accumulator
  fp.lse = nullptr; fp.carry = nullptr; fp.merged_acc = acc; fp.row_lse = row_lse;
  if ((e = ua::sm100::launch_fwd_merge(s, gate_dtype, kc, vc, xq, fp, st))) return e;
  return convert_any(dtype, acc, merged, BH * s.R * (size_t)s.L * s.D, st);
}

int ua_row_dot(long long rows, int head_dim, int dtype, const void* a, const void* b, float* out, void* stream) {
  if (rows <= 0 || head_dim <= 0) return UA_ERR_BAD_DIMS;
  if (dtype != UA_F32 && dtype != UA_BF16) return UA_ERR_BAD_DTYPE;
  if (!a || !b || !out) return UA_ERR_NULL_POINTER;
  if (!aligned16(a) || !aligned16(b)) return UA_ERR_ALIGNMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int tpr = head_dim * (dtype == UA_F32 ? 4 : 2) / 16;
  if (tpr < 1 || tpr > 32 || (tpr & (tpr - 1)) || tpr * 16 != head_dim * (dtype == UA_F32 ? 4 : 2)) return UA_ERR_UNSUPPORTED;
  const unsigned blocks = (unsigned)((rows * tpr + ua::aux::kMergeThreads - 1) / ua::aux::kMergeThreads);
#define UA_ROW_DOT(T, TPR) \
  ua::aux::row_dot_kernel<T, TPR><<<blocks, ua::aux::kMergeThreads, 0, st>>>(static_cast<const T*>(a), static_cast<const T*>(b), out, rows)
  if (dtype == UA_BF16) {
    if (tpr == 16) UA_ROW_DOT(bf16, 16); else if (tpr == 8) UA_ROW_DOT(bf16, 8); else if (tpr == 4) UA_ROW_DOT(bf16, 4);
    else if (tpr == 2) UA_ROW_DOT(bf16, 2); else if (tpr == 1) UA_ROW_DOT(bf16, 1); else return UA_ERR_UNSUPPORTED;
  } else {
    if (tpr == 32) UA_ROW_DOT(float, 32); else if (tpr == 16) UA_ROW_DOT(float, 16); else if (tpr == 8) UA_ROW_DOT(float, 8);
    else if (tpr == 4) UA_ROW_DOT(float, 4); else if (tpr == 2) UA_ROW_DOT(float, 2); else UA_ROW_DOT(float, 1);
  }
#undef UA_ROW_DOT
  return cudaGetLastError() == cudaSuccess ? UA_OK : UA_ERR_CUDA;
}

int ua_bwd_merged(const UaDims* dims, int dtype, int gate_dtype, const void* kc, const void* vc, const void* xq,
                  const void* static_src, const void* static_dest, const void* g_merged, const float* row_lse,
                  const float* row_delta, const void* carry_in, void* dkc, void* dvc, void* dxq, void* dstatic_src,
                  void* dstatic_dest, void* workspace, size_t workspace_bytes, void* stream) {
  int e = check_dims(dims);
  if (e) return e;
  if (!dtype_ok(dtype, gate_dtype)) return UA_ERR_BAD_DTYPE;
  if (!kc || !vc || !xq || !static_src || !static_dest || !g_merged || !row_lse || !row_delta || !dkc || !dvc || !dxq ||
      !dstatic_src || !dstatic_dest)
    return UA_ERR_NULL_POINTER;
  if (!aligned16(kc) || !aligned16(vc) || !aligned16(xq) || !aligned16(g_merged) || !aligned16(dvc) || !aligned16(dkc) ||
      !aligned16(dxq))
    return UA_ERR_ALIGNMENT;
  ua::Shape s = to_shape(dims);
  if (!ua::sm100::bwd2_supported(s, dtype)) return UA_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BwdWorkspaceTc w = bwd_layout_tc(s);
  if (!workspace || workspace_bytes < w.total || (reinterpret_cast<uintptr_t>(workspace) & 255u)) return UA_ERR_WORKSPACE;
  char* ws = static_cast<char*>(workspace);
  if (cudaMemsetAsync(ws, 0, w.acc_bytes, st) != cudaSuccess) return UA_ERR_CUDA;
  float* carry_tab = carry_in ? const_cast<float*>(static_cast<const float*>(carry_in)) : reinterpret_cast<float*>(ws + w.off_carry);
  if (!carry_in) {
    ua::sm100::FwdParams fp{};
    fp.s = s; fp.ssrc = static_src; fp.sdest = static_dest; fp.out = nullptr; fp.lse = nullptr; fp.denom = nullptr;
    fp.status = reinterpret_cast<int*>(ws); fp.carry = carry_tab;
    ua::sm100::whole_sequence(fp);
    if ((e = ua::sm100::launch_fwd<true>(s, gate_dtype, kc, nullptr, nullptr, fp, false, st))) return e;
  }
  ua::sm100::Bwd2Params qp{};
  if (!aligned16(row_lse) || !aligned16(row_delta) || !aligned16(static_dest) || !aligned16(carry_tab)) return UA_ERR_ALIGNMENT;
  qp.s = s; ua::sm100::whole_sequence(qp); qp.ssrc = static_src; qp.sdest = static_dest; qp.g_denom = nullptr;
  qp.lse = nullptr; qp.row_lse = row_lse; qp.row_delta = row_delta; qp.carry = carry_tab;
  qp.acc_dk = reinterpret_cast<float*>(ws + w.off_dk);
  qp.acc_dq = reinterpret_cast<float*>(ws + w.off_dq);
  qp.acc_dt = reinterpret_cast<float*>(ws + w.off_dt);
  qp.acc_dkr = reinterpret_cast<float*>(ws + w.off_dkr);
  qp.dvc = static_cast<bf16*>(dvc); qp.dss = dstatic_src; qp.status = reinterpret_cast<int*>(ws);
  qp.trace = nullptr;
  e = ua::sm100::launch_bwd2(s, gate_dtype, true, kc, vc, xq, g_merged, qp, st);
  if (e) return e;
  const size_t BHs = (size_t)s.B * s.H;
  if ((e = convert_any(dtype, qp.acc_dk, dkc, BHs * s.L * s.D, st))) return e;
  if ((e = convert_any(dtype, qp.acc_dq, dxq, BHs * s.R * s.L * s.D, st))) return e;
  if ((e = convert_any(gate_dtype, qp.acc_dt, dstatic_dest, BHs * s.L, st))) return e;
  return UA_OK;
}

int ua_merge_bwd(const UaDims* dims, int dtype, const void* out_cm, const float* lse_cm, const void* g_merged,
                 void* g_out_cm, float* g_lse_cm, int flags, void* stream) {
  int e = check_dims(dims);
  if (e) return e;
  if (dtype != UA_F32 && dtype != UA_BF16) return UA_ERR_BAD_DTYPE;
  if (!out_cm || !lse_cm || !g_merged || !g_out_cm || !g_lse_cm) return UA_ERR_NULL_POINTER;
  if (!aligned16(out_cm) || !aligned16(g_merged) || !aligned16(g_out_cm)) return UA_ERR_ALIGNMENT;
  ua::Shape s = to_shape(dims);
  const long long rows = (long long)s.B * s.H * s.R * s.L;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int tpr = s.D * (dtype == UA_F32 ? 4 : 2) / 16;
  const unsigned blocks = (unsigned)((rows * tpr + ua::aux::kMergeThreads - 1) / ua::aux::kMergeThreads);
  const int skip = (flags & UA_FLAG_SKIP_MASKED_FILL) ? 1 : 0;
#define UA_MERGE_BWD(T, TPR)                                                                                          \
  ua::aux::merge_bwd_kernel<T, TPR><<<blocks, ua::aux::kMergeThreads, 0, st>>>(                                       \
      static_cast<const T*>(out_cm), lse_cm, static_cast<const T*>(g_merged), static_cast<T*>(g_out_cm), g_lse_cm, rows, \
      s.N, s.R, s.L, skip)
  if (dtype == UA_BF16 && s.D == 64) UA_MERGE_BWD(bf16, 8);
  else if (dtype == UA_BF16 && s.D == 128) UA_MERGE_BWD(bf16, 16);
  else if (dtype == UA_BF16 && s.D == 32) UA_MERGE_BWD(bf16, 4);
  else if (dtype == UA_BF16 && s.D == 16) UA_MERGE_BWD(bf16, 2);
  else if (dtype == UA_BF16 && s.D == 8) UA_MERGE_BWD(bf16, 1);
  else if (dtype == UA_F32 && s.D == 128) UA_MERGE_BWD(float, 32);
  else if (dtype == UA_F32 && s.D == 64) UA_MERGE_BWD(float, 16);
  else if (dtype == UA_F32 && s.D == 32) UA_MERGE_BWD(float, 8);
  else if (dtype == UA_F32 && s.D == 16) UA_MERGE_BWD(float, 4);
  else if (dtype == UA_F32 && s.D == 8) UA_MERGE_BWD(float, 2);
  else if (dtype == UA_F32 && s.D == 4) UA_MERGE_BWD(float, 1);
  else return UA_ERR_UNSUPPORTED;
#undef UA_MERGE_BWD
  return cudaGetLastError() == cudaSuccess ? UA_OK : UA_ERR_CUDA;
}

}  // extern "C"
