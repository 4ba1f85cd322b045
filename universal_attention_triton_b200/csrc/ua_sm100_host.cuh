// Host-side launchers of the sm_100a tensor-core kernels: TMA descriptor
// construction and launch configuration.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/ua_b200.h"
#include "ua_bwd2_sm100.cuh"
#include "ua_bwd_masked_sm100.cuh"
#include "ua_fwd_sm100.cuh"

namespace ua {
namespace sm100 {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
    if (q != cudaDriverEntryPointSuccess) return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// 2-D bf16 tensor [rows][D] row-major, boxes of box_rows (128 or 64) rows x 64 elements, 128-byte swizzle.
inline bool make_rows_map(CUtensorMap* map, const void* base, uint64_t rows, int D, int box_rows = 128) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t gdim[2] = {(cuuint64_t)D, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)D * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// 2-D fp32 tensor [rows][64] row-major (the dQ / dK accumulators), boxes of 128 rows x 32 floats, 128-byte swizzle:
// the target of the backward kernel's shared-memory -> global reductions.
inline bool make_f32_rows_map(CUtensorMap* map, const void* base, uint64_t rows, int D = 64, int box_rows = 128) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t gdim[2] = {(cuuint64_t)D, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)D * 4};
  cuuint32_t box[2] = {32, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

inline bool fwd_supported(const Shape& s, int dtype) {
  return dtype == UA_BF16 && s.C == 128 && (s.D == 64 || s.D == 128);
}

// Fills the row-range fields of FwdParams for a call over the whole sequence.
inline void whole_sequence(FwdParams& p) {
  p.j_begin = 0; p.j_end = p.s.N; p.Lr = p.s.L; p.r0 = 0; p.carry_in = nullptr; p.total_out = nullptr;
}

// Forward (kCarryOnly = false) or decay-only pass (kCarryOnly = true: no values, queries or outputs) over the row
// tiles [p.j_begin, p.j_end).  xq / static_dest / out hold p.Lr rows; keys, values, static_src the whole sequence.
template <int D, typename TG, bool kCarryOnly, int kOut = kOutTiles>
int launch_fwd_t(const Shape& s, const void* kc, const void* vc, const void* xq, const FwdParams& p, bool fill_masked,
                 cudaStream_t st) {
  using Cfg = FwdCfg<D>;
  CUtensorMap tmK, tmV, tmQ;
  const uint64_t BH = (uint64_t)s.B * s.H;
  if (!make_rows_map(&tmK, kc, BH * s.L, D)) return UA_ERR_CUDA;
  if (kCarryOnly) {
    tmV = tmK; tmQ = tmK;          // not used by the decay-only pass
  } else if (!make_rows_map(&tmV, vc, BH * s.L, D) || !make_rows_map(&tmQ, xq, BH * s.R * p.Lr, D)) {
    return UA_ERR_CUDA;
  }
  // without an output tensor only the log-sum-exp (and the decay-prefix table) is wanted: the statistics-only kernel
  auto kern = (!kCarryOnly && kOut == kOutTiles && p.out == nullptr) ? fwd_kernel<D, TG, kCarryOnly, kOutStats>
                                                                     : fwd_kernel<D, TG, kCarryOnly, kOut>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess) return UA_ERR_CUDA;
  FwdParams q = p;
  q.vc = vc;
  q.fill_masked = (fill_masked && !kCarryOnly) ? 1 : 0;
  kern<<<(unsigned)(BH * s.N), 512, Cfg::kSmemBytes, st>>>(tmK, tmV, tmQ, q);
  return cudaGetLastError() == cudaSuccess ? UA_OK : UA_ERR_CUDA;
}

template <bool kCarryOnly>
int launch_fwd(const Shape& s, int gate_dtype, const void* kc, const void* vc, const void* xq, const FwdParams& p,
               bool fill_masked, cudaStream_t st) {
  if (s.D == 64) {
    return gate_dtype == UA_F32 ? launch_fwd_t<64, float, kCarryOnly>(s, kc, vc, xq, p, fill_masked, st)
                                : launch_fwd_t<64, __nv_bfloat16, kCarryOnly>(s, kc, vc, xq, p, fill_masked, st);
  }
  return gate_dtype == UA_F32 ? launch_fwd_t<128, float, kCarryOnly>(s, kc, vc, xq, p, fill_masked, st)
                              : launch_fwd_t<128, __nv_bfloat16, kCarryOnly>(s, kc, vc, xq, p, fill_masked, st);
}

// The forward in merged-output mode (p.merged_acc, p.row_lse set; nothing is written to out / lse / denom).
inline int launch_fwd_merge(const Shape& s, int gate_dtype, const void* kc, const void* vc, const void* xq, const FwdParams& p,
                            cudaStream_t st) {
  if (s.D == 64) {
    return gate_dtype == UA_F32 ? launch_fwd_t<64, float, false, kOutMerged>(s, kc, vc, xq, p, false, st)
                                : launch_fwd_t<64, __nv_bfloat16, false, kOutMerged>(s, kc, vc, xq, p, false, st);
  }
  return gate_dtype == UA_F32 ? launch_fwd_t<128, float, false, kOutMerged>(s, kc, vc, xq, p, false, st)
                              : launch_fwd_t<128, __nv_bfloat16, false, kOutMerged>(s, kc, vc, xq, p, false, st);
}

// Shapes of the keys-on-lanes backward kernel.
inline bool bwd2_supported(const Shape& s, int dtype) { return dtype == UA_BF16 && s.C == 128 && (s.D == 64 || s.D == 128); }

// Columns of a half tile per worker thread: 16 (sixteen worker warps, 96 registers each) at head_dim 64, 32 (eight worker
// warps, ~200 registers each) at head_dim 128.  At head_dim 64 sixteen warps (four per scheduler hide the TMEM and
// shared-memory latencies) that hand dS over at once are 5-6 % faster than eight that defer the tail of a head, in every
// build; sixteen that defer are slower than either (measured).
#ifndef UA_BWD2_COLS_64
#define UA_BWD2_COLS_64 16
#endif
#ifndef UA_BWD2_COLS_128
#define UA_BWD2_COLS_128 32
#endif
template <int D> constexpr int bwd2_cols() { return D == 64 ? UA_BWD2_COLS_64 : UA_BWD2_COLS_128; }

// Fills the row-range fields of Bwd2Params for a call over the whole sequence.
inline void whole_sequence(Bwd2Params& p) {
  p.j_begin = 0; p.j_end = p.s.N; p.Lr = p.s.L; p.r0 = 0; p.heads = p.s.R;
  p.suffix_in = nullptr; p.dctot_out = nullptr; p.acc_dv = nullptr; p.acc_ds = nullptr;
}

// Backward over the row tiles [p.j_begin, p.j_end) (the caller sets the range fields, e.g. with whole_sequence()).
// With p.heads == 0 (correction pass) xq, g_out and p.acc_dq are not touched and may be null.
template <int D, typename TG, int kMode>
int launch_bwd2_t(const Shape& s, const void* kc, const void* vc, const void* xq, const void* g_out, const Bwd2Params& p,
                  cudaStream_t st) {
  using Cfg = Bwd2Cfg<D>;
  CUtensorMap tmK, tmV, tmQ, tmG, tmDQ, tmDK;
  const uint64_t BH = (uint64_t)s.B * s.H;
  if (!make_rows_map(&tmK, kc, BH * s.L, D, 64) || !make_rows_map(&tmV, vc, BH * s.L, D, 64) ||
      !make_f32_rows_map(&tmDK, p.acc_dkr, BH * s.L, D, 64))
    return UA_ERR_CUDA;
  if (p.heads == 0) {
    tmQ = tmK; tmG = tmK; tmDQ = tmDK;       // never used
  } else if (!make_rows_map(&tmQ, xq, BH * s.R * p.Lr, D, 64) ||
             !make_rows_map(&tmG, g_out, (kMode == 2 ? BH : BH * s.N) * s.R * p.Lr, D, 64) ||
             !make_f32_rows_map(&tmDQ, p.acc_dq, BH * s.R * p.Lr, D, 64)) {
    return UA_ERR_CUDA;
  }
  constexpr int kCols = bwd2_cols<D>();
  auto kern = p.heads > 0 ? bwd2_kernel<D, TG, kMode, kCols, true> : bwd2_kernel<D, TG, kMode, kCols, false>;
  const int threads = 32 * (8 + 4 * (64 / kCols));
  // the forward's output tiles at hand (per-chunk form, head_dim 64): the row term comes from them
  CUtensorMap tmO = tmG;
  if constexpr (kMode == 1 && Cfg::kOutTiles) {
    if (p.heads > 0 && p.out_tiles != nullptr) {
      if (!make_rows_map(&tmO, p.out_tiles, BH * s.N * s.R * p.Lr, D, 64)) return UA_ERR_CUDA;
      kern = bwd2_kernel<D, TG, 1, kCols, true, true>;
    }
  }
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess) return UA_ERR_CUDA;
  kern<<<(unsigned)(BH * s.N), threads, Cfg::kSmemBytes, st>>>(tmK, tmV, tmQ, tmG, tmDQ, tmDK, tmO, p);
  // the row-side dK joins the accumulator; d static_dest of the range's rows comes out of it
  const int row_begin = p.j_begin * 128, row_end = p.j_end * 128;
  const long long warps = (long long)BH * (row_end - row_begin);
  if (warps > 0)
    row_side_finish_kernel<D, TG><<<(unsigned)((warps + 7) / 8), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(kc), static_cast<const TG*>(p.sdest), p.acc_dkr, p.acc_dk, p.acc_dt, (int)BH, s.L, p.Lr,
        p.r0, row_begin, row_end);
  return cudaGetLastError() == cudaSuccess ? UA_OK : UA_ERR_CUDA;
}

inline int launch_bwd2(const Shape& s, int gate_dtype, bool merged, const void* kc, const void* vc, const void* xq,
                       const void* g_out, const Bwd2Params& p, cudaStream_t st) {
#define UA_BWD2(D_, TG_) (merged ? launch_bwd2_t<D_, TG_, 2>(s, kc, vc, xq, g_out, p, st) : launch_bwd2_t<D_, TG_, 1>(s, kc, vc, xq, g_out, p, st))
  if (s.D == 64) return gate_dtype == UA_F32 ? UA_BWD2(64, float) : UA_BWD2(64, __nv_bfloat16);
  return gate_dtype == UA_F32 ? UA_BWD2(128, float) : UA_BWD2(128, __nv_bfloat16);
#undef UA_BWD2
}

// Fills the row-range fields of MaskedParams for a call over the whole sequence.
inline void whole_sequence(MaskedParams& p) {
  p.j_begin = 0; p.j_end = p.s.N; p.Lr = p.s.L; p.r0 = 0; p.acc_dv = nullptr;
}

// Rows before a chunk over the row tiles [p.j_begin, p.j_end): prep (per-chunk constants), sweep (one pass over the upstream
// gradient), finish (dK_i, and dV_i for a row range).  The caller has zeroed (or shares) acc_dq / acc_dk / acc_dv.
template <int D>
int launch_masked_t(const Shape& s, const void* kc, const void* vc, const void* xq, const void* g_out, float* acc_dq, MaskedParams p,
                    cudaStream_t st) {
  using Cfg = MkCfg<D>;
  const uint64_t BH = (uint64_t)s.B * s.H;
  CUtensorMap tmQ, tmG, tmDQ;
  if (!make_rows_map(&tmQ, xq, BH * s.R * p.Lr, D) || !make_rows_map(&tmG, g_out, BH * s.N * s.R * p.Lr, D) ||
      !make_f32_rows_map(&tmDQ, acc_dq, BH * s.R * p.Lr, D))
    return UA_ERR_CUDA;
  static const int jp_env = []() { const char* e = getenv("UA_MASKED_TILES"); return e ? atoi(e) : 0; }();
  p.jp = jp_env > 0 ? jp_env : 8;
  p.items_per_bh = 0;
  const int jcap = (s.N - 1 < p.j_end) ? s.N - 1 : p.j_end;      // no row tile at or after the last chunk is before any chunk
  for (int g = 0; g * Cfg::kG < s.N; ++g) {
    int jmax = (((g + 1) * Cfg::kG < s.N) ? (g + 1) * Cfg::kG : s.N) - 1;
    if (jmax > jcap) jmax = jcap;
    if (jmax > p.j_begin) p.items_per_bh += (jmax - p.j_begin + p.jp - 1) / p.jp;
  }
  if (p.items_per_bh == 0) return UA_OK;
  const auto* k16 = static_cast<const __nv_bfloat16*>(kc);
  const auto* v16 = static_cast<const __nv_bfloat16*>(vc);
  const int prep_smem = 2 * 128 * D * 2 + 2 * D * 4;
  auto prep = masked_prep_kernel<D>;
  if (cudaFuncSetAttribute(prep, cudaFuncAttributeMaxDynamicSharedMemorySize, prep_smem) != cudaSuccess) return UA_ERR_CUDA;
  prep<<<(unsigned)(BH * s.N), 256, prep_smem, st>>>(k16, v16, p);
  auto sweep = masked_sweep_kernel<D>;
  if (cudaFuncSetAttribute(sweep, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess) return UA_ERR_CUDA;
  sweep<<<(unsigned)(BH * p.items_per_bh * Cfg::kKB), 384, Cfg::kSmemBytes, st>>>(tmQ, tmG, tmDQ, p);
  masked_finish_kernel<D><<<(unsigned)(BH * s.N), 128, 0, st>>>(v16, p);
  return cudaGetLastError() == cudaSuccess ? UA_OK : UA_ERR_CUDA;
}

inline int launch_masked(const Shape& s, const void* kc, const void* vc, const void* xq, const void* g_out, float* acc_dq,
                         const MaskedParams& p, cudaStream_t st) {
  return s.D == 64 ? launch_masked_t<64>(s, kc, vc, xq, g_out, acc_dq, p, st) : launch_masked_t<128>(s, kc, vc, xq, g_out, acc_dq, p, st);
}

}  // namespace sm100
}  // namespace ua
