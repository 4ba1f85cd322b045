/*
 * C ABI of the B200 (sm_100a) Universal Attention library  --  libua_b200.so
 *
 * Plain pointers and sizes only; every pointer is DEVICE memory owned by the
 * caller, every call is asynchronous on the given CUDA stream (passed as a
 * void* holding a cudaStream_t; NULL = the default stream), nothing is
 * allocated, nothing synchronises.  Return value: 0 on success, otherwise a
 * UA_ERR_* code (ua_error_string() gives the text).  The library keeps no
 * state between calls and may be called from any host thread.
 *
 * These entry points are what a binding of the reference's operator boundary
 * attaches to.  Reference interfaces they replace:
 *   - UniversalAttention.forward / .backward, 1-D signature
 *       universal_attention_autograd.py:9-38, :47-99
 *   - UniversalAttention2.forward / .backward, 2-D signature
 *       universal_attention_autograd.py:104-163, :172-276
 *   - the Triton launchers _universal_attention_fwd / _universal_attention_bwd
 *       Universal_Attention/triton/universal_attention_kernel.py:192-239, :793-862
 *   - SMVecMatMul (merge over key chunks)
 *       universal_attention_autograd.py:278-297
 *
 * Tensor layouts.  b = batch, h = kv heads, r = query heads per kv head,
 * n = key chunks, c = keys per chunk, L = n*c rows, d = head dim.
 *   kc, vc        (b,h,n,c,d)   contiguous                    [dtype]
 *   xq            (b,h,r,L,d)   contiguous (the 2-D form (b,h,r,_n,_c,d) is the same memory)
 *   static_src    (b,h,n,c)     gates in (0,1)                [gate_dtype]
 *   static_dest   (b,h,L)       gates in (0,1)                [gate_dtype]
 *   out_cm        (b,h,n,r,L,d) "chunk-major": the reference's out (b,h,r,L,d,n)
 *                               is out_cm viewed with its axes permuted (0,1,3,4,5,2)
 *   lse_cm        (b,h,n,r,L)   fp32 log-sum-exp per (row, key chunk); the
 *                               reference's denom (b,h,r,L,n) is the (0,1,3,4,2) view
 *   denom_cm      (b,h,n,r,L)   lse rounded to dtype (may be NULL)
 */
#ifndef UA_B200_H_
#define UA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct UaDims {
  int32_t batch;      /* b  */
  int32_t kv_heads;   /* h  */
  int32_t q_per_kv;   /* r  */
  int32_t n_chunks;   /* n_ */
  int32_t chunk;      /* c_ */
  int32_t head_dim;   /* d  */
} UaDims;

enum { UA_F32 = 0, UA_BF16 = 1 };

enum {
  UA_OK = 0,
  UA_ERR_BAD_DIMS = 1,       /* non-positive dims, chunk not a multiple of 16, head_dim not a multiple of 4 ... */
  UA_ERR_BAD_DTYPE = 2,
  UA_ERR_NULL_POINTER = 3,
  UA_ERR_WORKSPACE = 4,      /* workspace missing, too small or not 256-byte aligned */
  UA_ERR_UNSUPPORTED = 5,    /* no kernel for this shape (tile does not fit shared memory) */
  UA_ERR_CUDA = 6,           /* a CUDA runtime call failed; cudaGetLastError() has the cause */
  UA_ERR_ALIGNMENT = 7,      /* a tensor pointer is not 16-byte aligned */
  UA_ERR_DEVICE = 8,         /* wrong GPU architecture (needs compute capability 10.x) */
  UA_ERR_TIMEOUT = 9,        /* a bounded device-side wait ran out; reported by ua_workspace_status() */
  UA_ERR_STATIC_LIMIT = 10   /* ua_bwd_static: the problem needs more scratch than UA_STATIC_SCRATCH_BYTES */
};

/* Flags for ua_fwd / ua_bwd. */
enum {
  /* Backward: skip the gradient that flows through fully masked blocks (rows
   * before a key chunk, where the reference's softmax is uniform).  That
   * gradient is exactly zero whenever SMVecMatMul consumes (out, denom), as in
   * the reference driver (main.py:55-62); it is non-zero for arbitrary
   * upstream gradients (universal_attention_kernel.py:1261-1262). */
  UA_FLAG_SKIP_MASKED_GRADS = 1,
  /* Forward: do not write the fully masked blocks of out/lse/denom (the caller
   * promises never to read them). */
  UA_FLAG_SKIP_MASKED_FILL = 2,
  /* Force the generic fp32 SIMT kernels even where a tensor-core kernel exists. */
  UA_FLAG_FORCE_SIMT = 4
};

int ua_version(void);
const char* ua_error_string(int code);

/* Bytes of scratch ua_fwd / ua_bwd need for these dims (256-byte aligned
 * device memory, contents irrelevant on entry; the first word holds the
 * status read by ua_workspace_status(), the rest is garbage on exit). */
size_t ua_fwd_workspace_bytes(const UaDims* dims, int dtype, int flags);
size_t ua_bwd_workspace_bytes(const UaDims* dims, int dtype, int flags);

/* Forward.  Replaces UniversalAttention(2).forward (universal_attention_autograd.py:9-38,
 * :104-163) and _universal_attention_fwd (universal_attention_kernel.py:192-239).
 * Writes out_cm, lse_cm and, if not NULL, denom_cm. */
int ua_fwd(const UaDims* dims, int dtype, int gate_dtype,
           const void* kc, const void* vc, const void* xq,
           const void* static_src, const void* static_dest,
           void* out_cm, float* lse_cm, void* denom_cm,
           void* workspace, size_t workspace_bytes, int flags, void* stream);

/* Backward.  Replaces UniversalAttention(2).backward (universal_attention_autograd.py:47-99,
 * :172-276) and _universal_attention_bwd (universal_attention_kernel.py:793-862).
 * Only the five inputs are needed (everything is recomputed, as the reference
 * does: universal_attention_autograd.py:166-169).  g_out_cm has the layout of
 * out_cm, g_denom_cm that of lse_cm with element type g_denom_dtype (the
 * reference receives fp32 there under mixed precision, :48).  Gradients have
 * the layout and dtype of their inputs and are overwritten. */
int ua_bwd(const UaDims* dims, int dtype, int gate_dtype,
           const void* kc, const void* vc, const void* xq,
           const void* static_src, const void* static_dest,
           const void* g_out_cm, const void* g_denom_cm, int g_denom_dtype,
           void* dkc, void* dvc, void* dxq, void* dstatic_src, void* dstatic_dest,
           void* workspace, size_t workspace_bytes, int flags, void* stream);

/* Optional hand-over of the decay-prefix table from forward to backward.  The
 * backward sweeps the rows downwards and needs, per key and row tile, the decay
 * prefix at the start of the tile; by default ua_bwd recomputes that table with a
 * pre-pass.  ua_fwd_keep() is ua_fwd() that also stores the table it has in
 * registers anyway into carry_out (ua_carry_bytes() bytes, fp32; 0 bytes means
 * this shape has no table and carry_out is ignored), and ua_bwd_kept() is ua_bwd()
 * that reads it from carry_in instead of running the pre-pass (carry_in may be
 * NULL: then it is ua_bwd()).  lse_cm (optional, NULL allowed): the fp32
 * log-sum-exp (b,h,n,r,L) that the forward wrote; with it the tensor-core backward
 * forms the probabilities as exp(s - lse) and skips its per-row max / sum (other
 * kernels ignore it).  Same inputs must be given to both calls.  The
 * reference keeps nothing but the five inputs (universal_attention_autograd.py:
 * 166-169); this is the "tiny extra saved tensor" variant of the same recompute. */
size_t ua_carry_bytes(const UaDims* dims, int dtype, int flags);
int ua_fwd_keep(const UaDims* dims, int dtype, int gate_dtype,
                const void* kc, const void* vc, const void* xq,
                const void* static_src, const void* static_dest,
                void* out_cm, float* lse_cm, void* denom_cm, void* carry_out,
                void* workspace, size_t workspace_bytes, int flags, void* stream);
int ua_bwd_kept(const UaDims* dims, int dtype, int gate_dtype,
                const void* kc, const void* vc, const void* xq,
                const void* static_src, const void* static_dest,
                const void* g_out_cm, const void* g_denom_cm, int g_denom_dtype, const void* carry_in,
                const float* lse_cm,
                void* dkc, void* dvc, void* dxq, void* dstatic_src, void* dstatic_dest,
                void* workspace, size_t workspace_bytes, int flags, void* stream);
/* ua_bwd_kept() for a caller that still holds the forward's output tiles out_cm (b,h,n,r,L,d), as an autograd graph does
 * whenever a later node saved them (SMVecMatMul does: universal_attention_autograd.py:286-288).  The softmax gradient
 * needs sum_k P dP per row; since P V = out, that is the dot product of the row's output and its upstream gradient, which
 * the tensor-core kernel then takes from the tiles instead of summing over the keys (about a sixth of its time).  out_cm
 * must be what ua_fwd wrote for the same inputs (rows before a chunk are not read); NULL: ua_bwd_kept().  Kernels
 * other than the tensor-core one ignore it.  The reference recomputes everything (universal_attention_autograd.py:
 * 166-169); its Triton backward has no use for the tiles. */
int ua_bwd_saved(const UaDims* dims, int dtype, int gate_dtype,
                 const void* kc, const void* vc, const void* xq,
                 const void* static_src, const void* static_dest,
                 const void* g_out_cm, const void* g_denom_cm, int g_denom_dtype, const void* carry_in,
                 const float* lse_cm, const void* out_cm,
                 void* dkc, void* dvc, void* dxq, void* dstatic_src, void* dstatic_dest,
                 void* workspace, size_t workspace_bytes, int flags, void* stream);

/* ---- Sequence-chunk sharding (long contexts).  No counterpart in the reference, which is single-device. ----
 *
 * A rank owns one or more contiguous ranges of row tiles (128 rows each) and computes those rows against ALL key
 * chunks.  kc, vc and static_src always cover the whole sequence.  The row-indexed tensors (xq_rows (b,h,r,Ls,d),
 * static_dest_rows (b,h,Ls), out_cm_rows (b,h,n,r,Ls,d), lse/denom_cm_rows (b,h,n,r,Ls), and in the backward
 * g_out_cm_rows, g_denom_cm_rows, dxq_rows_f32, ddest_rows_f32) hold "slabs" of Ls = rows_total rows, in which the
 * range occupies the rows [row_offset, row_offset + 128 * (tile_end - tile_begin)); several ranges (e.g. the two halves
 * of a zig-zag assignment) can share the slabs.  Tensor-core shapes only: bf16, chunk 128, head_dim 64 or 128 forward,
 * head_dim 64 backward; UA_ERR_UNSUPPORTED otherwise.
 *
 *   ua_decay_totals_rows  decay-only pass: total_out (b,h,n,128) = carry_in (or 0) + the sum of every key's
 *                         log-retention over the rows of the range.  Ranks run it first and exchange the totals.
 *   ua_fwd_rows           forward for the rows of the range; carry_in (b,h,n,128) fp32 or NULL (= zeros): per key,
 *                         the sum of its log-retention over ALL rows before the range (= sum of the totals of the
 *                         ranges before it).
 *   ua_bwd_rows           gradients of everything the rows of the range touch, ADDED into caller-zeroed fp32 buffers:
 *                         dk_f32, dv_f32 (b,h,L,d), dsrc_f32 (b,h,L) cover ALL keys (partial sums, to be added over the
 *                         ranges / ranks); dxq_rows_f32 (b,h,r,Ls,d), ddest_rows_f32 (b,h,Ls) the rows of the range.
 *                         carry_in as above.  suffix_in (b,h,n,128) or NULL: reverse decay carry entering from later
 *                         rows.  dctot_out (b,h,n,128) or NULL (overwritten): per key, the sum of the decay-prefix
 *                         gradient dC over the rows of the range -- what the ranges before it need.
 *   ua_bwd_rows_suffix    every gradient is linear in the reverse carry: after exchanging the dctot tables,
 *                         suffix = sum of dctot over the ranges AFTER this one, and this decay-only pass adds what it
 *                         induces into dk_f32, dsrc_f32 and ddest_rows_f32 (no queries, values or upstream gradients).
 * Workspace: 256 bytes, except ua_bwd_rows (ua_bwd_rows_workspace_bytes()) and ua_bwd_rows_suffix
 * (ua_bwd_rows_suffix_workspace_bytes(): an fp32 (b*h, L, d) scratch for the row-side dK, from which d static_dest
 * is taken after the sweep). */
typedef struct UaRows {
  int32_t tile_begin;   /* first row tile of the range (global tile index) */
  int32_t tile_end;     /* one past the last */
  int32_t rows_total;   /* Ls: rows per slab of the row-indexed tensors */
  int32_t row_offset;   /* row of the slab where the range starts (multiple of 128) */
} UaRows;

int ua_decay_totals_rows(const UaDims* dims, int dtype, int gate_dtype, const UaRows* rows,
                         const void* kc, const void* static_src, const void* static_dest_rows,
                         const float* carry_in, float* total_out,
                         void* workspace, size_t workspace_bytes, void* stream);
int ua_fwd_rows(const UaDims* dims, int dtype, int gate_dtype, const UaRows* rows,
                const void* kc, const void* vc, const void* xq_rows,
                const void* static_src, const void* static_dest_rows, const float* carry_in,
                void* out_cm_rows, float* lse_cm_rows, void* denom_cm_rows,
                void* workspace, size_t workspace_bytes, int flags, void* stream);
/* ua_fwd_rows that also hands over the decay-prefix table of the range's row tiles (carry_table_out:
 * ua_carry_bytes(dims, dtype, 0) bytes; entries of other row tiles are left alone, so the ranges of one rank can share
 * one table), for ua_bwd_rows_kept. */
int ua_fwd_rows_keep(const UaDims* dims, int dtype, int gate_dtype, const UaRows* rows,
                     const void* kc, const void* vc, const void* xq_rows,
                     const void* static_src, const void* static_dest_rows, const float* carry_in,
                     void* out_cm_rows, float* lse_cm_rows, void* denom_cm_rows, float* carry_table_out,
                     void* workspace, size_t workspace_bytes, int flags, void* stream);
size_t ua_bwd_rows_workspace_bytes(const UaDims* dims, int dtype);
size_t ua_bwd_rows_suffix_workspace_bytes(const UaDims* dims, int dtype);
int ua_bwd_rows(const UaDims* dims, int dtype, int gate_dtype, const UaRows* rows,
                const void* kc, const void* vc, const void* xq_rows,
                const void* static_src, const void* static_dest_rows,
                const void* g_out_cm_rows, const void* g_denom_cm_rows, int g_denom_dtype,
                const float* carry_in, const float* suffix_in,
                float* dk_f32, float* dv_f32, float* dxq_rows_f32, float* dsrc_f32, float* ddest_rows_f32, float* dctot_out,
                void* workspace, size_t workspace_bytes, int flags, void* stream);
/* ua_bwd_rows given what the forward of the same range produced: carry_table (ua_fwd_rows_keep) and the fp32
 * lse_cm_rows slab (ua_fwd_rows); with both, no part of the forward is run again (carry_in is then not read). */
int ua_bwd_rows_kept(const UaDims* dims, int dtype, int gate_dtype, const UaRows* rows,
                     const void* kc, const void* vc, const void* xq_rows,
                     const void* static_src, const void* static_dest_rows,
                     const void* g_out_cm_rows, const void* g_denom_cm_rows, int g_denom_dtype,
                     const float* carry_in, const float* suffix_in, const float* carry_table, const float* lse_cm_rows,
                     float* dk_f32, float* dv_f32, float* dxq_rows_f32, float* dsrc_f32, float* ddest_rows_f32, float* dctot_out,
                     void* workspace, size_t workspace_bytes, int flags, void* stream);
int ua_bwd_rows_suffix(const UaDims* dims, int dtype, int gate_dtype, const UaRows* rows,
                       const void* kc, const void* vc, const void* static_src, const void* static_dest_rows,
                       const float* suffix, float* dk_f32, float* dsrc_f32, float* ddest_rows_f32,
                       void* workspace, size_t workspace_bytes, void* stream);

/* Backward for callers that must not allocate.  No counterpart in the reference.
 *
 * Some hosts of this library cannot hand it a workspace: an inference or
 * training runtime that has frozen its memory plan, a plugin slot that only
 * passes the operator's inputs and outputs, code running under a memory pool
 * whose owner forbids cudaMalloc after start-up.  ua_bwd_static() is ua_bwd()
 * with the scratch taken from a fixed buffer of UA_STATIC_SCRATCH_BYTES that is
 * part of the library image on the device (every GPU context that loads the
 * library carries it from load until exit, used or not).  The call allocates
 * nothing, neither directly nor through a library.
 *
 *  - Limit: ua_bwd_workspace_bytes(dims, dtype, flags) must not exceed
 *    UA_STATIC_SCRATCH_BYTES (ua_static_scratch_bytes() returns it at run time);
 *    larger problems are refused with UA_ERR_STATIC_LIMIT and nothing is launched.
 *  - The first call on each device looks up the buffer's device address (with that
 *    device current).  Make that first call outside any stream capture.
 *  - There is one buffer per device and every call uses it, so two calls whose
 *    kernels can overlap on the GPU (different streams, no dependency) race; keep
 *    the calls of one device in stream order.  The buffer keeps what the previous
 *    call left; each call first clears the part that has to start at zero.
 *  - ua_static_status() is ua_workspace_status() for this buffer (it synchronises).
 * Inputs, outputs, flags and results are those of ua_bwd(). */
#define UA_STATIC_SCRATCH_BYTES (16u * 1024u * 1024u)
size_t ua_static_scratch_bytes(void);
int ua_bwd_static(const UaDims* dims, int dtype, int gate_dtype,
                  const void* kc, const void* vc, const void* xq,
                  const void* static_src, const void* static_dest,
                  const void* g_out_cm, const void* g_denom_cm, int g_denom_dtype,
                  void* dkc, void* dvc, void* dxq, void* dstatic_src, void* dstatic_dest,
                  int flags, void* stream);
int ua_static_status(void* stream);

/* The kernels never trap and never spin without bound: a device-side wait that
 * runs out makes the kernel give up and set a status word at the start of the
 * workspace it was given.  ua_workspace_status() copies that word back and
 * SYNCHRONISES the stream: 0 = every kernel of the last ua_fwd/ua_bwd call
 * that used this workspace completed, UA_ERR_TIMEOUT otherwise.  After a
 * timeout of the tensor-core backward the second 32-bit word of the workspace
 * says where the first block to give up was waiting:
 * (barrier index + 1) | thread << 8 | (phase & 0x7ff) << 20.  No counterpart
 * in the reference (its kernels have no device-side waits). */
int ua_workspace_status(const void* workspace, void* stream);

/* Self-test of that give-up path, for a host that wants to see it work before it relies on it: launches one block
 * whose two waiters (a single thread and a whole warp, the two forms the kernels use) wait on an mbarrier that
 * nothing ever completes, with a wall-time limit of limit_us microseconds (1 .. 100000) instead of the kernels'
 * 2 s.  The waits run out, the block sets the status word of `workspace` (>= 256 bytes, 256-byte aligned) the way the
 * kernels do and returns; nothing traps and the context stays usable.  ua_workspace_status(workspace) then reports
 * UA_ERR_TIMEOUT, and the second word holds (barrier index + 1) | thread << 8 of the first waiter to give up.
 * No counterpart in the reference. */
int ua_selftest_wait_timeout(void* workspace, size_t workspace_bytes, unsigned limit_us, void* stream);

/* Input prologue.  The reference's driver builds the operator's inputs from token-major projections with transposes
 * and views (main.py:24-31): query_state (b,s,n,d) -> xq (b,n_kv,rep,s,d) (query head kv * rep + r), key_state /
 * value_state (b,s,n_kv,d) -> kc / vc (b,n_kv,s,d) (= (b,n_kv,n_chunks,chunk,d)), gate_state (b,s,2,n_kv) ->
 * static_src, static_dest (b,n_kv,s).  ua_prepare_inputs does this in one pass and, on request, what a model applies
 * on the way (Universal_Attention/triton/_debug.py:470-475): UA_PREP_NORMALIZE_KEYS divides every key by (|k| + 1e-6)
 * (key_norm (b,n_kv,s) fp32 receives |k|: the backward needs it), UA_PREP_SIGMOID_GATES passes the gate logits through a
 * sigmoid.  ua_prepare_inputs_bwd maps the gradients of the five outputs back to the four projections (kc, static_src,
 * static_dest: the forward's outputs).  head_dim * element size must be a multiple of 16 bytes, at most 512. */
enum UaPrepFlags { UA_PREP_NORMALIZE_KEYS = 1, UA_PREP_SIGMOID_GATES = 2 };
int ua_prepare_inputs(int batch, int seq, int n_heads, int n_kv_heads, int head_dim, int dtype, int flags,
                      const void* query_state, const void* key_state, const void* value_state, const void* gate_state,
                      void* xq, void* kc, void* vc, void* static_src, void* static_dest, float* key_norm, void* stream);
int ua_prepare_inputs_bwd(int batch, int seq, int n_heads, int n_kv_heads, int head_dim, int dtype, int flags,
                          const void* g_xq, const void* g_kc, const void* g_vc,
                          const void* g_static_src, const void* g_static_dest,
                          const void* kc, const float* key_norm, const void* static_src, const void* static_dest,
                          void* d_query_state, void* d_key_state, void* d_value_state, void* d_gate_state, void* stream);

/* Incremental (decode) step: row t of the forward against cached keys and values.  No counterpart in the reference
 * (which always processes whole sequences, universal_attention_autograd.py:9-38); it is the serving form of the same
 * arithmetic.  dims: n_chunks * chunk = capacity L_cap of the caches.  k_cache, v_cache (b,h,L_cap,d), src_cache
 * (b,h,L_cap): rows 0..t filled (row t = the new token).  q_t (b,h,r,d), dest_t (b,h): the new row.  decay_state
 * (b,h,L_cap) fp32, in/out: for every key its decay prefix up to the previous row; entries 0..t are updated (zero it
 * before t = 0).  Outputs for the n_t = t / chunk + 1 key chunks that hold keys <= t: out_t (b,h,n_t,r,d) in `dtype`,
 * lse_t (b,h,n_t,r) fp32 -- row t of out_cm / lse_cm of ua_fwd.  Steps must be issued in order t = 0, 1, 2, ...
 * chunk a multiple of 32 up to 1024, q_per_kv <= 8. */
int ua_decode_step(const UaDims* dims, int dtype, int gate_dtype, int t,
                   const void* k_cache, const void* v_cache, const void* src_cache,
                   const void* q_t, const void* dest_t, float* decay_state,
                   void* out_t, float* lse_t, void* stream);

/* Layout converters between chunk-major storage and the reference's contiguous
 * layouts: out (b,h,r,L,d,n) <-> out_cm (b,h,n,r,L,d), with inner = d; and
 * denom (b,h,r,L,n) <-> denom_cm (b,h,n,r,L) with inner = 1.  Element size
 * elem_bytes in {2,4}.  to_reference != 0: chunk-major -> reference layout. */
int ua_relayout(const UaDims* dims, int inner, int elem_bytes, int to_reference,
                const void* src, void* dst, void* stream);

/* Merge over key chunks on chunk-major storage: SMVecMatMul.forward
 * (universal_attention_autograd.py:280-283): merged (b,h,r,L,d) =
 * sum_i softmax_i(lse)[i] * out[..., i].  weights are taken from lse_cm (fp32). */
int ua_merge_fwd(const UaDims* dims, int dtype, const void* out_cm, const float* lse_cm,
                 void* merged, void* stream);

/* ua_merge_fwd that also returns, per row, the log-sum-exp over ALL key chunks: row_lse (b,h,r,L) fp32 (NULL: not
 * wanted).  It is what ua_bwd_merged needs. */
int ua_merge_fwd_stats(const UaDims* dims, int dtype, const void* out_cm, const float* lse_cm,
                       void* merged, float* row_lse, void* stream);

/* The merged output WITHOUT the (b,h,n,r,L,d) tensor `out`: merged (b,h,r,L,d) = SMVecMatMul(UniversalAttention(...))
 * (main.py:55-56; universal_attention_autograd.py:9-38, :278-283) and row_lse (b,h,r,L) fp32, in two passes of the forward
 * kernel: the first leaves only the per-chunk log-sum-exp, the second adds every chunk's share exp(m - row_lse) P~ V to
 * an fp32 accumulator, which is rounded once at the end.  Memory: (b,h,n,r,L) + (b,h,r,L,d) floats of scratch instead of
 * two n-fold tensors; time: about 1.7 forwards.  carry_out as for ua_fwd_keep (NULL allowed).  Pairs with ua_bwd_merged.
 * bf16, chunk 128, head_dim 64 or 128.  No counterpart in the reference. */
size_t ua_fwd_merged_workspace_bytes(const UaDims* dims, int dtype);
int ua_fwd_merged(const UaDims* dims, int dtype, int gate_dtype,
                  const void* kc, const void* vc, const void* xq,
                  const void* static_src, const void* static_dest,
                  void* merged, float* row_lse, void* carry_out,
                  void* workspace, size_t workspace_bytes, void* stream);

/* out[row] = a[row] . b[row] for `rows` rows of head_dim elements (fp32 result).  With a = the gradient of the merged
 * output and b = the merged output this is the row_delta of ua_bwd_merged. */
int ua_row_dot(long long rows, int head_dim, int dtype, const void* a, const void* b, float* out, void* stream);

/* Backward of the COMPOSITION  merged = SMVecMatMul(UniversalAttention(kc, vc, xq, static_src, static_dest))
 * (the flow of the reference's driver, main.py:55-62; operator universal_attention_autograd.py:9-99, merge :278-297)
 * in one kernel, for callers that only consume the merged output (b,h,r,L,d).  The merged output is the softmax over
 * ALL keys of a row, so with row_lse (ua_merge_fwd_stats) and row_delta = g_merged . merged (ua_row_dot) the
 * probabilities are exp(s - row_lse) and dS = P (dP - row_delta): neither the (b,h,n,r,L,d) gradient of `out` nor
 * `out` itself is read, and the rows before a key chunk contribute nothing.  The reference has no fused form; values
 * equal ua_merge_bwd followed by ua_bwd up to rounding (the reference rounds the merge weights and `out` to the input
 * dtype).  carry_in as for ua_bwd_kept (NULL allowed).  Workspace: ua_bwd_workspace_bytes().  bf16, chunk 128,
 * head_dim 64 or 128 (UA_ERR_UNSUPPORTED otherwise: use ua_merge_bwd + ua_bwd). */
int ua_bwd_merged(const UaDims* dims, int dtype, int gate_dtype,
                  const void* kc, const void* vc, const void* xq,
                  const void* static_src, const void* static_dest,
                  const void* g_merged, const float* row_lse, const float* row_delta, const void* carry_in,
                  void* dkc, void* dvc, void* dxq, void* dstatic_src, void* dstatic_dest,
                  void* workspace, size_t workspace_bytes, void* stream);

/* SMVecMatMul.backward (universal_attention_autograd.py:291-297) producing
 * chunk-major gradients: g_out_cm (dtype) and g_lse_cm (fp32).  head_dim must be a
 * power of two between 8 (bf16) / 4 (fp32) and 128.  With UA_FLAG_SKIP_MASKED_FILL the
 * (row, chunk) blocks with row < chunk index * chunk size -- the rows before a key
 * chunk, whose merge weight is exactly zero -- are left unwritten: valid when the consumer is ua_bwd with
 * UA_FLAG_SKIP_MASKED_GRADS, which never reads them. */
int ua_merge_bwd(const UaDims* dims, int dtype, const void* out_cm, const float* lse_cm,
                 const void* g_merged, void* g_out_cm, float* g_lse_cm, int flags, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* UA_B200_H_ */
