/*
 * b200ops.h -- C ABI of the B200 (sm_100a) decode operator library, libb200ops.so.
 *
 * One entry point per operator of the reference's `ascend910a_extras.ops` API.  Each
 * replaces the two-phase CANN pair the reference FFI calls for the same operator,
 *     aclnn<Op>GetWorkspaceSize(tensors..., &workspaceSize, &executor)
 *     aclnn<Op>(workspace, workspaceSize, executor, stream)
 * (call sites are cited per function below, by path inside the reference project).
 *
 * Conventions
 *   - All data pointers are DEVICE pointers of the current CUDA device; tensors are dense,
 *     row-major ("contiguous") with the shapes written beside each argument.
 *   - "f16" = IEEE binary16.  Accumulation is always fp32; results are rounded once (RNE).
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).  Every
 *     call only enqueues work; nothing synchronises.  No call allocates device memory unless
 *     its comment says so: operators that need scratch take a caller-owned `workspace` whose
 *     minimum size comes from the matching *_workspace_size() query (the same split the
 *     reference makes between GetWorkspaceSize and the launch).
 *   - Return value: 0 on success, a negative B200OPS_E* code otherwise.  The failing
 *     thread can read a message with b200ops_last_error().  Argument violations that the
 *     reference reports through TORCH_CHECK are reported as B200OPS_EINVAL with the same
 *     condition.
 *   - There is no CPU path: without a CUDA device every launch returns B200OPS_ECUDA.
 */
#ifndef B200OPS_H_
#define B200OPS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200OPS_OK 0
#define B200OPS_EINVAL (-1)   /* argument check failed                       */
#define B200OPS_ECUDA (-2)    /* a CUDA runtime / driver call failed         */
#define B200OPS_EWORKSPACE (-3) /* workspace pointer null or too small       */
#define B200OPS_EUNSUPPORTED (-4) /* shape outside what the kernels implement */

/* KV-cache layouts understood by reshape_and_cache and paged_attention. */
#define B200OPS_KV_LAYOUT_NZ 0  /* [num_pages, num_kv_heads*head_dim/16, page_size, 16]  (reference-native) */
#define B200OPS_KV_LAYOUT_NHD 1 /* [num_pages, page_size, num_kv_heads, head_dim]        (vLLM standard)    */

/* Library version (major*10000 + minor*100 + patch). */
int b200ops_version(void);

/* Message of the last failure on the calling thread ("" if none). Never NULL. */
const char* b200ops_last_error(void);

/*
 * Tuning variables (B200OPS_GMM_PAIR, B200OPS_GMM_KSPLIT, B200OPS_GMM_SHORT, B200OPS_PA_MODE,
 * B200OPS_PA_STAGES, B200OPS_PA_CHUNK_TOKENS, B200OPS_RMSNORM_VPT, B200OPS_RMSNORM_CTA_WARPS,
 * B200OPS_RAC_DEDUP, B200OPS_PDL) are read from the environment once per process, at their
 * first use; no launch calls getenv after that.  This call forgets what was read, so that the
 * next use looks at the environment again (for tests and tuning sessions that change a
 * variable mid-process).  No counterpart in the reference.
 */
void b200ops_reload_options(void);

/*
 * Device report: SM count, shared memory, L2, memory size/clock/bus, printed to stdout.
 * Replaces native::print_info (csrc/ffi/bind.cpp:26-51).  If `buf` is non-NULL the same
 * text is also copied there (truncated to buf_len, always NUL-terminated).
 */
int b200ops_print_info(int device_id, char* buf, size_t buf_len);

/*
 * Fused residual add + RMSNorm.
 * Replaces aclnnAddRMSNormExGetWorkspaceSize / aclnnAddRMSNormEx (csrc/ffi/ops.cpp:303,308;
 * kernel csrc/opdev/op_kernel/add_rms_norm_ex.cpp:3-123).
 *   s = f16(x + residual); y = f16(s / sqrt(mean(s^2) + eps) * weight); residual_out = s
 *   x, residual, y, residual_out : f16 [num_tokens, dim];  weight : f16 [dim]
 * Requires dim % 64 == 0 (csrc/ffi/ops.cpp:245).  No workspace.
 */
int b200ops_add_rms_norm(const void* x, const void* residual, const void* weight, float eps,
                         void* y, void* residual_out, int64_t num_tokens, int64_t dim,
                         void* stream);

/*
 * SwiGLU: y[t, j] = silu(x[t, j]) * x[t, d + j],  x : f16 [num_tokens, 2*d], y : f16 [num_tokens, d].
 * Replaces aclnnSwiGluExGetWorkspaceSize / aclnnSwiGluEx (csrc/ffi/ops.cpp:138,143; kernel
 * csrc/opdev/op_kernel/swi_glu_ex.cpp:3-68).  `two_d` is x's last dimension; requires
 * two_d >= 64 and two_d % 64 == 0 (csrc/ffi/ops.cpp:113).  No workspace.
 */
int b200ops_swiglu(const void* x, void* y, int64_t num_tokens, int64_t two_d, void* stream);

/*
 * Rotary embedding, half-split ("neox") form, out of place, on q and k in one launch.
 * Replaces aclnnRopeExGetWorkspaceSize / aclnnRopeEx (csrc/ffi/ops.cpp:76,81; kernel
 * csrc/opdev/op_kernel/rope_ex.cpp:3-122).
 *   q, out_q : f16 [bs, num_heads, head_dim];  k, out_k : f16 [bs, num_kv_heads, head_dim]
 *   position_ids : int32 [bs];  cos_cache, sin_cache : f16 [max_pos, head_dim/2]
 *   out[..., :h] = x[..., :h]*cos - x[..., h:]*sin;  out[..., h:] = x[..., h:]*cos + x[..., :h]*sin
 * A position outside [0, max_pos) is an error the device cannot report; rows with such a
 * position are written as zeros and the call still returns 0.  Requires head_dim % 16 == 0.
 */
int b200ops_rope(const void* q, const void* k, const int32_t* position_ids,
                 const void* cos_cache, const void* sin_cache, void* out_q, void* out_k,
                 int64_t bs, int64_t num_heads, int64_t num_kv_heads, int64_t head_dim,
                 int64_t max_pos, void* stream);

/*
 * Scatter this step's K (and optionally V) rows into the paged KV cache, in place.
 * Replaces aclnnReshapeAndCacheExGetWorkspaceSize / aclnnReshapeAndCacheEx
 * (csrc/ffi/ops.cpp:387,394; kernel csrc/opdev/op_kernel/reshape_and_cache_ex.cpp:3-71).
 *   key, value : f16 [num_tokens, num_kv_heads, head_size];  slot_indices : int32 [num_tokens]
 *   cache_dims = the four sizes of key_cache (value_cache has the same shape)
 *   layout NZ  [pages, C, P, 16]:  cache[s/P, c, s%P, j] = flat(key[t])[c*16 + j]  for c*16+j < Hkv*D, c < C
 *   layout NHD [pages, P, Hkv, D]: cache[s/P, s%P, h, d] = key[t, h, d]
 * Slots < 0 or >= pages*P are skipped (reshape_and_cache_ex.cpp:50).  `value` and
 * `value_cache` may both be NULL (key-only form, ascend910a_extras/ops.py:40-43); if only
 * one of them is NULL values are not written, as in the reference kernel (:24-25,62-64).
 * Bit-exact copy.  No workspace.
 * A slot named by several tokens: with num_tokens <= 4096 the LAST of them is kept, as in the
 * reference's sequential loop (:47-61).  Larger batches skip that check: the slot then holds
 * the row of one of those tokens (a whole row when Hkv*D is a multiple of 16), not
 * necessarily the last.
 */
int b200ops_reshape_and_cache(const void* key, const void* value, void* key_cache,
                              void* value_cache, const int32_t* slot_indices,
                              int64_t num_tokens, int64_t num_kv_heads, int64_t head_size,
                              const int64_t cache_dims[4], int layout, void* stream);

/*
 * Decode attention over the paged KV cache (one query token per sequence, GQA).
 * Replaces aclnnPagedAttentionExGetWorkspaceSize / aclnnPagedAttentionEx
 * (csrc/ffi/ops.cpp:454,459; tiling csrc/opdev/op_host/paged_attention_ex.cpp:8-59; kernel
 * csrc/opdev/op_kernel/paged_attention_ex.cpp:3-471).
 *   q, out : f16 [bs, num_heads, head_dim];  block_tables : int32 [bs, max_pages_per_seq]
 *   context_lens : int32 [bs];  caches in `layout` with `num_pages` pages of `page_size` tokens
 *   out[b,h] = softmax(q[b,h] . K[b, h/(Hq/Hkv), :L_b]^T / sqrt(head_dim)) . V[b, h/(Hq/Hkv), :L_b]
 * A sequence with context_len <= 0 gets zeros.  A block-table entry outside [0, num_pages)
 * that lies inside a sequence's context names no page: the tokens of that page are left out
 * of the softmax (every kernel path behaves the same; the reference validates nothing here).
 * Scratch (split-context partials) lives in `workspace`; ask
 * b200ops_paged_attention_workspace_size() for the minimum size.
 */
size_t b200ops_paged_attention_workspace_size(int64_t bs, int64_t num_heads,
                                              int64_t num_kv_heads, int64_t head_dim,
                                              int64_t page_size, int64_t max_pages_per_seq);
int b200ops_paged_attention(const void* q, const void* key_cache, const void* value_cache,
                            const int32_t* block_tables, const int32_t* context_lens, void* out,
                            int64_t bs, int64_t num_heads, int64_t num_kv_heads,
                            int64_t head_dim, int64_t num_pages, int64_t page_size,
                            int64_t max_pages_per_seq, int layout, void* workspace,
                            size_t workspace_size, void* stream);

/*
 * Decode attention that allocates nothing (no counterpart in the reference).
 *
 * For hosts that cannot obtain device memory at call time: an engine that has already
 * handed all free HBM to its own arena, or a request path on which cudaMalloc is banned
 * because it synchronises the device and can fail.  Same arguments as
 * b200ops_paged_attention() without the workspace: the split-context scratch is a fixed
 * array of B200OPS_PAGED_ATTENTION_STATIC_SCRATCH_BYTES inside the library image, present
 * on every GPU that loads the library until the process exits.  Shapes whose
 * b200ops_paged_attention_workspace_size() exceeds that return B200OPS_EWORKSPACE.
 * The first call on each device looks up the array's device address (with that device
 * current); make that first call before starting any stream capture.  That first call is also
 * when the CUDA runtime may load the library's device code and set the array's memory aside
 * (module loading is lazy by default): a host that is about to claim all remaining HBM for
 * its own arena must make one warm-up call per device BEFORE it does so (any small valid
 * shape will do), or run with CUDA_MODULE_LOADING=EAGER; otherwise that first call can fail
 * with an out-of-memory error.  The array's bytes are charged to every CUDA context that
 * loads the library, whether or not this entry point is ever called.  All calls share the
 * one array, which keeps whatever the previous call left in it: two calls whose kernels
 * overlap on the GPU (different streams, no ordering) race on it -- order them on one
 * stream or with events.  Calls no cudaMalloc/cudaFree and no allocating library routine.
 */
#define B200OPS_PAGED_ATTENTION_STATIC_SCRATCH_BYTES (32u << 20)
int b200ops_paged_attention_static(const void* q, const void* key_cache, const void* value_cache,
                                   const int32_t* block_tables, const int32_t* context_lens,
                                   void* out, int64_t bs, int64_t num_heads, int64_t num_kv_heads,
                                   int64_t head_dim, int64_t num_pages, int64_t page_size,
                                   int64_t max_pages_per_seq, int layout, void* stream);

/*
 * Grouped (per-expert) NT GEMM: y[gl[e-1]:gl[e], :] = x[gl[e-1]:gl[e], :] @ w[e]  (gl[-1] = 0).
 * Replaces aclnnGroupedMatMulExGetWorkspaceSize / aclnnGroupedMatMulEx
 * (csrc/ffi/ops.cpp:211,216; kernel csrc/opdev/op_kernel/grouped_mat_mul_ex.cpp:5-45 and
 * csrc/opdev/op_kernel/matmul_core.h:7-221).
 *   x : f16 [num_tokens, k];  w : f16, STORAGE [num_experts, n, k] (k contiguous; the torch
 *   view is [E, k, n] with strides (n*k, 1, k), csrc/ffi/ops.cpp:171-172);
 *   group_list : int64 [num_experts], inclusive cumulative row ends;  y : f16 [num_tokens, n]
 * Requires k % 64 == 0 and n % 64 == 0 (csrc/ffi/ops.cpp:173).  Rows past gl[E-1] are not
 * written.  Empty groups are skipped (grouped_mat_mul_ex.cpp:40).
 * Workspace: optional.  With a workspace of b200ops_grouped_matmul_workspace_size() bytes (0 for
 * shapes that cannot benefit: many waves of output tiles by the row bound) the kernel may
 * spread the work evenly over the SMs instead of handing out whole output tiles: tiles cut by
 * a range boundary are summed from fp32 partial tiles in the workspace (a problem with fewer
 * tiles than SMs thereby runs split-K, one whose tiles do not fill the last wave loses no
 * wave).  The call zeroes the counters it needs itself.  With workspace == NULL the same result
 * is computed tile by tile.  A single group of at most 256 rows (a dense projection) splits k
 * over thread-block clusters instead and needs no workspace either way.  The kernel is chosen
 * from the shape alone; every choice sums fp16 products in fp32 and rounds once, so results
 * agree within the last fp16 bit, and each choice by itself is bitwise repeatable.
 */
size_t b200ops_grouped_matmul_workspace_size(int64_t num_tokens, int64_t k, int64_t num_experts,
                                             int64_t n);
int b200ops_grouped_matmul(const void* x, const void* w, const int64_t* group_list, void* y,
                           int64_t num_tokens, int64_t k, int64_t num_experts, int64_t n,
                           void* workspace, size_t workspace_size, void* stream);

/*
 * Dense NT product y = x . w^T:  x f16 [m, k], w f16 [n, k], y f16 [m, n], all contiguous.
 * Replaces matmul_impl(stream, x, w, y, m, n, k) of the reference's earlier single-call
 * interface (_csrc/ffi.cpp:71-75, called from native::matmul :408-442; kernel
 * _csrc/kernels/matmul.cpp:3-28 over csrc/opdev/op_kernel/matmul_core.h).  Like the reference
 * (whose multiple-of-64 check is commented out, _csrc/ffi.cpp:423-424) any m, n, k >= 1 is
 * accepted: with k and n multiples of 64 (and 16-byte aligned pointers) the product runs on the
 * tensor-core kernels of b200ops_grouped_matmul as a single group; every other shape runs a
 * plain tiled kernel.  fp32 accumulation, one rounding.  No workspace, nothing allocated.
 */
int b200ops_matmul(const void* x, const void* w, void* y, int64_t m, int64_t n, int64_t k, void* stream);

/*
 * Split + rotary embedding + KV-cache scatter in one launch, for the decode step
 * (the reference runs them as three graph nodes after the QKV projection,
 * csrc/ffi/graph.cpp:207-283; no single FFI call of the reference corresponds to this).
 *   qkv f16 [num_tokens, (num_heads + 2*num_kv_heads) * head_dim] (q heads, then k, then v)
 *   q_out f16 [num_tokens, num_heads, head_dim] = rope(q);  rope(k) and v are written into
 *   key_cache / value_cache at slot_indices[t] (layout and cache_dims as in
 *   b200ops_reshape_and_cache).  Bit-identical to b200ops_rope followed by
 *   b200ops_reshape_and_cache on the split tensors.
 */
int b200ops_fused_qkv_rope_cache(const void* qkv, const int32_t* position_ids, const void* cos_cache,
                                 const void* sin_cache, const int32_t* slot_indices, void* q_out,
                                 void* key_cache, void* value_cache, int64_t num_tokens,
                                 int64_t num_heads, int64_t num_kv_heads, int64_t head_dim,
                                 int64_t max_pos, const int64_t cache_dims[4], int layout, void* stream);

/*
 * The same launch with the per-head RMSNorm of Qwen3-style layers between the split and the
 * rotary embedding (the reference's graph builder inserts two RmsNorm nodes there,
 * csrc/ffi/graph.cpp:252-255): q heads are normalised over head_dim with q_norm_weight [head_dim]
 * f16, k heads with k_norm_weight, y = x / sqrt(mean(x^2) + eps) * w rounded to f16, then rotated.
 * Either weight may be NULL (that tensor is not normalised); head_dim must then be a power of
 * two times 16, at most 512.
 */
int b200ops_fused_qkv_norm_rope_cache(const void* qkv, const void* q_norm_weight, const void* k_norm_weight,
                                      float eps, const int32_t* position_ids, const void* cos_cache,
                                      const void* sin_cache, const int32_t* slot_indices, void* q_out,
                                      void* key_cache, void* value_cache, int64_t num_tokens,
                                      int64_t num_heads, int64_t num_kv_heads, int64_t head_dim,
                                      int64_t max_pos, const int64_t cache_dims[4], int layout, void* stream);

/*
 * MoE routing glue: the steps around grouped_matmul that the reference leaves to its caller
 * (its grouped_matmul expects rows pre-sorted by expert and cumulative group ends,
 * csrc/opdev/op_kernel/grouped_mat_mul_ex.cpp:29-38; the sorting lives in the companion
 * plugin named in the reference's README.md:3).  None of these has a counterpart in the
 * reference's FFI.  All metadata stays on the device, so a decode step needs no host sync.
 *
 * route_topk: logits = x . router_weight^T (fp32 accumulate, rounded to f16), softmax over
 *   experts in fp32, the top_k experts per token (ties to the lower index) and their
 *   probabilities.  x f16 [num_tokens, hidden]; router_weight f16 [num_experts, hidden];
 *   expert_ids int32 [num_tokens, top_k]; expert_weights f32 [num_tokens, top_k].
 * permute: stable counting sort of the num_slots = num_tokens*top_k routed slots by expert.
 *   slot_to_row[s] = destination row of slot s; counts[e] = rows of expert e (int32);
 *   group_list[e] = inclusive cumulative ends (int64), the form grouped_matmul takes.
 *   world == 1: rows are packed expert-major from row 0.  world > 1 (experts placed
 *   contiguously, num_experts/world per rank): rows for rank r start at r*segment_rows and are
 *   packed by expert inside that segment -- the layout an equal-split all-to-all sends.
 *   A segment holds at most segment_rows rows; with segment_rows >= num_slots nothing can be
 *   lost.  A smaller capacity trades exchange volume for the risk of overflow: rows that do
 *   not fit get slot_to_row = -1 (finalize then leaves their contribution out), counts are
 *   clamped, and *overflow (int32, may be NULL) receives the number of dropped rows so the
 *   caller can repeat the step with a larger capacity.
 * ep_plan: on the receiving rank.  all_counts int32 [world, num_experts] (every rank's
 *   `counts`, all-gathered).  grouped_to_received[d] = row of the received buffer
 *   ([world segments of segment_rows]) that supplies grouped (expert-major) row d;
 *   group_list int64 [num_experts/world] local cumulative ends; total_rows int32 [1].
 * copy_rows: for i < *n_valid (n_max if n_valid is NULL):
 *   dst[dst_index ? dst_index[i] : i] = src[(src_index ? src_index[i] : i) / src_div];
 *   rows of row_elems f16; negative indices skip the row.
 * finalize: y[t] = sum_k expert_weights[t,k] * rows[slot_to_row[t*top_k+k]], fp32 accumulate.
 */
int b200ops_moe_route_topk(const void* x, const void* router_weight, int32_t* expert_ids,
                           float* expert_weights, int64_t num_tokens, int64_t hidden,
                           int64_t num_experts, int64_t top_k, void* stream);
int b200ops_moe_permute(const int32_t* expert_ids, int32_t* slot_to_row, int32_t* counts,
                        int64_t* group_list, int32_t* overflow, int64_t num_slots, int64_t num_experts,
                        int64_t world, int64_t segment_rows, void* stream);
int b200ops_moe_ep_plan(const int32_t* all_counts, int32_t* grouped_to_received, int64_t* group_list,
                        int32_t* total_rows, int64_t world, int64_t num_experts, int64_t rank,
                        int64_t segment_rows, void* stream);
int b200ops_moe_copy_rows(void* dst, const void* src, const int32_t* dst_index, const int32_t* src_index,
                          int64_t src_div, const int32_t* n_valid, int64_t n_max, int64_t row_elems,
                          void* stream);
int b200ops_moe_finalize(const void* rows, const int32_t* slot_to_row, const float* expert_weights,
                         void* y, int64_t num_tokens, int64_t top_k, int64_t row_elems, void* stream);

/*
 * The gate/up projection of a gated MLP with SwiGLU in the GEMM's epilogue: replaces
 * b200ops_grouped_matmul (csrc/ffi/ops.cpp:157-233) followed by b200ops_swiglu
 * (csrc/ffi/ops.cpp:126-154) on its result, without the [num_tokens, two_d] intermediate.
 * w [num_experts, two_d, k] f16, k contiguous: rows [0, d) are the gate projection, rows
 * [d, 2d) the up projection, d = two_d / 2 a multiple of 64.  y [num_tokens, d] f16.  The
 * accumulators are rounded to f16 before SwiGLU, so without a workspace the result equals the
 * two-call form bit for bit.  Workspace: optional, as for b200ops_grouped_matmul;
 * b200ops_grouped_matmul_workspace_size(num_tokens, k, num_experts, two_d) gives its size (with
 * it, sums of cut tiles may differ from the two-call form in the last bit).
 */
int b200ops_grouped_matmul_swiglu(const void* x, const void* w, const int64_t* group_list, void* y,
                                  int64_t num_tokens, int64_t k, int64_t num_experts, int64_t two_d,
                                  void* workspace, size_t workspace_size, void* stream);

/*
 * grouped_matmul whose epilogue performs the return leg of the expert-parallel exchange
 * (GEMM + peer store in one kernel; no counterpart in the reference).  Same computation as
 * b200ops_grouped_matmul, but result row r is stored into the buffer of rank
 * row_index[r] / cap at row my_rank * cap + row_index[r] % cap (rows with a negative index
 * are not stored).  peer_out is a HOST array of `world` addresses, valid on this device, of
 * every rank's [world * cap, n] f16 return buffer; row_index is device int32 [num_tokens]
 * (the grouped_to_received map of b200ops_moe_ep_plan).  Follow it with b200ops_peer_barrier.
 */
int b200ops_grouped_matmul_scatter(const void* x, const void* w, const int64_t* group_list,
                                   int64_t num_tokens, int64_t k, int64_t num_experts, int64_t n,
                                   void* workspace, size_t workspace_size, const int32_t* row_index,
                                   void* const* peer_out, int64_t world, int64_t cap, int64_t my_rank,
                                   void* stream);

/*
 * Expert-parallel exchange over peer memory (NVLink), an alternative to an all-to-all
 * collective; no counterpart in the reference, which has no multi-device code.
 *
 * push_rows: for logical row i < *n_valid (n_max if n_valid is NULL) with idx = index[i] >= 0:
 *   row i / src_div of `src` (f16, row_elems wide) is stored into the buffer of peer idx / cap
 *   at row my_rank * cap + idx % cap.  peer_rows[r] is the address, valid on THIS device, of
 *   rank r's receive buffer ([world * cap, row_elems] f16; peer_rows[my_rank] is the local
 *   one).  If `counts` is given, its num_counts int32 values are also stored into row my_rank
 *   of every peer's count table peer_counts[r] ([world, num_counts] int32).  The arrays of peer
 *   addresses are HOST arrays of `world` entries.
 * peer_barrier: announces "this rank has finished pushing" to every peer and waits (at most two
 *   seconds) for the same announcement from every peer.  peer_flags[r] = address of rank r's
 *   flag array ([world] uint32, zero-initialised once); my_flags = the local one; state =
 *   [2] uint32 in local memory, zero-initialised once: state[0] counts barriers, state[1]
 *   becomes 100 + r if peer r never arrived (the kernel then returns instead of hanging).
 *   Launch it on the same stream right after the pushes; kernels after it may read what the
 *   peers pushed.  All ranks must call it the same number of times.
 */
int b200ops_moe_push_rows(const void* src, const int32_t* index, int64_t src_div, const int32_t* n_valid,
                          int64_t n_max, void* const* peer_rows, int64_t world, int64_t cap,
                          int64_t my_rank, int64_t row_elems, const int32_t* counts, int64_t num_counts,
                          void* const* peer_counts, void* stream);
int b200ops_peer_barrier(void* const* peer_flags, void* my_flags, void* state, int64_t world,
                         int64_t my_rank, void* stream);

/*
 * The same exchange as three launches around the two expert GEMMs (no counterpart in the
 * reference).  Slots (an expert, or one replica of a replicated expert) are placed
 * contiguously on ranks, num_slots / world per rank ("spr").  Buffers every rank provides in
 * memory its peers have mapped: a receive buffer [world][spr][cap] rows of `hidden` f16, a return
 * buffer [num_slots][cap] rows of the MLP's output width, a table of count words uint32
 * [world][spr] (rows in the low 20 bits, the step number above them: the counts double as the
 * "dispatched" announcement) and a flag array uint32 [world] ("returned"), all zero-initialised
 * once; cap < 2^20.  Local only:
 * cursor int32 [num_slots] and state uint32 [5], zero-initialised once; overflow int32 [2] (may
 * be NULL).  Arrays of peer addresses are HOST arrays of `world` entries (entry my_rank = the
 * local buffer).
 *
 * dispatch: one CTA per token.  With router_weight: route as b200ops_moe_route_topk does and
 *   store the choices in expert_ids_out / expert_weights_out; otherwise read expert_ids_in
 *   [num_tokens, top_k].  An expert id becomes a slot: the id itself, or, with expert_slots
 *   int32 [num_experts, max_replicas] and num_replicas int32 [num_experts], replica
 *   (token_offset + t) % num_replicas[e] of the expert.  The token's row is stored into the
 *   slot owner's receive buffer, in the sub-segment (my_rank, slot), at the next free row;
 *   slot_to_row[t*top_k+k] = row of the LOCAL return buffer where the result will arrive
 *   (-1: invalid id, or the sub-segment was full; overflow[0] counts the latter).  Row order
 *   inside a sub-segment depends on scheduling; results do not.  The last CTA to finish
 *   sends every peer the count words of that peer's slots for this step.
 * gather: waits (at most two seconds per source, then state[1] = 100 + source) until every
 *   source's count words carry the step, then copies the received rows into expert-major order:
 *   grouped [max_rows, hidden], grouped_to_received[d] = receive-buffer row of grouped row d,
 *   group_list int64 [spr], total_rows int32 [1].  Rows beyond max_rows are left out and
 *   counted in overflow[1].
 * (expert MLP: b200ops_grouped_matmul_swiglu on `grouped`, then b200ops_grouped_matmul_scatter
 *   with row_index = grouped_to_received, peer_out = the return buffers, cap = spr * cap.)
 * combine: announces "returned" to every peer, waits for every peer's announcement (same
 *   limit), then y[t] = sum_k expert_weights[t,k] * returned[slot_to_row[t*top_k+k]].
 * All ranks must run the three calls the same number of times, in this order.
 */
int b200ops_moe_dispatch(const void* x, const void* router_weight, const int32_t* expert_ids_in,
                         int32_t* expert_ids_out, float* expert_weights_out, const int32_t* expert_slots,
                         const int32_t* num_replicas, int64_t max_replicas, int64_t token_offset,
                         int32_t* slot_to_row, void* const* peer_recv, void* const* peer_counts,
                         int32_t* cursor, void* state, int32_t* overflow,
                         int64_t num_tokens, int64_t hidden, int64_t num_experts, int64_t top_k,
                         int64_t num_slots, int64_t world, int64_t cap, int64_t my_rank, void* stream);
int b200ops_moe_gather(const void* recv, const void* counts, void* state, int32_t* overflow, void* grouped, int32_t* grouped_to_received, int64_t* group_list,
                       int32_t* total_rows, int64_t hidden, int64_t world, int64_t slots_per_rank, int64_t cap,
                       int64_t max_rows, void* stream);
int b200ops_moe_combine(const void* returned, const int32_t* slot_to_row, const float* expert_weights, void* y,
                        void* const* peer_flags, void* my_flags, void* state, int64_t num_tokens, int64_t top_k,
                        int64_t row_elems, int64_t world, int64_t my_rank, void* stream);

/*
 * Health word of the pipelined kernels (grouped_matmul, paged_attention's TMA path).  Their
 * producer/consumer waits are bounded; a wait that runs out ends the kernel and leaves a
 * non-zero code here.  This call synchronises the device, returns the code in *status
 * (0 = healthy) and clears it.  Diagnostic only; it has no counterpart in the reference.
 */
int b200ops_pipeline_status(int* status);

#ifdef __cplusplus
}
#endif
#endif /* B200OPS_H_ */
