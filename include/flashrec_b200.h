/*
 * flashrec_b200 — C ABI of the sm_100a kernels for the quantized SID decode step.
 *
 * Every entry point takes raw DEVICE pointers, explicit sizes/strides and the
 * cudaStream_t to launch on; none allocates, synchronises or throws (unless its
 * comment says otherwise). The return value is a status code: 0 on success,
 * negative otherwise. Row-major contiguous layouts unless a stride is given.
 * "e4m3" is float8_e4m3fn (max 448). Each declaration names the function of the
 * reference engine (path inside its `python/flashrec/` tree) that it stands in
 * for.
 */
#ifndef FLASHREC_B200_H_
#define FLASHREC_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef __CUDA_RUNTIME_H__
typedef struct CUstream_st* cudaStream_t;
#endif

enum fr_status {
  FR_OK = 0,
  FR_ERR_BAD_ARG = -1,     /* null / misaligned pointer, negative size, shape mismatch */
  FR_ERR_UNSUPPORTED = -2, /* shape outside what the kernel was built for */
  FR_ERR_CUDA = -3,        /* a CUDA runtime / driver call or the launch failed */
  FR_ERR_TIMEOUT = -4      /* a bounded device-side wait gave up (see fr_device_status) */
};

/* Library / build identification: returns a static string. */
const char* fr_version(void);

/* Reads and clears the sticky device-side status word on the current device
 * (0 = clean, otherwise the FR_ERR_* code and site recorded by a kernel whose
 * bounded wait ran out). Synchronises the device; meant for tests and error
 * paths, not the step loop. */
int fr_device_status(int* status_out, int* site_out);

/* ---- activation quantisers (HBM bound) ---------------------------------- */

/* RMSNorm -> per-row e4m3. If `residual` is non-null it is updated in place
 * (residual += x, rounded to bf16) and the norm runs on the updated residual.
 * x, residual: bf16 [rows, hidden]; weight: bf16 [hidden]; q_out: e4m3
 * [rows, hidden]; scale_out: f32 [rows]. hidden % 8 == 0.
 * Reference: RMSNorm.quant_fp8 (layers/norm.py:28-42) ->
 * rmsnorm_per_token_quant_fp8 / fused_add_rmsnorm_per_token_quant_fp8
 * (kernel/rms_fp8.py:120-145). */
int fr_rms_quant_fp8(const void* x, void* residual, const void* weight, float eps, void* q_out, float* scale_out,
                     int rows, int hidden, cudaStream_t stream);

/* bf16 RMSNorm (optionally residual += x first). y_out: bf16 [rows, hidden].
 * Reference: rmsnorm / fused_add_rmsnorm (kernel/sglops.py:34-61). */
int fr_rmsnorm_bf16(const void* x, void* residual, const void* weight, float eps, void* y_out, int rows, int hidden,
                    cudaStream_t stream);

/* Per-row e4m3 quantisation, scale = max(amax,1e-12)/448. x is bf16
 * (x_is_f32 == 0, hidden % 8 == 0) or f32 (x_is_f32 != 0, hidden % 4 == 0).
 * Reference: per_token_quant_fp8 (kernel/sglops.py:84-96) and
 * quantize_weight_fp8 (layers/linear.py:26-32). */
int fr_token_quant_fp8(const void* x, int x_is_f32, void* q_out, float* scale_out, int rows, int hidden,
                       cudaStream_t stream);

/* silu(x[:, :d]) * x[:, d:] -> per-row e4m3. x: bf16 [rows, 2d]; q_out: e4m3
 * [rows, d]; scale_out: f32 [rows]. d % 8 == 0, d <= 16384.
 * First use on a device (of this entry, fr_silu_mul_bf16 or fr_gemm_fp8_silu_mul, which share
 * a 128 KB device table of exactly evaluated silu values): the table is filled by a kernel on
 * `stream` and the call waits for that stream once. Make that first call outside any stream
 * capture: under capture nothing can be waited for, so the fill is recorded into the graph (and
 * into every later graph, until a call outside capture has completed the set-up).
 * Reference: silu_and_mul_per_token_quant_fp8 (kernel/silu_fp8.py:86-119). */
int fr_silu_mul_quant_fp8(const void* x, void* q_out, float* scale_out, int rows, int d, cudaStream_t stream);

/* Unquantised SwiGLU, bf16 out [rows, d]. First use on a device fills the shared silu
 * table and waits for `stream` once, as described for fr_silu_mul_quant_fp8: make that call
 * outside stream capture.
 * Reference: silu_and_mul (kernel/sglops.py:143-151). */
int fr_silu_mul_bf16(const void* x, void* y_out, int rows, int d, cudaStream_t stream);

/* ---- W8A8 FP8 GEMM (tensor-core bound) ----------------------------------- */

/* out[m,n] = cast((sum_k a[m,k] b[n,k]) * scale_a[m] * scale_b[n]) (+ bias[n]).
 * a: e4m3 [M,K] pitch lda; b: e4m3 [N,K] pitch ldb (the weight as stored; the
 * reference passes its `.t()` view); scale_a f32 [M]; scale_b f32 [N]; bias
 * bf16 [N] or NULL; out: bf16 (out_is_f32 == 0) or f32 [M,N] pitch ldo
 * (elements). K % 16 == 0; pitches in elements, multiples of 16 for a/b.
 * block_n_hint: 0 = choose, 64 / 128 / 256 = one CTA per 128 x block_n tile,
 * 512 = CTA pairs (cluster of 2, tcgen05 cta_group::2) on 256 x 256 tiles,
 * 1024 = split-K over a cluster of up to 8 CTAs per 128 x 256 or 128 x 128 tile (few rows, long K; no bias;
 * the tile width is chosen per shape, 1024 + 128 / 1024 + 256 name it).
 * Reports FR_ERR_TIMEOUT through fr_device_status if a pipeline wait gives up.
 * Reference: Linear.forward_fp8 -> fp8_scaled_mm (layers/linear.py:134-172,
 * kernel/sglops.py:99-140). */
int fr_gemm_fp8_w8a8(const void* a, const void* b, const float* scale_a, const float* scale_b, const void* bias,
                     void* out, int out_is_f32, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldo,
                     int block_n_hint, cudaStream_t stream);

/* residual_inout[m, n] = bf16( bf16( (sum_k a[m,k] b[n,k]) * scale_a[m] * scale_b[n] ) + residual_inout[m, n] ):
 * the GEMM of fr_gemm_fp8_w8a8 (bf16 output, no bias) with the add half of the
 * reference's fused add + RMSNorm folded into its epilogue, in place on the bf16
 * residual stream [M, N] (row pitch ldr elements, 16-byte aligned rows). The
 * caller then normalises residual_inout without an add (fr_rms_quant_fp8 with
 * residual = NULL); the bits equal GEMM -> fused_add_rmsnorm
 * (kernel/sglops.py:49-61, models/qwen3.py:205-214). */
int fr_gemm_fp8_w8a8_add(const void* a, const void* b, const float* scale_a, const float* scale_b,
                         void* residual_inout, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldr,
                         int block_n_hint, cudaStream_t stream);

/* The qkv projection with fr_qk_norm_rope_kv_fp8 applied in the GEMM epilogue: the accumulator
 * tile (two whole heads of 128 columns) is scaled and rounded to bf16 exactly as fr_gemm_fp8_w8a8
 * would store it, then Q and K heads get the per-head RMSNorm and the NeoX rotation of the row's
 * position; Q goes to q_out (bf16 [M, n_q * 128], row pitch ldq elements), K (rounded to bf16
 * first) and V go as e4m3 to k_cache / v_cache[loc[m], head, :] (byte strides ck_*, cv_*; slots
 * outside [0, num_slots) are skipped). The [M, (n_q + 2 n_kv) * 128] qkv matrix is never written.
 * b: merged qkv weight e4m3 [(n_q + 2 n_kv) * 128, K]. head_dim == 128, n_q and n_kv even.
 * Same bits as the two calls in sequence.
 * Reference: Qwen3Attention.forward, qkv_proj followed by fused_qk_norm_rope_store_fp8
 * (models/qwen3.py:76-108, kernel/qk_rope_kv.py:165-250). */
int fr_gemm_fp8_qkv_rope(const void* a, const void* b, const float* scale_a, const float* scale_b, void* q_out,
                         int64_t ldq, int M, int n_q, int n_kv, int head_dim, int K, int64_t lda, int64_t ldb,
                         const int64_t* positions, const int64_t* loc, const void* q_weight, const void* k_weight,
                         float eps, const float* cos_sin, int max_pos, void* k_cache, void* v_cache, int64_t ck_s,
                         int64_t ck_h, int64_t cv_s, int64_t cv_h, int num_slots, cudaStream_t stream);

/* gate_up GEMM with SwiGLU fused into the epilogue. b_interleaved / its scales:
 * the [2d, K] gate_up weight with rows regrouped per 256-row tile as
 * [gate rows 128t .. 128t+127 | up rows 128t .. 128t+127] (N = 2d, d % 128 == 0).
 * y_out: bf16 [M, d] = bf16(silu(bf16 gate) * bf16 up), identical to what
 * fr_gemm_fp8_w8a8 followed by fr_silu_mul_bf16 produces; row_amax: f32 [M],
 * must be ZERO on entry, receives max|y| per row (then feed
 * fr_quant_known_amax_fp8). Together they reproduce fr_gemm_fp8_w8a8 +
 * fr_silu_mul_quant_fp8 bit for bit while moving half the bytes. mode: 0 = choose,
 * 1 = one CTA per 128 x 256 tile, 2 = CTA pairs on 256 x 256 tiles.
 * First use on a device fills the shared silu table and waits for `stream` once, as described
 * for fr_silu_mul_quant_fp8: make that call outside stream capture.
 * Reference: Qwen3MLP.forward (models/qwen3.py:144-172). */
int fr_gemm_fp8_silu_mul(const void* a, const void* b_interleaved, const float* scale_a,
                         const float* scale_b_interleaved, void* y_out, float* row_amax, int M, int N, int K,
                         int64_t lda, int64_t ldb, int64_t ldo, int mode, cudaStream_t stream);

/* Per-row e4m3 quantisation of bf16 rows whose max|y| is already known:
 * scale = max(row_amax, 1e-12) / 448. q_out e4m3 [rows, d], scale_out f32 [rows].
 * Reference: the quantisation half of silu_and_mul_per_token_quant_fp8
 * (kernel/silu_fp8.py:57-71). */
int fr_quant_known_amax_fp8(const void* y, const float* row_amax, void* q_out, float* scale_out, int rows, int d,
                            cudaStream_t stream);

/* ---- attention-side data movement (HBM bound) ---------------------------- */

/* Per-head RMSNorm of Q and K + NeoX RoPE; Q is rewritten in place (bf16), K is
 * rounded to bf16 then e4m3 and V to e4m3, both scattered to slot loc[t] of the
 * KV pool (unscaled). q/k/v: bf16 views [T, heads, D] with element strides
 * (token, head), D contiguous; positions, loc: int64 [T]; weights bf16 [D];
 * cos_sin: f32 [max_pos, D] = [cos(0..D/2) | sin(0..D/2)]; caches e4m3 with
 * byte strides (slot, head). D in {64, 128}. Slots outside [0, num_slots) are
 * skipped, positions are clamped.
 * Reference: fused_qk_norm_rope_store_fp8 (kernel/qk_rope_kv.py:165-250). */
int fr_qk_norm_rope_kv_fp8(void* q, const void* k, const void* v, int64_t q_t, int64_t q_h, int64_t k_t, int64_t k_h,
                           int64_t v_t, int64_t v_h, const int64_t* positions, const int64_t* loc,
                           const void* q_weight, const void* k_weight, float eps, const float* cos_sin, int max_pos,
                           void* k_cache, void* v_cache, int64_t ck_s, int64_t ck_h, int64_t cv_s, int64_t cv_h, int T,
                           int n_q, int n_kv, int D, int num_slots, cudaStream_t stream);

/* NeoX rotation only (no norm) of Q and K, both rewritten in place as bf16: x1' = x1 cos - x2 sin,
 * x2' = x2 cos + x1 sin in fp32, one rounding. q, k, v, positions, cos_sin as in
 * fr_qk_norm_rope_kv_fp8. With k_cache / v_cache given (both or neither), the rotated K (its
 * bf16 value) and V are also converted to e4m3 and scattered to slot loc[t]; with both NULL,
 * v and loc are not read.
 * Reference: apply_rope_inplace and apply_rope_and_store_kv (kernel/sglops.py:65-82, 155-205:
 * sgl-kernel's apply_rope_with_cos_sin_cache_inplace), RotaryEmbedding.forward
 * (layers/rotary.py:43-71) followed by TokenToKVPool.store (kvcache/pool.py:121-139). */
int fr_rope_neox_inplace(void* q, void* k, const void* v, int64_t q_t, int64_t q_h, int64_t k_t, int64_t k_h,
                         int64_t v_t, int64_t v_h, const int64_t* positions, const int64_t* loc, const float* cos_sin,
                         int max_pos, void* k_cache, void* v_cache, int64_t ck_s, int64_t ck_h, int64_t cv_s,
                         int64_t cv_h, int T, int n_q, int n_kv, int D, int num_slots, cudaStream_t stream);

/* K/V scatter into the e4m3 pool: cache[loc[t], h, :] = e4m3(src[t, h, :]). src is bf16
 * (src_is_e4m3 == 0; element strides, converted here) or e4m3 already (src_is_e4m3 != 0: byte
 * strides, 16-byte aligned rows, a plain copy — TokenToKVPool.store casts before it calls
 * store_kv_cache).
 * Reference: TokenToKVPool.store (kvcache/pool.py:121-139), store_kv_cache (kernel/sglops.py:207-222). */
int fr_store_kv_fp8(const void* k, const void* v, int64_t k_t, int64_t k_h, int64_t v_t, int64_t v_h,
                    const int64_t* loc, void* k_cache, void* v_cache, int64_t ck_s, int64_t ck_h, int64_t cv_s,
                    int64_t cv_h, int T, int n_kv, int D, int num_slots, int src_is_e4m3, cudaStream_t stream);

/* indptr_out[0..n] = exclusive scan of seq_lens; out[indptr[i] + j] =
 * req_to_token[rows[i], j] for j < seq_lens[i]. req_to_token int32 with element
 * row stride; rows int64 [n]; seq_lens int32 [n]; out int32 [out_capacity].
 * Reference: gather_kv_indices (attention/kv_indices.py:63-132). */
int fr_gather_kv_indices(const int32_t* req_to_token, int64_t row_stride, const int64_t* rows, const int32_t* seq_lens,
                         int32_t* indptr_out, int32_t* out, int n, int out_capacity, cudaStream_t stream);

/* One decode tick on the row -> slot table, for a whole wave of requests. Batch row i
 * (table row rows[i]) belongs to request g with group_indptr[g] <= i < group_indptr[g+1];
 * seq_lens[i] is the row's length AFTER the tick. In this order:
 *  1. (parents_rel != NULL) the decode window, columns [prefix_len[i], seq_lens[i] - 1), is taken
 *     from the row of parent p = clamp(parents_rel[i], 0, k-1) of the same request (k rows),
 *     all rows reading the table as it was before the call:
 *     remap_by_parents (scheduler/kv_remap.py:30-66), called per request at scheduler.py:1598-1610.
 *  2. (new_slot != NULL) table[rows[i], seq_lens[i] - 1] = new_slot[i]: the batched write_decode
 *     of scheduler/scheduler.py:1305-1310. With new_slot == NULL the window ends at seq_lens[i].
 *  3. indptr_out = exclusive scan of seq_lens, out = the rows' slots [:seq_lens[i]] after 1 and 2:
 *     gather_kv_indices (attention/kv_indices.py:63-132).
 * rows, parents_rel, new_slot: int64 [n]; group_indptr: int32 [n_groups + 1]; prefix_len,
 * seq_lens: int32 [n] (equal within a request); out: int32 [out_capacity], which must hold the
 * whole list (entries past it are dropped from the list AND from the table update, and the status
 * word read by fr_device_status is set to FR_ERR_BAD_ARG, site 41: size it from the host's own sum
 * of seq_lens). rows must be distinct; rows outside [0, n_table_rows) are
 * skipped; a parent whose row is outside the table, or a row whose group is empty or reaches
 * outside the batch, keeps its own window; seq_lens are clamped to n_cols.
 * No allocation, no host sync: graph-capturable. */
int fr_kv_table_step(int32_t* req_to_token, int64_t row_stride, int n_table_rows, int n_cols, const int64_t* rows,
                     const int32_t* group_indptr, int n_groups, const int64_t* parents_rel, const int32_t* prefix_len,
                     const int32_t* seq_lens, const int64_t* new_slot, int32_t* indptr_out, int32_t* out, int n,
                     int out_capacity, cudaStream_t stream);

/* table[dst_rows[r * beam_width + b], :m] = table[src_rows[r], :m] for every request r and beam b.
 * src_rows int64 [n_requests], dst_rows int64 [n_requests * beam_width]; a destination row must
 * not be another request's source row.
 * Reference: ModelEngine.copy_prefill_to_beams_many (engine/engine.py:252-274). */
int fr_kv_table_fanout(int32_t* req_to_token, int64_t row_stride, int n_table_rows, const int64_t* src_rows,
                       const int64_t* dst_rows, int n_requests, int beam_width, int m, cudaStream_t stream);

/* out[t, :] = table[ids[t], :] (bf16, hidden % 8 == 0).
 * Reference: nn.Embedding in Qwen3ForCausalLM.forward (models/qwen3.py:266). */
int fr_embedding_bf16(const void* table, const int64_t* ids, void* out, int T, int hidden, int vocab,
                      cudaStream_t stream);

/* ---- decode attention over the e4m3 KV pool ------------------------------ */

/* shared_len_out[g] = longest slot-list prefix common to all rows of group g,
 * rows [group_rows[g], group_rows[g+1]) (at most max_group_rows of them).
 * indptr int32 [n_rows+1], indices int32.
 * Reference: takes the place of AttentionBackend.prepare / _plan_decode
 * (attention/flashinfer.py:201-209, 262-349); runs on the device, capturable. */
int fr_decode_attn_plan(const int32_t* indptr, const int32_t* indices, const int32_t* group_rows, int n_groups,
                        int max_group_rows, int32_t* shared_len_out, cudaStream_t stream);

/* Bytes of scratch fr_decode_attn_fp8 needs for its tensor-core path: bf16
 * copies of K and of V transposed for the shared prefix (at most max_shared_len
 * tokens) of every group and kv head. */
int64_t fr_decode_attn_scratch_bytes(int n_groups, int hkv, int max_shared_len);

/* out[r,h,:] = softmax(q[r,h,:] . K^T * sm_scale) . V over the row's slot list.
 * q: bf16 [n_rows, hq, 128] (element strides token/head); caches e4m3 with byte
 * strides (slot, kv head), 16-byte aligned rows; out: bf16 [n_rows, hq, 128]
 * with token stride o_t. hq / hkv in {1,2,4,8}. Slots are clamped to the pool.
 * scratch (optional, caller-owned, 16-byte aligned, at least
 * fr_decode_attn_scratch_bytes(...) bytes; contents need not be preserved
 * between calls): when given, the groups' shared prefixes (capped at
 * max_shared_len tokens) run on tcgen05 tensor cores; when NULL, a kernel
 * without scratch (mma.sync) is used. Results agree within the bf16 tolerance.
 * Reference: AttentionBackend.forward decode branch (attention/flashinfer.py:
 * 212-238) / _sdpa (:380-431). */
int fr_decode_attn_fp8(const void* q, int64_t q_t, int64_t q_h, const void* k_cache, const void* v_cache,
                       int64_t ck_s, int64_t ck_h, int64_t cv_s, int64_t cv_h, const int32_t* indptr,
                       const int32_t* indices, const int32_t* group_rows, const int32_t* shared_len, void* out,
                       int64_t o_t, int n_rows, int n_groups, int hq, int hkv, int head_dim, int max_group_rows,
                       int num_slots, float sm_scale, void* scratch, int64_t scratch_bytes, int max_shared_len,
                       cudaStream_t stream);

/* fr_decode_attn_fp8 for the later decode steps of the same requests: the scratch
 * still holds the widened prefixes an earlier call (either entry) on the same
 * scratch, groups and KV pool wrote, and only tokens [prepared_len[g],
 * shared_len[g]) of group g are widened now (prepared_len: int32 [n_groups], the
 * shared_len that earlier call saw). Valid while the first prepared_len[g] slots
 * of every group are the slots that call saw and their KV bytes are unchanged
 * (the prompt of a request during its decode steps). scratch and prepared_len
 * are required. Has no counterpart in the reference, whose attention re-reads
 * the e4m3 pool every step (attention/flashinfer.py:212-238). */
int fr_decode_attn_reuse_fp8(const void* q, int64_t q_t, int64_t q_h, const void* k_cache, const void* v_cache,
                       int64_t ck_s, int64_t ck_h, int64_t cv_s, int64_t cv_h, const int32_t* indptr,
                       const int32_t* indices, const int32_t* group_rows, const int32_t* shared_len, void* out,
                       int64_t o_t, int n_rows, int n_groups, int hq, int hkv, int head_dim, int max_group_rows,
                       int num_slots, float sm_scale, void* scratch, int64_t scratch_bytes, int max_shared_len,
                       const int32_t* prepared_len, cudaStream_t stream);

/* Causal attention of a prefill (extend) batch over the e4m3 pool, on the tensor cores.
 * Request g owns query tokens [qo_indptr[g], qo_indptr[g+1]) of q / out and the slot list
 * kv_indices[kv_indptr[g] .. kv_indptr[g+1]) (its cached prefix followed by the extend tokens'
 * own slots, already written to the pool); token e of the request sees keys [0, prefix + e] with
 * prefix = keys - extend tokens. q, out, caches, sm_scale as in fr_decode_attn_fp8; head_dim 128.
 * scratch: fr_decode_attn_scratch_bytes(n_requests, hkv, max_kv_len) bytes; max_extend_len and
 * max_kv_len bound the requests' extend and key counts (keys past max_kv_len would be ignored).
 * Reference: AttentionBackend.forward prefill branch, FlashInfer BatchPrefillWithPagedKVCache
 * planned causal with page_size 1 (attention/flashinfer.py:351-378), and its SDPA twin
 * (_sdpa, attention/flashinfer.py:380-431: mask s <= prefix + e). */
int fr_prefill_attn_fp8(const void* q, int64_t q_t, int64_t q_h, const void* k_cache, const void* v_cache,
                        int64_t ck_s, int64_t ck_h, int64_t cv_s, int64_t cv_h, const int32_t* qo_indptr,
                        const int32_t* kv_indptr, const int32_t* kv_indices, void* out, int64_t o_t, int n_tokens,
                        int n_requests, int hq, int hkv, int head_dim, int max_extend_len, int max_kv_len,
                        int num_slots, float sm_scale, void* scratch, int64_t scratch_bytes, cudaStream_t stream);

/* ---- trie-constrained SID head ------------------------------------------- */

enum fr_trie_kind { FR_TRIE_NONE = 0, FR_TRIE_DENSE = 1, FR_TRIE_CSR = 2, FR_TRIE_BITMAP = 3 };

/* Device-resident catalog trie (all pointers are DEVICE pointers; the struct
 * itself is read on the host). Node -1 = unconstrained, invalid_node = no legal
 * continuation. Token t maps to column rel = t - token_base in [0, vsz).
 *   DENSE : allow u8 [n_rows, vsz], next i32/i64 [n_rows, vsz] — the layout of
 *           BeamValidPathTrie._allow_table/_next_node (search/trie.py:211-266).
 *   CSR   : csr_keys i64 [n_edges] sorted (node * vsz + rel), csr_child i64
 *           [n_edges] — BeamValidPathTrie._csr_keys/_csr_child (search/trie.py:292-343).
 *   BITMAP: bitmap u32 [n_rows, words_per_node] over the codes of the node's own
 *           level, level_off i32 [n_rows] = rel of that level's code 0, child_base
 *           i64 [n_rows] = id of the node's first child (children are numbered
 *           consecutively in code order) or -1 when the children are leaves. */
typedef struct fr_trie {
  int32_t kind;
  int32_t next_is_i32;
  const void* allow;
  const void* next;
  const void* csr_keys;
  const void* csr_child;
  int64_t n_edges;
  const void* bitmap;
  const void* child_base;
  const void* level_off;
  int32_t words_per_node;
  int32_t reserved_;
  int64_t n_rows;
  int64_t vsz;
  int64_t token_base;
  int64_t invalid_node;
} fr_trie;

/* Row statistics of fp32 logits [rows, cols] (pitch ld): row_max, row_logsum =
 * log(sum exp(x - max)); if logprobs_out is non-null also writes
 * (x - max) - logsum with pitch ldo.
 * Reference: F.log_softmax in RestrictedLMHead.compute_level (logits.py:118-138). */
int fr_logsumexp_rows(const float* logits, int64_t ld, float* row_max, float* row_logsum, float* logprobs_out,
                      int64_t ldo, int rows, int cols, cudaStream_t stream);

/* Per-row sorted top-k (value descending, ties: smaller index). If row_max /
 * row_logsum are given the values are the log-probs (x - max) - logsum.
 * vals_out f32 [rows, k], idx_out i64 [rows, k]; cols * 4 bytes must fit in
 * shared memory (cols <= 49152).
 * Reference: torch.topk(..., sorted=True) in the expand path
 * (scheduler/scheduler.py:1476-1482, engine/graph.py:185-194). */
int fr_topk_rows(const float* x, int64_t ld, const float* row_max, const float* row_logsum, float* vals_out,
                 int64_t* idx_out, int rows, int cols, int k, cudaStream_t stream);

/* Catalog trie built on the device, straight into the CSR layout (FR_TRIE_CSR) of `fr_trie`.
 * items: int32 [n_items, depth] (device), items[i][l] in [0, sizes[l]); sizes: int64 [depth] (HOST).
 * keys_out / child_out: int64 [edge_capacity] (device; n_items * depth always suffices): edges in
 * ascending key order, key = node * vsz + (token - token_base) with vsz = sum(sizes), child = node
 * id or -1 at the last level. counts_out: int64 [3 + 2 * (depth + 1)] (device): [0] distinct items
 * (-1 if an item code was out of range: the outputs are then invalid), [1] internal nodes
 * (= invalid_node), [2] edges, [3 + d] first node id of depth d (d = 0..depth), then the first
 * edge of each depth. Node numbering as the reference: root 0, prefixes by (length, prefix) order.
 * workspace: fr_trie_build_workspace_bytes(n_items) bytes, 16-byte aligned. depth <= 8,
 * prod(sizes) < 2^62, n_items < 2^31. No host synchronisation.
 * Reference: BeamValidPathTrie._ensure_gpu_cache / _build_csr_cache (search/trie.py:222-251,
 * 300-327), which walk Python dicts. */
int64_t fr_trie_build_workspace_bytes(int64_t n_items);
int fr_trie_build_csr(const int32_t* items, int64_t n_items, int depth, const int64_t* sizes, int64_t* keys_out,
                      int64_t* child_out, int64_t edge_capacity, int64_t* counts_out, void* workspace,
                      int64_t workspace_bytes, cudaStream_t stream);

/* The bitmap layout (FR_TRIE_BITMAP) from the CSR arrays of fr_trie_build_csr: bitmap_out u32
 * [n_nodes + 1, words] (bit c of row n = code c of node n's own level is a legal continuation),
 * child_base_out int64 [n_nodes + 1] (id of the node's first child, children being consecutive in
 * code order; -1 at the last level and for childless rows), level_off_out int32 [n_nodes + 1]
 * (token offset of the node's level). sizes, node_start (= counts_out[3 ..] read back): HOST arrays
 * of depth and depth + 1 entries; words * 32 >= max(sizes). */
int fr_trie_csr_to_bitmap(const int64_t* keys, const int64_t* child, int64_t n_edges, int depth,
                          const int64_t* sizes, const int64_t* node_start, uint32_t* bitmap_out,
                          int64_t* child_base_out, int32_t* level_off_out, int words, cudaStream_t stream);

/* scores_out = allowed(node_ids[r], cand_tokens[r,c]) ? scores_in : neg_inf.
 * Reference: trie_mask_candidates (kernel/beam_trie.py:82-117) and the CSR
 * branch of BeamValidPathTrie.mask_candidates (search/trie.py:491-500). */
int fr_trie_mask(float* scores_out, const float* scores_in, const int64_t* cand_tokens, const int64_t* node_ids,
                 const fr_trie* trie, float neg_inf, int64_t rows, int64_t cols, cudaStream_t stream);

/* out[n,k] = next(node_ids[n, clamp(parents[n,k])], tokens[n,k]).
 * Reference: trie_advance_nodes(_batched) (kernel/beam_trie.py:120-197),
 * BeamValidPathTrie.advance_node_ids (search/trie.py:531-589). */
int fr_trie_advance(int64_t* out, const int64_t* node_ids, const int64_t* parents, const int64_t* tokens,
                    const fr_trie* trie, int N, int BW, int K, cudaStream_t stream);

/* out[n,b,:] = token_ids[n, clamp(parents[n,b]), :]; out[n,b,col] = new_tokens[n,b].
 * Reference: beam_expand_token_ids (kernel/beam_trie.py:200-232). */
int fr_beam_expand(int64_t* out, const int64_t* token_ids, const int64_t* parents, const int64_t* new_tokens, int N,
                   int BW, int L, int col, cudaStream_t stream);

/* Fused mask + sorted top-K over BW*C explicit candidates + token-row expand +
 * node advance, one request per CTA; K <= 4096. The input planes are [N, BW, ..], the output
 * planes [N, max(BW, K), ..]: K > BW is a request fanning out from fewer input beams than it
 * selects (level 0 from one prefill row, init_from_prefill_batch, search/expand.py:168-237).
 * scratch: f32 [N, BW*C], required when masking. In/out planes must not alias.
 * out_child (optional): node after the step for each winner.
 * Reference: genrec_mask_topk_expand / call_genrec_cuda (kernel/beam_trie.py:
 * 536-684, kernel/csrc/beam_trie.cuh:548-936). */
int fr_mask_topk_expand(float* out_vals, int64_t* out_parents, int64_t* out_tokens, int64_t* out_indices,
                        int64_t* out_child, float* scratch, const float* cum, const float* top_logprobs,
                        const int64_t* top_tokens, const int64_t* node_in, const int64_t* token_ids_in,
                        int64_t* token_ids_out, int64_t* node_ids_out, const uint8_t* do_expand, const int32_t* col_n,
                        const fr_trie* trie, int N, int BW, int C, int K, int L, int apply_mask, int apply_expand,
                        int apply_advance, cudaStream_t stream);

/* fr_mask_topk_expand for callers that cannot hand over a workspace (a decode
 * worker in a server whose device memory was fully carved up at start-up and
 * that may not call the allocator during a tick): same arguments minus
 * `scratch`; the masked scores go to a fixed 8 MiB array inside the library.
 * When the call masks (apply_mask, a trie and node_in given), N * BW * C must
 * not exceed 2 * 1024 * 1024 (FR_ERR_UNSUPPORTED otherwise); unmasked calls do
 * not use the array and have no such limit. The first call on a device
 * resolves the array's address (cached per device ordinal, without a lock; the
 * cache does not survive cudaDeviceReset); make it before any stream capture.
 * Calls on one device share the array: do not let two of them overlap on the
 * GPU. No counterpart in the reference. */
int fr_mask_topk_expand_static(float* out_vals, int64_t* out_parents, int64_t* out_tokens, int64_t* out_indices,
                               int64_t* out_child, const float* cum, const float* top_logprobs,
                               const int64_t* top_tokens, const int64_t* node_in, const int64_t* token_ids_in,
                               int64_t* token_ids_out, int64_t* node_ids_out, const uint8_t* do_expand,
                               const int32_t* col_n, const fr_trie* trie, int N, int BW, int C, int K, int L,
                               int apply_mask, int apply_expand, int apply_advance, cudaStream_t stream);

/* One beam expansion step with stop tokens, for G independent groups of R frontier rows with C candidates
 * each: rank the R * C extensions by cum[r] + top_logprobs[r, c] (+ perturb[r, c] when given: rank noise,
 * e.g. Gumbel(0, 1) for sampling without replacement; the reported scores never carry it), take the C best
 * in order, and walk them: a candidate whose token is not a stop token survives while fewer than K survivors
 * rank before it; a stop-token candidate is finished while fewer than K survivors rank before it. Survivors
 * go to next_tokens / parent_idx / new_cum [G, K] in rank order, finished candidates to fin_* [G, C];
 * unused slots are zero; num_survivors / num_finished [G] (int64) count them. Ties rank by lower flat index
 * r * C + c. C <= 4096. workspace: fr_joint_select_workspace_bytes(G, C) bytes, 16-byte aligned.
 * Reference: joint_select (search/select.py:98-161), one group per call there. */
int64_t fr_joint_select_workspace_bytes(int G, int C);
int fr_joint_select(int64_t* next_tokens, int64_t* parent_idx, float* new_cum, int64_t* num_survivors,
                    int64_t* fin_tokens, int64_t* fin_parent, float* fin_cum, int64_t* num_finished,
                    const float* cum, const float* top_logprobs, const int64_t* top_tokens, const float* perturb,
                    const int64_t* stop_ids, int n_stop, void* workspace, int64_t workspace_bytes, int G, int R,
                    int C, int K, cudaStream_t stream);

/* The K best of the R * C extensions of each group, in order, all finished (the step that ends by length):
 * tokens / parent_idx / cum_out [G, K]; indices_scratch int64 [G, K] receives the flat indices. perturb as above.
 * Reference: select_final_topk (search/select.py:164-179). */
int fr_select_final_topk(int64_t* tokens, int64_t* parent_idx, float* cum_out, int64_t* indices_scratch,
                         const float* cum, const float* top_logprobs, const int64_t* top_tokens,
                         const float* perturb, int G, int R, int C, int K, cudaStream_t stream);

/* The same step with the candidates taken straight from the level's fp32
 * logits [N*BW, level_width] and their row statistics: every code of the level
 * is a candidate (score = cum + (logit - max) - logsum), so no legal SID is
 * lost to a per-beam pre-selection. token = level_tok_base + idx_base + c;
 * flat index = b * idx_width + idx_base + c (idx_base / idx_width describe a
 * token-range shard of a wider level; 0 / level_width otherwise). With a CSR
 * trie only the node's own edges are visited.
 * Reference: RestrictedLMHead.compute_level + expand_step (logits.py:118-138,
 * search/expand.py:240-372) with the candidate width set to the level width. */
int fr_sid_beam_step(float* out_vals, int64_t* out_parents, int64_t* out_tokens, int64_t* out_indices,
                     int64_t* out_child, const float* cum, const float* logits, int64_t ld, const float* row_max,
                     const float* row_logsum, const int64_t* node_in, const int64_t* token_ids_in,
                     int64_t* token_ids_out, int64_t* node_ids_out, const uint8_t* do_expand, const int32_t* col_n,
                     const fr_trie* trie, int64_t level_tok_base, int64_t idx_base, int64_t idx_width, int N, int BW,
                     int level_width, int K, int L, int apply_expand, int apply_advance, cudaStream_t stream);

/* The SID head of one level and the beam step in one call, without the [N*BW, level_width] fp32 logits
 * matrix: the head GEMM (a: e4m3 hidden rows [N*BW, K_dim] with per-row scales, w: the level's e4m3 head
 * rows [level_width, K_dim] with per-channel scales; the arithmetic of fr_gemm_fp8_w8a8 with fp32 output)
 * keeps, in its epilogue, only (max, log-sum-exp) per row and 256-code tile and the logits of the codes the
 * row's trie node allows (bitmap tries are indexed by node in the epilogue; for CSR / dense tries a per-row
 * bit mask is built first); the tile statistics are combined per row (the unmasked normaliser over the whole
 * level, as logits.py:136-137), and the beam step of fr_sid_beam_step runs over the compact candidate lists.
 * Winners, scores, planes: bit-identical to fr_gemm_fp8_w8a8 (fp32 out, CTA pairs) -> fr_sid_beam_step given
 * the same row statistics. BW % 32 == 0, idx_base % 32 == 0.
 * phase 0: everything. phase 1: GEMM + candidates + row statistics only (row_max / row_logsum, f32 [N*BW],
 * receive the statistics of this call's codes: a token-range shard exchanges them). phase 2: the beam step
 * only, on the candidates phase 1 left in the workspace, with row_max / row_logsum given (the statistics of
 * the whole row). In phase 0 row_max / row_logsum are optional outputs.
 * out_records (optional, 16-byte aligned, 16 bytes x [N, K]): the winners once more as {score bits, flat
 * index u32, child node as two 32-bit halves}, the record a token-range shard hands to fr_topk_merge_shards.
 * workspace: fr_sid_head_topk_workspace_bytes(N, BW, level_width, cand_capacity) bytes, 16-byte aligned;
 * cand_capacity = candidate records per request (an upper bound on the legal continuations of its live
 * beams; records beyond it are dropped and the status word gets FR_ERR_UNSUPPORTED, site 51).
 * Reference: RestrictedLMHead.compute_level (logits.py:118-138) + the expand step
 * (search/expand.py:240-372, kernel/beam_trie.py:536-684), which materialise the [T, K] fp32 log-probs. */
int64_t fr_sid_head_topk_workspace_bytes(int N, int BW, int level_width, int cand_capacity);
int fr_sid_head_topk(float* out_vals, int64_t* out_parents, int64_t* out_tokens, int64_t* out_indices,
                     int64_t* out_child, void* out_records, const void* a, const float* scale_a, int64_t lda, const void* w,
                     const float* scale_w, int64_t ldw, int K_dim, const float* cum, const int64_t* node_in,
                     const int64_t* token_ids_in, int64_t* token_ids_out, int64_t* node_ids_out,
                     const uint8_t* do_expand, const int32_t* col_n, const fr_trie* trie, int64_t level_tok_base,
                     int64_t idx_base, int64_t idx_width, int N, int BW, int level_width, int K, int L,
                     int apply_expand, int apply_advance, int phase, float* row_max, float* row_logsum,
                     void* workspace, int64_t workspace_bytes, int cand_capacity, cudaStream_t stream);

/* Merge S per-shard sorted winner lists ([S, N, K] values / flat indices /
 * child nodes, or the same as 16-byte records in shard_records, e.g. after ONE
 * all-gather; the three arrays may then be NULL) into the global sorted top-K, then
 * expand / advance as above. S * K <= 16384. trie (optional): with it, the slots
 * past the last live winner get the child node fr_sid_beam_step gives them (the
 * edge of code 0 from beam 0's node), so sharded and unsharded node planes agree
 * there too; NULL writes node 0. No counterpart in the reference (it has no
 * multi-GPU path); the ordering rule is the one above. */
int fr_topk_merge_shards(float* out_vals, int64_t* out_parents, int64_t* out_tokens, int64_t* out_indices,
                         int64_t* out_child, const float* shard_vals, const int64_t* shard_indices,
                         const int64_t* shard_child, const void* shard_records, const int64_t* node_in,
                         const int64_t* token_ids_in,
                         int64_t* token_ids_out, int64_t* node_ids_out, const uint8_t* do_expand, const int32_t* col_n,
                         const fr_trie* trie, int64_t level_tok_base, int64_t idx_width, int S, int N, int BW, int K,
                         int L, int apply_expand, int apply_advance, cudaStream_t stream);

/* Combine per-shard row statistics (max, logsum) into the statistics of the concatenated row.
 * Shard s has its maxima at shard_max + s * shard_stride and its log-sums at shard_logsum +
 * s * shard_stride (floats; shard_stride 0 = rows, i.e. two dense [S, rows] arrays; 2 * rows when each
 * shard sent one [2, rows] block). No counterpart in the reference. */
int fr_lse_combine_shards(const float* shard_max, const float* shard_logsum, float* row_max, float* row_logsum, int S,
                          int rows, int64_t shard_stride, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* FLASHREC_B200_H_ */
