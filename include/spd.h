/*
 * spd.h — C ABI of libspd.so, the B200 (sm_100a) implementation of Semi-PD's concurrent
 * prefill + decode forward path.
 *
 * Every entry point is `extern "C"`, takes raw device pointers, explicit sizes / strides and the
 * CUDA stream to launch on, performs no allocation and no host synchronisation (so the calls can
 * be captured into CUDA graphs), and returns 0 on success, a positive cudaError_t on a CUDA
 * failure, or a negative SPD_E_* code on an argument error.  Nothing here throws.  The text of
 * the most recent failure on the calling thread is available from spd_last_error_string().
 *
 * Each declaration cites the reference interface it replaces.  Paths are relative to the
 * reference checkout (infinigence/Semi-PD @ 2565f9f): S/ = python/sglang/srt/, K/ = sgl-kernel/.
 */
#ifndef SPD_H_
#define SPD_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* spd_stream_t; /* cudaStream_t */

/* element types of activations / weights / KV pool */
#define SPD_BF16 0
#define SPD_F16 1
#define SPD_F32 2 /* the operators of the "32-bit capable ops" section only */

/* argument-check error codes (CUDA errors are returned as positive cudaError_t values) */
#define SPD_E_BADARG (-1)   /* null pointer, non-positive size, bad enum */
#define SPD_E_ALIGN (-2)    /* pointer or stride not 16-byte aligned / dim not multiple of 8 */
#define SPD_E_SHAPE (-3)    /* unsupported shape (head_dim, group size, K multiple …) */
#define SPD_E_WORKSPACE (-4)/* workspace too small */
#define SPD_E_DRIVER (-5)   /* driver entry point missing (green contexts, tensor maps) */

/* ---------------------------------------------------------------------------------------------
 * library / device
 * ------------------------------------------------------------------------------------------- */
int spd_version(void);
const char* spd_last_error_string(void);
/* replaces semi_pd_ipc.get_device_sm_count (semi-pd-ipc/ipc.cpp:87-92) */
int spd_device_sm_count(int device, int* sm_count);

/* ---------------------------------------------------------------------------------------------
 * SM partitions — replaces the per-process MPS caps (CUDA_MPS_ACTIVE_THREAD_PERCENTAGE set in
 * S/entrypoints/engine.py:591-593,632-634) with two CUDA green contexts that own DISJOINT SM
 * sets inside one process.  `prefill_sms + decode_sms` may not exceed the device SM count; the
 * driver rounds each group to its SM-group granularity and reports the granted counts.
 * The returned streams belong to the partition; destroy with spd_partition_destroy.
 * ------------------------------------------------------------------------------------------- */
typedef struct spd_partition spd_partition_t;
int spd_partition_create(int device, int prefill_sms, int decode_sms, spd_partition_t** out);
int spd_partition_sm_counts(const spd_partition_t* p, int* prefill_sms, int* decode_sms);
/* which = 0: prefill stream, 1: decode stream */
int spd_partition_stream(const spd_partition_t* p, int which, spd_stream_t* stream);
int spd_partition_destroy(spd_partition_t* p);

/* ---------------------------------------------------------------------------------------------
 * elementwise ops — twins of torch.ops.sgl_kernel.* (K/csrc/torch_extension.cc:49-73)
 * ------------------------------------------------------------------------------------------- */
/* out[t,:] = x[t,:] * rsqrt(mean(x[t,:]^2) + eps) * w      (fp32 math)
 * replaces sgl_kernel.rmsnorm (K/python/sgl_kernel/elementwise.py:9-19; semantics
 * S/layers/layernorm.py:59-76).  Rows are `x_stride` / `out_stride` elements apart. */
int spd_rmsnorm(void* out, const void* x, const void* w, int64_t tokens, int64_t dim,
                int64_t x_stride, int64_t out_stride, float eps, int dtype, spd_stream_t stream);
/* residual += x (rounded to dtype, stored) ; x = rmsnorm(residual) * w — both IN PLACE.
 * replaces sgl_kernel.fused_add_rmsnorm (K/csrc/elementwise/fused_add_rms_norm_kernel.cu:24-55) */
int spd_fused_add_rmsnorm(void* x, void* residual, const void* w, int64_t tokens, int64_t dim,
                          float eps, int dtype, spd_stream_t stream);
/* out[t, :d] = silu(x[t, :d]) * x[t, d:2d]
 * replaces sgl_kernel.silu_and_mul (K/csrc/elementwise/activation.cu:36-50) */
int spd_silu_and_mul(void* out, const void* x, int64_t tokens, int64_t d, int dtype,
                     spd_stream_t stream);
/* In-place rotary embedding of q [T, Hq, D] and k [T, Hk, D] (token strides in elements) using the
 * fp32 cos_sin_cache [max_pos, rot_dim] (cos || sin) indexed by pos_ids [T] (int64).
 * interleave = 0: NeoX halves, 1: GPT-J pairs.
 * replaces sgl_kernel.apply_rope_pos_ids_cos_sin_cache (K/csrc/elementwise/rope.cu:22-89) */
int spd_rope_inplace(void* q, void* k, const float* cos_sin_cache, const int64_t* pos_ids,
                     int64_t tokens, int num_q_heads, int num_k_heads, int head_dim, int rot_dim,
                     int64_t q_stride, int64_t k_stride, int interleave, int dtype,
                     spd_stream_t stream);
/* Fused: RoPE on q and k in place (as above) AND scatter of the rotated k rows and the v rows into
 * the KV pool at out_cache_loc[t]:  k_pool[loc[t]] = k[t], v_pool[loc[t]] = v[t]  (pool rows are
 * Hk*D contiguous elements).  Replaces rope (above) + MHATokenToKVPool.set_kv_buffer
 * (S/mem_cache/memory_pool.py:316-346).  loc is int64. */
int spd_rope_kvwrite(void* q, void* k, const void* v, void* k_pool, void* v_pool,
                     const float* cos_sin_cache, const int64_t* pos_ids, const int64_t* loc,
                     int64_t tokens, int num_q_heads, int num_k_heads, int head_dim, int rot_dim,
                     int64_t q_stride, int64_t k_stride, int64_t v_stride, int interleave,
                     int dtype, spd_stream_t stream);
/* k_pool[loc[t]] = k[t]; v_pool[loc[t]] = v[t] — set_kv_buffer alone (S/mem_cache/memory_pool.py:316-346).
 * v and v_pool may both be NULL: single-buffer pools (MLATokenToKVPool.set_kv_buffer, :426-452). */
int spd_kv_write(const void* k, const void* v, void* k_pool, void* v_pool, const int64_t* loc,
                 int64_t tokens, int64_t row_elems, int64_t k_stride, int64_t v_stride, int dtype,
                 spd_stream_t stream);
/* out[i, :] = table[idx[i], :]   (row_elems 16-bit elements per row; idx int64).
 * Embedding lookup (S/layers/vocab_parallel_embedding.py:469-490) and the last-token gather of
 * the logits processor (S/layers/logits_processor.py:244-262). */
int spd_gather_rows(void* out, const void* table, const int64_t* idx, int64_t n, int64_t row_elems,
                    int64_t table_rows, int dtype, spd_stream_t stream);
/* ids[b] = argmax_v logits[b, v] (first maximal index, as torch.argmax) — greedy branch of
 * Sampler.forward (S/layers/sampler.py:73-77,171).  logits fp32 [B, V] with row stride ld. */
int spd_argmax_f32(int32_t* ids, const float* logits, int64_t batch, int64_t vocab, int64_t ld,
                   spd_stream_t stream);
/* Greedy sampling over a vocab-SHARDED lm_head (ParallelLMHead, S/layers/vocab_parallel_embedding.py
 * + the all-gather of S/layers/logits_processor.py:426-427) without moving the logits:
 * spd_argmax_partial_f32 writes one 16-byte row per request {f32 max, i32 index_offset + argmax,
 * 0, 0} for this rank's [B, vocab] shard; after an all-gather of those rows ([parts][B] rows),
 * spd_argmax_merge picks the winner (ties -> smallest index == torch.argmax of the full row). */
int spd_argmax_partial_f32(void* pairs, const float* logits, int64_t batch, int64_t vocab, int64_t ld,
                           int64_t index_offset, spd_stream_t stream);
int spd_argmax_merge(int32_t* ids, const void* pairs, int parts, int64_t batch, spd_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * batch metadata (integer work; bit-exact)
 * ------------------------------------------------------------------------------------------- */
/* positions[extend_start_loc[r] + j] = prefix_lens[r] + j ; extend_start_loc = exclusive cumsum of
 * extend_lens.  Optionally (token_req != NULL) also writes the request index of every token.
 * replaces compute_position_kernel (S/model_executor/forward_batch_info.py:393-446) */
int spd_compute_positions(int64_t* positions, int32_t* extend_start_loc, int32_t* token_req,
                          const int32_t* prefix_lens, const int32_t* extend_lens, int64_t batch,
                          spd_stream_t stream);
/* positions[b] = max(seq_lens[b] - 1, 0) — clamp_position (forward_batch_info.py:466-468) */
int spd_decode_positions(int64_t* positions, const int64_t* seq_lens, int64_t batch,
                         spd_stream_t stream);
/* kv_indices[kv_indptr[b] + j] = req_to_token[req_pool_indices[b], kv_start[b] + j], j < lens[b]
 * replaces create_flashinfer_kv_indices_triton (S/layers/attention/utils.py:5-39).
 * kv_start may be NULL (= 0). req_pool_indices / lens int64 or int32 per `idx64`. */
int spd_build_kv_indices(int32_t* kv_indices, const int32_t* req_to_token,
                         const int64_t* req_pool_indices, const int32_t* lens,
                         const int32_t* kv_indptr, const int32_t* kv_start, int64_t batch,
                         int64_t req_to_token_stride, spd_stream_t stream);
/* req_to_token[req[b], pre[b] + j] = out_cache_loc[cumsum(ext)[b] + j], j < ext[b]
 * replaces write_req_to_token_pool_triton (S/managers/schedule_batch.py:1446-1480) */
int spd_write_req_to_token(int32_t* req_to_token, const int64_t* req_pool_indices,
                           const int64_t* pre_lens, const int64_t* seq_lens,
                           const int64_t* extend_lens, const int64_t* out_cache_loc, int64_t batch,
                           int64_t req_to_token_stride, spd_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * OPT-family ops (BASELINE configs[0]: opt-125m plumbing + logit check).  The reference has no OPT
 * model; these follow torch.nn.LayerNorm / F.relu / the `residual + hidden_states` adds of
 * transformers' modeling_opt.py (OPTDecoderLayer.forward), fp32 math, 16-bit I/O.
 * spd_layernorm: out = (x - mean) / sqrt(var + eps) * gamma + beta per row (dim <= 8192).
 * spd_bias_act_residual: out = act(x + bias) + residual, rows contiguous; bias / residual may be
 * NULL; act: 0 = identity, 1 = ReLU.  out may alias x.
 * ------------------------------------------------------------------------------------------- */
int spd_layernorm(void* out, const void* x, const void* gamma, const void* beta, int64_t tokens,
                  int64_t dim, int64_t x_stride, int64_t out_stride, float eps, int dtype,
                  spd_stream_t stream);
int spd_bias_act_residual(void* out, const void* x, const void* bias, const void* residual,
                          int64_t tokens, int64_t dim, int act, int dtype, spd_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * GEMM — C[M,N] = A[M,K] * W[N,K]^T, 16-bit inputs, fp32 accumulation in TMEM (tcgen05 + TMA).
 * replaces UnquantizedLinearMethod.apply = F.linear (S/layers/linear.py:165-172) for
 * W_qkv / W_o / W_gate_up / W_down and the lm_head matmul (S/layers/logits_processor.py:416-419).
 * lda/ldw/ldc are row strides in elements.  out_f32 == 1: C is fp32 holding the dtype-rounded
 * result (== `.float()` of the 16-bit product, logits_processor.py:440); out_f32 == 2: C is the
 * fp32 accumulator itself (routers and logits of models that want them in 32-bit).
 * epilogue: SPD_EPI_NONE, or SPD_EPI_SILU_MUL: W is [2N, K] (gate rows || up rows, the
 * MergedColumnParallelLinear order, S/models/llama.py:67-73) and C[M,N] = silu(A Wg^T) * (A Wu^T),
 * both products rounded to dtype first (== gate_up_proj followed by SiluAndMul).
 * workspace: device scratch for the stream-K partials and their "published" flags
 * (spd_gemm_workspace_bytes()), zero-initialised ONCE by the caller and then owned by one stream
 * (the kernels re-arm the flags themselves; two streams must not share one workspace).  May be
 * NULL: the call then never splits a tile.
 * sm_budget: number of SMs the call may occupy (0 = all); a worker running on a green-context
 * partition passes its partition's SM count so that persistent grids and the stream-K split match it.
 * ------------------------------------------------------------------------------------------- */
#define SPD_EPI_NONE 0
#define SPD_EPI_SILU_MUL 1
int64_t spd_gemm_workspace_bytes(void);
int spd_gemm(void* C, const void* A, const void* W, int64_t M, int64_t N, int64_t K, int64_t lda,
             int64_t ldw, int64_t ldc, int dtype, int out_f32, int epilogue, void* workspace,
             int64_t workspace_bytes, int sm_budget, spd_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * attention over the token-granular paged KV pool (page_size = 1; slot 0 is the dummy slot).
 * Pool layout per layer: k_pool, v_pool [slots, Hk, D] (S/mem_cache/memory_pool.py:231-250).
 * Slots of request r are req_to_token[req_pool_indices[r], 0 .. seq_len).
 * ------------------------------------------------------------------------------------------- */
/* Ragged chunked-prefill ("extend") attention, causal over [prefix || new]:
 * query token j of request r (row extend_start_loc[r] + j of q) attends keys 0 .. prefix_r + j.
 * The new tokens' K/V must already be in the pool.  q/out: [T, Hq, D], token stride in elements.
 * replaces FlashInferAttnBackend.forward_extend's ragged + paged + merge_state kernels
 * (S/layers/attention/flashinfer_backend.py:386-452); semantics
 * S/layers/attention/torch_native_backend.py:26-109.
 * sm_budget: SMs of the caller's partition (0 = whole device) — the kernel is persistent, one CTA
 * per SM. */
int spd_attn_prefill_ragged(void* out, const void* q, const void* k_pool, const void* v_pool,
                            const int32_t* req_to_token, const int64_t* req_pool_indices,
                            const int32_t* prefix_lens, const int32_t* extend_lens,
                            const int32_t* extend_start_loc, int64_t batch, int64_t total_tokens,
                            int64_t max_extend_len, int num_q_heads, int num_kv_heads,
                            int head_dim, int64_t q_stride, int64_t out_stride,
                            int64_t req_to_token_stride, float sm_scale, int dtype,
                            int sm_budget, spd_stream_t stream);
/* Batched paged-decode attention: one query row per request over its seq_lens[b] cached rows
 * (including the token just written).  Split-KV with an in-kernel merge; workspace from
 * spd_attn_decode_workspace_bytes().  replaces FlashInferAttnBackend.forward_decode
 * (flashinfer_backend.py:454-488); semantics torch_native_backend.py:111-179. */
int64_t spd_attn_decode_workspace_bytes(int64_t max_batch, int num_q_heads, int head_dim);
int spd_attn_decode_paged(void* out, const void* q, const void* k_pool, const void* v_pool,
                          const int32_t* req_to_token, const int64_t* req_pool_indices,
                          const int64_t* seq_lens, int64_t batch, int num_q_heads,
                          int num_kv_heads, int head_dim, int64_t q_stride, int64_t out_stride,
                          int64_t req_to_token_stride, float sm_scale, int dtype, void* workspace,
                          int64_t workspace_bytes, int sm_budget, spd_stream_t stream);
/* Plain SIMT implementations of the two calls above (no tensor cores).  Bring-up / on-device
 * cross-check only; the product path never calls them. */
int spd_attn_prefill_simt(void* out, const void* q, const void* k_pool, const void* v_pool,
                          const int32_t* req_to_token, const int64_t* req_pool_indices,
                          const int32_t* prefix_lens, const int32_t* extend_lens,
                          const int32_t* extend_start_loc, int64_t batch, int64_t total_tokens,
                          int64_t max_extend_len, int num_q_heads, int num_kv_heads, int head_dim,
                          int64_t q_stride, int64_t out_stride, int64_t req_to_token_stride,
                          float sm_scale, int dtype, spd_stream_t stream);
int spd_attn_decode_simt(void* out, const void* q, const void* k_pool, const void* v_pool,
                         const int32_t* req_to_token, const int64_t* req_pool_indices,
                         const int64_t* seq_lens, int64_t batch, int num_q_heads, int num_kv_heads,
                         int head_dim, int64_t q_stride, int64_t out_stride,
                         int64_t req_to_token_stride, float sm_scale, int dtype, void* workspace,
                         int64_t workspace_bytes, spd_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * tensor-parallel all-reduce over NVLink peer memory (one process per GPU) — the `spd_allreduce`
 * of SURVEY §8b's export list.  Replaces the custom all-reduce the reference sends every
 * RowParallelLinear output below 8 MiB through (S/layers/linear.py:1265-1266 →
 * S/distributed/parallel_state.py:376-436 → device_communicators/custom_all_reduce.py:147-160,
 * 447-480; alternative K/csrc/allreduce/trt_reduce_internal.cu:190-300); the reference sends larger
 * messages (prefill batches) to ncclAllReduce (parallel_state.py:431-436) — the host side here
 * passes them through this entry point in pieces of at most max_message_bytes.
 *
 * spd_comm_create allocates this rank's symmetric buffer (3 x max_message_bytes + 8 KB) on the
 * current device and writes its 64-byte cudaIpcMemHandle to ipc_handle_out; the caller gathers
 * all ranks' handles (rank order) with any host-side transport and passes them to
 * spd_comm_connect, which maps the peers (cudaIpcOpenMemHandle).  One communicator belongs to
 * ONE stream: the prefill and the decode worker of a GPU each create their own, like the
 * reference's separate NCCL worlds for P and D (S/managers/scheduler.py:250-259).
 *
 * spd_allreduce: out[i] = sum over ranks of in[i], i < count (16-bit elements, count % 8 == 0,
 * count*2 <= max_message_bytes), fp32 accumulation in rank order — bit-identical on all ranks.
 * `in` and `out` are ordinary device buffers (out may alias in).  All ranks must issue the same
 * sequence of calls (same counts) on a communicator.  The call is stream-ordered, allocation- and
 * sync-free and may be captured into a CUDA graph and replayed any number of times (the barrier
 * sequence numbers live in device memory).  algo: 0 = auto (the reference's dispatch: one-shot
 * below 512 KB for <= 4 ranks / 256 KB for 8 ranks, two-shot above), 1 = one-shot, 2 = two-shot.
 * A peer that does not arrive within SPD_AR_TIMEOUT_MS (default 10000) sets a sticky error that
 * spd_comm_status reports; the GPU never hangs.
 * ------------------------------------------------------------------------------------------- */
#define SPD_IPC_HANDLE_BYTES 64
typedef struct spd_comm spd_comm_t;
int spd_comm_create(int rank, int world, int64_t max_message_bytes, spd_comm_t** out,
                    void* ipc_handle_out);
int spd_comm_connect(spd_comm_t* comm, const void* all_handles);
int64_t spd_comm_max_bytes(const spd_comm_t* comm);
int spd_comm_status(spd_comm_t* comm, int* timed_out);
int spd_allreduce(spd_comm_t* comm, void* out, const void* in, int64_t count, int dtype, int algo,
                  spd_stream_t stream);
/* The all-reduce fused with its consumer (round 2): x = sum over ranks of in[rows, dim];
 * residual += x (rounded to the dtype as fused_add_rmsnorm stores it); out = RMSNorm(residual) * weight
 * — S/layers/linear.py:1265-1266 (tensor_model_parallel_all_reduce after o_proj / down_proj)
 * followed by S/layers/layernorm.py:46-57 (fused_add_rmsnorm) in ONE kernel over the peer-mapped
 * slots.  Bit-identical to spd_allreduce + spd_fused_add_rmsnorm.  dim % 8 == 0, dim <= 8192,
 * rows * dim * 2 <= max_message_bytes; out may alias in.  Same ordering / graph-capture rules. */
int spd_allreduce_add_rmsnorm(spd_comm_t* comm, void* out, const void* in, void* residual,
                              const void* weight, int64_t rows, int64_t dim, float eps, int dtype,
                              spd_stream_t stream);
/* out[r * bytes_per_rank + i] = rank r's in[i] (bytes_per_rank % 16 == 0, <= max_message_bytes):
 * the all-gather after the vocab-sharded lm_head (S/layers/logits_processor.py:426-427), here of
 * the per-shard (max, argmax) rows below — and of small logits blocks.  Same ordering /
 * graph-capture rules as spd_allreduce. */
int spd_allgather(spd_comm_t* comm, void* out, const void* in, int64_t bytes_per_rank,
                  spd_stream_t stream);
int spd_comm_destroy(spd_comm_t* comm);

/* ---------------------------------------------------------------------------------------------
 * DeepSeek-V2-Lite path (BASELINE configs[3]): absorbed MLA attention over the latent KV pool,
 * grouped GEMMs and the MoE plumbing.
 * ------------------------------------------------------------------------------------------- */
/* Grouped GEMM on the tcgen05 kernel of spd_gemm (normal regime, 128-row tiles).
 * rows mode (tile_group != NULL) — the two expert GEMMs of the fused MoE
 *   (S/layers/moe/fused_moe_triton/fused_moe.py:961-1168): A [M, K] holds the routed tokens sorted by
 *   expert in 128-row tiles (spd_moe_align / spd_moe_gather), tile_group[i] = expert of rows
 *   [128 i, 128 i + 128) or < 0 (unused tile, skipped); W = the experts' weights stacked,
 *   [num_groups * N, K] — with SPD_EPI_SILU_MUL [num_groups * 2N, K], gate rows || up rows per expert;
 *   C [M, N].  a_group_stride must be 0.
 * cols mode (tile_group == NULL) — block-diagonal products, the absorbed-MLA BMMs
 *   torch.bmm(q_nope, w_kc) / torch.bmm(attn_out, w_vc) (S/models/deepseek_v2.py:667,702):
 *   C[:, g*N:(g+1)*N] = A[:, g*a_group_stride : g*a_group_stride + K] * W[g*N:(g+1)*N, :K]^T,
 *   A [M, a_cols] with row stride lda, N % 128 == 0, K % 64 == 0.  c_group_stride > 0 places group g's
 *   N output columns at column g * c_group_stride of C instead of g * N.
 * w_group_col_stride > 0 (rows mode, no epilogue): the experts' weights are concatenated along K
 *   instead of stacked — W [N, num_groups * w_group_col_stride], expert g = columns
 *   [g * stride, g * stride + K) — the layout the decode-sized dense path multiplies as ONE GEMM. */
int spd_gemm_grouped(void* C, const void* A, const void* W, int64_t M, int64_t N, int64_t K, int64_t lda,
                     int64_t ldw, int64_t ldc, int num_groups, const int32_t* tile_group,
                     int64_t a_group_stride, int64_t a_cols, int64_t c_group_stride, int64_t w_group_col_stride,
                     int dtype, int epilogue, int sm_budget, spd_stream_t stream);
/* Router: softmax over the experts (fp32) + greedy top-k; weights = prob (renormalised over the k
 * if renormalize) * scale.  logits [tokens, num_experts] 16-bit.  replaces select_experts /
 * fused_topk (S/layers/moe/topk.py:79-120,128-163). */
int spd_moe_route(int32_t* topk_ids, float* topk_w, const void* logits, int64_t tokens, int num_experts,
                  int top_k, float scale, int renormalize, int dtype, spd_stream_t stream);
/* Expert alignment: sorts the tokens*top_k routing entries by expert, every expert padded to whole
 * 128-row tiles.  row_token[max_rows]: source token of each sorted row (-1 = padding);
 * inv_pos[tokens*top_k]: sorted row of entry (token, j); tile_group[max_rows/128]: expert per tile
 * (-1 = unused).  max_rows >= spd_moe_align_rows().  replaces moe_align_block_size
 * (K/csrc/moe/moe_align_kernel.cu:28,44). */
int64_t spd_moe_align_rows(int64_t tokens, int top_k, int num_experts);
int spd_moe_align(int32_t* row_token, int32_t* inv_pos, int32_t* tile_group, const int32_t* topk_ids,
                  int64_t tokens, int top_k, int num_experts, int64_t max_rows, spd_stream_t stream);
/* xs[r, :] = x[row_token[r], :] (zeros for padding rows) */
int spd_moe_gather(void* xs, const void* x, const int32_t* row_token, int64_t rows, int64_t dim,
                   int64_t x_stride, int dtype, spd_stream_t stream);
/* out[t, :] = (shared ? shared[t, :] : 0) + sum_j topk_w[t, j] * y[inv_pos[t*top_k + j], :]
 * (the weighted sum of fused_moe + the shared experts' output, S/models/deepseek_v2.py:205-218) */
int spd_moe_combine(void* out, const void* y, const void* shared, const int32_t* inv_pos, const float* topk_w,
                    int64_t tokens, int top_k, int64_t dim, int dtype, spd_stream_t stream);
/* Decode-sized batches run every expert as two plain spd_gemm calls over the stacked weights;
 * between them: act[t, e*inter + i] = w(t, e) * silu(gate_up[t, e, i]) * gate_up[t, e, inter + i],
 * w(t, e) = 0 for experts token t did not select.  gate_up [tokens, num_experts * 2 * inter]. */
int spd_moe_dense_act(void* act, const void* gate_up, const int32_t* topk_ids, const float* topk_w,
                      int64_t tokens, int top_k, int num_experts, int64_t inter, int dtype,
                      spd_stream_t stream);
/* Absorbed MLA attention (MQA over the latent pool), decode (seq_lens != NULL: one query per request
 * over its seq_lens[b] rows) or ragged extend (seq_lens == NULL: query token j of request r, row
 * extend_start_loc[r] + j of q, attends keys 0 .. prefix_lens[r] + j).  kv_pool [slots, kv_lora_rank +
 * rope_dim] = MLATokenToKVPool rows (S/mem_cache/memory_pool.py:379-452); K = the whole row, V = its
 * first kv_lora_rank columns; q [tokens, H, kv_lora_rank + rope_dim] (q_nope already multiplied by
 * w_kc), out [tokens, H, kv_lora_rank].  replaces DeepseekV2AttentionMLA.forward_absorb's attention
 * call (S/models/deepseek_v2.py:684-700 → S/layers/attention/triton_ops/decode_attention.py:235-470,
 * extend_attention.py:291-410). */
int64_t spd_attn_mla_workspace_bytes(int num_heads, int kv_lora_rank);
int spd_attn_mla(void* out, const void* q, const void* kv_pool, const int32_t* req_to_token,
                 const int64_t* req_pool_indices, const int64_t* seq_lens, const int32_t* prefix_lens,
                 const int32_t* extend_start_loc, int64_t batch, int64_t total_tokens, int num_heads,
                 int kv_lora_rank, int rope_dim, int64_t q_stride, int64_t out_stride,
                 int64_t req_to_token_stride, float sm_scale, int dtype, void* workspace,
                 int64_t workspace_bytes, int sm_budget, spd_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * 32-bit capable ops — the operators of the hybrid (windowed attention + retention + MoE) model
 * family.  dtype is SPD_BF16 / SPD_F16 / SPD_F32 (activations, weights and KV pool alike); softmax,
 * norms, routing, the residual stream and recurrent state are fp32 whatever the dtype.  The
 * reference has no such models; the calling conventions follow the ops above.
 * ------------------------------------------------------------------------------------------- */
/* x[r, :] += a[r, :] (+ b[r, :])   (x fp32 residual stream, a / b nullable, dtype elements);
 * out[r, :] = x[r, :] / sqrt(mean(x[r, :]^2) + eps) * (weight_offset + w[:])   (out nullable) */
int spd_residual_rmsnorm(void* out, float* x, const void* a, const void* b, const void* w, int64_t rows,
                         int64_t dim, float eps, float weight_offset, int dtype, spd_stream_t stream);
/* x[r, :] = table[idx[r], :] as fp32 (embedding lookup into the fp32 residual stream) */
int spd_embed_f32(float* x, const void* table, const int64_t* idx, int64_t rows, int64_t dim,
                  int64_t table_rows, int dtype, spd_stream_t stream);
/* out[r, i] = act(x[r, i]) * x[r, inter + i]; act 0 = SiLU, 1 = tanh-form GELU.  x [rows, 2 inter].
 * act 2: with g = min(x[r, i], p0) and u = clamp(x[r, inter + i], -p0, p0), out = g sigmoid(p1 g) (u + 1)
 * (p0, p1 are read by act 2 only) */
int spd_act_and_mul(void* out, const void* x, int64_t rows, int64_t inter, int act, float p0, float p1, int dtype,
                    spd_stream_t stream);
/* out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * gate(g[t, h, :]), gate = SiLU (gate_act 0) or
 * sigmoid (gate_act 1);  o fp32 [tokens, heads * vdim] contiguous, g dtype with row stride g_stride, out dtype
 * contiguous */
/* w (nullable, dtype): a weight on the normed values, element h * w_head_stride + c for head h (stride 0:
 * one vector of vdim shared by the heads) */
int spd_headnorm_gate(void* out, const float* o, const void* g, int64_t tokens, int heads, int vdim,
                      int64_t g_stride, float eps, const void* w, int w_head_stride, int gate_act, int dtype,
                      spd_stream_t stream);
/* C = A W^T on the CUDA cores with fp32 accumulation in ascending-k order (any M, N, K; any dtype).
 * tile_group != NULL: rows of A are grouped in 128-row tiles (spd_moe_align) and rows
 * [g * w_group_rows, +N) of W multiply the tiles of group g = tile_group[row / 128] (< 0: skipped). */
int spd_linear_simt(void* C, const void* A, const void* W, int64_t M, int64_t N, int64_t K, int64_t lda,
                    int64_t ldw, int64_t ldc, const int32_t* tile_group, int64_t w_group_rows, int dtype,
                    int out_f32, spd_stream_t stream);
/* Routing from fp32 logits (row stride ld): score = softmax (score_func 0) or sigmoid (1) of the logits,
 * the top_k largest scores are chosen (ties: smaller expert id), weights = score (renormalised over the
 * chosen ones if renormalize) x scale.
 * correction (fp32 [experts], nullable) biases the SELECTION only (weights stay unbiased).  num_groups > 1: the
 * experts are cut into equal runs of neighbours, a run ranks by its top-2 biased scores added together, and
 * selection is restricted to the keep_groups highest-ranked runs. */
int spd_moe_route_scores(int32_t* topk_ids, float* topk_w, const float* logits, int64_t ld, int64_t tokens,
                         int num_experts, int top_k, int score_func, int renormalize, float scale,
                         const float* correction, int num_groups, int keep_groups, spd_stream_t stream);
/* xs[r, :] = w(r) * x[row_token[r], :] with w(r) the routing weight of the entry sorted to row r (1 if
 * topk_w == NULL); zeros for padding rows — experts that weight their INPUT */
int spd_moe_gather_scaled(void* xs, const void* x, const int32_t* row_token, const int32_t* inv_pos,
                          const float* topk_w, int64_t rows, int top_k, int64_t dim, int64_t x_stride,
                          int dtype, spd_stream_t stream);
/* out[t, :] = sum_j (topk_w ? topk_w[t, j] : 1) * y[inv_pos[t * top_k + j], :]
 *           + (shared ? (shared_gate ? sigmoid(shared_gate[t * gate_stride]) : 1) * shared[t, :] : 0) */
int spd_moe_combine_gated(void* out, const void* y, const int32_t* inv_pos, const float* topk_w,
                          const void* shared, const float* shared_gate, int64_t gate_stride, int64_t tokens,
                          int top_k, int64_t dim, int dtype, spd_stream_t stream);
/* k_pool[loc[t]] = k[t], v_pool[loc[t]] = v[t] with different row sizes for keys and values */
int spd_kv_store(const void* k, const void* v, void* k_pool, void* v_pool, const int64_t* loc,
                 int64_t tokens, int64_t k_row_elems, int64_t v_row_elems, int64_t k_stride,
                 int64_t v_stride, int dtype, spd_stream_t stream);
/* Softmax attention over the paged pool with the options of the hybrid family, decode (seq_lens !=
 * NULL: one query per request at position seq_lens[b] - 1) or ragged extend (query j of request r is row
 * extend_start_loc[r] + j of q, position prefix_lens[r] + j).  Query i sees keys j with 0 <= i - j <
 * window (window <= 0: all j <= i).  score = (q . k) * sm_scale * temp(i) - slopes[h] * (i - j) with
 * temp(i) = 1 + qtemp_coef * ln(floor((i + 1) / qtemp_every) + 1) (qtemp_every <= 0: 1); slopes nullable.
 * sinks != NULL: exp(sinks[h]) joins the softmax denominator.  key size head_dim, value size v_dim;
 * k_pool [slots, kv_heads, head_dim], v_pool [slots, kv_heads, v_dim]; out [tokens, heads * v_dim].
 * max_extend_len (extend): an upper bound of extend_lens known on the host; > 0 lets 16-bit prefill
 * take the tensor-core kernel (64-row query tiles), 0 keeps the CUDA-core kernel. */
int spd_attn_general(void* out, const void* q, const void* k_pool, const void* v_pool,
                     const int32_t* req_to_token, const int64_t* req_pool_indices, const int64_t* seq_lens,
                     const int32_t* prefix_lens, const int32_t* extend_lens, const int32_t* extend_start_loc,
                     int64_t batch, int64_t total_tokens, int num_q_heads, int num_kv_heads, int head_dim,
                     int v_dim, int64_t q_stride, int64_t out_stride, int64_t req_to_token_stride,
                     float sm_scale, int window, const float* sinks, const float* slopes, float qtemp_coef,
                     int qtemp_every, int64_t max_extend_len, int dtype, spd_stream_t stream);
/* Retention (linear attention with a fixed per-head decay, no softmax): per head
 *   S_t = decay[h] S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t
 * with q, k rotated over their first rot_dims dimensions (rotate-half pairing, cos_sin [positions,
 * rot_dims] fp32 = cos || sin) and k scaled by k_scale afterwards.  state [slots, heads, head_dim, v_dim]
 * fp32 is read at slot req_pool_indices[r] unless the request starts at position 0 (zero state then),
 * and written back.  Decode (seq_lens != NULL) or ragged extend as spd_attn_general; in decode rows
 * whose out_cache_loc is 0 (padding of a captured batch) leave the state untouched.  o fp32 [tokens,
 * heads * v_dim].  in_act 1: q, k and v pass through SiLU (in fp32) as they are read, before the rotation. */
int spd_retention(float* o, const void* q, const void* k, const void* v, float* state,
                  const int64_t* req_pool_indices, const int64_t* seq_lens, const int64_t* out_cache_loc,
                  const int32_t* prefix_lens, const int32_t* extend_lens, const int32_t* extend_start_loc,
                  int64_t batch, int num_heads, int head_dim, int v_dim, int64_t q_stride, int64_t k_stride,
                  int64_t v_stride, const float* decay, const float* cos_sin, int rot_dims,
                  int64_t max_positions, float k_scale, int in_act, int dtype, spd_stream_t stream);

/* spd_residual_rmsnorm with a second weight: out2 = the same normed row times (weight_offset + w2)
 * (out2 and w2 both NULL or both given) */
int spd_residual_rmsnorm2(void* out, void* out2, float* x, const void* a, const void* b, const void* w,
                          const void* w2, int64_t rows, int64_t dim, float eps, float weight_offset, int dtype,
                          spd_stream_t stream);
/* block-diagonal spd_linear_simt: for g < num_groups, C[:, g * c_group_cols : + N] =
 * A[:, g * a_group_cols : + K] W[g * N : (g + 1) * N, :K]^T */
int spd_linear_simt_block_diag(void* C, const void* A, const void* W, int64_t M, int64_t N, int64_t K,
                               int64_t lda, int64_t ldw, int64_t ldc, int num_groups, int64_t a_group_cols,
                               int64_t c_group_cols, int dtype, spd_stream_t stream);
/* Linear attention with a decay per key channel that depends on the token; per head, state S [head_dim,
 * v_dim] fp32 at slot req_pool_indices[r] (zero for a request that starts at position 0), written back.
 *   form 0: w = sigmoid(z + z_bias)^(1 / tau);  S_t = diag(w_t) S_(t-1) + k_t v_t^T;  o_t = S_t^T (q_t q_scale)
 *   form 1: w = exp(-exp(z + z_bias));  o_t = (S_(t-1) + diag(bonus[h]) k_t v_t^T)^T (q_t q_scale);
 *           S_t = diag(w_t) S_(t-1) + k_t v_t^T
 * q, k, z [tokens, heads * head_dim], v [tokens, heads * v_dim] (dtype, row strides given); z_bias (nullable)
 * and bonus fp32 [heads * head_dim].  Decode / ragged extend and padded rows as spd_retention.  o fp32. */
int spd_gated_recurrence(float* o, const void* q, const void* k, const void* v, const void* z, float* state,
                         const int64_t* req_pool_indices, const int64_t* seq_lens, const int64_t* out_cache_loc,
                         const int32_t* prefix_lens, const int32_t* extend_lens, const int32_t* extend_start_loc,
                         int64_t batch, int num_heads, int head_dim, int v_dim, int64_t q_stride, int64_t k_stride,
                         int64_t v_stride, int64_t z_stride, const float* z_bias, const float* bonus, int form,
                         float q_scale, float tau, int dtype, spd_stream_t stream);
/* out[s, t, :] = h[t, :] + (h[t - 1, :] - h[t, :]) * mu[s, :] for s < n_mix (out [n_mix, total_rows, dim]);
 * the row before a request's first new row is shift_state[req_pool_indices[r]] (fp32 [slots, dim]; zeros at
 * position 0), which then receives the request's last row.  max_rows_per_request: host-side bound of
 * extend_lens (0: total_rows). */
int spd_token_shift_mix(void* out, const void* h, const void* mu, float* shift_state,
                        const int64_t* req_pool_indices, const int64_t* seq_lens, const int64_t* out_cache_loc,
                        const int32_t* prefix_lens, const int32_t* extend_lens, const int32_t* extend_start_loc,
                        int64_t batch, int64_t total_rows, int64_t max_rows_per_request, int64_t dim, int n_mix,
                        int dtype, spd_stream_t stream);
/* x[r, 2i] = table[idx[r], 2i] + sin(positions[r] f_i), x[r, 2i + 1] = table[idx[r], 2i + 1] + cos(positions[r] f_i),
 * f_i = freq_hi[i] + freq_lo[i] (fp32 [ceil(dim / 2)] each) */
int spd_embed_sincos(float* x, const void* table, const int64_t* idx, const int64_t* positions,
                     const float* freq_hi, const float* freq_lo, int64_t rows, int64_t dim, int64_t table_rows,
                     int dtype, spd_stream_t stream);
/* out[r, :] = [a[r, :] | b[r, :]] converted to dtype (a, b fp32 [rows, dim]; out [rows, 2 dim]) */
int spd_cast_concat(void* out, const float* a, const float* b, int64_t rows, int64_t dim, int dtype,
                    spd_stream_t stream);
/* out[r, c] = act(x[r * x_stride + c]); act 0 SiLU, 1 tanh-form GELU, 2 relu squared, 3 tanh, 4 relu */
int spd_activation(void* out, const void* x, int64_t rows, int64_t cols, int64_t x_stride, int act, int dtype,
                   spd_stream_t stream);
/* y = x[r, :dim] / sqrt(mean(x[r, :dim]^2) + eps) * w; pool[loc[r] * pool_stride + :] = y (pool nullable) and
 * out[r, :] = y (out nullable, contiguous) */
int spd_rmsnorm_store(void* pool, void* out, const void* x, const void* w, const int64_t* loc, int64_t rows,
                      int64_t dim, int64_t x_stride, int64_t pool_stride, float eps, int dtype,
                      spd_stream_t stream);
/* out[t, h, :] = o[t, h, :] * sigmoid(g[t, h]) (o row stride o_stride, g row stride g_stride, out contiguous) */
int spd_head_gate_sigmoid(void* out, const void* o, const void* g, int64_t tokens, int heads, int vdim,
                          int64_t o_stride, int64_t g_stride, int dtype, spd_stream_t stream);
/* x[i] *= alpha for i < n */
int spd_scale_f32(float* x, int64_t n, float alpha, spd_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * A residual kept as several streams (hyper-connections), the rotary step of an attention with
 * biased projections, and the exponentially gated matrix memory (csrc/stream_ops.cu, matrix_memory.cu)
 * ------------------------------------------------------------------------------------------- */
/* X[r, s, :] = table[idx[r], :] / sqrt(mean(.^2) + eps) * w for s < streams (X fp32 [rows, streams, dim];
 * w NULL: the raw row) */
int spd_embed_norm_streams(float* X, const void* table, const int64_t* idx, const void* w, int64_t rows,
                           int64_t dim, int64_t table_rows, int streams, float eps, int dtype,
                           spd_stream_t stream);
/* Per token r (X fp32 [tokens, streams, dim], in place):
 *   write (a != NULL): y = sa a[r] + sb b[r] + sbias bias (b, bias nullable; a, b dtype [tokens, dim], bias fp32
 *     [dim]); X'[t] = sum_s mix[s * streams + t] X[s] + mult * outw[t] * y  (mix, outw fp32)
 *   read (out != NULL): u = sum_s inw[s] X'[s] (inw NULL: all 1); out[r] = u / sqrt(mean(u^2) + eps) * w
 * rows_idx != NULL (read only): out row r comes from token rows_idx[r]; `rows` counts out rows. */
int spd_streams_mix_norm(void* out, float* X, const void* a, const void* b, const float* bias, float sa, float sb,
                         float sbias, const float* mix, const float* outw, float mult, const float* inw,
                         const void* w, const int64_t* rows_idx, int64_t rows, int64_t dim, int streams,
                         float eps, int dtype, spd_stream_t stream);
/* q_out[t] = rot(q[t] + q_bias), k_pool[loc[t]] = rot(k[t] + k_bias), rotation of the first rot_dims dimensions
 * of every head by position positions[t] (rotate-half pairing, cos_sin [max_positions, rot_dims] fp32 =
 * cos || sin); v_pool[loc[t]] = v[t], or, with v NULL, the biased keys before the rotation (v_pool nullable;
 * biases fp32, nullable). */
int spd_rotary_bias_store(void* q_out, const void* q, const void* k, const void* v, const float* q_bias,
                          const float* k_bias, void* k_pool, void* v_pool, const int64_t* loc,
                          const int64_t* positions, const float* cos_sin, int rot_dims, int64_t max_positions,
                          int64_t tokens, int num_q_heads, int num_kv_heads, int head_dim, int v_dim,
                          int64_t q_stride, int64_t k_stride, int64_t v_stride, int64_t q_out_stride, int dtype,
                          spd_stream_t stream);
/* floats per slot of the vector state of spd_matrix_memory: per head and block of 32 value columns, n
 * [head_dim] and m */
int64_t spd_matrix_memory_vector_dim(int num_heads, int head_dim, int v_dim);
/* Exponentially gated matrix memory per (request, head): with i = softcap(zi + i_bias), f =
 * logsigmoid(softcap(zf + f_bias)), softcap(z) = cap tanh(z / cap) (cap <= 0: z),
 *   m' = max(f + m, i); S' = e^(f + m - m') S + e^(i - m') k v^T; n' = e^(f + m - m') n + e^(i - m') k;
 *   o = S'^T (q q_scale) / (max(|n' . q q_scale|, e^(-m')) + 1e-6)
 * S [slots, heads, head_dim, v_dim] and vec [slots, vec_stride] fp32 at slot req_pool_indices[r] (S = n = 0,
 * m = 0 for a request that starts at position 0), written back.  q, k [tokens, heads * head_dim], v [tokens,
 * heads * v_dim], zi, zf [tokens, heads] (dtype, row strides given); biases fp32 [heads], nullable.  Decode /
 * ragged extend and padded rows as spd_retention.  o fp32 [tokens, heads * v_dim]. */
int spd_matrix_memory(float* o, const void* q, const void* k, const void* v, const void* zi, const void* zf,
                      float* state, float* vec, int64_t vec_stride, const int64_t* req_pool_indices,
                      const int64_t* seq_lens, const int64_t* out_cache_loc, const int32_t* prefix_lens,
                      const int32_t* extend_lens, const int32_t* extend_start_loc, int64_t batch, int num_heads,
                      int head_dim, int v_dim, int64_t q_stride, int64_t k_stride, int64_t v_stride,
                      int64_t zi_stride, int64_t zf_stride, const float* i_bias, const float* f_bias, float cap,
                      float q_scale, int dtype, spd_stream_t stream);

/* spd_attn_general with three more options.  softcap > 0: score <- softcap * tanh(score / softcap) after the
 * scale and before the distance bias.  num_v_heads (0: num_kv_heads): the value pool has fewer heads than the
 * key pool and key head g reads value head g mod num_v_heads (several attention maps over one set of values).
 * v_slot_stride (0: num_v_heads * v_dim): elements between two slots of v_pool — with v_pool = k_pool,
 * num_v_heads = 1 and v_slot_stride = head_dim, the values are the first v_dim columns of the key rows (a latent
 * cache). */
int spd_attn_general_ex(void* out, const void* q, const void* k_pool, const void* v_pool,
                        const int32_t* req_to_token, const int64_t* req_pool_indices, const int64_t* seq_lens,
                        const int32_t* prefix_lens, const int32_t* extend_lens, const int32_t* extend_start_loc,
                        int64_t batch, int64_t total_tokens, int num_q_heads, int num_kv_heads, int head_dim,
                        int v_dim, int64_t q_stride, int64_t out_stride, int64_t req_to_token_stride,
                        float sm_scale, int window, const float* sinks, const float* slopes, float qtemp_coef,
                        int qtemp_every, int64_t max_extend_len, float softcap, int num_v_heads,
                        int64_t v_slot_stride, int dtype, spd_stream_t stream);
/* x[t, :] = table[idx[t], :] * scale + pair[row, :] (fp32) with row = (prev * mul_prev + idx[t] * mul_cur) mod
 * buckets, or `buckets` (the table's last row) for the first token of a request; pair == NULL: no pair term.
 * prev is the token before in the same request: the row before in the batch, or prev_state[slot] (int32
 * [slots], slot = req_pool_indices[r]) for the first row of a portion that does not start at position 0;
 * afterwards prev_state[slot] holds the request's last token of this batch.  Decode (seq_lens != NULL; rows
 * with out_cache_loc == 0 are padding and leave the state alone) or ragged extend as spd_attn_general. */
int spd_embed_pair(float* x, const void* table, const void* pair, const int64_t* idx, int32_t* prev_state,
                   const int64_t* req_pool_indices, const int64_t* seq_lens, const int64_t* out_cache_loc,
                   const int32_t* prefix_lens, const int32_t* extend_lens, const int32_t* extend_start_loc,
                   int64_t batch, int64_t tokens, int64_t dim, int64_t table_rows, float scale, int64_t buckets,
                   int64_t mul_prev, int64_t mul_cur, int dtype, spd_stream_t stream);
/* x (fp32 [*, dim], in place) += a + x0 + vec (a [*, dim] in dtype, x0 fp32 [*, dim], vec fp32 [dim]; each
 * nullable), then out[r, :] = tanh(alpha * x[row, :]) * w + b in dtype (w, b [dim]; out, w, b all NULL: update
 * only).  rows (int64 [n_rows], nullable) selects the rows that are normed; nothing is added then. */
int spd_residual_tanh_norm(void* out, float* x, const void* a, const float* x0, const float* vec, const void* w,
                           const void* b, const int64_t* rows, int64_t n_rows, int64_t dim, float alpha, int dtype,
                           spd_stream_t stream);
/* One strided piece of a rotary step: head h of token t is read at src + t * src_row + h * src_head (elements),
 * bias (fp32 [heads * head_dim], nullable) is added, the first `rot` channels are rotated, and the head is
 * written to dst + (to_pool ? loc[t] : t) * dst_row + h * dst_head. */
typedef struct {
  const void* src;
  const float* bias;
  void* dst;
  int64_t src_row, dst_row;
  int32_t heads, head_dim, rot, src_head, dst_head, to_pool;
} spd_rotary_segment_t;
/* Up to four segments in one launch.  cos_sin fp32 [max_positions, rot_max] = cos || sin (rot_max / 2 each) of
 * position * f_i; a segment with rot < rot_max uses the first rot / 2 of both.  paired != 0: channel 2 i turns
 * with 2 i + 1, else channel i with i + rot / 2: (u, v) -> (u cos - v sin, v cos + u sin). */
int spd_rotary_segments(const spd_rotary_segment_t* segments, int num_segments, const int64_t* positions,
                        const int64_t* loc, const float* cos_sin, int rot_max, int64_t max_positions, int paired,
                        int64_t tokens, int dtype, spd_stream_t stream);
/* out[t, h, c] = y * sigmoid(gate[t, h * vdim + c]) with y = a[t, h, c], or — a2 given (same strides as a) —
 * y = d / sqrt(mean_c(d^2) + eps) * post, d = a - lambda * a2 (the difference of two attention maps at unit RMS
 * per head). */
int spd_heads_gate(void* out, const void* a, const void* a2, const void* gate, int64_t tokens, int heads, int vdim,
                   int64_t a_stride, int64_t gate_stride, int64_t out_stride, float lambda, float eps, float post,
                   int dtype, spd_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* SPD_H_ */
