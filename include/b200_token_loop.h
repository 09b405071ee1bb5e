/*
 * b200_token_loop.h — C ABI of the B200 (sm_100a) per-step token loop.
 *
 * This library replaces the device side of sglang.cpp's per-step forward pass
 * (Engine::forward_batch, src/engine/engine.cc:495-544 of the reference) with
 * hand-written sm_100a kernels.  Every entry point takes plain device pointers,
 * sizes, strides (in elements) and a CUDA stream; none allocates or touches
 * LibTorch types.  Each declaration cites the reference interface it stands in
 * for, by the file's path inside the reference project.
 *
 * Conventions
 *   - All entry points return B200_OK (0) or a B200_ERR_* code;
 *     b200_last_error() gives the text for the calling thread.
 *   - bf16 tensors are raw uint16 storage ("bf16*" below means const void* /
 *     void* pointing at __nv_bfloat16 data).  Index tensors are int32.
 *   - `stream` is a cudaStream_t passed as void*; NULL is the legacy default
 *     stream.  Calls are asynchronous unless stated otherwise.
 *   - Nothing here synchronises the device unless stated otherwise.
 */
#ifndef B200_TOKEN_LOOP_H_
#define B200_TOKEN_LOOP_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_API __attribute__((visibility("default")))

typedef void* b200_stream_t;

enum {
    B200_OK = 0,
    B200_ERR_INVALID_ARGUMENT = 1, /* the reference would TORCH_CHECK-fail here */
    B200_ERR_CUDA = 2,             /* a CUDA runtime / driver call failed */
    B200_ERR_TIMEOUT = 3,          /* a bounded in-kernel wait ran out */
    B200_ERR_UNSUPPORTED = 4,      /* shape / dtype outside what the kernels cover */
    B200_ERR_STATE = 5             /* object used in the wrong state */
};

/* ---- library ------------------------------------------------------------- */

/* Text of the last error returned to the calling thread ("" if none). */
B200_API const char* b200_last_error(void);

/* ABI version of this header (bumped on incompatible change). */
B200_API int b200_abi_version(void);

/* Reads (synchronously) and clears the device status words that kernels with
 * bounded waits or index checks write: out[0] = wait site that timed out (0 =
 * none), out[1] = offending index + 1 (0 = none).  Synchronises `stream`. */
B200_API int b200_read_device_status(int32_t out[2], b200_stream_t stream);

/* ---- normalisation (include/sglang/layers/normalization.h:6-22) ---------- */

/* RMSNorm::forward / forward_inplace (src/layers/normalization.cu:236-269):
 * out[r,:] = x[r,:] * rsqrt(mean(x[r,:]^2) + eps) * weight, fp32 math, bf16
 * storage.  out may alias x.  x, out: [rows, hidden] contiguous. */
B200_API int b200_rmsnorm(void* out, const void* x, const void* weight, int rows, int hidden,
                          float eps, b200_stream_t stream);

/* RMSNorm::fused_add_forward_inplace (src/layers/normalization.cu:386-416):
 * residual <- x + residual (fp32 add, stored bf16); x <- rmsnorm(fp32 sum) * weight. */
B200_API int b200_fused_add_rmsnorm(void* x, void* residual, const void* weight, int rows,
                                    int hidden, float eps, b200_stream_t stream);

/* fused_qk_rmsnorm_inplace_3d_strided and RMSNorm::forward_inplace_3d_strided
 * (src/layers/normalization.cu:271-384): per-(token, head) RMSNorm over head_dim,
 * in place, on strided views q [tokens, q_heads, head_dim] and k [tokens,
 * k_heads, head_dim].  Either of q / k may be NULL (with 0 heads) for the
 * single-tensor form.  Strides are in elements. */
B200_API int b200_qk_rmsnorm_strided(void* q, void* k, const void* q_weight, const void* k_weight,
                                     int tokens, int q_heads, int k_heads, int head_dim,
                                     int64_t q_stride_token, int64_t q_stride_head,
                                     int64_t k_stride_token, int64_t k_stride_head, float eps,
                                     b200_stream_t stream);

/* ---- rotary embedding (include/sglang/layers/rotary_embedding.h:11-22) ---- */

/* RotaryEmbedding::forward_inplace (src/layers/rotary_embedding.cu:96-190):
 * NeoX (rotate-half) RoPE applied in place to q [tokens, q_heads, head_dim] and
 * k [tokens, k_heads, head_dim] from fp32 tables cos/sin [max_pos, rotary_dim/2]
 * and int32 positions [tokens].  fp32 math, bf16 storage. */
B200_API int b200_rope_neox_inplace(void* q, void* k, const float* cos_table,
                                    const float* sin_table, const int32_t* positions, int tokens,
                                    int q_heads, int k_heads, int head_dim, int rotary_dim,
                                    int max_pos, int64_t q_stride_token, int64_t q_stride_head,
                                    int64_t k_stride_token, int64_t k_stride_head,
                                    b200_stream_t stream);

/* ---- KV pool (include/sglang/kvcache/base.h:78-90) ------------------------ */

/* MHAKVCache::store_kv (src/kvcache/mha_kvcache.cu:12-41,113-155):
 * k_cache[out_loc[t], :, :] = k[t, :, :] and the same for v.  k_cache / v_cache:
 * one layer's [slots, kv_heads, head_dim] contiguous; k / v: strided rows of
 * kv_heads*head_dim elements. */
B200_API int b200_store_kv(void* k_cache, void* v_cache, const void* k, const void* v,
                           const int32_t* out_loc, int tokens, int kv_heads, int head_dim,
                           int64_t k_stride_token, int64_t v_stride_token, int64_t num_slots,
                           b200_stream_t stream);

/* The three steps AttentionLayer::forward runs before attention
 * (src/layers/attention_layer.cc:17-47), as one pass over the packed qkv rows
 * [tokens, (q_heads + 2*kv_heads)*head_dim]: optional per-head QK RMSNorm
 * (q_weight/k_weight NULL = none), NeoX RoPE, then the KV-pool store of the
 * rotated k and of v at out_loc.  q is rewritten in place; with
 * write_k_back != 0 the k rows are too (as the reference leaves them).
 * Rounding points match the unfused sequence (bf16 after the norm, bf16 after
 * the rotation). */
B200_API int b200_qknorm_rope_store(void* qkv, const void* q_weight, const void* k_weight,
                                    const float* cos_table, const float* sin_table,
                                    const int32_t* positions, const int32_t* out_loc,
                                    void* k_cache, void* v_cache, int tokens, int q_heads,
                                    int kv_heads, int head_dim, int max_pos, int64_t num_slots,
                                    float eps, int write_k_back, b200_stream_t stream);

/* ---- activation (include/sglang/layers/activation.h:8-11) ----------------- */

/* silu_and_mul / gelu_and_mul (src/layers/activation.cu:15-75):
 * out[t, j] = act(in[t, j]) * in[t, d + j]; in [tokens, 2*d], out [tokens, d]. */
B200_API int b200_silu_and_mul(void* out, const void* in, int tokens, int d, b200_stream_t stream);
B200_API int b200_gelu_and_mul(void* out, const void* in, int tokens, int d, b200_stream_t stream);

/* ---- embedding and index tables ------------------------------------------- */

/* torch::nn::Embedding as used by the models (src/models/qwen3.cc:38-43,56):
 * out[t, :] = table[ids[t], :].  ids int32; an id outside [0, vocab) writes a
 * zero row and records the index in the device status word. */
B200_API int b200_embedding(void* out, const void* table, const int32_t* ids, int tokens,
                            int hidden, int vocab, b200_stream_t stream);

/* gather_int32_2d (src/kernels/token_pool.cu:31-49,93-133):
 * out[i] = table[req[i], pos[i]], 0 when either index is out of range. */
B200_API int b200_gather_int32_2d(int32_t* out, const int32_t* table, int64_t rows, int64_t stride,
                                  int64_t cols, const int32_t* req_indices,
                                  const int32_t* positions, int64_t count, b200_stream_t stream);

/* write_token_pool (src/kernels/token_pool.cu:10-29,53-91):
 * table[req[i], pos[i]] = tokens[i], skipped when either index is out of range. */
B200_API int b200_write_token_pool(int32_t* table, int64_t rows, int64_t stride, int64_t cols,
                                   const int32_t* req_indices, const int32_t* positions,
                                   const int32_t* tokens, int64_t count, b200_stream_t stream);

/* ---- linear (include/sglang/layers/linear.h:7-73) -------------------------- */

enum {
    B200_EPILOGUE_NONE = 0,
    /* y[m, j] = silu(bf16(acc[m, j])) * bf16(acc[m, N/2 + j]), j < N/2: the
     * gate_up projection followed by silu_and_mul (src/models/utils.cc:41-57). */
    B200_EPILOGUE_SWIGLU = 1,
    B200_EPILOGUE_GEGLU = 2,     /* tanh-approximated GELU, as gelu_and_mul (src/layers/activation.cu:11-13) */
    B200_EPILOGUE_GEGLU_ERF = 3  /* exact GELU, as torch::gelu in MoELayer::forward (src/moe/moe.cc:80) */
};

/* LinearBase::forward (src/layers/linear.cc:24-26): y = x W^T (+ bias), bf16 in,
 * fp32 accumulate on the tcgen05 tensor cores, bf16 out.  x [M, K] with row
 * stride ldx, w [N, K] contiguous, y [M, N_out] contiguous where N_out = N (or
 * N/2 with a gated epilogue).  K must be a multiple of 64, N of 16. */
B200_API int b200_linear(void* y, const void* x, const void* w, const void* bias, int M, int N,
                         int K, int64_t ldx, int epilogue, b200_stream_t stream);

/* ---- mixture of experts (include/sglang/moe/moe.h:9-35) -------------------- */

/* Bytes of scratch b200_moe_forward needs (routing tables and the permuted activations). */
B200_API int64_t b200_moe_workspace_bytes(int tokens, int num_experts, int top_k, int hidden_size,
                                          int intermediate_size);

/* The routing half of MoELayer::forward (src/moe/moe.cc:47-55): fp32 softmax of bf16 router
 * logits [tokens, num_experts], top_k largest per token (lower expert index on ties), optional
 * renormalisation w / (sum w + 1e-8), weights rounded to bf16 as the reference casts them.
 * topk_ids int32 [tokens, top_k], topk_weights float [tokens, top_k], expert_counts int32
 * [num_experts + 1] (histogram; cleared by the call). */
B200_API int b200_moe_route(int32_t* topk_ids, float* topk_weights, int32_t* expert_counts,
                            const void* router_logits, int tokens, int num_experts, int top_k,
                            int renormalize, b200_stream_t stream);

/* MoELayer::forward (src/moe/moe.cc:36-96) for tp_size 1 (the caller all-reduces under TP):
 * out[t] = sum over the token's top_k experts e, in k order with bf16 accumulation, of
 * w[t,k] * down_e(act(gate_e x_t) * up_e x_t).  hidden_states / out bf16 [tokens, hidden_size];
 * gate_up_proj bf16 [E, 2*I, hidden]; down_proj bf16 [E, hidden, I]; activation 0 = silu,
 * 1 = gelu (exact, as torch::gelu).  No host synchronisation: six launches. */
B200_API int b200_moe_forward(void* out, const void* hidden_states, const void* router_logits,
                              const void* gate_up_proj, const void* down_proj, int tokens,
                              int num_experts, int top_k, int hidden_size, int intermediate_size,
                              int renormalize, int activation, void* workspace,
                              int64_t workspace_bytes, b200_stream_t stream);

/* One rank's share of MoELayer::forward under expert parallelism.  No counterpart in the
 * reference, whose MoELayer gives every rank a slice of every expert's intermediate dimension
 * (src/moe/moe.cc:12-30); here the rank holds whole experts [expert_begin, expert_begin +
 * num_local_experts) of the router's num_experts: gate_up_proj bf16 [num_local_experts, 2*I,
 * hidden], down_proj bf16 [num_local_experts, hidden, I].  Routing runs over all experts; only
 * the local experts' terms are summed into out (rows with none are zero); the all-reduce the
 * caller runs next (tensor_model_parallel_all_reduce, src/moe/moe.cc:92-94) adds the ranks. */
B200_API int b200_moe_forward_local(void* out, const void* hidden_states, const void* router_logits,
                                    const void* gate_up_proj, const void* down_proj, int tokens,
                                    int num_experts, int top_k, int hidden_size,
                                    int intermediate_size, int renormalize, int activation,
                                    int expert_begin, int num_local_experts, void* workspace,
                                    int64_t workspace_bytes, b200_stream_t stream);

/* ---- attention (include/sglang/attention/backend.h:24-41) ------------------ */

/* Bytes of scratch b200_attention_decode needs for up to max_batch requests
 * with q_heads / kv_heads local heads. */
B200_API int64_t b200_attention_decode_workspace_bytes(int max_batch, int q_heads, int kv_heads,
                                                       int head_dim);

/* FlashInferBackend::forward for a decode batch
 * (src/attention/flashinfer_backend.cu:553-595): out[b, h, :] = softmax(q[b, h]
 * . K_b^T / sqrt(d)) V_b over the seq_lens[b] keys whose KV-pool slots are
 * page_table[table_idx[b], 0 .. seq_lens[b]).  page_table holds one slot per
 * token position; page_size states that positions [j*page_size, (j+1)*page_size)
 * of a row are consecutive slots starting at a multiple of page_size (1 = no
 * such guarantee, as the reference Engine runs).  q [batch, q_heads, head_dim]
 * with strides; out [batch, q_heads*head_dim] contiguous.  k_cache / v_cache:
 * one layer's [num_slots, kv_heads, head_dim].  workspace: zero-initialised
 * once by the caller, then owned by the calls (they leave it zeroed where it
 * must be).  Split-KV is decided on the device; no host plan. */
B200_API int b200_attention_decode(void* out, const void* q, int64_t q_stride_token,
                                   int64_t q_stride_head, const void* k_cache, const void* v_cache,
                                   int64_t num_slots, const int32_t* page_table,
                                   int64_t page_table_stride, const int32_t* table_idx,
                                   const int32_t* seq_lens, int batch, int q_heads, int kv_heads,
                                   int head_dim, int page_size, float sm_scale, void* workspace,
                                   int64_t workspace_bytes, b200_stream_t stream);

/* No counterpart in the reference.  The same computation as b200_attention_decode for callers
 * that cannot allocate device memory when they need it (a process whose device-memory budget is
 * already owned by one pool, or a step loop that must not run into cudaMalloc's device-wide
 * synchronisation): there is no workspace argument, the split-KV scratch is an 8 MiB array built
 * into the library image (every GPU that loads the library carries it until exit).  The call makes
 * no cudaMalloc / cudaFree and no other allocating call.  Shapes whose partial results need more
 * than that array (see b200_attention_decode_workspace_bytes; 64 requests x 16 query heads need
 * under 2 MiB) are refused with B200_ERR_UNSUPPORTED.  The first call on a device looks up the
 * array's device address (cudaGetSymbolAddress) with that device current; make that first call
 * before any stream capture begins.  All calls share the one array and it keeps the previous
 * call's contents (the call clears the words that must start at zero): two calls whose kernels
 * overlap on the GPU race.  What the kernel reports (a wait that ran out, a page-table slot out of
 * range) goes to two words inside the same array, NOT to the words b200_read_device_status reads:
 * read them with b200_attention_decode_noalloc_status. */
B200_API int b200_attention_decode_noalloc(void* out, const void* q, int64_t q_stride_token,
                                           int64_t q_stride_head, const void* k_cache,
                                           const void* v_cache, int64_t num_slots,
                                           const int32_t* page_table, int64_t page_table_stride,
                                           const int32_t* table_idx, const int32_t* seq_lens,
                                           int batch, int q_heads, int kv_heads, int head_dim,
                                           int page_size, float sm_scale, b200_stream_t stream);

/* No counterpart in the reference.  Reads what the kernels of b200_attention_decode_noalloc reported
 * on the current device since the last read, after synchronising `stream`: out[0] = site of a wait
 * that ran out (0 = none), out[1] = offending slot + 1 of a page-table entry outside the pool (0 =
 * none; the kernel read slot 0 instead, nothing faulted).  Non-zero words are cleared by the read, so
 * a report survives later calls until somebody looks.  Allocates nothing. */
B200_API int b200_attention_decode_noalloc_status(int32_t out[2], b200_stream_t stream);

/* FlashInferBackend::forward for a prefill (extend) batch
 * (src/attention/flashinfer_backend.cu:596-678): causal attention of ragged
 * query rows against paged keys.  Request b owns query rows
 * [qo_indptr[b], qo_indptr[b+1]), which are the LAST extend positions of its
 * seq_lens[b] keys (the first seq_lens[b] - extend_len are the cached prefix).
 * max_extend_len bounds the longest request's extend length (grid sizing). */
B200_API int b200_attention_prefill(void* out, const void* q, int64_t q_stride_token,
                                    int64_t q_stride_head, const void* k_cache,
                                    const void* v_cache, int64_t num_slots,
                                    const int32_t* page_table, int64_t page_table_stride,
                                    const int32_t* table_idx, const int32_t* seq_lens,
                                    const int32_t* qo_indptr, int batch, int max_extend_len,
                                    int q_heads, int kv_heads, int head_dim, int page_size,
                                    float sm_scale, b200_stream_t stream);

/* ---- sampler (include/sglang/engine/engine.h:36-55) ------------------------- */

/* Sampler::sample, all-greedy branch (src/engine/engine.cc:294-298): argmax over
 * bf16 logits [rows, vocab] (row stride ld), first index on ties, int32 out. */
B200_API int b200_argmax(int32_t* out, const void* logits, int rows, int vocab, int64_t ld,
                         b200_stream_t stream);

/* Sampler::sample, stochastic branch (src/engine/engine.cc:299-338) with the candidate set of
 * sample_row (engine.cc:126-158): logits / temperature, keep the top_k largest, then drop sorted
 * entries whose inclusive cumulative probability exceeds top_p (never the first), renormalise and
 * draw.  bf16 logits [rows, vocab]; temperatures / top_k / top_p per row as Sampler::prepare
 * clamps them (top_k, top_p may be NULL = off; a row with temperature <= 1e-6 is greedy).  The
 * draw uses Philox keyed by seeds[row] (NULL = row index) and step_index, so it is reproducible;
 * the reference draws from torch's global generator instead.  candidate_mask (NULL or uint8
 * [rows, vocab]) receives 1 for every token of the final candidate set.  Ties are ordered by
 * index. */
B200_API int b200_sample(int32_t* out, const void* logits, int rows, int vocab, int64_t ld,
                         const float* temperatures, const int32_t* top_k, const float* top_p,
                         const uint64_t* seeds, uint64_t step_index, uint8_t* candidate_mask,
                         b200_stream_t stream);

/* flashinfer_sample_from_probs / _top_k_ / _top_p_ / _top_k_top_p_sample_from_probs
 * (include/sglang/engine/sampling.h:12-34; src/engine/sampling.cu:65-192): one token per row of
 * fp32 probabilities [rows, vocab] (contiguous), drawn with the caller's uniform number
 * uniform[row] in [0, 1) by inverse CDF over the tokens FlashInfer's rejection samplers accept:
 * those among the top_k largest probabilities (ties included) whose strictly larger probabilities
 * sum to less than top_p.  top_k / top_p: per-row device arrays, or NULL to use the scalar
 * (top_k_value < 1 or >= vocab and top_p_value >= 1 switch the filter off).  Always succeeds (the
 * reference's `success` flags are all true).  Reproducible: masses are summed in fixed point. */
B200_API int b200_sample_from_probs(int32_t* out, const float* probs, int rows, int vocab,
                                    const int32_t* top_k, int top_k_value, const float* top_p,
                                    float top_p_value, const float* uniform, b200_stream_t stream);

/* ---- tensor-parallel all-reduce (include/sglang/distributed/distributed.h:24) --- */

/* One process per GPU.  A communicator owns this rank's two exchange buffers (call parity 0 / 1)
 * of buffer_bytes each and a flag table, in device memory that the peers map through CUDA IPC.
 * Set-up (the part the reference does with an NCCL unique id, src/distributed/distributed.cc:
 * 142-173): every rank creates, exports its 64-byte handle, the host code gathers all handles
 * in rank order (torch.distributed / MPI / a file), every rank connects. */
typedef struct b200_comm b200_comm;
B200_API int b200_comm_create(int rank, int world, int64_t buffer_bytes, b200_comm** out);
B200_API int b200_comm_handle_bytes(void);
B200_API int b200_comm_export(b200_comm* comm, void* handle_out);
B200_API int b200_comm_connect(b200_comm* comm, const void* all_handles);
/* The same communicator over memory the host obtained elsewhere (a symmetric allocation): region =
 * this rank's block of b200_comm_region_bytes(buffer_bytes) zeroed bytes, 256-byte aligned;
 * peer_regions[world] = every rank's block as this process addresses it; multicast_region = the
 * NVLink multicast address of the blocks, or NULL.  With a multicast address the all-reduce is
 * summed inside the switch (multimem.ld_reduce) and delivered with one store (multimem.st); the
 * order of the additions is then the switch's, not rank order.  The memory stays the caller's. */
B200_API int64_t b200_comm_region_bytes(int64_t buffer_bytes);
B200_API int b200_comm_create_on(int rank, int world, int64_t buffer_bytes, void* region, b200_comm** out);
B200_API int b200_comm_connect_pointers(b200_comm* comm, const void* const* peer_regions,
                                        const void* multicast_region);
B200_API int b200_comm_uses_multicast(b200_comm* comm);
/* Device address of this rank's exchange buffer for the given parity: the producer of the
 * partial sum (the row-parallel GEMM) writes there. */
B200_API void* b200_comm_buffer(b200_comm* comm, int parity);
B200_API int b200_comm_destroy(b200_comm* comm);
/* The longest one kernel waits for its peers' announcement before it gives up, leaves its outputs
 * untouched and reports through the device status words (sites 401-403).  Default 2 s; the
 * reference's only time-out is the NCCL rendezvous (src/distributed/distributed.cc:106-120,145). */
B200_API int b200_comm_set_wait_limit_ns(b200_comm* comm, uint64_t nanoseconds);
/* Failure-path testing on ONE GPU, no counterpart in the reference: instead of b200_comm_connect,
 * map every peer onto this rank's own buffers.  A peer's announcement then never arrives by
 * itself, so a call runs into the wait limit and returns — unless the host plays the peers' part
 * first with b200_comm_loopback_announce(call_number), call numbers counting from 1 per
 * communicator (failed calls count too).  The all-reduce of such a communicator returns
 * world x this rank's partial. */
B200_API int b200_comm_connect_loopback(b200_comm* comm);
B200_API int b200_comm_loopback_announce(b200_comm* comm, uint32_t call_number, b200_stream_t stream);

/* tensor_model_parallel_all_reduce (src/distributed/distributed.cc:205-226): out[rows, hidden]
 * = bf16(sum over ranks, in rank order, fp32) of the partials in the exchange buffers of
 * `parity`.  One-shot: every rank reads every peer's partial over NVLink with plain loads.
 * Successive calls must alternate parity.  The wait for the peers is bounded; a time-out is
 * reported through the device status words. */
B200_API int b200_allreduce(b200_comm* comm, int parity, void* out, int rows, int hidden,
                            b200_stream_t stream);
/* The all-reduce above fused with the RMSNorm::fused_add_forward_inplace that the models run on
 * its result (src/models/qwen3.cc:24,31; src/layers/linear.cc:52-55,73-76):
 * residual <- bf16(all-reduce) + residual; x_out <- rmsnorm(sum) * weight. */
B200_API int b200_allreduce_fused_add_rmsnorm(b200_comm* comm, int parity, void* x_out,
                                              void* residual, const void* weight, int rows,
                                              int hidden, float eps, int round_sum_first,
                                              b200_stream_t stream);

/* ---- step runner (include/sglang/engine/engine.h:57-103) -------------------- */

/* The fields of ModelConfig the forward pass reads (include/sglang/models/config.h:15-42). */
typedef struct b200_model_config {
    int32_t num_layers;
    int32_t hidden_size;
    int32_t num_qo_heads;
    int32_t num_kv_heads;
    int32_t head_dim;
    int32_t intermediate_size;
    int32_t vocab_size;
    float rms_norm_eps;
    float rope_theta;
    int32_t max_position;
    int32_t tie_word_embeddings;
    int32_t qk_norm;        /* per-head q/k RMSNorm (Qwen3, Qwen3-MoE) */
    int32_t fused_residual; /* 1: Qwen3 wiring (src/models/qwen3.cc:21-35); 0: Llama wiring (src/models/llama.cc:15-29) */
    int32_t attention_bias; /* qkv bias (Qwen2) */
    int32_t hidden_act;     /* 0 = silu, 1 = gelu */
    int32_t num_experts;    /* 0 = dense MLP */
    int32_t num_experts_per_tok;
    int32_t moe_intermediate_size;
    int32_t norm_topk_prob;
} b200_model_config;

/* The fields of EngineConfig that size device state (include/sglang/engine/config.h:13-32). */
typedef struct b200_engine_config {
    int32_t page_size;         /* tokens per KV page (the reference Engine runs 1) */
    int32_t num_pages;         /* usable pages; one more is allocated as the dummy page */
    int32_t max_running_req;   /* page-table rows; row max_running_req is the dummy request's */
    int32_t max_seq_len;
    int32_t max_extend_tokens; /* most tokens one prefill step may carry */
    int32_t tp_rank;
    int32_t tp_size;
    int32_t expert_parallel;   /* MoE models under tp_size > 1: 0 = every rank holds a slice of every
                                  expert's intermediate dimension (the reference's layout), 1 = rank r
                                  holds whole experts [r*E/tp, (r+1)*E/tp) */
} b200_engine_config;

enum { B200_PHASE_PREFILL = 0, B200_PHASE_DECODE = 1 };

/* One scheduler step, as Scheduler::prepare_batch describes it on the host
 * (src/scheduler/scheduler.cc:275-358): all arrays are HOST memory and are copied
 * by the call.  Requests [num_reqs, num_padded_reqs) are padding (the dummy
 * request of GraphRunner::pad_batch, src/engine/engine.cc:628-645). */
typedef struct b200_step {
    int32_t phase;
    int32_t num_reqs;
    int32_t num_padded_reqs;
    const int32_t* table_idx;   /* [num_padded_reqs] page-table row (Req::table_idx) */
    const int32_t* cached_lens; /* [num_padded_reqs] keys already in the pool (Req::cached_len) */
    const int32_t* extend_lens; /* [num_padded_reqs] tokens run this step (Req::extend_len; 1 in decode) */
    const int32_t* write_pos;   /* [num_reqs] token-pool column that receives the sampled token, < 0 = none */
    const float* temperatures;  /* [num_reqs] or NULL = every request greedy (BatchSamplingArgs, engine.h:22-26) */
    const int32_t* top_k;       /* [num_reqs] or NULL */
    const float* top_p;         /* [num_reqs] or NULL */
    const uint64_t* seeds;      /* [num_reqs] or NULL: per-request RNG seed (no counterpart in the reference) */
    uint64_t step_index;        /* offsets the per-request random stream */
} b200_step;

typedef struct b200_engine b200_engine;

/* Engine::Engine (src/engine/engine.cc:412-489): allocates weights (uninitialised), the KV
 * pool [2, L, (num_pages+1)*page_size, kv_heads/tp, head_dim], the page table and token pool
 * [max_running_req+1, align32(max_seq_len)] (dummy row filled with slot num_pages*page_size),
 * RoPE tables and activation buffers on the current device. */
B200_API int b200_engine_create(const b200_model_config* model, const b200_engine_config* config,
                                b200_engine** out);
B200_API int b200_engine_destroy(b200_engine* engine);

/* Device address and size of a named tensor: "embed", "lm_head", "final_norm", "rope_cos",
 * "rope_sin", "page_table", "token_pool", "kv_cache", "logits", "next_tokens", and per layer
 * "qkv", "qkv_bias", "o", "gate_up", "down", "input_norm", "post_norm", "q_norm", "k_norm",
 * "router", "experts_gate_up", "experts_down" (layouts: src/models/weight_loader.cc:27-33,455,497). */
B200_API int b200_engine_tensor(b200_engine* engine, const char* name, int layer, void** device_ptr,
                                int64_t* nbytes);
/* Synchronous host-to-device copy into a named tensor (nbytes must equal its size). */
B200_API int b200_engine_load(b200_engine* engine, const char* name, int layer, const void* host,
                              int64_t nbytes);

/* CacheManager::write_page_table / the token-pool fill (src/scheduler/prefill.cc:144-187):
 * table[rows[i], positions[i]] = values[i] from host arrays; which = 0 page table, 1 token pool. */
B200_API int b200_engine_write_table(b200_engine* engine, int which, const int32_t* rows,
                                     const int32_t* positions, const int32_t* values, int64_t count);

/* GraphRunner::capture_graphs (src/engine/engine.cc:670-730): captures CUDA graphs per padded decode
 * batch size — one that ends in argmax and one that ends in the sampling kernel (the reference
 * samples outside its graph, src/engine/engine.cc:504-523; here the sampling parameters and the
 * step index live in device memory, so the sampled step replays too).  batch_sizes NULL or count 0:
 * the reference's default list 1, 2, 4, 8, 16, ... and max_running_req (determine_batch_sizes,
 * :592-616).  A later decode step runs at the smallest captured size >= its num_padded_reqs
 * (GraphRunner::pad_batch, :628-645): the step runner adds dummy-request rows itself. */
B200_API int b200_engine_capture_graphs(b200_engine* engine, const int32_t* batch_sizes, int count);

/* Engine::forward_batch (src/engine/engine.cc:495-544) together with the device half of
 * Scheduler::prepare_batch (scheduler.cc:329-334: out_loc / input_ids gathers) and the token
 * write-back (scheduler.cc:403-412).  Asynchronous: next_tokens_host [num_reqs] (pinned memory
 * recommended) is valid after b200_engine_synchronize (ForwardOutput::synchronize). */
B200_API int b200_engine_step(b200_engine* engine, const b200_step* step, int32_t* next_tokens_host);
B200_API int b200_engine_synchronize(b200_engine* engine);

/* The same step reporting through the engine's result ring instead of a device-to-host copy and a
 * stream synchronisation: what ForwardOutput's pinned tensor + event (src/engine/engine.cc:526-531)
 * and the scheduler's per-request finish test (src/scheduler/scheduler.cc:449-455) are in the
 * reference.  The step's last kernel writes, into pinned host memory, the sampled tokens, one finish
 * flag per request (1 when write_pos[i] < 0, i.e. the request cannot decode further, or when the
 * token equals the end-of-sequence id and ignore_eos[i] is 0; a chunked prefill request also has
 * write_pos < 0 and its flag, like its token, means nothing), and the device status words.
 * b200_engine_wait blocks on that step's own event only - steps enqueued behind it keep running -
 * and returns pointers into the slot, valid until b200_engine_result_slots() further steps have
 * been enqueued; a ticket older than that is refused.  Its return code is the step's:
 * B200_ERR_TIMEOUT / B200_ERR_INVALID_ARGUMENT as b200_engine_synchronize reports them.
 * ignore_eos: [num_reqs] or NULL (nobody ignores).  b200_engine_set_eos_token: Engine::eos_token_id
 * (include/sglang/engine/engine.h:71); negative (the default) = the model has none. */
B200_API int b200_engine_set_eos_token(b200_engine* engine, int32_t eos_token_id);
B200_API int b200_engine_result_slots(void);
B200_API int b200_engine_step_async(b200_engine* engine, const b200_step* step, const uint8_t* ignore_eos,
                                    int64_t* ticket);
B200_API int b200_engine_wait(b200_engine* engine, int64_t ticket, const int32_t** tokens,
                              const uint8_t** finished);

/* Copies the bf16 logits [rows, vocab] of the last step to host memory (synchronous). */
B200_API int b200_engine_read_logits(b200_engine* engine, void* host, int rows);

/* Tensor parallelism (engine created with tp_size > 1): export this rank's IPC handle
 * (b200_comm_handle_bytes bytes) and connect to all ranks' handles before the first step. */
B200_API int b200_engine_comm_export(b200_engine* engine, void* handle_out);
B200_API int b200_engine_comm_connect(b200_engine* engine, const void* all_handles);
/* The same over memory the host obtained elsewhere - a symmetric allocation whose peer addresses,
 * and the NVLink multicast address of the whole group where the fabric has one, the host already
 * knows (torch.distributed's symmetric memory in the tests; no counterpart in the reference, whose
 * all-reduce is NCCL's).  region: this rank's block of b200_engine_comm_region_bytes() zeroed bytes,
 * 256-byte aligned; peer_regions[tp_size]: every rank's block as this process addresses it;
 * multicast_region: the multicast address of the blocks or NULL.  With a multicast address the
 * all-reduce is reduced inside the switch (multimem.ld_reduce) and its result delivered to every
 * rank with one store (multimem.st); the sum's order of additions is then the switch's, not rank
 * order.  Replaces the communicator created with the engine; call before capturing graphs.  The
 * memory stays the caller's and must outlive the engine. */
B200_API int64_t b200_engine_comm_region_bytes(b200_engine* engine);
B200_API int b200_engine_comm_attach(b200_engine* engine, void* region, const void* const* peer_regions,
                                     const void* multicast_region);
/* The engine's communicator, for b200_comm_set_wait_limit_ns and the loop-back test hooks
 * (NULL when the engine was created with tp_size 1). */
B200_API b200_comm* b200_engine_comm(b200_engine* engine);

/* No counterpart in the reference.  With B200_DECODE_CHAIN=1 in the environment when the engine is
 * created, decode steps of at most 64 tokens of a dense, unsharded model run everything between two
 * attention launches (o_proj, add + norm, gate_up, activation, down, add + norm, the next layer's
 * qkv, QK-norm, RoPE, KV store) as one persistent kernel of 8-CTA clusters whose CTAs must all be
 * resident at once, instead of one kernel per operator (the default, and the faster of the two on
 * B200).  Returns the number of CTAs that kernel runs with on the current device, or 0 when the
 * device cannot hold it. */
B200_API int b200_decode_chain_grid(void);

/* The stream the engine enqueues on (Engine::stream_), as a cudaStream_t. */
B200_API b200_stream_t b200_engine_stream(b200_engine* engine);

/* Measurement aid with no counterpart in the reference (it profiles with steady_clock timers,
 * src/engine/engine.cc:36-87): while on, steps run eagerly (no graph replay) with a CUDA event
 * pair around each attention launch.  b200_engine_read_profile synchronises and returns the
 * summed attention time of the last step, how many attention launches that covers, and the
 * number of kernels the last step launched (also valid for graph replays, profiling or not). */
B200_API int b200_engine_set_profiling(b200_engine* engine, int on);
B200_API int b200_engine_read_profile(b200_engine* engine, float* attention_ms,
                                      int32_t* attention_launches, int32_t* kernel_launches);
/* The same for the fused all-reduce launches of the last profiled step (tensor parallelism). */
B200_API int b200_engine_read_profile_allreduce(b200_engine* engine, float* allreduce_ms,
                                                int32_t* launches);

/* Device time of the last step in milliseconds (CUDA events around it); synchronises. */
B200_API int b200_engine_last_step_ms(b200_engine* engine, float* ms);

#ifdef __cplusplus
}
#endif

#endif /* B200_TOKEN_LOOP_H_ */
