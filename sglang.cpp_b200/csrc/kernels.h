// Internal launch interface shared by the C-ABI wrappers and the step runner.
// Every function enqueues work on `stream` and returns a B200_* status.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

int launch_rmsnorm(void* out, const void* x, const void* weight, int rows, int hidden, float eps,
                   cudaStream_t stream);
// round_sum_first: normalise the bf16-rounded sum (separate add then norm, as the Llama wiring
// does) instead of the fp32 sum (the fused FlashInfer form the Qwen3 wiring uses).
int launch_fused_add_rmsnorm(void* x, void* residual, const void* weight, int rows, int hidden,
                             float eps, bool round_sum_first, cudaStream_t stream);
int launch_qknorm_rope_store(void* qkv, const void* q_weight, const void* k_weight,
                             const float* cos_table, const float* sin_table,
                             const int32_t* positions, const int32_t* out_loc, void* k_cache,
                             void* v_cache, int tokens, int q_heads, int kv_heads, int head_dim,
                             int max_pos, int64_t num_slots, float eps, int write_k_back,
                             int* status, cudaStream_t stream);
int launch_act_and_mul(void* out, const void* in, int tokens, int d, bool gelu, cudaStream_t stream);
// ssq (optional, [ssq_slots, ssq_stride]): slot 0 receives each row's sum of squares in 2^-24 fixed
// point and the other slots are zeroed for the tokens of this call.
int launch_embedding(void* out, const void* table, const int32_t* ids, int tokens, int hidden,
                     int vocab, int* status, cudaStream_t stream, unsigned long long* ssq = nullptr,
                     int ssq_slots = 0, int ssq_stride = 0);
// out[n, k] = bf16(w[n, k] * scale[k]): a norm weight folded into the columns of the matrix that follows it.
int launch_scale_columns(void* out, const void* w, const void* scale, int64_t rows, int K, cudaStream_t stream);
// Optional write-back of the chosen tokens into the token pool by the kernel that chooses them
// (token_pool[table_idx[i], write_pos[i]] = token[i] for i < count, positions outside the table
// skipped): what a separate scatter launch would do behind it.
struct TokenWriteBack {
    int32_t* pool = nullptr;
    int64_t rows = 0, stride = 0, cols = 0;
    const int32_t* table_idx = nullptr;
    const int32_t* write_pos = nullptr;
    int count = 0;
};
// step_index_dev (optional): the step index is read from device memory instead of the argument, so a
// captured graph replays with a new value.
int launch_sample(int32_t* out, const void* logits, int rows, int vocab, int64_t ld,
                  const float* temperatures, const int32_t* top_k, const float* top_p,
                  const uint64_t* seeds, uint64_t step_index, uint8_t* mask, cudaStream_t stream,
                  const uint64_t* step_index_dev = nullptr, const TokenWriteBack* write_back = nullptr);
int launch_argmax(int32_t* out, const void* logits, int rows, int vocab, int64_t ld,
                  cudaStream_t stream, const TokenWriteBack* write_back = nullptr);

// Tensor map of a 2-D bf16 tensor [outer, inner] copied in [box_outer, box_inner] boxes with the
// 128-byte swizzle, from a small per-thread cache (the same buffers come back every layer).
int cached_tmap(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t pitch,
                uint32_t box_inner, uint32_t box_outer);

// Large-M GEMM (prefill batches): persistent 128 x 256 output tiles on the tcgen05 tensor cores.
int launch_tile_gemm(void* y, const void* x, const void* w, const void* bias, int M, int N, int K,
                     int64_t ldx, int epilogue, int* status, cudaStream_t stream);

int launch_grouped_tile_gemm(void* y, const void* x, const void* w, const int32_t* counts,
                             const int32_t* offsets, int num_groups, int64_t total_rows, int N, int K,
                             int epilogue, int* status, cudaStream_t stream);

// Fusions of a split-K GEMM of at most 256 rows with the residual stream of a decode step.  Row
// statistics travel as sums of squares in 2^-24 fixed point (integer atomics: the same bits whatever
// order the CTAs finish in).
//  - ssq_in: the rows of x are un-normalised and w has the norm weight folded into its columns; the
//    accumulator of row m is multiplied by rsqrt(ssq_in[m] / 2^24 / norm_width + eps).
//  - residual: y is not written; residual[m, n] becomes bf16(bf16(acc) + residual[m, n]) and
//    ssq_out[m] grows by the squares of those sums (of the stored bf16 values if ssq_of_rounded).
//  - heads: the projection is a packed qkv projection with 128-wide heads; instead of y[:, all] the
//    epilogue writes the rotated (and, with norm weights, RMS-normalised) q heads into y and the k / v
//    heads into the pool at out_loc - what launch_qknorm_rope_store does after a plain projection.
struct HeadEpilogue {
    const void* q_norm_w = nullptr;   // [128] bf16 or NULL
    const void* k_norm_w = nullptr;
    const float* cos_t = nullptr;     // [max_pos, 64]
    const float* sin_t = nullptr;
    const int32_t* positions = nullptr;
    const int32_t* out_loc = nullptr;
    void* k_cache = nullptr;          // [num_slots, kv_heads, 128] bf16
    void* v_cache = nullptr;
    int q_heads = 0, kv_heads = 0, max_pos = 1;
    int64_t num_slots = 0;
    float eps = 0.f;
};
struct SkinnyFusion {
    const unsigned long long* ssq_in = nullptr;
    float eps = 0.f;
    int norm_width = 1;
    void* residual = nullptr;
    unsigned long long* ssq_out = nullptr;
    bool ssq_of_rounded = false;
    const HeadEpilogue* heads = nullptr;
};
// The K split launch_linear picks for a slab of this shape (the fusions need it above 1).
int skinny_gemm_split(int M, int N, int K, int epilogue);

// y[M, n_out] = x[M, K] w[N, K]^T (+bias / gated epilogue); any M (slabs of 256 rows).
int launch_linear(void* y, const void* x, const void* w, const void* bias, int M, int N, int K,
                  int64_t ldx, int epilogue, int* status, cudaStream_t stream,
                  const SkinnyFusion* fuse = nullptr);

int launch_grouped_gemm(void* y, const void* x, const void* w, const int32_t* counts,
                        const int32_t* offsets, int num_groups, int max_rows_per_group,
                        int64_t total_rows, int N, int K, int epilogue, int* status,
                        cudaStream_t stream);

int64_t moe_workspace_bytes(int tokens, int E, int top_k, int H, int I);
int launch_moe_forward(void* out, const void* hidden, const void* router_logits, const void* gate_up,
                       const void* down, int tokens, int E, int top_k, int H, int I, int renorm,
                       int activation, int expert_begin, int num_local_experts, void* workspace,
                       int* status, cudaStream_t stream);

// Decode-step layer chain (decode_chain.cu): o_proj -> add + norm -> gate_up -> act -> down ->
// add + norm -> the next layer's qkv -> QK-norm -> RoPE -> KV store, as one persistent kernel.
struct DecodeChainArgs {
    int tokens, hidden, inter, q_heads, kv_heads, max_pos;
    float eps;
    bool round_first, gelu;
    const void* attn_out;        // [tokens, q_heads * 128] bf16, the attention output of this layer
    void* residual;              // [tokens, hidden] bf16, updated in place
    void* mlp_act;               // [tokens, inter] bf16 scratch (the activated gate_up output)
    void* x_out;                 // last layer only: [tokens, hidden] down_proj output (no residual add)
    void* qkv_out;               // [tokens, (q + 2 kv) * 128]: the q heads of the next layer are written
    const void *w_o, *w_gate_up, *w_down;
    const void* w_qkv_next;      // NULL for the last layer: the chain then ends after down_proj
    const void *post_norm_w, *next_input_norm_w, *q_norm_w, *k_norm_w;   // q / k norm weights may be NULL
    const float *cos_t, *sin_t;
    const int32_t *positions, *out_loc;
    void *k_cache_next, *v_cache_next;
    int64_t num_slots;
    void* scratch;               // decode_chain_scratch_bytes(hidden), zero-initialised once
    int* status;
};
int decode_chain_max_grid();
int64_t decode_chain_scratch_bytes(int hidden);
bool decode_chain_supported(int tokens, int hidden, int q_heads, int kv_heads, int head_dim, int inter,
                            bool has_bias);
int launch_decode_chain(const DecodeChainArgs& args, cudaStream_t stream);

int64_t decode_workspace_bytes(int max_batch, int q_heads, int kv_heads);
int make_kv_tmap(CUtensorMap* out, const void* cache, int64_t num_slots, int kv_heads, int page_size);
int launch_attention_decode(void* out, const void* q, int64_t q_st, int64_t q_sh,
                            const CUtensorMap& tmap_k, const CUtensorMap& tmap_v, int64_t num_slots,
                            const int32_t* page_table, int64_t pt_stride, const int32_t* table_idx,
                            const int32_t* seq_lens, int batch, int q_heads, int kv_heads,
                            int page_size, float sm_scale, void* workspace, int64_t workspace_bytes,
                            int* status, cudaStream_t stream, bool kv_evict_first = false);
bool attention_prefill_tc_supported(const void* q, int64_t q_st, int64_t q_sh, const void* out);
int launch_attention_prefill_tc(void* out, const void* q, int64_t q_st, int64_t q_sh, const void* k_cache,
                                const void* v_cache, int64_t num_slots, const int32_t* page_table,
                                int64_t pt_stride, const int32_t* table_idx, const int32_t* seq_lens,
                                const int32_t* qo_indptr, int batch, int max_extend_len, int q_heads,
                                int kv_heads, int page_size, float sm_scale, int* status,
                                cudaStream_t stream);
int launch_attention_prefill_tc2(void* out, const void* q, int64_t q_st, int64_t q_sh, const void* k_cache,
                                const void* v_cache, int64_t num_slots, const int32_t* page_table,
                                int64_t pt_stride, const int32_t* table_idx, const int32_t* seq_lens,
                                const int32_t* qo_indptr, int batch, int max_extend_len, int q_heads,
                                int kv_heads, int page_size, float sm_scale, int* status,
                                cudaStream_t stream);
int launch_attention_prefill(void* out, const void* q, int64_t q_st, int64_t q_sh, const void* k_cache,
                             const void* v_cache, int64_t num_slots, const int32_t* page_table,
                             int64_t pt_stride, const int32_t* table_idx, const int32_t* seq_lens,
                             const int32_t* qo_indptr, int batch, int max_extend_len, int q_heads,
                             int kv_heads, int page_size, float sm_scale, int* status,
                             cudaStream_t stream);

}  // namespace b200
