// Step runner: the device state and per-step driver that stand where the
// reference's Engine / GraphRunner / model classes do.
//
// One object owns the weights (packed exactly as the reference's loader packs
// them), the KV pool, the page table and token pool, RoPE tables and activation
// buffers, all from cudaMalloc on the current device.  A step takes the host-side
// description of a batch (per-request rows and lengths), uploads it in ONE copy
// from a pinned staging block, derives every per-token quantity on the device,
// runs the layer stack, selects tokens and writes them back to the token pool.
// Decode steps replay one CUDA graph per padded batch size.
#include <math.h>
#include <string.h>

#include <map>
#include <string>
#include <vector>

#include "common.cuh"
#include "kernels.h"

namespace b200 {
namespace {

static inline int align_ceil(int a, int b) { return (a + b - 1) / b * b; }

// ---- small device kernels that only the step runner needs ----------------------

// Per-token quantities from per-request ones (the host loops of
// Scheduler::prepare_batch plus its two gathers, moved to the device).
//   meta layout (int32): table_idx[Bp] | cached[Bp] | qo_indptr[Bp + 1]
__global__ void prepare_tokens_kernel(const int32_t* __restrict__ meta, int Bp, int T,
                                      const int32_t* __restrict__ page_table,
                                      const int32_t* __restrict__ token_pool, int64_t pt_stride,
                                      int pt_rows, int pt_cols, int32_t* __restrict__ positions,
                                      int32_t* __restrict__ out_loc, int32_t* __restrict__ input_ids,
                                      int32_t* __restrict__ seq_lens) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int32_t* table_idx = meta;
    const int32_t* cached = meta + Bp;
    const int32_t* qo = meta + 2 * Bp;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < Bp) seq_lens[i] = cached[i] + (qo[i + 1] - qo[i]);
    if (i >= T) return;
    int lo = 0, hi = Bp;  // request b with qo[b] <= i < qo[b+1]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (qo[mid] <= i) lo = mid; else hi = mid;
    }
    const int pos = cached[lo] + (i - qo[lo]);
    const int row = table_idx[lo];
    const bool ok = row >= 0 && row < pt_rows && pos >= 0 && pos < pt_cols;
    positions[i] = pos;
    out_loc[i] = ok ? page_table[row * pt_stride + pos] : 0;
    input_ids[i] = ok ? token_pool[row * pt_stride + pos] : 0;
}

// dst[b, :] = src[qo_indptr[b + 1] - 1, :]   (select_lm_head_input, src/models/utils.cc:8-19)
__global__ void select_last_rows_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src,
                                        const int32_t* __restrict__ qo, int vec_per_row) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int b = blockIdx.x;
    const int64_t row = qo[b + 1] - 1;
    for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x)
        dst[static_cast<int64_t>(b) * vec_per_row + v] = src[row * vec_per_row + v];
}

__global__ void scatter_int32_kernel(int32_t* __restrict__ table, int64_t rows, int64_t stride,
                                     int64_t cols, const int32_t* __restrict__ r,
                                     const int32_t* __restrict__ p, const int32_t* __restrict__ v,
                                     int64_t count) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const int64_t rr = r[i], pp = p[i];
    if (rr < 0 || rr >= rows || pp < 0 || pp >= cols) return;
    table[rr * stride + pp] = v[i];
}

// Last kernel of a step that reports through the result ring: the sampled tokens, one finish flag per
// request (what Scheduler::process_forward_output derives on the host, src/scheduler/scheduler.cc:449-455:
// the request cannot decode further - the host passed no write position - or the token is the
// end-of-sequence id and the request does not ignore it), the two device status words and, last, the
// step's ticket, all written into pinned host memory.
__global__ void publish_step_kernel(int32_t* __restrict__ tokens_out, uint8_t* __restrict__ finished_out,
                                    const uint8_t* __restrict__ ignore_eos, int32_t* __restrict__ status_out,
                                    const int32_t* __restrict__ next_tokens, const int32_t* __restrict__ write_pos,
                                    const int* __restrict__ status, int B, int eos, unsigned long long ticket) {
    pdl_launch_dependents();
    pdl_wait_prior();
    for (int i = threadIdx.x; i < B; i += blockDim.x) {
        const int32_t tok = next_tokens[i];
        tokens_out[i] = tok;
        finished_out[i] = (write_pos[i] < 0 || (eos >= 0 && !ignore_eos[i] && tok == eos)) ? 1 : 0;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        status_out[0] = status[0];
        status_out[1] = status[1];
        __threadfence_system();
        *reinterpret_cast<volatile unsigned long long*>(status_out + 2) = ticket;
    }
}

__global__ void fill_int32_kernel(int32_t* p, int32_t v, int64_t n) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}

struct LayerWeights {
    __nv_bfloat16 *qkv = nullptr, *qkv_bias = nullptr, *o = nullptr, *gate_up = nullptr, *down = nullptr;
    __nv_bfloat16 *input_norm = nullptr, *post_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr;
    __nv_bfloat16 *router = nullptr, *experts_gate_up = nullptr, *experts_down = nullptr;
    // qkv and gate_up with the norm weight in front of them folded into their columns (decode steps
    // whose GEMMs carry the add + norm in their epilogues)
    __nv_bfloat16 *qkv_folded = nullptr, *gate_up_folded = nullptr;
    CUtensorMap tmap_k, tmap_v;
};

struct Tensor {
    void* ptr;
    int64_t bytes;
};

}  // namespace
}  // namespace b200

using namespace b200;

struct b200_comm;
extern "C" {
int b200_comm_create(int rank, int world, int64_t buffer_bytes, b200_comm** out);
int64_t b200_comm_region_bytes(int64_t buffer_bytes);
int b200_comm_create_on(int rank, int world, int64_t buffer_bytes, void* region, b200_comm** out);
int b200_comm_connect_pointers(b200_comm* c, const void* const* peer_regions, const void* multicast_region);
int b200_comm_export(b200_comm* c, void* handle_out);
int b200_comm_connect(b200_comm* c, const void* all_handles);
void* b200_comm_buffer(b200_comm* c, int parity);
int b200_comm_destroy(b200_comm* c);
}
namespace b200 {
int launch_allreduce(b200_comm* c, int parity, int mode, void* out, void* residual, const void* weight,
                     int rows, int hidden, float eps, bool round_first, int* status, cudaStream_t stream);
}

struct b200_engine {
    b200_model_config m;
    b200_engine_config c;
    int device = 0;
    int hq = 0, hkv = 0, inter = 0, qkv_dim = 0;  // per-rank sizes
    int moe_inter = 0, experts_local = 0, expert_begin = 0;  // per-rank expert layout
    int64_t num_slots = 0;
    int pt_rows = 0, pt_cols = 0;
    int max_tokens = 0, max_batch = 0;
    float sm_scale = 0.f;

    std::vector<void*> allocs;
    std::map<std::string, Tensor> named;  // "name" or "name.<layer>"
    std::vector<LayerWeights> layers;

    __nv_bfloat16 *embed = nullptr, *lm_head = nullptr, *final_norm = nullptr;
    float *rope_cos = nullptr, *rope_sin = nullptr;
    __nv_bfloat16* kv_cache = nullptr;
    int32_t *page_table = nullptr, *token_pool = nullptr;

    // activations
    __nv_bfloat16 *x = nullptr, *residual = nullptr, *qkv = nullptr, *attn_out = nullptr, *h = nullptr,
                  *sel = nullptr, *logits = nullptr;
    int32_t *positions = nullptr, *out_loc = nullptr, *input_ids = nullptr, *seq_lens = nullptr,
            *next_tokens = nullptr;
    void* attn_ws = nullptr;
    int64_t attn_ws_bytes = 0;
    __nv_bfloat16* router_logits = nullptr;
    void* moe_ws = nullptr;

    // per-step metadata: pinned staging + device mirror
    int32_t* meta_host = nullptr;
    int32_t* meta_dev = nullptr;
    int meta_ints = 0;
    int32_t *scatter_host = nullptr, *scatter_dev = nullptr;
    int64_t scatter_cap = 0;

    cudaStream_t stream = nullptr;
    cudaEvent_t ev_meta_done = nullptr, ev_step_begin = nullptr, ev_step_end = nullptr,
                ev_scatter_done = nullptr;
    bool meta_in_flight = false, scatter_in_flight = false;
    int* status = nullptr;

    std::map<int, cudaGraphExec_t> graphs;          // padded decode batch size -> graph ending in argmax
    std::map<int, cudaGraphExec_t> graphs_sampled;  // ... ending in the sampling kernel
    std::map<int, int> graph_launches;              // kernels inside each captured graph

    // Optional per-kernel timing of the attention launches of eager steps.
    bool profile_attention = false;
    bool capturing = false;
    std::vector<cudaEvent_t> prof_events;   // 2 per layer
    std::vector<cudaEvent_t> prof_events_ar;  // 2 per all-reduce call
    int prof_ar_recorded = 0;
    int prof_pairs_recorded = 0;
    int launches_last_step = 0;
    b200_comm* comm = nullptr;  // tensor parallelism: exchange buffers for the fused all-reduce
    int64_t comm_buffer_bytes = 0;

    // Results of the steps in flight: a ring of pinned, device-mapped slots the last kernel of a step
    // writes straight into (tokens, finish flags, the device status words, the ticket), one event each.
    struct ResultSlot {
        int32_t* tokens = nullptr;         // [max_batch]
        uint8_t* finished = nullptr;       // [max_batch]
        uint8_t* ignore_eos = nullptr;     // [max_batch], written by the host before the launch
        int32_t* status = nullptr;         // [2] + 64-bit ticket behind them
        cudaEvent_t done = nullptr;
        int64_t ticket = -1;
        int num_reqs = 0;
    };
    static constexpr int kResultSlots = 4;
    ResultSlot ring[kResultSlots];
    uint8_t* ring_host = nullptr;
    int64_t next_ticket = 0;
    int32_t eos_token_id = -1;
    void* chain_scratch = nullptr;  // fp32 sums, partial sums of squares and barrier words of the decode layer chain
    // B200_DECODE_CHAIN=1: decode steps run everything between two attention launches as one
    // persistent kernel (decode_chain.cu).  Off by default: measured on B200 it is the slower of the
    // two paths (each of its phases pays several ~1 us round trips to L2 that separate launches hide
    // behind one another under programmatic dependent launch).
    bool use_chain = false;
    // Decode steps of a dense, unsharded model of at most 256 tokens: no add + norm kernels.  o_proj and
    // down_proj add the residual in their split-K epilogue and accumulate each row's sum of squares;
    // qkv_proj and gate_up_proj read the un-normalised residual against weights with the norm weight
    // folded in, and scale their accumulator by the row's 1 / rms.  B200_FOLD_NORM=0 turns it off.
    bool use_fold = true;
    bool use_fold_heads = true;         // B200_FOLD_HEADS=0: QK-norm + RoPE + K/V store stay a kernel of their own
    bool folded_valid = false;          // the folded copies match qkv / gate_up / the norm weights
    unsigned long long* ssq = nullptr;  // [2 * layers + 1, kSsqStride] sums of squares of the residual rows
    static constexpr int kSsqStride = 256;
    bool use_pdl = true;  // B200_PDL=0 turns programmatic dependent launches off
    bool kv_evict_first = true;  // B200_KV_EVICT_FIRST=0: K/V loads with the default L2 policy
    // Seeds are 64-bit: keep them 8-byte aligned inside the int32 staging block.  The 64-bit step
    // index follows them, so a captured graph reads a fresh one on every replay.
    static int seed_offset(int Bp) { return (7 * Bp + 1 + 1) & ~1; }
    static int step_index_offset(int Bp) { return seed_offset(Bp) + 2 * Bp; }
};

namespace {

int dev_alloc(b200_engine* e, void** out, int64_t bytes, bool zero) {
    void* p = nullptr;
    if (bytes <= 0) bytes = 16;
    B200_CHECK_CUDA(cudaMalloc(&p, static_cast<size_t>(bytes)));
    e->allocs.push_back(p);
    if (zero) B200_CHECK_CUDA(cudaMemset(p, 0, static_cast<size_t>(bytes)));
    *out = p;
    return B200_OK;
}

template <typename T>
int named_alloc(b200_engine* e, T** out, const std::string& name, int64_t elems, bool zero = false) {
    void* p = nullptr;
    const int64_t bytes = elems * static_cast<int64_t>(sizeof(T));
    int err = dev_alloc(e, &p, bytes, zero);
    if (err != B200_OK) return err;
    *out = static_cast<T*>(p);
    e->named[name] = Tensor{p, bytes};
    return B200_OK;
}

#define B200_TRY(expr)                  \
    do {                                \
        int err__ = (expr);             \
        if (err__ != B200_OK) return err__; \
    } while (0)

int build_rope_tables(b200_engine* e) {
    // cos/sin [max_position, head_dim / 2] in fp32, with the reference's sequence of fp32
    // operations (src/layers/rotary_embedding.cu:80-93): inv_freq = 1 / base^(2j / d),
    // freq = t * inv_freq, cos(freq), sin(freq), every step rounded to fp32.  The reference runs
    // these steps as torch CPU ops, whose vectorised pow / cos / sin differ from libm's in the last
    // bit of some entries; a host that needs torch's exact bit pattern loads its own tables over
    // "rope_cos" / "rope_sin" (b200_engine_load).
    const int half = e->m.head_dim / 2;
    const int64_t n = static_cast<int64_t>(e->m.max_position) * half;
    std::vector<float> c(n), s(n), inv(half);
    const float base = e->m.rope_theta, dim = static_cast<float>(e->m.head_dim);
    for (int j = 0; j < half; ++j) inv[j] = 1.0f / powf(base, static_cast<float>(2 * j) / dim);
    for (int64_t t = 0; t < e->m.max_position; ++t)
        for (int j = 0; j < half; ++j) {
            const float f = static_cast<float>(t) * inv[j];
            c[t * half + j] = cosf(f);
            s[t * half + j] = sinf(f);
        }
    B200_CHECK_CUDA(cudaMemcpy(e->rope_cos, c.data(), n * sizeof(float), cudaMemcpyHostToDevice));
    B200_CHECK_CUDA(cudaMemcpy(e->rope_sin, s.data(), n * sizeof(float), cudaMemcpyHostToDevice));
    return B200_OK;
}

// Do the four projections of a layer all split along K (the fusions live in the split-K epilogue; the
// split does not depend on the number of tokens)?
bool fold_shapes_ok(const b200_engine* e) {
    const int H = e->m.hidden_size, D = e->m.head_dim;
    return skinny_gemm_split(1, e->qkv_dim, H, B200_EPILOGUE_NONE) > 1 &&
           skinny_gemm_split(1, H, e->hq * D, B200_EPILOGUE_NONE) > 1 &&
           skinny_gemm_split(1, 2 * e->inter, H, B200_EPILOGUE_SWIGLU) > 1 &&
           skinny_gemm_split(1, H, e->inter, B200_EPILOGUE_NONE) > 1;
}

// Can this step run with the add + norm kernels folded into the GEMMs around them?  (The statistics
// buffer exists only for dense, unsharded engines whose shapes qualify.)
bool fold_supported(const b200_engine* e, int phase, int T) {
    return e->ssq != nullptr && phase == B200_PHASE_DECODE && T <= b200_engine::kSsqStride;
}

// Rebuilds the folded weight copies after a weight was loaded.  Enqueued on the engine's stream, never
// inside a graph capture (the callers run it first).
int ensure_folded(b200_engine* e) {
    if (e->ssq == nullptr || e->folded_valid) return B200_OK;
    const int H = e->m.hidden_size;
    for (LayerWeights& L : e->layers) {
        B200_TRY(launch_scale_columns(L.qkv_folded, L.qkv, L.input_norm, e->qkv_dim, H, e->stream));
        B200_TRY(launch_scale_columns(L.gate_up_folded, L.gate_up, L.post_norm, 2 * static_cast<int64_t>(e->inter), H,
                                      e->stream));
    }
    e->folded_valid = true;
    return B200_OK;
}

// The layer stack on `T` tokens of `Bp` requests; everything is enqueued on e->stream.
int enqueue_forward(b200_engine* e, int phase, int B, int Bp, int T, int max_extend,
                    bool sampling = false, uint64_t step_index = 0) {
    const b200_model_config& m = e->m;
    cudaStream_t s = e->stream;
    const int hidden = m.hidden_size, d = m.head_dim;
    const uint64_t launches_before = kernel_launch_count();
    const int32_t* meta_table_idx = e->meta_dev;
    const int32_t* meta_qo = e->meta_dev + 2 * Bp;

    const bool fold = fold_supported(e, phase, T);
    // The residual stream starts at zero, so the first fused add+norm leaves residual = embedding
    // (what the reference's layer 0 does with `residual = x`).  With the norms folded into the GEMMs
    // the embedding is written into the residual directly.
    if (!fold) B200_CHECK_CUDA(cudaMemsetAsync(e->residual, 0, static_cast<size_t>(T) * hidden * 2, s));
    // From here on the step is an unbroken chain of kernels.  With programmatic dependent
    // launches each kernel's prologue (barrier set-up, TMEM allocation, weight-tile TMA loads)
    // overlaps the tail of its predecessor; every kernel waits (griddepcontrol.wait) before it
    // reads or writes anything a predecessor touches.
    struct PdlScope {
        ~PdlScope() { set_pdl_launches(false); }
    } pdl_scope;
    set_pdl_launches(false);  // the first kernel follows a memset / copy: ordinary dependency
    {
        const int n = T > Bp ? T : Bp;
        B200_CHECK_CUDA(launch_kernel(prepare_tokens_kernel, dim3(div_ceil(n, 256)), dim3(256), 0, s,
                                      dim3(1, 1, 1), static_cast<const int32_t*>(e->meta_dev), Bp, T,
                                      static_cast<const int32_t*>(e->page_table),
                                      static_cast<const int32_t*>(e->token_pool),
                                      static_cast<int64_t>(e->pt_cols), e->pt_rows, e->pt_cols, e->positions,
                                      e->out_loc, e->input_ids, e->seq_lens));
    }
    // (Per-kernel event timing wants each kernel to start after its predecessor ends.)
    // The embedding is launched as an ordinary dependent of the prepare kernel: every later kernel
    // of the step can then rely on seq_lens / positions / out_loc being complete even in code it
    // runs ahead of griddepcontrol.wait (a kernel can only start after the embedding has).
    if (fold)
        B200_TRY(launch_embedding(e->residual, e->embed, e->input_ids, T, hidden, m.vocab_size, e->status, s, e->ssq,
                                  2 * m.num_layers + 1, b200_engine::kSsqStride));
    else
        B200_TRY(launch_embedding(e->x, e->embed, e->input_ids, T, hidden, m.vocab_size, e->status, s));
    set_pdl_launches(e->use_pdl && !(e->profile_attention && !e->capturing));
    const bool round_first = m.fused_residual == 0;
    // Under tensor parallelism the row-parallel projections (o_proj, down_proj, the MoE output)
    // leave a partial sum: they write it into this rank's exchange buffer, and the add + norm
    // that follows becomes the fused all-reduce kernel.  Two calls per layer alternate the
    // buffers, so the parity of a call is fixed across steps (and inside a captured graph).
    const bool tp = e->c.tp_size > 1;
    int ar_calls = 0;
    bool x_is_partial = false;  // does the running `x` sit in an exchange buffer awaiting reduction?
    auto proj_out = [&]() -> __nv_bfloat16* {
        if (!tp) return e->x;
        x_is_partial = true;
        return static_cast<__nv_bfloat16*>(b200_comm_buffer(e->comm, ar_calls & 1));
    };
    auto add_norm = [&](const __nv_bfloat16* w) -> int {
        if (tp && x_is_partial) {
            x_is_partial = false;
            const int call = ar_calls++;
            const bool timed_ar = e->profile_attention && !e->capturing;
            if (timed_ar) {
                while (static_cast<int>(e->prof_events_ar.size()) < 2 * (call + 1)) {
                    cudaEvent_t ev = nullptr;
                    B200_CHECK_CUDA(cudaEventCreate(&ev));
                    e->prof_events_ar.push_back(ev);
                }
                B200_CHECK_CUDA(cudaEventRecord(e->prof_events_ar[2 * call], s));
            }
            int rc = launch_allreduce(e->comm, call & 1, 1, e->x, e->residual, w, T, hidden, m.rms_norm_eps,
                                      round_first, e->status, s);
            if (timed_ar) {
                B200_CHECK_CUDA(cudaEventRecord(e->prof_events_ar[2 * call + 1], s));
                e->prof_ar_recorded = call + 1;
            }
            return rc;
        }
        return launch_fused_add_rmsnorm(e->x, e->residual, w, T, hidden, m.rms_norm_eps, round_first, s);
    };
    const int epi = m.hidden_act == 1 ? B200_EPILOGUE_GEGLU : B200_EPILOGUE_SWIGLU;
    // The head epilogue of the qkv projection wants the split-K form of the small-batch kernel; beyond
    // two exchange rounds (128 tokens) the separate kernel is the faster of the two, and on a sharded
    // engine (few heads per rank) it is no gain: Llama-3-8B at batch 128 ran 7.21 against 7.44 ms with it
    // on one GPU, 5.52 against 5.51 on two, 3.33 against 3.31 on eight.
    const bool heads_in_qkv = e->use_fold_heads && d == 128 && T <= 128 && !tp &&
                              skinny_gemm_split(T, e->qkv_dim, hidden, B200_EPILOGUE_NONE) > 1;

    // Decode batches of at most 64 tokens of a dense, unsharded model: everything between two attention
    // launches is one persistent kernel (decode_chain.cu) instead of seven launches.
    const bool chain = !fold && phase == B200_PHASE_DECODE && e->use_chain && !tp && m.num_experts == 0 &&
                       decode_chain_supported(T, hidden, e->hq, e->hkv, d, e->inter, m.attention_bias != 0);
    if (chain) {
        auto caches = [&](int l, __nv_bfloat16** kc, __nv_bfloat16** vc) {
            *kc = e->kv_cache + static_cast<int64_t>(l) * e->num_slots * e->hkv * d;
            *vc = *kc + static_cast<int64_t>(m.num_layers) * e->num_slots * e->hkv * d;
        };
        __nv_bfloat16 *kc = nullptr, *vc = nullptr;
        caches(0, &kc, &vc);
        LayerWeights& L0 = e->layers[0];
        B200_TRY(add_norm(L0.input_norm));
        B200_TRY(launch_linear(e->qkv, e->x, L0.qkv, nullptr, T, e->qkv_dim, hidden, hidden, B200_EPILOGUE_NONE,
                               e->status, s));
        B200_TRY(launch_qknorm_rope_store(e->qkv, L0.q_norm, L0.k_norm, e->rope_cos, e->rope_sin, e->positions,
                                          e->out_loc, kc, vc, T, e->hq, e->hkv, d, m.max_position, e->num_slots,
                                          m.rms_norm_eps, 0, e->status, s));
        for (int l = 0; l < m.num_layers; ++l) {
            LayerWeights& L = e->layers[l];
            const bool timed = e->profile_attention && !e->capturing;
            if (timed) {
                while (static_cast<int>(e->prof_events.size()) < 2 * m.num_layers) {
                    cudaEvent_t ev = nullptr;
                    B200_CHECK_CUDA(cudaEventCreate(&ev));
                    e->prof_events.push_back(ev);
                }
                B200_CHECK_CUDA(cudaEventRecord(e->prof_events[2 * l], s));
            }
            B200_TRY(launch_attention_decode(e->attn_out, e->qkv, e->qkv_dim, d, L.tmap_k, L.tmap_v, e->num_slots,
                                             e->page_table, e->pt_cols, meta_table_idx, e->seq_lens, Bp, e->hq,
                                             e->hkv, e->c.page_size, e->sm_scale, e->attn_ws, e->attn_ws_bytes,
                                             e->status, s, e->kv_evict_first));
            if (timed) {
                B200_CHECK_CUDA(cudaEventRecord(e->prof_events[2 * l + 1], s));
                e->prof_pairs_recorded = l + 1;
            }
            const bool last = l + 1 == m.num_layers;
            DecodeChainArgs a = {};
            a.tokens = T;
            a.hidden = hidden;
            a.inter = e->inter;
            a.q_heads = e->hq;
            a.kv_heads = e->hkv;
            a.max_pos = m.max_position;
            a.eps = m.rms_norm_eps;
            a.round_first = round_first;
            a.gelu = m.hidden_act == 1;
            a.attn_out = e->attn_out;
            a.residual = e->residual;
            a.mlp_act = e->h;
            a.x_out = e->x;
            a.qkv_out = e->qkv;
            a.w_o = L.o;
            a.w_gate_up = L.gate_up;
            a.w_down = L.down;
            a.post_norm_w = L.post_norm;
            if (!last) {
                LayerWeights& N = e->layers[l + 1];
                a.w_qkv_next = N.qkv;
                a.next_input_norm_w = N.input_norm;
                a.q_norm_w = N.q_norm;
                a.k_norm_w = N.k_norm;
                caches(l + 1, &kc, &vc);
                a.k_cache_next = kc;
                a.v_cache_next = vc;
            }
            a.cos_t = e->rope_cos;
            a.sin_t = e->rope_sin;
            a.positions = e->positions;
            a.out_loc = e->out_loc;
            a.num_slots = e->num_slots;
            a.scratch = e->chain_scratch;
            a.status = e->status;
            B200_TRY(launch_decode_chain(a, s));
        }
    }

    for (int l = 0; l < (fold ? m.num_layers : 0); ++l) {
        LayerWeights& L = e->layers[l];
        unsigned long long* ssq_l = e->ssq + static_cast<int64_t>(2 * l) * b200_engine::kSsqStride;
        SkinnyFusion normed, into_residual;
        normed.eps = m.rms_norm_eps;
        normed.norm_width = hidden;
        into_residual.residual = e->residual;
        into_residual.ssq_of_rounded = round_first;
        normed.ssq_in = ssq_l;
        __nv_bfloat16* k_cache = e->kv_cache + static_cast<int64_t>(l) * e->num_slots * e->hkv * d;
        __nv_bfloat16* v_cache = k_cache + static_cast<int64_t>(m.num_layers) * e->num_slots * e->hkv * d;
        if (heads_in_qkv) {
            // ... and the QK-norm, the rotation and the K/V store ride in the qkv projection's epilogue
            HeadEpilogue he;
            he.q_norm_w = L.q_norm;
            he.k_norm_w = L.k_norm;
            he.cos_t = e->rope_cos;
            he.sin_t = e->rope_sin;
            he.positions = e->positions;
            he.out_loc = e->out_loc;
            he.k_cache = k_cache;
            he.v_cache = v_cache;
            he.q_heads = e->hq;
            he.kv_heads = e->hkv;
            he.max_pos = m.max_position;
            he.num_slots = e->num_slots;
            he.eps = m.rms_norm_eps;
            normed.heads = &he;
            B200_TRY(launch_linear(e->qkv, e->residual, L.qkv_folded, L.qkv_bias, T, e->qkv_dim, hidden, hidden,
                                   B200_EPILOGUE_NONE, e->status, s, &normed));
            normed.heads = nullptr;
        } else {
            B200_TRY(launch_linear(e->qkv, e->residual, L.qkv_folded, L.qkv_bias, T, e->qkv_dim, hidden, hidden,
                                   B200_EPILOGUE_NONE, e->status, s, &normed));
            B200_TRY(launch_qknorm_rope_store(e->qkv, L.q_norm, L.k_norm, e->rope_cos, e->rope_sin, e->positions,
                                              e->out_loc, k_cache, v_cache, T, e->hq, e->hkv, d, m.max_position,
                                              e->num_slots, m.rms_norm_eps, 0, e->status, s));
        }
        const bool timed = e->profile_attention && !e->capturing;
        if (timed) {
            while (static_cast<int>(e->prof_events.size()) < 2 * m.num_layers) {
                cudaEvent_t ev = nullptr;
                B200_CHECK_CUDA(cudaEventCreate(&ev));
                e->prof_events.push_back(ev);
            }
            B200_CHECK_CUDA(cudaEventRecord(e->prof_events[2 * l], s));
        }
        B200_TRY(launch_attention_decode(e->attn_out, e->qkv, e->qkv_dim, d, L.tmap_k, L.tmap_v, e->num_slots,
                                         e->page_table, e->pt_cols, meta_table_idx, e->seq_lens, Bp, e->hq, e->hkv,
                                         e->c.page_size, e->sm_scale, e->attn_ws, e->attn_ws_bytes, e->status, s,
                                         e->kv_evict_first));
        if (timed) {
            B200_CHECK_CUDA(cudaEventRecord(e->prof_events[2 * l + 1], s));
            e->prof_pairs_recorded = l + 1;
        }
        into_residual.ssq_out = ssq_l + b200_engine::kSsqStride;
        B200_TRY(launch_linear(nullptr, e->attn_out, L.o, nullptr, T, hidden, e->hq * d, e->hq * d,
                               B200_EPILOGUE_NONE, e->status, s, &into_residual));
        normed.ssq_in = ssq_l + b200_engine::kSsqStride;
        B200_TRY(launch_linear(e->h, e->residual, L.gate_up_folded, nullptr, T, 2 * e->inter, hidden, hidden, epi,
                               e->status, s, &normed));
        into_residual.ssq_out = ssq_l + 2 * b200_engine::kSsqStride;
        B200_TRY(launch_linear(nullptr, e->h, L.down, nullptr, T, hidden, e->inter, e->inter, B200_EPILOGUE_NONE,
                               e->status, s, &into_residual));
    }

    for (int l = 0; l < (chain || fold ? 0 : m.num_layers); ++l) {
        LayerWeights& L = e->layers[l];
        B200_TRY(add_norm(L.input_norm));
        __nv_bfloat16* k_cache = e->kv_cache + static_cast<int64_t>(l) * e->num_slots * e->hkv * d;
        __nv_bfloat16* v_cache = k_cache + static_cast<int64_t>(m.num_layers) * e->num_slots * e->hkv * d;
        if (heads_in_qkv) {
            // (sharded and MoE engines, short prefill batches: the head epilogue alone, on normalised rows)
            HeadEpilogue he;
            he.q_norm_w = L.q_norm;
            he.k_norm_w = L.k_norm;
            he.cos_t = e->rope_cos;
            he.sin_t = e->rope_sin;
            he.positions = e->positions;
            he.out_loc = e->out_loc;
            he.k_cache = k_cache;
            he.v_cache = v_cache;
            he.q_heads = e->hq;
            he.kv_heads = e->hkv;
            he.max_pos = m.max_position;
            he.num_slots = e->num_slots;
            he.eps = m.rms_norm_eps;
            SkinnyFusion with_heads;
            with_heads.heads = &he;
            B200_TRY(launch_linear(e->qkv, e->x, L.qkv, L.qkv_bias, T, e->qkv_dim, hidden, hidden, B200_EPILOGUE_NONE,
                                   e->status, s, &with_heads));
        } else {
            B200_TRY(launch_linear(e->qkv, e->x, L.qkv, L.qkv_bias, T, e->qkv_dim, hidden, hidden,
                                   B200_EPILOGUE_NONE, e->status, s));
            B200_TRY(launch_qknorm_rope_store(e->qkv, L.q_norm, L.k_norm, e->rope_cos, e->rope_sin,
                                              e->positions, e->out_loc, k_cache, v_cache, T, e->hq, e->hkv,
                                              d, m.max_position, e->num_slots, m.rms_norm_eps, 0, e->status, s));
        }
        const bool timed = e->profile_attention && !e->capturing;
        if (timed) {
            while (static_cast<int>(e->prof_events.size()) < 2 * m.num_layers) {
                cudaEvent_t ev = nullptr;
                B200_CHECK_CUDA(cudaEventCreate(&ev));
                e->prof_events.push_back(ev);
            }
            B200_CHECK_CUDA(cudaEventRecord(e->prof_events[2 * l], s));
        }
        if (phase == B200_PHASE_DECODE) {
            B200_TRY(launch_attention_decode(e->attn_out, e->qkv, e->qkv_dim, d, L.tmap_k, L.tmap_v,
                                             e->num_slots, e->page_table, e->pt_cols, meta_table_idx,
                                             e->seq_lens, Bp, e->hq, e->hkv, e->c.page_size, e->sm_scale,
                                             e->attn_ws, e->attn_ws_bytes, e->status, s, e->kv_evict_first));
        } else {
            B200_TRY(launch_attention_prefill(e->attn_out, e->qkv, e->qkv_dim, d, k_cache, v_cache,
                                              e->num_slots, e->page_table, e->pt_cols, meta_table_idx,
                                              e->seq_lens, meta_qo, Bp, max_extend, e->hq, e->hkv,
                                              e->c.page_size, e->sm_scale, e->status, s));
        }
        if (timed) {
            B200_CHECK_CUDA(cudaEventRecord(e->prof_events[2 * l + 1], s));
            e->prof_pairs_recorded = l + 1;
        }
        B200_TRY(launch_linear(proj_out(), e->attn_out, L.o, nullptr, T, hidden, e->hq * d, e->hq * d,
                                   B200_EPILOGUE_NONE, e->status, s));
        B200_TRY(add_norm(L.post_norm));
        if (m.num_experts > 0) {
            // MoEMLP::forward (src/models/utils.cc:82-91): router logits, then the expert layer.
            B200_TRY(launch_linear(e->router_logits, e->x, L.router, nullptr, T, m.num_experts, hidden, hidden,
                                   B200_EPILOGUE_NONE, e->status, s));
            B200_TRY(launch_moe_forward(proj_out(), e->x, e->router_logits, L.experts_gate_up, L.experts_down, T,
                                        m.num_experts, m.num_experts_per_tok, hidden, e->moe_inter,
                                        m.norm_topk_prob, m.hidden_act == 1 ? 1 : 0, e->expert_begin,
                                        e->experts_local, e->moe_ws, e->status, s));
            continue;
        }
        B200_TRY(launch_linear(e->h, e->x, L.gate_up, nullptr, T, 2 * e->inter, hidden, hidden, epi,
                                   e->status, s));
        B200_TRY(launch_linear(proj_out(), e->h, L.down, nullptr, T, hidden, e->inter, e->inter,
                                   B200_EPILOGUE_NONE, e->status, s));
    }
    if (fold)
        B200_TRY(launch_rmsnorm(e->x, e->residual, e->final_norm, T, hidden, m.rms_norm_eps, s));
    else
        B200_TRY(add_norm(e->final_norm));
    const __nv_bfloat16* head_in = e->x;
    if (phase == B200_PHASE_PREFILL) {
        B200_CHECK_CUDA(launch_kernel(select_last_rows_kernel, dim3(Bp), dim3(128), 0, s, dim3(1, 1, 1),
                                      reinterpret_cast<uint4*>(e->sel), reinterpret_cast<const uint4*>(e->x),
                                      meta_qo, hidden / 8));
        head_in = e->sel;
    }
    B200_TRY(launch_linear(e->logits, head_in, e->lm_head, nullptr, Bp, m.vocab_size, hidden, hidden,
                           B200_EPILOGUE_NONE, e->status, s));
    // Token write-back, token_pool[table_idx[i], write_pos[i]] = next_tokens[i], by the kernel that picks the token.
    TokenWriteBack wb;
    wb.pool = e->token_pool;
    wb.rows = e->pt_rows;
    wb.stride = e->pt_cols;
    wb.cols = e->pt_cols;
    wb.table_idx = meta_table_idx;
    wb.write_pos = e->meta_dev + 3 * Bp + 1;
    wb.count = B;
    if (sampling) {
        // meta layout after write_pos[Bp]: temperatures | top_k | top_p | seeds (2 ints each)
        const int32_t* sp = e->meta_dev + 4 * Bp + 1;
        B200_TRY(launch_sample(e->next_tokens, e->logits, B, m.vocab_size, m.vocab_size,
                               reinterpret_cast<const float*>(sp), sp + Bp,
                               reinterpret_cast<const float*>(sp + 2 * Bp),
                               reinterpret_cast<const uint64_t*>(e->meta_dev + e->seed_offset(Bp)), step_index,
                               nullptr, s,
                               reinterpret_cast<const uint64_t*>(e->meta_dev + e->step_index_offset(Bp)), &wb));
    } else {
        B200_TRY(launch_argmax(e->next_tokens, e->logits, B, m.vocab_size, m.vocab_size, s, &wb));
    }
    e->launches_last_step = static_cast<int>(kernel_launch_count() - launches_before);
    return B200_OK;
}

// Fills the pinned staging block for a step of Bp padded requests; returns T and the longest extend
// length.  Rows past st->num_padded_reqs (the step runner padding a decode batch up to a captured
// graph size, GraphRunner::pad_batch, src/engine/engine.cc:628-645) are the dummy request: its table
// row, no cached tokens, one token, nothing written back.
int stage_step(b200_engine* e, const b200_step* st, int Bp, int* T_out, int* max_ext_out) {
    const int B = st->num_reqs, Bc = st->num_padded_reqs;
    int32_t* mh = e->meta_host;
    int T = 0, max_ext = 0;
    for (int i = 0; i < Bp; ++i) {
        const bool own = i < Bc;
        const int ext = own ? st->extend_lens[i] : 1;
        const int cached = own ? st->cached_lens[i] : 0;
        mh[i] = own ? st->table_idx[i] : e->c.max_running_req;
        mh[Bp + i] = cached;
        mh[2 * Bp + i] = T;
        if (ext < 0) {
            set_last_error("step: extend_lens[%d] is negative", i);
            return B200_ERR_INVALID_ARGUMENT;
        }
        if (cached < 0 || cached + ext > e->pt_cols) {
            set_last_error("step: request %d needs %d positions, the page table has %d columns", i, cached + ext,
                           e->pt_cols);
            return B200_ERR_INVALID_ARGUMENT;
        }
        T += ext;
        if (ext > max_ext) max_ext = ext;
    }
    mh[3 * Bp] = T;
    for (int i = 0; i < Bp; ++i) mh[3 * Bp + 1 + i] = (i < B && st->write_pos) ? st->write_pos[i] : -1;
    if (st->temperatures) {
        float* tf = reinterpret_cast<float*>(mh + 4 * Bp + 1);
        int32_t* tk = mh + 5 * Bp + 1;
        float* tp = reinterpret_cast<float*>(mh + 6 * Bp + 1);
        uint64_t* sd = reinterpret_cast<uint64_t*>(mh + b200_engine::seed_offset(Bp));
        for (int i = 0; i < Bp; ++i) {
            // Clamping as Sampler::prepare does (src/engine/engine.cc:264-275).
            const float t = i < B ? st->temperatures[i] : 0.f;
            tf[i] = t > 1e-6f ? t : 1e-6f;
            const int k = (i < B && st->top_k) ? st->top_k[i] : -1;
            tk[i] = k >= 1 ? k : e->m.vocab_size;
            const float pp = (i < B && st->top_p) ? st->top_p[i] : 1.f;
            tp[i] = pp < 1e-6f ? 1e-6f : (pp > 1.f ? 1.f : pp);
            sd[i] = (i < B && st->seeds) ? st->seeds[i] : static_cast<uint64_t>(i);
        }
        *reinterpret_cast<uint64_t*>(mh + b200_engine::step_index_offset(Bp)) = st->step_index;
    }
    *T_out = T;
    *max_ext_out = max_ext;
    return B200_OK;
}

}  // namespace

extern "C" {

int b200_engine_create(const b200_model_config* model, const b200_engine_config* config,
                       b200_engine** out) {
    B200_CHECK_ARG(model && config && out, "engine_create: NULL argument");
    const b200_model_config& m = *model;
    const b200_engine_config& c = *config;
    B200_CHECK_ARG(m.num_layers > 0 && m.hidden_size > 0 && m.vocab_size > 0, "engine_create: bad model size");
    B200_CHECK_ARG(m.head_dim == 128, "engine_create: head_dim must be 128 (as the reference's attention is)");
    B200_CHECK_ARG(m.hidden_size % 64 == 0 && m.intermediate_size % 64 == 0,
                   "engine_create: hidden and intermediate sizes must be multiples of 64");
    B200_CHECK_ARG(c.tp_size >= 1 && c.tp_rank >= 0 && c.tp_rank < c.tp_size, "engine_create: bad TP rank/size");
    B200_CHECK_ARG(m.num_qo_heads % c.tp_size == 0, "num_qo_heads must be divisible by tp_size");
    // Fewer KV heads than ranks: each KV head is replicated on tp_size / num_kv_heads ranks.
    B200_CHECK_ARG(m.num_kv_heads % c.tp_size == 0 || c.tp_size % m.num_kv_heads == 0,
                   "num_kv_heads must divide, or be divisible by, tp_size");
    if (m.num_experts > 0 && c.expert_parallel) {
        B200_CHECK_ARG(m.num_experts % c.tp_size == 0, "num_experts must be divisible by tp_size");
        B200_CHECK_ARG(m.moe_intermediate_size % 64 == 0, "MoELayer intermediate size must be a multiple of 64");
    } else if (m.num_experts > 0) {
        B200_CHECK_ARG(m.moe_intermediate_size % (64 * c.tp_size) == 0,
                       "MoELayer intermediate size / tp_size must be a multiple of 64");
    }
    B200_CHECK_ARG(m.intermediate_size % (64 * c.tp_size) == 0 || m.num_experts > 0,
                   "intermediate_size / tp_size must be a multiple of 64");
    B200_CHECK_ARG(c.page_size >= 1 && (c.page_size & (c.page_size - 1)) == 0,
                   "engine_create: page_size must be a power of two");
    B200_CHECK_ARG(c.num_pages >= 1 && c.max_running_req >= 1 && c.max_seq_len >= 1 && c.max_extend_tokens >= 1,
                   "engine_create: bad engine sizes");
    const int hkv = m.num_kv_heads >= c.tp_size ? m.num_kv_heads / c.tp_size : 1;
    B200_CHECK_ARG(hkv <= 8 && 8 % hkv == 0, "engine_create: kv heads per rank must be 1, 2, 4 or 8");

    b200_engine* e = new b200_engine();
    e->m = m;
    e->c = c;
    B200_CHECK_CUDA(cudaGetDevice(&e->device));
    e->hq = m.num_qo_heads / c.tp_size;
    e->hkv = hkv;
    if (m.num_experts > 0) {
        const bool ep = c.expert_parallel != 0;
        e->moe_inter = ep ? m.moe_intermediate_size : m.moe_intermediate_size / c.tp_size;
        e->experts_local = ep ? m.num_experts / c.tp_size : m.num_experts;
        e->expert_begin = ep ? c.tp_rank * e->experts_local : 0;
    }
    e->inter = m.intermediate_size / c.tp_size;
    e->qkv_dim = (e->hq + 2 * e->hkv) * m.head_dim;
    e->num_slots = static_cast<int64_t>(c.num_pages + 1) * c.page_size;
    e->pt_rows = c.max_running_req + 1;
    e->pt_cols = align_ceil(c.max_seq_len, 32);
    e->max_batch = c.max_running_req + 1;
    e->max_tokens = c.max_extend_tokens > e->max_batch ? c.max_extend_tokens : e->max_batch;
    e->sm_scale = 1.0f / sqrtf(static_cast<float>(m.head_dim));
    int err = B200_OK;
    e->status = device_status_words(&err);
    if (err != B200_OK) { delete e; return err; }
    if (const char* v = getenv("B200_PDL")) e->use_pdl = atoi(v) != 0;
    if (const char* v = getenv("B200_DECODE_CHAIN")) e->use_chain = atoi(v) != 0;
    if (const char* v = getenv("B200_KV_EVICT_FIRST")) e->kv_evict_first = atoi(v) != 0;

    auto fail = [&](int code) { b200_engine_destroy(e); return code; };
#define E_TRY(expr) do { int c__ = (expr); if (c__ != B200_OK) return fail(c__); } while (0)

    const int64_t H = m.hidden_size, D = m.head_dim;
    E_TRY(named_alloc(e, &e->embed, "embed", static_cast<int64_t>(m.vocab_size) * H));
    if (m.tie_word_embeddings) {
        e->lm_head = e->embed;
        e->named["lm_head"] = e->named["embed"];
    } else {
        E_TRY(named_alloc(e, &e->lm_head, "lm_head", static_cast<int64_t>(m.vocab_size) * H));
    }
    E_TRY(named_alloc(e, &e->final_norm, "final_norm", H));
    E_TRY(named_alloc(e, &e->rope_cos, "rope_cos", static_cast<int64_t>(m.max_position) * (D / 2)));
    E_TRY(named_alloc(e, &e->rope_sin, "rope_sin", static_cast<int64_t>(m.max_position) * (D / 2)));
    E_TRY(build_rope_tables(e));
    E_TRY(named_alloc(e, &e->kv_cache, "kv_cache", 2 * static_cast<int64_t>(m.num_layers) * e->num_slots * e->hkv * D, true));
    E_TRY(named_alloc(e, &e->page_table, "page_table", static_cast<int64_t>(e->pt_rows) * e->pt_cols, true));
    E_TRY(named_alloc(e, &e->token_pool, "token_pool", static_cast<int64_t>(e->pt_rows) * e->pt_cols, true));
    {
        // Dummy request: row max_running_req points every position at the extra page.
        int32_t* row = e->page_table + static_cast<int64_t>(c.max_running_req) * e->pt_cols;
        fill_int32_kernel<<<div_ceil(e->pt_cols, 256), 256>>>(row, c.num_pages * c.page_size, e->pt_cols);
        if (cudaGetLastError() != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
            set_last_error("engine_create: initialising the dummy page-table row failed");
            return fail(B200_ERR_CUDA);
        }
    }
    e->layers.resize(m.num_layers);
    for (int l = 0; l < m.num_layers; ++l) {
        LayerWeights& L = e->layers[l];
        const std::string sfx = "." + std::to_string(l);
        E_TRY(named_alloc(e, &L.qkv, "qkv" + sfx, static_cast<int64_t>(e->qkv_dim) * H));
        if (m.attention_bias) E_TRY(named_alloc(e, &L.qkv_bias, "qkv_bias" + sfx, e->qkv_dim));
        E_TRY(named_alloc(e, &L.o, "o" + sfx, H * e->hq * D));
        E_TRY(named_alloc(e, &L.input_norm, "input_norm" + sfx, H));
        E_TRY(named_alloc(e, &L.post_norm, "post_norm" + sfx, H));
        if (m.qk_norm) {
            E_TRY(named_alloc(e, &L.q_norm, "q_norm" + sfx, D));
            E_TRY(named_alloc(e, &L.k_norm, "k_norm" + sfx, D));
        }
        if (m.num_experts > 0) {
            const int64_t ie = e->moe_inter, el = e->experts_local;
            E_TRY(named_alloc(e, &L.router, "router" + sfx, static_cast<int64_t>(m.num_experts) * H));
            E_TRY(named_alloc(e, &L.experts_gate_up, "experts_gate_up" + sfx, el * 2 * ie * H));
            E_TRY(named_alloc(e, &L.experts_down, "experts_down" + sfx, el * H * ie));
        } else {
            E_TRY(named_alloc(e, &L.gate_up, "gate_up" + sfx, 2 * static_cast<int64_t>(e->inter) * H));
            E_TRY(named_alloc(e, &L.down, "down" + sfx, H * e->inter));
        }
        const __nv_bfloat16* kc = e->kv_cache + static_cast<int64_t>(l) * e->num_slots * e->hkv * D;
        const __nv_bfloat16* vc = kc + static_cast<int64_t>(m.num_layers) * e->num_slots * e->hkv * D;
        E_TRY(make_kv_tmap(&L.tmap_k, kc, e->num_slots, e->hkv, c.page_size));
        E_TRY(make_kv_tmap(&L.tmap_v, vc, e->num_slots, e->hkv, c.page_size));
    }
    const int64_t Tm = e->max_tokens;
    const int64_t inter_buf = m.num_experts > 0 ? m.moe_intermediate_size : e->inter;
    E_TRY(named_alloc(e, &e->x, "x", Tm * H));
    E_TRY(named_alloc(e, &e->residual, "residual", Tm * H));
    E_TRY(named_alloc(e, &e->qkv, "qkv_act", Tm * e->qkv_dim));
    E_TRY(named_alloc(e, &e->attn_out, "attn_out", Tm * e->hq * D));
    E_TRY(named_alloc(e, &e->h, "mlp_act", Tm * inter_buf));
    E_TRY(named_alloc(e, &e->sel, "sel", static_cast<int64_t>(e->max_batch) * H));
    E_TRY(named_alloc(e, &e->logits, "logits", static_cast<int64_t>(e->max_batch) * m.vocab_size));
    E_TRY(named_alloc(e, &e->positions, "positions", Tm));
    E_TRY(named_alloc(e, &e->out_loc, "out_loc", Tm));
    E_TRY(named_alloc(e, &e->input_ids, "input_ids", Tm));
    E_TRY(named_alloc(e, &e->seq_lens, "seq_lens", e->max_batch));
    E_TRY(named_alloc(e, &e->next_tokens, "next_tokens", e->max_batch, true));
    e->comm_buffer_bytes = Tm * H * 2;
    if (c.tp_size > 1) E_TRY(b200_comm_create(c.tp_rank, c.tp_size, e->comm_buffer_bytes, &e->comm));
    if (m.num_experts > 0) {
        E_TRY(named_alloc(e, &e->router_logits, "router_logits", Tm * m.num_experts));
        E_TRY(dev_alloc(e, &e->moe_ws,
                        moe_workspace_bytes(static_cast<int>(Tm), m.num_experts, m.num_experts_per_tok, m.hidden_size,
                                            e->moe_inter),
                        false));
    }
    if (const char* v = getenv("B200_FOLD_NORM")) e->use_fold = atoi(v) != 0;
    if (const char* v = getenv("B200_FOLD_HEADS")) e->use_fold_heads = atoi(v) != 0;
    if (e->use_fold && c.tp_size == 1 && m.num_experts == 0 && fold_shapes_ok(e)) {
        for (LayerWeights& L : e->layers) {
            void* p = nullptr;
            E_TRY(dev_alloc(e, &p, static_cast<int64_t>(e->qkv_dim) * H * 2, false));
            L.qkv_folded = static_cast<__nv_bfloat16*>(p);
            E_TRY(dev_alloc(e, &p, 2 * static_cast<int64_t>(e->inter) * H * 2, false));
            L.gate_up_folded = static_cast<__nv_bfloat16*>(p);
        }
        void* p = nullptr;
        E_TRY(dev_alloc(e, &p, static_cast<int64_t>(2 * m.num_layers + 1) * b200_engine::kSsqStride * 8, true));
        e->ssq = static_cast<unsigned long long*>(p);
    }
    E_TRY(dev_alloc(e, &e->chain_scratch, decode_chain_scratch_bytes(m.hidden_size), true));
    e->attn_ws_bytes = decode_workspace_bytes(e->max_batch, e->hq, e->hkv);
    E_TRY(dev_alloc(e, &e->attn_ws, e->attn_ws_bytes, true));

    e->meta_ints = 9 * e->max_batch + 16;
    if (cudaMallocHost(&e->meta_host, e->meta_ints * sizeof(int32_t)) != cudaSuccess) {
        set_last_error("engine_create: pinned staging allocation failed");
        return fail(B200_ERR_CUDA);
    }
    E_TRY(named_alloc(e, &e->meta_dev, "step_meta", e->meta_ints, true));
    {
        const size_t rows = (static_cast<size_t>(e->max_batch) + 15) & ~size_t(15);
        const size_t slot_bytes = rows * 4 + rows + rows + 16;
        if (cudaHostAlloc(reinterpret_cast<void**>(&e->ring_host), slot_bytes * b200_engine::kResultSlots,
                          cudaHostAllocMapped) != cudaSuccess) {
            set_last_error("engine_create: pinned result ring allocation failed");
            return fail(B200_ERR_CUDA);
        }
        memset(e->ring_host, 0, slot_bytes * b200_engine::kResultSlots);
        for (int i = 0; i < b200_engine::kResultSlots; ++i) {
            uint8_t* base = e->ring_host + slot_bytes * i;
            auto& slot = e->ring[i];
            slot.tokens = reinterpret_cast<int32_t*>(base);
            slot.finished = base + rows * 4;
            slot.ignore_eos = base + rows * 5;
            slot.status = reinterpret_cast<int32_t*>(base + rows * 6);
            if (cudaEventCreateWithFlags(&slot.done, cudaEventDisableTiming) != cudaSuccess) {
                set_last_error("engine_create: event creation failed");
                return fail(B200_ERR_CUDA);
            }
        }
    }
    if (cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&e->ev_meta_done, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&e->ev_scatter_done, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreate(&e->ev_step_begin) != cudaSuccess || cudaEventCreate(&e->ev_step_end) != cudaSuccess) {
        set_last_error("engine_create: stream / event creation failed");
        return fail(B200_ERR_CUDA);
    }
    if (cudaDeviceSynchronize() != cudaSuccess) {
        set_last_error("engine_create: device error during initialisation");
        return fail(B200_ERR_CUDA);
    }
#undef E_TRY
    *out = e;
    return B200_OK;
}

int b200_engine_destroy(b200_engine* e) {
    if (!e) return B200_OK;
    if (e->stream) cudaStreamSynchronize(e->stream);
    for (auto& g : e->graphs) cudaGraphExecDestroy(g.second);
    for (auto& g : e->graphs_sampled) cudaGraphExecDestroy(g.second);
    for (cudaEvent_t ev : e->prof_events) cudaEventDestroy(ev);
    for (cudaEvent_t ev : e->prof_events_ar) cudaEventDestroy(ev);
    if (e->comm) b200_comm_destroy(e->comm);
    for (void* p : e->allocs) cudaFree(p);
    if (e->meta_host) cudaFreeHost(e->meta_host);
    if (e->scatter_host) cudaFreeHost(e->scatter_host);
    for (auto& slot : e->ring)
        if (slot.done) cudaEventDestroy(slot.done);
    if (e->ring_host) cudaFreeHost(e->ring_host);
    if (e->ev_meta_done) cudaEventDestroy(e->ev_meta_done);
    if (e->ev_scatter_done) cudaEventDestroy(e->ev_scatter_done);
    if (e->ev_step_begin) cudaEventDestroy(e->ev_step_begin);
    if (e->ev_step_end) cudaEventDestroy(e->ev_step_end);
    if (e->stream) cudaStreamDestroy(e->stream);
    delete e;
    return B200_OK;
}

int b200_engine_tensor(b200_engine* e, const char* name, int layer, void** device_ptr, int64_t* nbytes) {
    B200_CHECK_ARG(e && name, "engine_tensor: NULL argument");
    std::string key(name);
    auto it = e->named.find(key);
    if (it == e->named.end()) it = e->named.find(key + "." + std::to_string(layer));
    if (it == e->named.end()) {
        set_last_error("engine_tensor: no tensor named '%s' (layer %d)", name, layer);
        return B200_ERR_INVALID_ARGUMENT;
    }
    if (device_ptr) *device_ptr = it->second.ptr;
    if (nbytes) *nbytes = it->second.bytes;
    // A caller that asks for one of these may write it: the folded copies are rebuilt before the next step.
    const std::string stem = key.substr(0, key.find('.'));
    if (device_ptr && (stem == "qkv" || stem == "gate_up" || stem == "input_norm" || stem == "post_norm"))
        e->folded_valid = false;
    return B200_OK;
}

int b200_engine_load(b200_engine* e, const char* name, int layer, const void* host, int64_t nbytes) {
    B200_CHECK_ARG(host, "engine_load: host pointer is NULL");
    void* p = nullptr;
    int64_t bytes = 0;
    int err = b200_engine_tensor(e, name, layer, &p, &bytes);
    if (err != B200_OK) return err;
    B200_CHECK_ARG(bytes == nbytes, "engine_load: '%s' holds %lld bytes, got %lld", name,
                   static_cast<long long>(bytes), static_cast<long long>(nbytes));
    B200_CHECK_CUDA(cudaStreamSynchronize(e->stream));
    B200_CHECK_CUDA(cudaMemcpy(p, host, static_cast<size_t>(nbytes), cudaMemcpyHostToDevice));
    return B200_OK;
}

int b200_engine_write_table(b200_engine* e, int which, const int32_t* rows, const int32_t* positions,
                            const int32_t* values, int64_t count) {
    B200_CHECK_ARG(e, "engine_write_table: NULL engine");
    B200_CHECK_ARG(which == 0 || which == 1, "engine_write_table: which must be 0 (page table) or 1 (token pool)");
    B200_CHECK_ARG(count >= 0, "engine_write_table: negative count");
    if (count == 0) return B200_OK;
    B200_CHECK_ARG(rows && positions && values, "engine_write_table: NULL array");
    if (e->scatter_in_flight) {
        B200_CHECK_CUDA(cudaEventSynchronize(e->ev_scatter_done));
        e->scatter_in_flight = false;
    }
    if (count > e->scatter_cap) {
        int64_t cap = 1024;
        while (cap < count) cap <<= 1;
        if (e->scatter_host) cudaFreeHost(e->scatter_host);
        e->scatter_host = nullptr;
        B200_CHECK_CUDA(cudaMallocHost(&e->scatter_host, 3 * cap * sizeof(int32_t)));
        void* d = nullptr;
        B200_TRY(dev_alloc(e, &d, 3 * cap * sizeof(int32_t), false));
        e->scatter_dev = static_cast<int32_t*>(d);
        e->scatter_cap = cap;
    }
    memcpy(e->scatter_host, rows, count * sizeof(int32_t));
    memcpy(e->scatter_host + count, positions, count * sizeof(int32_t));
    memcpy(e->scatter_host + 2 * count, values, count * sizeof(int32_t));
    B200_CHECK_CUDA(cudaMemcpyAsync(e->scatter_dev, e->scatter_host, 3 * count * sizeof(int32_t),
                                    cudaMemcpyHostToDevice, e->stream));
    B200_CHECK_CUDA(cudaEventRecord(e->ev_scatter_done, e->stream));
    e->scatter_in_flight = true;
    int32_t* table = which == 0 ? e->page_table : e->token_pool;
    scatter_int32_kernel<<<static_cast<unsigned>((count + 255) / 256), 256, 0, e->stream>>>(
        table, e->pt_rows, e->pt_cols, e->pt_cols, e->scatter_dev, e->scatter_dev + count,
        e->scatter_dev + 2 * count, count);
    B200_CHECK_LAUNCH();
    return B200_OK;
}

int b200_engine_capture_graphs(b200_engine* e, const int32_t* batch_sizes, int count) {
    B200_CHECK_ARG(e && count >= 0, "engine_capture_graphs: NULL engine or negative count");
    std::vector<int> sizes;
    if (count == 0 || batch_sizes == nullptr) {
        // GraphRunner::determine_batch_sizes (src/engine/engine.cc:592-616): 1, 2, 4, 8, ... and the maximum
        const int mx = e->c.max_running_req;
        for (int bs : {1, 2, 4}) if (bs <= mx) sizes.push_back(bs);
        for (int bs = 8; bs <= mx; bs *= 2) sizes.push_back(bs);
        if (sizes.empty() || sizes.back() != mx) sizes.push_back(mx);
    } else {
        sizes.assign(batch_sizes, batch_sizes + count);
    }
    for (int Bp : sizes) {
        B200_CHECK_ARG(Bp >= 1 && Bp <= e->max_batch, "engine_capture_graphs: batch size %d out of range", Bp);
        for (int variant = 0; variant < 2; ++variant) {   // 0: ends in argmax; 1: ends in the sampling kernel
            auto& graphs = variant ? e->graphs_sampled : e->graphs;
            if (graphs.count(Bp)) continue;
            // Warm-up + capture run on the dummy request only (GraphRunner::capture_graphs does the
            // same): every row is the dummy row, one key each, nothing is written back.
            B200_CHECK_CUDA(cudaStreamSynchronize(e->stream));
            b200_step st = {};
            st.phase = B200_PHASE_DECODE;
            st.num_reqs = 0;
            st.num_padded_reqs = 0;      // every row is padding
            const float one = 1.0f;
            st.temperatures = variant ? &one : nullptr;   // non-NULL only switches the staging of sampling fields on
            int T = 0, max_ext = 0;
            B200_TRY(stage_step(e, &st, Bp, &T, &max_ext));
            const size_t bytes = (variant ? b200_engine::step_index_offset(Bp) + 2 : 4 * Bp + 1) * sizeof(int32_t);
            B200_CHECK_CUDA(cudaMemcpyAsync(e->meta_dev, e->meta_host, bytes, cudaMemcpyHostToDevice, e->stream));
            B200_TRY(ensure_folded(e));
            B200_TRY(enqueue_forward(e, B200_PHASE_DECODE, Bp, Bp, Bp, 1, variant != 0));  // eager warm-up
            B200_CHECK_CUDA(cudaStreamSynchronize(e->stream));
            cudaGraph_t graph = nullptr;
            B200_CHECK_CUDA(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal));
            e->capturing = true;
            int err = enqueue_forward(e, B200_PHASE_DECODE, Bp, Bp, Bp, 1, variant != 0);
            e->capturing = false;
            cudaError_t ce = cudaStreamEndCapture(e->stream, &graph);
            if (err != B200_OK) {
                if (graph) cudaGraphDestroy(graph);
                return err;
            }
            B200_CHECK_CUDA(ce);
            cudaGraphExec_t exec = nullptr;
            ce = cudaGraphInstantiate(&exec, graph, 0);
            cudaGraphDestroy(graph);
            B200_CHECK_CUDA(ce);
            graphs[Bp] = exec;
            e->graph_launches[Bp] = e->launches_last_step;
        }
    }
    return B200_OK;
}

// One step; the tokens go to `next_tokens_host` by a copy, or (slot != NULL) through the result ring.
static int run_step(b200_engine* e, const b200_step* st, int32_t* next_tokens_host, b200_engine::ResultSlot* slot) {
    B200_CHECK_ARG(e && st, "engine_step: NULL argument");
    B200_CHECK_ARG(st->phase == B200_PHASE_PREFILL || st->phase == B200_PHASE_DECODE, "engine_step: bad phase");
    const int B = st->num_reqs, Bp = st->num_padded_reqs;
    B200_CHECK_ARG(B >= 0 && Bp >= B && Bp <= e->max_batch, "engine_step: batch size out of range");
    if (Bp == 0) return B200_OK;
    B200_CHECK_ARG(st->table_idx && st->cached_lens && st->extend_lens, "engine_step: NULL request arrays");
    const bool sampling = st->temperatures != nullptr;
    if (e->meta_in_flight) {  // the staging block of the previous step must have been consumed
        B200_CHECK_CUDA(cudaEventSynchronize(e->ev_meta_done));
        e->meta_in_flight = false;
    }
    // A decode batch runs at the next captured size (GraphRunner::pad_batch takes the lower bound of the
    // captured sizes, src/engine/engine.cc:628-645): rows the caller did not pad are padded here.
    auto& graphs = sampling ? e->graphs_sampled : e->graphs;
    int Bg = Bp;
    if (st->phase == B200_PHASE_DECODE && !e->profile_attention) {
        auto it = graphs.lower_bound(Bp);
        if (it != graphs.end()) Bg = it->first;
    }
    int T = 0, max_ext = 0;
    B200_TRY(stage_step(e, st, Bg, &T, &max_ext));
    B200_CHECK_ARG(T <= e->max_tokens, "engine_step: %d tokens exceed max_extend_tokens %d", T, e->max_tokens);
    if (st->phase == B200_PHASE_DECODE)
        B200_CHECK_ARG(T == Bg, "engine_step: a decode step runs exactly one token per request");

    cudaStream_t s = e->stream;
    B200_TRY(ensure_folded(e));
    B200_CHECK_CUDA(cudaEventRecord(e->ev_step_begin, s));
    const size_t meta_bytes =
        (sampling ? b200_engine::step_index_offset(Bg) + 2 : 4 * Bg + 1) * sizeof(int32_t);
    B200_CHECK_CUDA(cudaMemcpyAsync(e->meta_dev, e->meta_host, meta_bytes, cudaMemcpyHostToDevice, s));
    B200_CHECK_CUDA(cudaEventRecord(e->ev_meta_done, s));
    e->meta_in_flight = true;
    // A captured graph covers all Bg rows; padded rows carry write_pos = -1 so nothing of
    // theirs is written back, and only the first B tokens are copied out.
    auto g = st->phase == B200_PHASE_DECODE ? graphs.find(Bg) : graphs.end();
    if (g != graphs.end() && !e->profile_attention) {
        B200_CHECK_CUDA(cudaGraphLaunch(g->second, s));
        e->launches_last_step = e->graph_launches[Bg];
    } else {
        B200_TRY(enqueue_forward(e, st->phase, B, Bg, T, max_ext, sampling, st->step_index));
    }
    if (next_tokens_host && B > 0)
        B200_CHECK_CUDA(cudaMemcpyAsync(next_tokens_host, e->next_tokens, B * sizeof(int32_t),
                                        cudaMemcpyDeviceToHost, s));
    if (slot) {
        B200_CHECK_CUDA(launch_kernel(publish_step_kernel, dim3(1), dim3(256), 0, s, dim3(1, 1, 1), slot->tokens,
                                      slot->finished, static_cast<const uint8_t*>(slot->ignore_eos), slot->status,
                                      static_cast<const int32_t*>(e->next_tokens),
                                      static_cast<const int32_t*>(e->meta_dev + 3 * Bg + 1),
                                      static_cast<const int*>(e->status), B, static_cast<int>(e->eos_token_id),
                                      static_cast<unsigned long long>(slot->ticket)));
        e->launches_last_step += 1;
        B200_CHECK_CUDA(cudaEventRecord(slot->done, s));
    }
    B200_CHECK_CUDA(cudaEventRecord(e->ev_step_end, s));
    return B200_OK;
}

int b200_engine_step(b200_engine* e, const b200_step* st, int32_t* next_tokens_host) {
    return run_step(e, st, next_tokens_host, nullptr);
}

int b200_engine_set_eos_token(b200_engine* e, int32_t eos_token_id) {
    B200_CHECK_ARG(e, "engine_set_eos_token: NULL engine");
    e->eos_token_id = eos_token_id;
    return B200_OK;
}

int b200_engine_result_slots(void) { return b200_engine::kResultSlots; }

int b200_engine_step_async(b200_engine* e, const b200_step* st, const uint8_t* ignore_eos, int64_t* ticket) {
    B200_CHECK_ARG(e && st && ticket, "engine_step_async: NULL argument");
    B200_CHECK_ARG(st->num_reqs >= 0 && st->num_reqs <= e->max_batch, "engine_step_async: batch size out of range");
    auto& slot = e->ring[e->next_ticket % b200_engine::kResultSlots];
    // The slot's previous step (kResultSlots tickets ago) has long finished in a loop that waits for
    // its tickets; if nobody waited, its result is overwritten and its ticket becomes stale.
    if (slot.ticket >= 0) B200_CHECK_CUDA(cudaEventSynchronize(slot.done));
    for (int i = 0; i < st->num_reqs; ++i) slot.ignore_eos[i] = ignore_eos ? ignore_eos[i] : 0;
    slot.ticket = e->next_ticket;
    slot.num_reqs = st->num_reqs;
    int err = run_step(e, st, nullptr, &slot);
    if (err != B200_OK) {
        slot.ticket = -1;
        return err;
    }
    *ticket = e->next_ticket++;
    return B200_OK;
}

int b200_engine_wait(b200_engine* e, int64_t ticket, const int32_t** tokens, const uint8_t** finished) {
    B200_CHECK_ARG(e, "engine_wait: NULL engine");
    B200_CHECK_ARG(ticket >= 0 && ticket < e->next_ticket, "engine_wait: ticket %lld was never issued",
                   static_cast<long long>(ticket));
    auto& slot = e->ring[ticket % b200_engine::kResultSlots];
    B200_CHECK_ARG(slot.ticket == ticket, "engine_wait: ticket %lld has left the ring (%d steps are kept)",
                   static_cast<long long>(ticket), b200_engine::kResultSlots);
    B200_CHECK_CUDA(cudaEventSynchronize(slot.done));
    if (tokens) *tokens = slot.tokens;
    if (finished) *finished = slot.finished;
    const int timeout_site = slot.status[0], bad_index = slot.status[1];
    if (timeout_site != 0 || bad_index != 0) {
        // rare: clear the device words for the steps that follow
        cudaStreamSynchronize(e->stream);
        cudaMemset(e->status, 0, 2 * sizeof(int));
        if (timeout_site != 0) {
            set_last_error("a bounded wait inside a kernel ran out (site %d)", timeout_site);
            return B200_ERR_TIMEOUT;
        }
        set_last_error("a kernel saw an out-of-range index (%d)", bad_index - 1);
        return B200_ERR_INVALID_ARGUMENT;
    }
    return B200_OK;
}

int b200_engine_synchronize(b200_engine* e) {
    B200_CHECK_ARG(e, "engine_synchronize: NULL engine");
    B200_CHECK_CUDA(cudaStreamSynchronize(e->stream));
    int host[2] = {0, 0};
    B200_CHECK_CUDA(cudaMemcpy(host, e->status, sizeof(host), cudaMemcpyDeviceToHost));
    if (host[0] != 0) {
        cudaMemset(e->status, 0, sizeof(host));
        set_last_error("a bounded wait inside a kernel ran out (site %d)", host[0]);
        return B200_ERR_TIMEOUT;
    }
    if (host[1] != 0) {
        cudaMemset(e->status, 0, sizeof(host));
        set_last_error("a kernel saw an out-of-range index (%d)", host[1] - 1);
        return B200_ERR_INVALID_ARGUMENT;
    }
    return B200_OK;
}

int b200_engine_read_logits(b200_engine* e, void* host, int rows) {
    B200_CHECK_ARG(e && host, "engine_read_logits: NULL argument");
    B200_CHECK_ARG(rows >= 0 && rows <= e->max_batch, "engine_read_logits: rows out of range");
    B200_CHECK_CUDA(cudaStreamSynchronize(e->stream));
    B200_CHECK_CUDA(cudaMemcpy(host, e->logits, static_cast<size_t>(rows) * e->m.vocab_size * 2,
                               cudaMemcpyDeviceToHost));
    return B200_OK;
}

b200_stream_t b200_engine_stream(b200_engine* e) { return e ? e->stream : nullptr; }

int b200_engine_comm_export(b200_engine* e, void* handle_out) {
    B200_CHECK_ARG(e && e->comm, "engine_comm_export: the engine was not created with tp_size > 1");
    return b200_comm_export(e->comm, handle_out);
}

int b200_engine_comm_connect(b200_engine* e, const void* all_handles) {
    B200_CHECK_ARG(e && e->comm, "engine_comm_connect: the engine was not created with tp_size > 1");
    return b200_comm_connect(e->comm, all_handles);
}

b200_comm* b200_engine_comm(b200_engine* e) { return e ? e->comm : nullptr; }

int64_t b200_engine_comm_region_bytes(b200_engine* e) {
    if (!e || !e->comm) return -1;
    return b200_comm_region_bytes(e->comm_buffer_bytes);
}

int b200_engine_comm_attach(b200_engine* e, void* region, const void* const* peer_regions,
                            const void* multicast_region) {
    B200_CHECK_ARG(e && e->comm, "engine_comm_attach: the engine was not created with tp_size > 1");
    B200_CHECK_ARG(region && peer_regions, "engine_comm_attach: NULL region");
    B200_CHECK_ARG(e->graphs.empty() && e->graphs_sampled.empty(),
                   "engine_comm_attach: attach before capturing graphs (they hold the exchange buffers' addresses)");
    B200_CHECK_CUDA(cudaStreamSynchronize(e->stream));
    b200_comm* fresh = nullptr;
    int err = b200_comm_create_on(e->c.tp_rank, e->c.tp_size, e->comm_buffer_bytes, region, &fresh);
    if (err != B200_OK) return err;
    err = b200_comm_connect_pointers(fresh, peer_regions, multicast_region);
    if (err != B200_OK) {
        b200_comm_destroy(fresh);
        return err;
    }
    b200_comm_destroy(e->comm);
    e->comm = fresh;
    return B200_OK;
}

int b200_engine_set_profiling(b200_engine* e, int on) {
    B200_CHECK_ARG(e, "engine_set_profiling: NULL engine");
    e->profile_attention = on != 0;
    e->prof_pairs_recorded = 0;
    return B200_OK;
}

int b200_engine_read_profile_allreduce(b200_engine* e, float* allreduce_ms, int32_t* launches) {
    B200_CHECK_ARG(e, "engine_read_profile_allreduce: NULL engine");
    B200_CHECK_CUDA(cudaStreamSynchronize(e->stream));
    float total = 0.f;
    for (int i = 0; i < e->prof_ar_recorded; ++i) {
        float ms = 0.f;
        B200_CHECK_CUDA(cudaEventElapsedTime(&ms, e->prof_events_ar[2 * i], e->prof_events_ar[2 * i + 1]));
        total += ms;
    }
    if (allreduce_ms) *allreduce_ms = total;
    if (launches) *launches = e->prof_ar_recorded;
    return B200_OK;
}

int b200_engine_read_profile(b200_engine* e, float* attention_ms, int32_t* attention_launches,
                             int32_t* kernel_launches) {
    B200_CHECK_ARG(e, "engine_read_profile: NULL engine");
    B200_CHECK_CUDA(cudaStreamSynchronize(e->stream));
    float total = 0.f;
    for (int i = 0; i < e->prof_pairs_recorded; ++i) {
        float ms = 0.f;
        B200_CHECK_CUDA(cudaEventElapsedTime(&ms, e->prof_events[2 * i], e->prof_events[2 * i + 1]));
        total += ms;
    }
    if (attention_ms) *attention_ms = total;
    if (attention_launches) *attention_launches = e->prof_pairs_recorded;
    if (kernel_launches) *kernel_launches = e->launches_last_step;
    return B200_OK;
}

int b200_engine_last_step_ms(b200_engine* e, float* ms) {
    B200_CHECK_ARG(e && ms, "engine_last_step_ms: NULL argument");
    B200_CHECK_CUDA(cudaEventSynchronize(e->ev_step_end));
    B200_CHECK_CUDA(cudaEventElapsedTime(ms, e->ev_step_begin, e->ev_step_end));
    return B200_OK;
}

}  // extern "C"
