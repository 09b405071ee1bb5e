// Mixture-of-experts layer: router top-k, token permute, grouped expert GEMMs, weighted combine.
//
// Stands where MoELayer::forward does (src/moe/moe.cc:36-96).  The reference walks
// top_k x num_experts host-synchronised iterations; here one step is six launches with no host
// involvement: route (softmax + top-k per token, expert histogram) -> scan -> scatter (rows
// grouped by expert) -> grouped gate_up GEMM with the gated activation in its epilogue ->
// grouped down GEMM -> combine in the reference's accumulation order (k ascending, bf16 after
// every multiply and add, as index_add_ on bf16 tensors does).
#include "common.cuh"
#include "kernels.h"

namespace b200 {
namespace {

constexpr int kMaxExpertsPerLane = 8;  // num_experts <= 256
constexpr int kMaxTopK = 16;

// One warp per token.
__global__ void __launch_bounds__(128)
moe_route_kernel(const __nv_bfloat16* __restrict__ logits, int tokens, int E, int top_k, int renorm,
                 int32_t* __restrict__ ids, float* __restrict__ weights, int32_t* __restrict__ counts) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= tokens) return;
    const __nv_bfloat16* row = logits + static_cast<int64_t>(t) * E;
    float v[kMaxExpertsPerLane];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
        const int e = lane + i * 32;
        v[i] = e < E ? __bfloat162float(row[e]) : -INFINITY;
        mx = fmaxf(mx, v[i]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
        v[i] = (lane + i * 32) < E ? __expf(v[i] - mx) : -1.f;  // -1 marks "not a candidate"
        if (v[i] > 0.f) sum += v[i];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    float wsel[kMaxTopK];
    int isel[kMaxTopK];
    float wsum = 0.f;
    for (int k = 0; k < top_k; ++k) {
        // Largest remaining probability; the lower expert index wins ties.
        float best = -1.f;
        int bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kMaxExpertsPerLane; ++i)
            if (v[i] > best) {
                best = v[i];
                bi = lane + i * 32;
            }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) {
                best = ob;
                bi = oi;
            }
        }
        if ((bi & 31) == lane) v[bi >> 5] = -1.f;
        wsel[k] = best * inv;
        isel[k] = bi;
        wsum += wsel[k];
    }
    if (lane == 0) {
        for (int k = 0; k < top_k; ++k) {
            float w = wsel[k];
            if (renorm) w = w / (wsum + 1e-8f);
            ids[t * top_k + k] = isel[k];
            weights[t * top_k + k] = round_bf16(w);  // the reference casts the weights to bf16
            atomicAdd(&counts[isel[k]], 1);
        }
    }
}

// Row ranges of the experts [e_begin, e_begin + e_count) this call computes (all of them unless
// the experts are partitioned over ranks); every other expert gets offset -1 = "not here".
__global__ void __launch_bounds__(256)
moe_scan_kernel(const int32_t* __restrict__ counts, int32_t* __restrict__ offsets,
                int32_t* __restrict__ cursor, int E, int e_begin, int e_count) {
    pdl_launch_dependents();
    pdl_wait_prior();
    __shared__ int s[256];
    const int e = threadIdx.x;
    const bool local = e >= e_begin && e < e_begin + e_count;
    s[e] = (e < E && local) ? counts[e] : 0;
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int i = 0; i < E; ++i) {
            const int c = s[i];
            s[i] = run;
            run += c;
        }
        offsets[E] = run;
    }
    __syncthreads();
    if (e < E) {
        offsets[e] = local ? s[e] : -1;
        cursor[e] = 0;
    }
}

// One CTA per (token, k) pair: claim a row in the expert's range and copy the token there.
__global__ void __launch_bounds__(128)
moe_scatter_kernel(const uint4* __restrict__ hidden, uint4* __restrict__ xp,
                   const int32_t* __restrict__ ids, const int32_t* __restrict__ offsets,
                   int32_t* __restrict__ cursor, int32_t* __restrict__ pos, int top_k, int vec_per_row) {
    pdl_launch_dependents();
    pdl_wait_prior();
    __shared__ int s_row;
    const int pair = blockIdx.x;
    if (threadIdx.x == 0) {
        const int e = ids[pair];
        const int base = offsets[e];
        s_row = base < 0 ? -1 : base + atomicAdd(&cursor[e], 1);
        pos[pair] = s_row;
    }
    __syncthreads();
    if (s_row < 0) return;  // another rank's expert
    const uint4* src = hidden + static_cast<int64_t>(pair / top_k) * vec_per_row;
    uint4* dst = xp + static_cast<int64_t>(s_row) * vec_per_row;
    for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) dst[v] = src[v];
}

// out[t] = fold over k of bf16(acc + bf16(y[pos[t,k]] * w[t,k])), acc starting at 0.
__global__ void __launch_bounds__(128)
moe_combine_kernel(uint4* __restrict__ out, const uint4* __restrict__ y, const int32_t* __restrict__ pos,
                   const float* __restrict__ weights, int top_k, int vec_per_row) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int t = blockIdx.x;
    for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int k = 0; k < top_k; ++k) {
            const float w = weights[t * top_k + k];
            const int row = pos[t * top_k + k];
            if (row < 0) continue;  // another rank's expert: its term arrives through the all-reduce
            const uint4 a = y[static_cast<int64_t>(row) * vec_per_row + v];
            const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                acc[2 * j] = round_bf16(acc[2 * j] + round_bf16(bf16_lo(aw[j]) * w));
                acc[2 * j + 1] = round_bf16(acc[2 * j + 1] + round_bf16(bf16_hi(aw[j]) * w));
            }
        }
        out[static_cast<int64_t>(t) * vec_per_row + v] =
            make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]),
                       pack_bf16(acc[6], acc[7]));
    }
}

struct MoeWorkspace {
    int32_t *ids, *counts, *offsets, *cursor, *pos;
    float* weights;
    __nv_bfloat16 *xp, *hact, *y2;
};

int64_t align256(int64_t x) { return (x + 255) / 256 * 256; }

int64_t carve(MoeWorkspace* w, uint8_t* base, int tokens, int E, int top_k, int H, int I) {
    const int64_t pairs = static_cast<int64_t>(tokens) * top_k;
    int64_t off = 0;
    auto take = [&](int64_t bytes) {
        uint8_t* p = base ? base + off : nullptr;
        off += align256(bytes);
        return p;
    };
    w->ids = reinterpret_cast<int32_t*>(take(pairs * 4));
    w->weights = reinterpret_cast<float*>(take(pairs * 4));
    w->pos = reinterpret_cast<int32_t*>(take(pairs * 4));
    w->counts = reinterpret_cast<int32_t*>(take((E + 1) * 4));
    w->offsets = reinterpret_cast<int32_t*>(take((E + 1) * 4));
    w->cursor = reinterpret_cast<int32_t*>(take((E + 1) * 4));
    w->xp = reinterpret_cast<__nv_bfloat16*>(take(pairs * H * 2));
    w->hact = reinterpret_cast<__nv_bfloat16*>(take(pairs * I * 2));
    w->y2 = reinterpret_cast<__nv_bfloat16*>(take(pairs * H * 2));
    return off;
}

}  // namespace

int64_t moe_workspace_bytes(int tokens, int E, int top_k, int H, int I) {
    MoeWorkspace w;
    return carve(&w, nullptr, tokens, E, top_k, H, I);
}

int launch_moe_route(int32_t* ids, float* weights, int32_t* counts, const void* logits, int tokens, int E,
                     int top_k, int renorm, cudaStream_t stream) {
    B200_CHECK_CUDA(cudaMemsetAsync(counts, 0, (E + 1) * sizeof(int32_t), stream));
    const bool pdl = pdl_launches_enabled();
    set_pdl_launches(false);  // follows a memset
    cudaError_t ce = launch_kernel(moe_route_kernel, dim3(div_ceil(tokens, 4)), dim3(128), 0, stream, dim3(1, 1, 1),
                                   static_cast<const __nv_bfloat16*>(logits), tokens, E, top_k, renorm, ids,
                                   weights, counts);
    set_pdl_launches(pdl);
    B200_CHECK_CUDA(ce);
    return B200_OK;
}

int launch_moe_forward(void* out, const void* hidden, const void* router_logits, const void* gate_up,
                       const void* down, int tokens, int E, int top_k, int H, int I, int renorm,
                       int activation, int expert_begin, int num_local_experts, void* workspace,
                       int* status, cudaStream_t stream) {
    if (tokens == 0) return B200_OK;
    MoeWorkspace w;
    carve(&w, static_cast<uint8_t*>(workspace), tokens, E, top_k, H, I);
    const int pairs = tokens * top_k;
    int err = launch_moe_route(w.ids, w.weights, w.counts, router_logits, tokens, E, top_k, renorm, stream);
    if (err != B200_OK) return err;
    B200_CHECK_CUDA(launch_kernel(moe_scan_kernel, dim3(1), dim3(256), 0, stream, dim3(1, 1, 1),
                                  static_cast<const int32_t*>(w.counts), w.offsets, w.cursor, E, expert_begin,
                                  num_local_experts));
    B200_CHECK_CUDA(launch_kernel(moe_scatter_kernel, dim3(pairs), dim3(128), 0, stream, dim3(1, 1, 1),
                                  static_cast<const uint4*>(hidden), reinterpret_cast<uint4*>(w.xp),
                                  static_cast<const int32_t*>(w.ids), static_cast<const int32_t*>(w.offsets),
                                  w.cursor, w.pos, top_k, H / 8));
    const int epi = activation == 1 ? B200_EPILOGUE_GEGLU_ERF : B200_EPILOGUE_SWIGLU;
    // A token picks distinct experts, so no expert gets more rows than there are tokens.
    // gate_up / down hold the local experts only, so group g is expert expert_begin + g.
    const int32_t* counts = w.counts + expert_begin;
    const int32_t* offsets = w.offsets + expert_begin;
    err = launch_grouped_gemm(w.hact, w.xp, gate_up, counts, offsets, num_local_experts, tokens, pairs, 2 * I, H,
                              epi, status, stream);
    if (err != B200_OK) return err;
    err = launch_grouped_gemm(w.y2, w.hact, down, counts, offsets, num_local_experts, tokens, pairs, H, I,
                              B200_EPILOGUE_NONE, status, stream);
    if (err != B200_OK) return err;
    B200_CHECK_CUDA(launch_kernel(moe_combine_kernel, dim3(tokens), dim3(128), 0, stream, dim3(1, 1, 1),
                                  static_cast<uint4*>(out), reinterpret_cast<const uint4*>(w.y2),
                                  static_cast<const int32_t*>(w.pos), static_cast<const float*>(w.weights),
                                  top_k, H / 8));
    return B200_OK;
}

}  // namespace b200

extern "C" {

int64_t b200_moe_workspace_bytes(int tokens, int num_experts, int top_k, int hidden_size, int intermediate_size) {
    if (tokens < 0 || num_experts <= 0 || top_k <= 0 || hidden_size <= 0 || intermediate_size <= 0) return -1;
    return b200::moe_workspace_bytes(tokens, num_experts, top_k, hidden_size, intermediate_size);
}

int b200_moe_route(int32_t* topk_ids, float* topk_weights, int32_t* expert_counts, const void* router_logits,
                   int tokens, int num_experts, int top_k, int renormalize, b200_stream_t stream) {
    B200_CHECK_ARG(tokens >= 0, "moe_route: tokens must be >= 0");
    B200_CHECK_ARG(num_experts > 0 && num_experts <= 256, "MoELayer requires 0 < num_experts <= 256");
    B200_CHECK_ARG(top_k > 0 && top_k <= b200::kMaxTopK, "MoELayer requires 0 < top_k <= 16");
    B200_CHECK_ARG(top_k <= num_experts, "MoELayer top_k must be <= num_experts");
    if (tokens == 0) return B200_OK;
    B200_CHECK_ARG(topk_ids && topk_weights && expert_counts && router_logits, "moe_route: NULL tensor");
    return b200::launch_moe_route(topk_ids, topk_weights, expert_counts, router_logits, tokens, num_experts,
                                  top_k, renormalize, static_cast<cudaStream_t>(stream));
}

int b200_moe_forward_local(void* out, const void* hidden_states, const void* router_logits,
                           const void* gate_up_proj, const void* down_proj, int tokens, int num_experts,
                           int top_k, int hidden_size, int intermediate_size, int renormalize,
                           int activation, int expert_begin, int num_local_experts, void* workspace,
                           int64_t workspace_bytes, b200_stream_t stream) {
    B200_CHECK_ARG(tokens >= 0, "MoELayer token count must be >= 0");
    B200_CHECK_ARG(num_experts > 0 && num_experts <= 256, "MoELayer requires 0 < num_experts <= 256");
    B200_CHECK_ARG(top_k > 0 && top_k <= b200::kMaxTopK, "MoELayer requires 0 < top_k <= 16");
    B200_CHECK_ARG(top_k <= num_experts, "MoELayer top_k must be <= num_experts");
    B200_CHECK_ARG(hidden_size > 0 && hidden_size % 64 == 0, "MoELayer hidden size must be a positive multiple of 64");
    B200_CHECK_ARG(intermediate_size > 0 && intermediate_size % 64 == 0,
                   "MoELayer intermediate size must be a positive multiple of 64");
    B200_CHECK_ARG(activation == 0 || activation == 1, "Unsupported MoE activation function");
    B200_CHECK_ARG(expert_begin >= 0 && num_local_experts > 0 && expert_begin + num_local_experts <= num_experts,
                   "moe_forward: local expert range outside [0, num_experts)");
    if (tokens == 0) return B200_OK;
    B200_CHECK_ARG(out && hidden_states && router_logits && gate_up_proj && down_proj && workspace,
                   "moe_forward: NULL tensor");
    B200_CHECK_ARG(workspace_bytes >= b200::moe_workspace_bytes(tokens, num_experts, top_k, hidden_size, intermediate_size),
                   "moe_forward: workspace too small");
    int err = B200_OK;
    int* status = b200::device_status_words(&err);
    if (err != B200_OK) return err;
    return b200::launch_moe_forward(out, hidden_states, router_logits, gate_up_proj, down_proj, tokens,
                                    num_experts, top_k, hidden_size, intermediate_size, renormalize, activation,
                                    expert_begin, num_local_experts, workspace, status,
                                    static_cast<cudaStream_t>(stream));
}

int b200_moe_forward(void* out, const void* hidden_states, const void* router_logits, const void* gate_up_proj,
                     const void* down_proj, int tokens, int num_experts, int top_k, int hidden_size,
                     int intermediate_size, int renormalize, int activation, void* workspace,
                     int64_t workspace_bytes, b200_stream_t stream) {
    return b200_moe_forward_local(out, hidden_states, router_logits, gate_up_proj, down_proj, tokens, num_experts,
                                  top_k, hidden_size, intermediate_size, renormalize, activation, 0,
                                  num_experts > 0 ? num_experts : 1, workspace, workspace_bytes, stream);
}

}  // extern "C"
