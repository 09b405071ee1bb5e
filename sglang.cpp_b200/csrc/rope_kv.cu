// Rotary embedding, KV-pool store, and the fused QK-norm + RoPE + store pass.
//
// HBM-bound elementwise work on rows of head_dim bf16.  One warp owns one
// (token, head) row; a lane holds the two halves of its NeoX pairs so the
// rotation needs no shuffles, and the norm needs one 5-step shuffle reduction.
#include "common.cuh"
#include "kernels.h"

namespace b200 {
namespace {

template <int N>
struct __align__(N * 2) BfVec {
    __nv_bfloat16 v[N];
};

// General in-place NeoX rotation (any even rotary_dim <= head_dim).
__global__ void __launch_bounds__(128)
rope_neox_kernel(__nv_bfloat16* q, __nv_bfloat16* k, const float* __restrict__ cos_t,
                 const float* __restrict__ sin_t, const int32_t* __restrict__ positions,
                 int64_t q_rows, int64_t total_rows, int q_heads, int k_heads, int head_dim,
                 int rotary_dim, int max_pos, int64_t qst, int64_t qsh, int64_t kst, int64_t ksh,
                 int* status) {
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= total_rows) return;
    __nv_bfloat16* p;
    int64_t t;
    if (row < q_rows) {
        t = row / q_heads;
        p = q + t * qst + (row - t * q_heads) * qsh;
    } else {
        const int64_t r = row - q_rows;
        t = r / k_heads;
        p = k + t * kst + (r - t * k_heads) * ksh;
    }
    int pos = positions[t];
    if (pos < 0 || pos >= max_pos) {
        if (lane == 0) atomicExch(&status[kStatusBadIndex], pos + 1);
        pos = min(max(pos, 0), max_pos - 1);
    }
    const int half = rotary_dim >> 1;
    const float* c = cos_t + static_cast<int64_t>(pos) * half;
    const float* s = sin_t + static_cast<int64_t>(pos) * half;
    for (int i = lane; i < half; i += 32) {
        const float x1 = __bfloat162float(p[i]);
        const float x2 = __bfloat162float(p[i + half]);
        const float cs = c[i], sn = s[i];
        p[i] = __float2bfloat16_rn(x1 * cs - x2 * sn);
        p[i + half] = __float2bfloat16_rn(x2 * cs + x1 * sn);
    }
}

// k_cache[out_loc[t]] = k[t], v likewise; 16-byte vectors, one warp per token.
__global__ void __launch_bounds__(128)
store_kv_kernel(uint4* __restrict__ k_cache, uint4* __restrict__ v_cache,
                const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                const int32_t* __restrict__ out_loc, int tokens, int vec_per_token, int64_t kst,
                int64_t vst, int64_t num_slots, int* status) {
    const int lane = threadIdx.x & 31;
    const int64_t t = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= tokens) return;
    const int64_t slot = out_loc[t];
    if (slot < 0 || slot >= num_slots) {
        if (lane == 0) atomicExch(&status[kStatusBadIndex], static_cast<int>(slot) + 1);
        return;
    }
    const uint4* ks = reinterpret_cast<const uint4*>(k + t * kst);
    const uint4* vs = reinterpret_cast<const uint4*>(v + t * vst);
    uint4* kd = k_cache + slot * vec_per_token;
    uint4* vd = v_cache + slot * vec_per_token;
    for (int i = lane; i < vec_per_token; i += 32) {
        kd[i] = ks[i];
        vd[i] = vs[i];
    }
}

// Fused pass over packed qkv rows.  D = head_dim (rotary_dim == head_dim).
// Row index r in [0, q_heads + 2*kv_heads): q head, then k head, then v head.
template <int D>
__global__ void __launch_bounds__(128)
qknorm_rope_store_kernel(__nv_bfloat16* qkv, const __nv_bfloat16* __restrict__ qw,
                         const __nv_bfloat16* __restrict__ kw, const float* __restrict__ cos_t,
                         const float* __restrict__ sin_t, const int32_t* __restrict__ positions,
                         const int32_t* __restrict__ out_loc, __nv_bfloat16* __restrict__ k_cache,
                         __nv_bfloat16* __restrict__ v_cache, int tokens, int q_heads,
                         int kv_heads, int max_pos, int64_t num_slots, float eps, int write_k_back,
                         int* status, int rows_per_warp) {
    // Eight lanes per row, 16-byte vectors (head_dim 128): lane `sub` of a row holds elements
    // [sub*EPL, sub*EPL + EPL) of each half, so the NeoX partner of an element is in the same lane.
    constexpr int LPR = 8;                  // lanes per row
    constexpr int RPP = 32 / LPR;           // rows a warp handles per pass
    constexpr int EPL = D / (2 * LPR);      // elements per lane per half
    using Vec = BfVec<EPL>;
    const int lane = threadIdx.x & 31;
    const int sub = lane % LPR;
    const unsigned group_mask = ((1u << LPR) - 1u) << (lane / LPR * LPR);
    const int rows_per_token = q_heads + 2 * kv_heads;
    const int64_t total_rows = static_cast<int64_t>(tokens) * rows_per_token;
    const int64_t row0 =
        (static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5)) * rows_per_warp * RPP +
        lane / LPR;

    pdl_launch_dependents();
    // What the first row needs besides the row itself - its token's position and slot, the rotation
    // entries of that position, the norm weights - does not come from the kernel before this one
    // (positions and out_loc are complete before any kernel of the layer stack starts): fetch it
    // ahead of the wait, so that only the row is loaded behind it.
    int pre_pos = 0, pre_slot = 0;
    float pre_c[EPL], pre_s[EPL];
    Vec pre_wa, pre_wb;
    if (row0 < total_rows) {
        const int64_t t = row0 / rows_per_token;
        const int r = static_cast<int>(row0 - t * rows_per_token);
        pre_pos = positions[t];
        pre_slot = out_loc[t];
        const int pc = min(max(pre_pos, 0), max_pos - 1);
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
            pre_c[e] = cos_t[static_cast<int64_t>(pc) * (D / 2) + sub * EPL + e];
            pre_s[e] = sin_t[static_cast<int64_t>(pc) * (D / 2) + sub * EPL + e];
        }
        const __nv_bfloat16* w = r < q_heads ? qw : kw;
        if (w != nullptr && r < q_heads + kv_heads) {
            pre_wa = *reinterpret_cast<const Vec*>(w + sub * EPL);
            pre_wb = *reinterpret_cast<const Vec*>(w + D / 2 + sub * EPL);
        }
    }
    pdl_wait_prior();
    if (row0 >= total_rows) return;

    // One row: a, b are its two halves, already loaded.
    auto process = [&](int64_t row, Vec a, Vec b) {
    const bool first = row == row0;
    const int64_t t = row / rows_per_token;
    const int r = static_cast<int>(row - t * rows_per_token);
    __nv_bfloat16* src = qkv + (t * rows_per_token + r) * D;

    const bool is_q = r < q_heads;
    const bool is_k = !is_q && r < q_heads + kv_heads;
    const int kvh = is_q ? 0 : (is_k ? r - q_heads : r - q_heads - kv_heads);

    int64_t slot = 0;
    if (!is_q) {
        slot = first ? pre_slot : out_loc[t];
        if (slot < 0 || slot >= num_slots) {
            if (sub == 0) atomicExch(&status[kStatusBadIndex], static_cast<int>(slot) + 1);
            slot = -1;
        }
    }

    if (!is_q && !is_k) {  // v row: plain copy into the pool
        if (slot >= 0) {
            __nv_bfloat16* dst = v_cache + (slot * kv_heads + kvh) * D;
            *reinterpret_cast<Vec*>(dst + sub * EPL) = a;
            *reinterpret_cast<Vec*>(dst + D / 2 + sub * EPL) = b;
        }
        return;
    }

    float x1[EPL], x2[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
        x1[e] = __bfloat162float(a.v[e]);
        x2[e] = __bfloat162float(b.v[e]);
    }

    const __nv_bfloat16* w = is_q ? qw : kw;
    if (w != nullptr) {
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) ss += x1[e] * x1[e] + x2[e] * x2[e];
#pragma unroll
        for (int o = LPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(group_mask, ss, o);
        const float scale = rsqrtf(ss / static_cast<float>(D) + eps);
        Vec wa = first ? pre_wa : *reinterpret_cast<const Vec*>(w + sub * EPL);
        Vec wb = first ? pre_wb : *reinterpret_cast<const Vec*>(w + D / 2 + sub * EPL);
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
            // bf16 rounding here is where the unfused norm kernel stores its result.
            x1[e] = round_bf16(x1[e] * scale * __bfloat162float(wa.v[e]));
            x2[e] = round_bf16(x2[e] * scale * __bfloat162float(wb.v[e]));
        }
    }

    int pos = first ? pre_pos : positions[t];
    if (pos < 0 || pos >= max_pos) {
        if (sub == 0) atomicExch(&status[kStatusBadIndex], pos + 1);
        pos = min(max(pos, 0), max_pos - 1);
    }
    const float* c = cos_t + static_cast<int64_t>(pos) * (D / 2) + sub * EPL;
    const float* s = sin_t + static_cast<int64_t>(pos) * (D / 2) + sub * EPL;
    Vec oa, ob;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
        const float cs = first ? pre_c[e] : c[e], sn = first ? pre_s[e] : s[e];
        oa.v[e] = __float2bfloat16_rn(x1[e] * cs - x2[e] * sn);
        ob.v[e] = __float2bfloat16_rn(x2[e] * cs + x1[e] * sn);
    }

    if (is_q || write_k_back) {
        *reinterpret_cast<Vec*>(src + sub * EPL) = oa;
        *reinterpret_cast<Vec*>(src + D / 2 + sub * EPL) = ob;
    }
    if (is_k && slot >= 0) {
        __nv_bfloat16* dst = k_cache + (slot * kv_heads + kvh) * D;
        *reinterpret_cast<Vec*>(dst + sub * EPL) = oa;
        *reinterpret_cast<Vec*>(dst + D / 2 + sub * EPL) = ob;
    }
    };

    // Rows of this warp, the next row's loads in flight while the current one is processed
    // (rows are adjacent in the qkv buffer: row * D elements from its start).
    const int64_t row_end = min(row0 + static_cast<int64_t>(rows_per_warp) * RPP, total_rows);
    Vec a = *reinterpret_cast<const Vec*>(qkv + row0 * D + sub * EPL);
    Vec b = *reinterpret_cast<const Vec*>(qkv + row0 * D + D / 2 + sub * EPL);
    for (int64_t row = row0; row < row_end; row += RPP) {
        Vec an = a, bn = b;
        if (row + RPP < row_end) {
            an = *reinterpret_cast<const Vec*>(qkv + (row + RPP) * D + sub * EPL);
            bn = *reinterpret_cast<const Vec*>(qkv + (row + RPP) * D + D / 2 + sub * EPL);
        }
        process(row, a, b);
        a = an;
        b = bn;
    }
}

}  // namespace

int launch_qknorm_rope_store(void* qkv, const void* q_weight, const void* k_weight,
                             const float* cos_table, const float* sin_table,
                             const int32_t* positions, const int32_t* out_loc, void* k_cache,
                             void* v_cache, int tokens, int q_heads, int kv_heads, int head_dim,
                             int max_pos, int64_t num_slots, float eps, int write_k_back,
                             int* status, cudaStream_t stream) {
    const int64_t rows = static_cast<int64_t>(tokens) * (q_heads + 2 * kv_heads);
    if (rows == 0) return B200_OK;
    // Few rows (decode): one row per warp for the most parallelism; many rows (prefill): four per
    // warp with the next row's loads in flight.
    const int rows_per_warp = rows >= 32768 ? 4 : 1;   // passes of 4 rows each
    const int warps_per_block = rows >= 32768 ? 4 : 1; // decode: one warp per CTA, spread over all SMs
    const int64_t rows_per_block = 4 * warps_per_block * rows_per_warp;
    const unsigned blocks = static_cast<unsigned>((rows + rows_per_block - 1) / rows_per_block);
#define B200_LAUNCH_QRS(D)                                                                       \
    B200_CHECK_CUDA(launch_kernel(                                                               \
        qknorm_rope_store_kernel<D>, dim3(blocks), dim3(32 * warps_per_block), 0, stream, dim3(1, 1, 1), \
        static_cast<__nv_bfloat16*>(qkv), static_cast<const __nv_bfloat16*>(q_weight),           \
        static_cast<const __nv_bfloat16*>(k_weight), cos_table, sin_table, positions, out_loc,   \
        static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), tokens,      \
        q_heads, kv_heads, max_pos, num_slots, eps, write_k_back, status, rows_per_warp))
    switch (head_dim) {
        case 64: B200_LAUNCH_QRS(64); break;
        case 128: B200_LAUNCH_QRS(128); break;
        case 256: B200_LAUNCH_QRS(256); break;
        default:
            set_last_error("qknorm_rope_store: head_dim %d not in {64,128,256}", head_dim);
            return B200_ERR_UNSUPPORTED;
    }
#undef B200_LAUNCH_QRS
    B200_CHECK_LAUNCH();
    return B200_OK;
}

}  // namespace b200

extern "C" {

int b200_rope_neox_inplace(void* q, void* k, const float* cos_table, const float* sin_table,
                           const int32_t* positions, int tokens, int q_heads, int k_heads,
                           int head_dim, int rotary_dim, int max_pos, int64_t q_stride_token,
                           int64_t q_stride_head, int64_t k_stride_token, int64_t k_stride_head,
                           b200_stream_t stream) {
    B200_CHECK_ARG(tokens >= 0 && q_heads >= 0 && k_heads >= 0, "rope: negative size");
    if (tokens == 0) return B200_OK;
    B200_CHECK_ARG(cos_table && sin_table && positions, "rope: NULL table or positions");
    B200_CHECK_ARG(rotary_dim % 2 == 0, "rotary_dim must be even");
    B200_CHECK_ARG(rotary_dim > 0 && rotary_dim <= head_dim, "rope: rotary_dim out of range");
    B200_CHECK_ARG(q_heads == 0 || q, "rope: q is NULL");
    B200_CHECK_ARG(k_heads == 0 || k, "rope: k is NULL");
    B200_CHECK_ARG(max_pos > 0, "rope: max_pos must be positive");
    int err = B200_OK;
    int* status = b200::device_status_words(&err);
    if (err != B200_OK) return err;
    const int64_t q_rows = static_cast<int64_t>(tokens) * q_heads;
    const int64_t total = q_rows + static_cast<int64_t>(tokens) * k_heads;
    if (total == 0) return B200_OK;
    const unsigned blocks = static_cast<unsigned>((total + 3) / 4);
    b200::rope_neox_kernel<<<blocks, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k), cos_table, sin_table,
        positions, q_rows, total, q_heads, k_heads, head_dim, rotary_dim, max_pos, q_stride_token,
        q_stride_head, k_stride_token, k_stride_head, status);
    B200_CHECK_LAUNCH();
    return B200_OK;
}

int b200_store_kv(void* k_cache, void* v_cache, const void* k, const void* v,
                  const int32_t* out_loc, int tokens, int kv_heads, int head_dim,
                  int64_t k_stride_token, int64_t v_stride_token, int64_t num_slots,
                  b200_stream_t stream) {
    B200_CHECK_ARG(tokens >= 0 && kv_heads > 0 && head_dim > 0, "store_kv: bad size");
    if (tokens == 0) return B200_OK;
    B200_CHECK_ARG(k_cache && v_cache && k && v && out_loc, "store_kv: NULL tensor");
    const int64_t elems = static_cast<int64_t>(kv_heads) * head_dim;
    B200_CHECK_ARG(elems % 8 == 0 && k_stride_token % 8 == 0 && v_stride_token % 8 == 0,
                   "store_kv: rows must be 16-byte aligned");
    int err = B200_OK;
    int* status = b200::device_status_words(&err);
    if (err != B200_OK) return err;
    if (tokens == 0) return B200_OK;
    const unsigned blocks = static_cast<unsigned>((tokens + 3) / 4);
    b200::store_kv_kernel<<<blocks, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint4*>(k_cache), static_cast<uint4*>(v_cache),
        static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), out_loc, tokens,
        static_cast<int>(elems / 8), k_stride_token, v_stride_token, num_slots, status);
    B200_CHECK_LAUNCH();
    return B200_OK;
}

int b200_qknorm_rope_store(void* qkv, const void* q_weight, const void* k_weight,
                           const float* cos_table, const float* sin_table,
                           const int32_t* positions, const int32_t* out_loc, void* k_cache,
                           void* v_cache, int tokens, int q_heads, int kv_heads, int head_dim,
                           int max_pos, int64_t num_slots, float eps, int write_k_back,
                           b200_stream_t stream) {
    B200_CHECK_ARG(tokens >= 0, "qknorm_rope_store: tokens must be >= 0");
    if (tokens == 0) return B200_OK;
    B200_CHECK_ARG(qkv && cos_table && sin_table && positions && out_loc && k_cache && v_cache,
                   "qknorm_rope_store: NULL tensor");
    B200_CHECK_ARG((q_weight == nullptr) == (k_weight == nullptr),
                   "qknorm_rope_store: q_weight and k_weight must both be set or both be NULL");
    B200_CHECK_ARG(tokens >= 0 && q_heads > 0 && kv_heads > 0, "qknorm_rope_store: bad size");
    B200_CHECK_ARG(max_pos > 0 && num_slots > 0, "qknorm_rope_store: bad table size");
    int err = B200_OK;
    int* status = b200::device_status_words(&err);
    if (err != B200_OK) return err;
    return b200::launch_qknorm_rope_store(qkv, q_weight, k_weight, cos_table, sin_table, positions,
                                          out_loc, k_cache, v_cache, tokens, q_heads, kv_heads,
                                          head_dim, max_pos, num_slots, eps, write_k_back, status,
                                          static_cast<cudaStream_t>(stream));
}

}  // extern "C"
