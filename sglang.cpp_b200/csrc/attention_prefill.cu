// Paged-KV causal prefill (extend) attention with ragged queries.
//
// One CTA owns (request, KV head, block of 128/G query tokens), G = q_heads /
// kv_heads: its 128 accumulator rows are (token, head-in-group) pairs that all
// read the same KV head, so every K/V byte staged in shared memory feeds all G
// query heads.  A producer warp streams 64-key tiles of that head through a
// 4-stage ring with TMA (3-D tensor map [128, kv_heads, slots], box [64, 1,
// keys-per-copy], 128-byte swizzle); eight consumer warps hold 16 rows each and
// run S = Q K^T, online softmax and O += P V with mma.sync m16n8k16 + ldmatrix.
// Queries are the LAST extend_len positions of the request, so tiles left of
// the diagonal need no mask and tiles right of it are never loaded.
#include "common.cuh"
#include "kernels.h"
#include "tensormap.cuh"

namespace b200 {
namespace {

constexpr int kD = 128;
constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kTileKeys = 64;
constexpr uint32_t kHalfBytes = kTileKeys * 128;   // 8 KB: 64 keys x 64 elements
constexpr uint32_t kStageBytes = 4 * kHalfBytes;   // K lo, K hi, V lo, V hi
constexpr int kStages = 4;

struct PrefillParams {
    __nv_bfloat16* out;
    const __nv_bfloat16* q;
    int64_t q_st, q_sh;
    const int32_t* page_table;
    int64_t pt_stride;
    const int32_t* table_idx;
    const int32_t* seq_lens;
    const int32_t* qo_indptr;
    int q_heads, kv_heads, group;
    int kpc;  // keys per TMA copy = min(page_size, 64)
    int64_t num_slots;
    float scale_log2;
    int* status;
};

__global__ void __launch_bounds__(kThreads, 1)
attention_prefill_kernel(const __grid_constant__ CUtensorMap tmap_k,
                         const __grid_constant__ CUtensorMap tmap_v, const PrefillParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kStages];
    __shared__ __align__(8) uint64_t empty_bar[kStages];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int G = p.group;
    const int QB = 128 / G;  // query tokens per CTA

    const int b = blockIdx.z;
    const int h = blockIdx.y;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), kConsumerWarps);
        }
        fence_mbar_init();
    }
    // Clear the ring once so that rows no copy ever wrote cannot hold NaN patterns.
    {
        uint4* z = reinterpret_cast<uint4*>(smem_raw + (smem_base - smem_u32(smem_raw)));
        for (uint32_t i = threadIdx.x; i < kStages * kStageBytes / 16; i += kThreads)
            z[i] = make_uint4(0, 0, 0, 0);
        fence_proxy_async_smem();
    }
    pdl_launch_dependents();
    pdl_wait_prior();
    __syncthreads();

    const int q_begin = p.qo_indptr[b];
    const int ext = p.qo_indptr[b + 1] - q_begin;
    const int len = p.seq_lens[b];
    const int nqb = (ext + QB - 1) / QB;
    // Heaviest blocks (the last tokens) are scheduled first.
    const int qb = nqb - 1 - static_cast<int>(blockIdx.x);
    if (qb < 0 || ext <= 0 || len <= 0) return;
    const int t0 = qb * QB;                       // first query token of this block
    const int t1 = min(t0 + QB, ext);
    const int pos0 = len - ext;                   // position of query token 0
    const int kv_end = min(len, pos0 + t1);       // keys [0, kv_end) are visible to this block
    const int ntiles = (kv_end + kTileKeys - 1) / kTileKeys;

    if (warp == kConsumerWarps) {
        // ================= producer =================
        const int32_t* pt_row = p.page_table + static_cast<int64_t>(p.table_idx[b]) * p.pt_stride;
        const uint32_t copy_bytes = static_cast<uint32_t>(p.kpc) * 128u;
        for (int kt = 0; kt < ntiles; ++kt) {
            const uint32_t slot = kt % kStages;
            const uint32_t parity = ((kt / kStages) & 1u) ^ 1u;
            if (!mbar_wait_bounded(smem_u32(&empty_bar[slot]), parity, p.status, 301)) return;
            const int k0 = kt * kTileKeys;
            const int valid = min(kTileKeys, kv_end - k0);
            const int ncopies = (valid + p.kpc - 1) / p.kpc;
            const uint32_t bar = smem_u32(&full_bar[slot]);
            if (lane == 0) mbar_arrive_expect_tx(bar, static_cast<uint32_t>(ncopies) * 4u * copy_bytes);
            __syncwarp();
            const uint32_t stage_base = smem_base + slot * kStageBytes;
            for (int ci = lane; ci < ncopies * 4; ci += 32) {
                const int copy = ci >> 2, which = ci & 3;
                int64_t sl = pt_row[k0 + copy * p.kpc];
                if (sl < 0 || sl + p.kpc > p.num_slots) {
                    atomicExch(&p.status[kStatusBadIndex], static_cast<int>(sl) + 1);
                    sl = 0;
                }
                tma_load_3d(stage_base + which * kHalfBytes + copy * copy_bytes,
                            which < 2 ? &tmap_k : &tmap_v, (which & 1) * 64, h, static_cast<int>(sl), bar);
            }
        }
        return;
    }

    // ================= consumers =================
    const int g = lane >> 2, t = lane & 3;
    const int mi = lane >> 3, r8 = lane & 7;
    // Rows of this warp: r = warp*16 + {g, g+8}; token = t0 + r / G; head = h*G + r % G.
    const int ra = warp * 16 + g, rb = ra + 8;
    const int tok_a = t0 + ra / G, tok_b = t0 + rb / G;
    const bool va = tok_a < t1, vb = tok_b < t1;
    const int head_a = h * G + ra % G, head_b = h * G + rb % G;
    const int pos_a = pos0 + tok_a, pos_b = pos0 + tok_b;  // last visible key of each row

    uint32_t qa[8][4];
    {
        const __nv_bfloat16* qa_ptr = p.q + static_cast<int64_t>(q_begin + tok_a) * p.q_st + head_a * p.q_sh;
        const __nv_bfloat16* qb_ptr = p.q + static_cast<int64_t>(q_begin + tok_b) * p.q_st + head_b * p.q_sh;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            const int d0 = ks * 16 + 2 * t;
            qa[ks][0] = va ? *reinterpret_cast<const uint32_t*>(qa_ptr + d0) : 0u;
            qa[ks][2] = va ? *reinterpret_cast<const uint32_t*>(qa_ptr + d0 + 8) : 0u;
            qa[ks][1] = vb ? *reinterpret_cast<const uint32_t*>(qb_ptr + d0) : 0u;
            qa[ks][3] = vb ? *reinterpret_cast<const uint32_t*>(qb_ptr + d0 + 8) : 0u;
        }
    }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    // Last key any row of this warp may see; tiles past it are skipped by the warp.
    const int warp_last_tok = min(t0 + (warp * 16 + 15) / G, t1 - 1);
    const int warp_kv_end = pos0 + warp_last_tok + 1;
    const int warp_first_pos = pos0 + t0 + (warp * 16) / G;
    bool failed = false;

    for (int kt = 0; kt < ntiles; ++kt) {
        const uint32_t slot = kt % kStages;
        const uint32_t parity = (kt / kStages) & 1u;
        if (!failed && !mbar_wait_bounded(smem_u32(&full_bar[slot]), parity, p.status, 302)) failed = true;
        const int k0 = kt * kTileKeys;
        if (!failed && k0 < warp_kv_end) {
            const uint32_t stage_base = smem_base + slot * kStageBytes;
            const int valid = min(kTileKeys, kv_end - k0);
            if (valid < kTileKeys) {
                for (int i = lane; i < (kTileKeys - valid) * 16; i += 32) {
                    const int j = valid + (i >> 4), c16 = i & 15;
                    const uint32_t a = stage_base + (2 + (c16 >> 3)) * kHalfBytes + j * 128u + (c16 & 7) * 16u;
                    asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(a), "r"(0u) : "memory");
                }
                fence_proxy_async_smem();
                __syncwarp();
            }
            const bool need_mask = (k0 + kTileKeys - 1 > warp_first_pos) || valid < kTileKeys;

            float s[8][4];
#pragma unroll
            for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {  // 16 keys per step
                const int j = kk * 16 + (mi >> 1) * 8 + r8;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const int c16 = ks * 2 + (mi & 1);
                    const uint32_t row_addr = stage_base + (c16 >> 3) * kHalfBytes + j * 128u;
                    uint32_t b00, b01, b10, b11;
                    ldmatrix_x4(swz128(row_addr, c16 & 7), b00, b01, b10, b11);
                    mma_bf16_16816(s[2 * kk], qa[ks], b00, b01);
                    mma_bf16_16816(s[2 * kk + 1], qa[ks], b10, b11);
                }
            }
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int n = 0; n < 8; ++n) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float v = s[n][e] * p.scale_log2;
                    if (need_mask) {
                        const int key = k0 + n * 8 + 2 * t + (e & 1);
                        const int lim = (e < 2) ? pos_a : pos_b;
                        if (key > lim || key >= kv_end) v = -INFINITY;
                    }
                    s[n][e] = v;
                    if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
                }
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            // A row can be fully masked in a tile (its diagonal lies left of the
            // tile): keep the running max finite-safe so exp2 never sees inf - inf.
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
            const float ms0 = mn0 == -INFINITY ? 0.f : mn0;
            const float ms1 = mn1 == -INFINITY ? 0.f : mn1;
            const float al0 = exp2f(m0 - ms0), al1 = exp2f(m1 - ms1);
            m0 = mn0;
            m1 = mn1;
            float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                s[n][0] = exp2f(s[n][0] - ms0);
                s[n][1] = exp2f(s[n][1] - ms0);
                s[n][2] = exp2f(s[n][2] - ms1);
                s[n][3] = exp2f(s[n][3] - ms1);
                sum0 += s[n][0] + s[n][1];
                sum1 += s[n][2] + s[n][3];
            }
            l0 = l0 * al0 + sum0;
            l1 = l1 * al1 + sum1;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                o[i][0] *= al0;
                o[i][1] *= al0;
                o[i][2] *= al1;
                o[i][3] *= al1;
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                uint32_t pa[4];
                pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
                pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
                const int j = kk * 16 + (mi & 1) * 8 + r8;
#pragma unroll
                for (int np = 0; np < 8; ++np) {
                    const int c16 = np * 2 + (mi >> 1);
                    const uint32_t row_addr = stage_base + (2 + (c16 >> 3)) * kHalfBytes + j * 128u;
                    uint32_t v0, v1, v2, v3;
                    ldmatrix_x4_trans(swz128(row_addr, c16 & 7), v0, v1, v2, v3);
                    mma_bf16_16816(o[2 * np], pa, v0, v1);
                    mma_bf16_16816(o[2 * np + 1], pa, v2, v3);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&empty_bar[slot]));
    }

    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const int Hq = p.q_heads;
    if (va) {
        const float inv = l0 > 0.f ? 1.f / l0 : 0.f;
        __nv_bfloat16* dst = p.out + (static_cast<int64_t>(q_begin + tok_a) * Hq + head_a) * kD;
#pragma unroll
        for (int i = 0; i < 16; ++i)
            *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t) = pack_bf16(o[i][0] * inv, o[i][1] * inv);
    }
    if (vb) {
        const float inv = l1 > 0.f ? 1.f / l1 : 0.f;
        __nv_bfloat16* dst = p.out + (static_cast<int64_t>(q_begin + tok_b) * Hq + head_b) * kD;
#pragma unroll
        for (int i = 0; i < 16; ++i)
            *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t) = pack_bf16(o[i][2] * inv, o[i][3] * inv);
    }
}

int make_kv_tmap_3d(CUtensorMap* out, const void* cache, int64_t num_slots, int kv_heads, int kpc) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) {
        set_last_error("cuTensorMapEncodeTiled is not available from this driver");
        return B200_ERR_CUDA;
    }
    const cuuint64_t dims[3] = {kD, static_cast<cuuint64_t>(kv_heads), static_cast<cuuint64_t>(num_slots)};
    const cuuint64_t strides[2] = {kD * 2, static_cast<cuuint64_t>(kv_heads) * kD * 2};
    const cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(kpc)};
    const cuuint32_t es[3] = {1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(cache), dims, strides,
                    box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_last_error("cuTensorMapEncodeTiled (3-D KV map) failed with CUresult %d", static_cast<int>(r));
        return B200_ERR_CUDA;
    }
    return B200_OK;
}

}  // namespace

int launch_attention_prefill(void* out, const void* q, int64_t q_st, int64_t q_sh, const void* k_cache,
                             const void* v_cache, int64_t num_slots, const int32_t* page_table,
                             int64_t pt_stride, const int32_t* table_idx, const int32_t* seq_lens,
                             const int32_t* qo_indptr, int batch, int max_extend_len, int q_heads,
                             int kv_heads, int page_size, float sm_scale, int* status,
                             cudaStream_t stream) {
    if (batch == 0 || max_extend_len == 0) return B200_OK;
    // The tensor-core kernel takes every call with 16-byte aligned query rows; the mma.sync kernel
    // below stays for the rest (and for comparison: B200_PREFILL_ATTN=mma).
    static const char choice = [] {
        const char* v = getenv("B200_PREFILL_ATTN");   // "mma": legacy path; "tc": one query tile per CTA
        return v && v[0] ? v[0] : ' ';
    }();
    const bool force_mma = choice == 'm';
    // Two query tiles per CTA (attention_prefill_tc2.cu) once a request can fill more than one tile.
    if (!force_mma && choice != 't' && attention_prefill_tc_supported(q, q_st, q_sh, out) &&
        max_extend_len > 128 / (q_heads / kv_heads))
        return launch_attention_prefill_tc2(out, q, q_st, q_sh, k_cache, v_cache, num_slots, page_table, pt_stride,
                                            table_idx, seq_lens, qo_indptr, batch, max_extend_len, q_heads,
                                            kv_heads, page_size, sm_scale, status, stream);
    if (!force_mma && attention_prefill_tc_supported(q, q_st, q_sh, out))
        return launch_attention_prefill_tc(out, q, q_st, q_sh, k_cache, v_cache, num_slots, page_table, pt_stride,
                                           table_idx, seq_lens, qo_indptr, batch, max_extend_len, q_heads,
                                           kv_heads, page_size, sm_scale, status, stream);
    PrefillParams p;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.q_st = q_st;
    p.q_sh = q_sh;
    p.page_table = page_table;
    p.pt_stride = pt_stride;
    p.table_idx = table_idx;
    p.seq_lens = seq_lens;
    p.qo_indptr = qo_indptr;
    p.q_heads = q_heads;
    p.kv_heads = kv_heads;
    p.group = q_heads / kv_heads;
    p.kpc = page_size < kTileKeys ? page_size : kTileKeys;
    p.num_slots = num_slots;
    p.scale_log2 = sm_scale * 1.4426950408889634f;
    p.status = status;
    CUtensorMap tk, tv;
    int err = make_kv_tmap_3d(&tk, k_cache, num_slots, kv_heads, p.kpc);
    if (err != B200_OK) return err;
    err = make_kv_tmap_3d(&tv, v_cache, num_slots, kv_heads, p.kpc);
    if (err != B200_OK) return err;
    const int QB = 128 / p.group;
    const int smem = kStages * kStageBytes + 1024;
    B200_CHECK_CUDA(cudaFuncSetAttribute(attention_prefill_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    dim3 grid(div_ceil(max_extend_len, QB), kv_heads, batch);
    B200_CHECK_CUDA(launch_kernel(attention_prefill_kernel, grid, dim3(kThreads), smem, stream,
                                  dim3(1, 1, 1), tk, tv, p));
    return B200_OK;
}

}  // namespace b200

extern "C" {

int b200_attention_prefill(void* out, const void* q, int64_t q_stride_token, int64_t q_stride_head,
                           const void* k_cache, const void* v_cache, int64_t num_slots,
                           const int32_t* page_table, int64_t page_table_stride,
                           const int32_t* table_idx, const int32_t* seq_lens,
                           const int32_t* qo_indptr, int batch, int max_extend_len, int q_heads,
                           int kv_heads, int head_dim, int page_size, float sm_scale,
                           b200_stream_t stream) {
    B200_CHECK_ARG(batch == 0 || max_extend_len == 0 ||
                       (out && q && k_cache && v_cache && page_table && table_idx && seq_lens && qo_indptr),
                   "attention_prefill: NULL tensor");
    B200_CHECK_ARG(head_dim == b200::kD, "attention_prefill: head_dim must be 128");
    B200_CHECK_ARG(batch >= 0 && batch <= 65535, "attention_prefill: batch must be in [0, 65535]");
    B200_CHECK_ARG(kv_heads >= 1 && q_heads % kv_heads == 0, "attention_prefill: q_heads must be a multiple of kv_heads");
    const int group = q_heads / kv_heads;
    B200_CHECK_ARG(group <= 16 && (group & (group - 1)) == 0,
                   "attention_prefill: group size must be a power of two <= 16");
    B200_CHECK_ARG(page_size >= 1 && (page_size & (page_size - 1)) == 0,
                   "attention_prefill: page_size must be a power of two");
    B200_CHECK_ARG(q_stride_token % 2 == 0 && q_stride_head % 2 == 0,
                   "attention_prefill: q strides must be even");
    B200_CHECK_ARG(max_extend_len >= 0 && num_slots > 0, "attention_prefill: bad size");
    int err = B200_OK;
    int* status = b200::device_status_words(&err);
    if (err != B200_OK) return err;
    return b200::launch_attention_prefill(out, q, q_stride_token, q_stride_head, k_cache, v_cache,
                                          num_slots, page_table, page_table_stride, table_idx,
                                          seq_lens, qo_indptr, batch, max_extend_len, q_heads,
                                          kv_heads, page_size, sm_scale, status,
                                          static_cast<cudaStream_t>(stream));
}

}  // extern "C"
