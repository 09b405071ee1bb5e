// Paged-KV causal prefill (extend) attention on the tcgen05 tensor cores.
//
// One CTA owns (request, KV head, block of 128/G query tokens), G = q_heads / kv_heads: its 128
// rows are (token, head-in-group) pairs that read the same KV head.  Roles:
//   warp 0      producer: 128-key K/V tiles through a 2-stage TMA ring (3-D tensor map
//               [128, kv_heads, slots], box [64, 1, keys-per-copy], 128-byte swizzle);
//   warp 1      one thread issues the MMAs: S = Q K^T (128 x 128 x 128, accumulator in TMEM,
//               two S buffers so the next tile's S is computed while this tile's softmax runs)
//               and PV = P V (V consumed MN-major, straight from the layout TMA delivers);
//   warps 2-9   two threads per query row (thread pair = TMEM lane; warps w and w+4 share a lane
//               quarter and take keys / head-dim columns 0-63 and 64-127): read S, online softmax
//               in the log2 domain (row maxima meet in shared memory), write P (bf16) into shared
//               memory in the swizzled K-major layout the MMA reads, then fold PV into the row's
//               output accumulator in registers.
// Queries are the LAST extend_len positions of the request, so tiles left of the diagonal need
// no mask and tiles right of it are never loaded.
#include "common.cuh"
#include "kernels.h"
#include "tcgen05.cuh"
#include "tensormap.cuh"

namespace b200 {
namespace {

constexpr int kD = 128;
constexpr int kTile = 128;                  // keys per K/V tile and query rows per CTA
constexpr int kThreads = 320;  // producer, MMA issuer, 8 softmax warps
constexpr uint32_t kAtomBytes = 128 * 128;  // 128 rows x 64 bf16: one swizzle atom column
constexpr uint32_t kQOff = 0;               // Q: 2 atoms (d 0-63, d 64-127)
constexpr uint32_t kPOff = 2 * kAtomBytes;  // P: 2 atoms (keys 0-63, 64-127)
constexpr uint32_t kKVOff = 4 * kAtomBytes; // ring: per stage K lo, K hi, V lo, V hi
constexpr uint32_t kStageBytes = 4 * kAtomBytes;
constexpr int kStages = 2;
constexpr uint32_t kSmemBytes = kKVOff + kStages * kStageBytes;
constexpr uint32_t kColS = 0, kColPV = 256;  // TMEM columns: S0, S1 (128 each), PV (128)

struct PrefillTcParams {
    __nv_bfloat16* out;
    const __nv_bfloat16* q;
    int64_t q_st, q_sh;
    const int32_t* page_table;
    int64_t pt_stride;
    const int32_t* table_idx;
    const int32_t* seq_lens;
    const int32_t* qo_indptr;
    int q_heads, kv_heads, group;
    int kpc;  // keys per TMA copy = min(page_size, 128)
    int whole_tile_boxes;  // the *_tile tensor maps copy 128 keys at once (kpc < 128 <= num_slots)
    int64_t num_slots;
    float scale_log2;
    int* status;
};

// MN-major operand under the 128-byte swizzle (V as the B operand of P V: rows are keys, 64
// head-dim elements per 128-byte row): 8-key groups 1024 bytes apart along K, the second 64
// head-dim elements one atom (16 KB) further.
__device__ __forceinline__ uint64_t mnmajor_sw128_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
    d |= static_cast<uint64_t>(kAtomBytes >> 4) << 16;  // leading byte offset: next 64 elements along N
    d |= static_cast<uint64_t>(1024 >> 4) << 32;        // stride byte offset: next 8 rows along K
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
// bf16 x bf16 -> fp32, M = 128, N = 128; A K-major, B K-major or MN-major.
__device__ __forceinline__ uint32_t idesc_128x128(bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) |
           (static_cast<uint32_t>(128 >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
}

__global__ void __launch_bounds__(kThreads, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap_k,
                            const __grid_constant__ CUtensorMap tmap_v,
                            const __grid_constant__ CUtensorMap tmap_k_tile,
                            const __grid_constant__ CUtensorMap tmap_v_tile, const PrefillTcParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t k_full[kStages];   // K and V have rings of their own: a K tile
    __shared__ __align__(8) uint64_t k_empty[kStages];  // is free as soon as its S = Q K^T is done,
    __shared__ __align__(8) uint64_t v_full[kStages];   // so the next K load does not wait for P V
    __shared__ __align__(8) uint64_t v_empty[kStages];
    __shared__ __align__(8) uint64_t s_full[2];
    __shared__ __align__(8) uint64_t p_full;
    __shared__ __align__(8) uint64_t pv_full;
    __shared__ uint32_t tmem_base_slot;
    __shared__ float s_max[2][2][kTile];   // [tile parity][column half][row]: row maxima of each half
    __shared__ float s_sum[2][kTile];      // [column half][row]: final partial row sums

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const int G = p.group;
    const int QB = kTile / G;  // query tokens per CTA
    const int b = blockIdx.z;
    const int h = blockIdx.y;

    pdl_launch_dependents();
    pdl_wait_prior();

    const int q_begin = p.qo_indptr[b];
    const int ext = p.qo_indptr[b + 1] - q_begin;
    const int len = p.seq_lens[b];
    const int nqb = (ext + QB - 1) / QB;
    const int qb = nqb - 1 - static_cast<int>(blockIdx.x);  // heaviest blocks first
    if (qb < 0 || ext <= 0 || len <= 0) return;             // whole CTA, before any barrier or TMEM use
    const int t0 = qb * QB;
    const int t1 = min(t0 + QB, ext);
    const int pos0 = len - ext;                   // position of query token 0
    const int kv_end = min(len, pos0 + t1);       // keys [0, kv_end) are visible to this block
    const int ntiles = (kv_end + kTile - 1) / kTile;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&k_full[s]), 1);
            mbar_init(smem_u32(&k_empty[s]), 1);
            mbar_init(smem_u32(&v_full[s]), 1);
            mbar_init(smem_u32(&v_empty[s]), 1);
        }
        mbar_init(smem_u32(&s_full[0]), 1);
        mbar_init(smem_u32(&s_full[1]), 1);
        mbar_init(smem_u32(&p_full), 8);   // one arrival per softmax warp
        mbar_init(smem_u32(&pv_full), 1);
        fence_mbar_init();
    }
    // Clear the ring once so that rows no copy ever wrote cannot hold NaN patterns.
    {
        uint4* z = reinterpret_cast<uint4*>(smem_gen + kKVOff);
        for (uint32_t i = threadIdx.x; i < kStages * kStageBytes / 16; i += kThreads)
            z[i] = make_uint4(0, 0, 0, 0);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), 512);
        tmem_relinquish();
    }
    // Q rows into shared memory in the swizzled K-major layout: row r = (token t0 + r / G,
    // head h * G + r % G); rows past the request's last token are zero.
    if (warp >= 2) {
        const int r = ((warp - 2) & 3) * 32 + lane;
        const int half = (warp - 2) >> 2;
        const int tok = t0 + r / G;
        const int head = h * G + r % G;
        const uint4* src = reinterpret_cast<const uint4*>(p.q + static_cast<int64_t>(q_begin + tok) * p.q_st +
                                                          static_cast<int64_t>(head) * p.q_sh);
        const bool valid = tok < t1;
#pragma unroll
        for (int c = half * 8; c < half * 8 + 8; ++c) {
            const uint4 v = valid ? src[c] : make_uint4(0, 0, 0, 0);
            const uint32_t row_addr = smem_base + kQOff + (c >> 3) * kAtomBytes + r * 128;
            const uint32_t a = swz128(row_addr, c & 7);
            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                         : "memory");
        }
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        // ================= producer =================
        const int32_t* pt_row = p.page_table + static_cast<int64_t>(p.table_idx[b]) * p.pt_stride;
        const uint32_t copy_bytes = static_cast<uint32_t>(p.kpc) * 128u;
        bool failed = false;
        for (int kt = 0; kt < ntiles && !failed; ++kt) {
            const uint32_t slot = kt % kStages;
            const uint32_t parity = static_cast<uint32_t>(kt / kStages - 1) & 1u;
            const int k0 = kt * kTile;
            const int valid = min(kTile, kv_end - k0);
            const int ncopies = (valid + p.kpc - 1) / p.kpc;
            const uint32_t stage_base = smem_base + kKVOff + slot * kStageBytes;
            // first slot of this lane's copies (copy = lane, lane + 32, ...: up to 128 with page size 1)
            int sl[4] = {0, 0, 0, 0};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int copy = i * 32 + lane;
                if (copy < ncopies) {
                    int64_t v = pt_row[k0 + copy * p.kpc];
                    if (v < 0 || v + p.kpc > p.num_slots) {
                        atomicExch(&p.status[kStatusBadIndex], static_cast<int>(v) + 1);
                        v = 0;
                    }
                    sl[i] = static_cast<int>(v);
                }
            }
            // A tile whose pages are consecutive slots (the usual outcome of allocating a prompt's
            // pages in one go) is fetched with two 128-key boxes per tensor instead of two per page.
            bool mine = true;
            const int first = __shfl_sync(0xffffffffu, sl[0], 0);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int copy = i * 32 + lane;
                if (copy < ncopies && sl[i] != first + copy * p.kpc) mine = false;
            }
            const bool whole = __all_sync(0xffffffffu, mine) && valid == kTile && p.whole_tile_boxes;
#pragma unroll
            for (int kv = 0; kv < 2; ++kv) {   // 0: K tile, 1: V tile
                if (kt >= kStages &&
                    !mbar_wait_bounded(smem_u32(kv == 0 ? &k_empty[slot] : &v_empty[slot]), parity, p.status, 311)) {
                    failed = true;
                    break;
                }
                const uint32_t bar = smem_u32(kv == 0 ? &k_full[slot] : &v_full[slot]);
                if (lane == 0) mbar_arrive_expect_tx(bar, static_cast<uint32_t>(ncopies) * 2u * copy_bytes);
                __syncwarp();
                if (whole) {
                    if (lane < 2)
                        tma_load_3d(stage_base + (kv * 2 + lane) * kAtomBytes, kv == 0 ? &tmap_k_tile : &tmap_v_tile,
                                    lane * 64, h, first, bar);
                    continue;
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int copy = i * 32 + lane;
                    if (copy < ncopies) {
                        const uint32_t dst = stage_base + kv * 2 * kAtomBytes + copy * copy_bytes;
                        tma_load_3d(dst, kv == 0 ? &tmap_k : &tmap_v, 0, h, sl[i], bar);
                        tma_load_3d(dst + kAtomBytes, kv == 0 ? &tmap_k : &tmap_v, 64, h, sl[i], bar);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        if (lane == 0) {
            const uint32_t idesc_s = idesc_128x128(false);
            const uint32_t idesc_pv = idesc_128x128(true);
            const uint32_t q_addr = smem_base + kQOff, p_addr = smem_base + kPOff;
            bool failed = false;
            auto issue_s = [&](int kt) {
                const uint32_t slot = kt % kStages;
                if (!mbar_wait_bounded(smem_u32(&k_full[slot]), static_cast<uint32_t>(kt / kStages) & 1u,
                                       p.status, 312)) {
                    failed = true;
                    return;
                }
                tc_fence_after();
                const uint32_t k_addr = smem_base + kKVOff + slot * kStageBytes;
                const uint32_t d = tmem_base + kColS + static_cast<uint32_t>(kt & 1) * 128u;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t off = (ks >> 2) * kAtomBytes + (ks & 3) * 32;
                    tc_mma_bf16(d, kmajor_sw128_desc(q_addr + off), kmajor_sw128_desc(k_addr + off), idesc_s,
                                ks > 0 ? 1u : 0u);
                }
                tc_commit(smem_u32(&s_full[kt & 1]));
                tc_commit(smem_u32(&k_empty[slot]));
            };
            issue_s(0);
            for (int kt = 0; kt < ntiles && !failed; ++kt) {
                if (kt + 1 < ntiles) issue_s(kt + 1);
                if (failed) break;
                const uint32_t slot = kt % kStages;
                if (!mbar_wait_bounded(smem_u32(&v_full[slot]), static_cast<uint32_t>(kt / kStages) & 1u, p.status, 316))
                    break;
                if (!mbar_wait_bounded(smem_u32(&p_full), static_cast<uint32_t>(kt) & 1u, p.status, 313)) break;
                tc_fence_after();
                const uint32_t v_addr = smem_base + kKVOff + slot * kStageBytes + 2 * kAtomBytes;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    // keys ks*16 .. +15: P columns inside atom ks/4; V rows 2048 bytes further per step
                    const uint32_t p_off = (ks >> 2) * kAtomBytes + (ks & 3) * 32;
                    tc_mma_bf16(tmem_base + kColPV, kmajor_sw128_desc(p_addr + p_off),
                                mnmajor_sw128_desc(v_addr + ks * 2048), idesc_pv, ks > 0 ? 1u : 0u);
                }
                tc_commit(smem_u32(&pv_full));
                tc_commit(smem_u32(&v_empty[slot]));
            }
        }
    } else {
        // ================= softmax / output rows =================
        const int qtr = warp & 3;                 // TMEM lane quarter this warp may read
        const int half = (warp - 2) >> 2;         // keys / head-dim columns [64*half, 64*half + 64)
        const int r = qtr * 32 + lane;            // query row = TMEM lane
        const int tok = t0 + r / G;
        const int head = h * G + r % G;
        const int limit = min(pos0 + tok, len - 1);   // last visible key of this row
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(qtr * 32) << 16) + static_cast<uint32_t>(half * 64);
        const float sc = p.scale_log2;
        float m_run = -INFINITY, l_run = 0.f;
        float o[64];
#pragma unroll
        for (int i = 0; i < 64; ++i) o[i] = 0.f;
        bool failed = false;
        auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + qtr) : "memory"); };
        auto ex2 = [](float x) {
            float y;
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
            return y;
        };
        const uint32_t p_row_addr = smem_base + kPOff + half * kAtomBytes + r * 128;
        uint32_t packed[32];    // this thread's 64 probabilities of the tile being prepared (bf16 pairs)
        float alpha_pending = 1.f;  // rescale factor that goes with the P V product not folded in yet

        // Scores of tile kt -> probabilities in `packed`, running max / sum updated; returns the factor
        // by which everything accumulated before this tile shrinks.  Every thread meets its partner at
        // the pair barrier once per call, also after a wait has run out (the output is then discarded).
        auto softmax_tile = [&](int kt) -> float {
            if (!failed && !mbar_wait_bounded(smem_u32(&s_full[kt & 1]), static_cast<uint32_t>(kt >> 1) & 1u,
                                              p.status, 314))
                failed = true;
            tc_fence_after();
            const uint32_t s_addr = lane_addr + kColS + static_cast<uint32_t>(kt & 1) * 128u;
            const int k0 = kt * kTile + half * 64;    // first key of this thread's columns
            const bool need_mask = k0 + 63 > limit;
            uint32_t sv[2][32];
            tmem_ld_32x32b_x32(s_addr, sv[0]);
            tmem_ld_32x32b_x32(s_addr + 32, sv[1]);
            tmem_ld_wait();
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                if (need_mask) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (k0 + c * 32 + i <= limit) mx = fmaxf(mx, __uint_as_float(sv[c][i]));
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(sv[c][i]));
                }
            }
            s_max[kt & 1][half][r] = mx;
            pair_sync();
            mx = fmaxf(mx, s_max[kt & 1][half ^ 1][r]);
            const float m_new = fmaxf(m_run, mx);
            const float alpha = m_new == -INFINITY ? 1.f : ex2((m_run - m_new) * sc);
            const float mb = m_new == -INFINITY ? 0.f : m_new * sc;
            float sum = 0.f;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float p0 = ex2(fmaf(__uint_as_float(sv[c][i]), sc, -mb));
                    float p1 = ex2(fmaf(__uint_as_float(sv[c][i + 1]), sc, -mb));
                    if (need_mask) {
                        if (k0 + c * 32 + i > limit) p0 = 0.f;
                        if (k0 + c * 32 + i + 1 > limit) p1 = 0.f;
                    }
                    sum += p0 + p1;
                    packed[c * 16 + (i >> 1)] = pack_bf16(p0, p1);
                }
            }
            l_run = l_run * alpha + sum;
            m_run = m_new;
            return alpha;
        };
        // `packed` -> this half's atom of P in shared memory, then tell the MMA thread.
        auto publish_p = [&]() {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t a = swz128(p_row_addr, j);
                asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(packed[4 * j]),
                             "r"(packed[4 * j + 1]), "r"(packed[4 * j + 2]), "r"(packed[4 * j + 3])
                             : "memory");
            }
            fence_proxy_async_smem();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&p_full));
        };

        // Software pipeline: the probabilities of tile kt+1 are computed while the tensor core runs
        // P V of tile kt; P of tile kt+1 is stored once that product has released the P buffer.
        alpha_pending = softmax_tile(0);
        publish_p();
        for (int kt = 0; kt < ntiles; ++kt) {
            float alpha_next = 1.f;
            if (kt + 1 < ntiles) alpha_next = softmax_tile(kt + 1);
            if (!failed && !mbar_wait_bounded(smem_u32(&pv_full), static_cast<uint32_t>(kt) & 1u, p.status, 315))
                failed = true;
            tc_fence_after();
            {
                uint32_t pv[2][32];
                tmem_ld_32x32b_x32(lane_addr + kColPV, pv[0]);
                tmem_ld_32x32b_x32(lane_addr + kColPV + 32, pv[1]);
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 2; ++c) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        o[c * 32 + i] = fmaf(o[c * 32 + i], alpha_pending, __uint_as_float(pv[c][i]));
                }
            }
            tc_fence_before();
            if (kt + 1 < ntiles) publish_p();
            alpha_pending = alpha_next;
        }
        // the row's normaliser is the sum of the two halves' partial sums (same alpha sequence)
        s_sum[half][r] = l_run;
        pair_sync();
        const float l_tot = l_run + s_sum[half ^ 1][r];
        if (!failed && tok < t1) {
            const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
            uint4* dst = reinterpret_cast<uint4*>(p.out + (static_cast<int64_t>(q_begin + tok) * p.q_heads + head) * kD +
                                                  half * 64);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                uint4 w;
                w.x = pack_bf16(o[c * 8 + 0] * inv, o[c * 8 + 1] * inv);
                w.y = pack_bf16(o[c * 8 + 2] * inv, o[c * 8 + 3] * inv);
                w.z = pack_bf16(o[c * 8 + 4] * inv, o[c * 8 + 5] * inv);
                w.w = pack_bf16(o[c * 8 + 6] * inv, o[c * 8 + 7] * inv);
                dst[c] = w;
            }
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

int make_kv_tmap_3d_tc(CUtensorMap* out, const void* cache, int64_t num_slots, int kv_heads, int kpc) {
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

// True when the tensor-core kernel can take the call: 16-byte aligned query rows.
bool attention_prefill_tc_supported(const void* q, int64_t q_st, int64_t q_sh, const void* out) {
    return (reinterpret_cast<uintptr_t>(q) & 15u) == 0 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0 &&
           q_st % 8 == 0 && q_sh % 8 == 0;
}

int launch_attention_prefill_tc(void* out, const void* q, int64_t q_st, int64_t q_sh, const void* k_cache,
                                const void* v_cache, int64_t num_slots, const int32_t* page_table,
                                int64_t pt_stride, const int32_t* table_idx, const int32_t* seq_lens,
                                const int32_t* qo_indptr, int batch, int max_extend_len, int q_heads,
                                int kv_heads, int page_size, float sm_scale, int* status,
                                cudaStream_t stream) {
    if (batch == 0 || max_extend_len == 0) return B200_OK;
    PrefillTcParams p;
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
    p.kpc = page_size < kTile ? page_size : kTile;
    p.num_slots = num_slots;
    p.scale_log2 = sm_scale * 1.4426950408889634f;
    p.status = status;
    CUtensorMap tk, tv;
    int err = make_kv_tmap_3d_tc(&tk, k_cache, num_slots, kv_heads, p.kpc);
    if (err != B200_OK) return err;
    err = make_kv_tmap_3d_tc(&tv, v_cache, num_slots, kv_heads, p.kpc);
    if (err != B200_OK) return err;
    CUtensorMap tk_tile, tv_tile;   // 128-key boxes for tiles whose pages are consecutive slots
    const int tile_box = num_slots >= kTile ? kTile : p.kpc;
    p.whole_tile_boxes = (tile_box == kTile && p.kpc < kTile) ? 1 : 0;
    err = make_kv_tmap_3d_tc(&tk_tile, k_cache, num_slots, kv_heads, tile_box);
    if (err != B200_OK) return err;
    err = make_kv_tmap_3d_tc(&tv_tile, v_cache, num_slots, kv_heads, tile_box);
    if (err != B200_OK) return err;
    const int QB = kTile / p.group;
    const int smem = kSmemBytes + 1024;
    B200_CHECK_CUDA(cudaFuncSetAttribute(attention_prefill_tc_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    dim3 grid(div_ceil(max_extend_len, QB), kv_heads, batch);
    B200_CHECK_CUDA(launch_kernel(attention_prefill_tc_kernel, grid, dim3(kThreads), smem, stream,
                                  dim3(1, 1, 1), tk, tv, tk_tile, tv_tile, p));
    return B200_OK;
}

}  // namespace b200
