// Paged-KV causal prefill (extend) attention on the tcgen05 tensor cores, two query tiles per CTA.
//
// One CTA owns (request, KV head, block of 2 x 128/G query tokens), G = q_heads / kv_heads: two tiles
// of 128 rows, each row a (token, head-in-group) pair that reads the same KV head.  The two tiles share
// every K/V tile the producer loads and take turns on the tensor core: while the rows of one tile are
// in their softmax, the MMAs of the other run.  Per tile and K/V tile:
//     S = Q K^T            128 x 128 x 128, accumulator in TMEM (columns i*128 ..)
//     softmax              two threads per row read S, keep a running row maximum and sum in the log2
//                          domain and write the probabilities back into TMEM as bf16, over the first
//                          half of the S columns they have just read
//     O += P V             P is the A operand straight from TMEM, V MN-major from the layout TMA
//                          delivers, O accumulates in TMEM (columns 256 + i*128 ..) for the whole row
// The row maximum used for the exponentials is only moved when the true maximum has grown by more than
// 2^8 since (the sum and the final division use the same reference, so the result is exact); on those
// rare occasions the row's O is rescaled in TMEM by the threads that own the row.  Nothing else touches
// O until the end, so the softmax threads carry no accumulator and no P tile goes through shared memory.
//
// Roles: warp 0 producer (K/V tiles through a 2-stage TMA ring, as in attention_prefill_tc.cu), warp 1
// one thread issues every MMA, warps 2-9 softmax of tile 0, warps 10-17 softmax of tile 1 (thread pair =
// TMEM lane; warps w and w+4 of a group share a lane quarter and take keys 0-63 / 64-127).
// Queries are the LAST extend_len positions of the request, so tiles left of the diagonal need no mask
// and tiles right of it are never loaded.
#include "common.cuh"
#include "kernels.h"
#include "tcgen05.cuh"
#include "tensormap.cuh"

namespace b200 {
namespace {

constexpr int kD = 128;
constexpr int kTile = 128;                  // keys per K/V tile and rows per query tile
constexpr int kThreads = 64 + 2 * 256;      // producer, MMA issuer, 2 x 8 softmax warps
constexpr uint32_t kAtomBytes = 128 * 128;  // 128 rows x 64 bf16: one swizzle atom column
constexpr uint32_t kQOff = 0;               // Q: 2 tiles x 2 atoms (d 0-63, d 64-127)
constexpr uint32_t kKVOff = 4 * kAtomBytes; // ring: per stage K lo, K hi, V lo, V hi
constexpr uint32_t kStageBytes = 4 * kAtomBytes;
constexpr int kStages = 2;
constexpr uint32_t kSmemBytes = kKVOff + kStages * kStageBytes;
constexpr uint32_t kColS = 0, kColO = 256;  // TMEM columns: S0, S1 (128 each), O0, O1 (128 each)
constexpr float kLazyLog2 = 8.0f;           // the reference maximum moves when the true one is 2^8 ahead

struct PrefillTc2Params {
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

// MN-major operand under the 128-byte swizzle (V as the B operand of P V: rows are keys, 64 head-dim
// elements per 128-byte row): 8-key groups 1024 bytes apart along K, the second 64 head-dim elements one
// atom (16 KB) further.
__device__ __forceinline__ uint64_t mnmajor_sw128_desc2(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
    d |= static_cast<uint64_t>(kAtomBytes >> 4) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
__device__ __forceinline__ uint32_t idesc2_128x128(bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) |
           (static_cast<uint32_t>(128 >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void tc_mma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]),
        "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]),
        "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
attention_prefill_tc2_kernel(const __grid_constant__ CUtensorMap tmap_k,
                             const __grid_constant__ CUtensorMap tmap_v,
                             const __grid_constant__ CUtensorMap tmap_k_tile,
                             const __grid_constant__ CUtensorMap tmap_v_tile, const PrefillTc2Params p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t k_full[kStages];
    __shared__ __align__(8) uint64_t k_empty[kStages];
    __shared__ __align__(8) uint64_t v_full[kStages];
    __shared__ __align__(8) uint64_t v_empty[kStages];
    __shared__ __align__(8) uint64_t s_full[2];    // per query tile: S of the current K/V tile is in TMEM
    __shared__ __align__(8) uint64_t p_full[2];    // per query tile: P is in TMEM (8 warp arrivals)
    __shared__ __align__(8) uint64_t pv_done[2];   // per query tile: O += P V has completed
    __shared__ uint32_t tmem_base_slot;
    __shared__ float s_max[2][2][2][kTile];   // [K/V tile parity][query tile][column half][row]
    __shared__ float s_sum[2][2][kTile];      // [query tile][column half][row]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const int G = p.group;
    const int QB = kTile / G;      // query tokens per tile
    const int b = blockIdx.z;
    const int h = blockIdx.y;

    pdl_launch_dependents();
    pdl_wait_prior();

    const int q_begin = p.qo_indptr[b];
    const int ext = p.qo_indptr[b + 1] - q_begin;
    const int len = p.seq_lens[b];
    const int nqb = (ext + 2 * QB - 1) / (2 * QB);
    const int qb = nqb - 1 - static_cast<int>(blockIdx.x);  // heaviest blocks first
    if (qb < 0 || ext <= 0 || len <= 0) return;             // whole CTA, before any barrier or TMEM use
    const int t0 = qb * 2 * QB;                   // first token of tile 0; tile 1 starts QB further
    const int t_end = min(t0 + 2 * QB, ext);
    const int pos0 = len - ext;                   // position of query token 0
    const int kv_end = min(len, pos0 + t_end);    // keys [0, kv_end) are visible to this block
    const int ntiles = (kv_end + kTile - 1) / kTile;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&k_full[s]), 1);
            mbar_init(smem_u32(&k_empty[s]), 1);
            mbar_init(smem_u32(&v_full[s]), 1);
            mbar_init(smem_u32(&v_empty[s]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&s_full[i]), 1);
            mbar_init(smem_u32(&p_full[i]), 8);   // one arrival per softmax warp of the tile
            mbar_init(smem_u32(&pv_done[i]), 1);
        }
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
    // Q rows into shared memory in the swizzled K-major layout: tile i, row r = (token t0 + i*QB + r / G,
    // head h * G + r % G); rows past the request's last token are zero.
    if (warp >= 2) {
        const int sw = warp - 2;                  // 0..15
        const int tile = sw >> 3;
        const int r = (sw & 3) * 32 + lane;
        const int half = (sw & 7) >> 2;
        const int tok = t0 + tile * QB + r / G;
        const int head = h * G + r % G;
        const uint4* src = reinterpret_cast<const uint4*>(p.q + static_cast<int64_t>(q_begin + tok) * p.q_st +
                                                          static_cast<int64_t>(head) * p.q_sh);
        const bool valid = tok < t_end;
#pragma unroll
        for (int c = half * 8; c < half * 8 + 8; ++c) {
            const uint4 v = valid ? src[c] : make_uint4(0, 0, 0, 0);
            const uint32_t row_addr = smem_base + kQOff + (tile * 2 + (c >> 3)) * kAtomBytes + r * 128;
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
            // A tile whose pages are consecutive slots is fetched with two 128-key boxes per tensor.
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
                    !mbar_wait_bounded(smem_u32(kv == 0 ? &k_empty[slot] : &v_empty[slot]), parity, p.status, 321)) {
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
            const uint32_t idesc_s = idesc2_128x128(false);
            const uint32_t idesc_pv = idesc2_128x128(true);
            bool failed = false;
            // S_i = Q_i K^T of K/V tile kt (the K tile's barrier is waited for by whoever comes first)
            auto issue_s = [&](int i, int kt) {
                const uint32_t slot = kt % kStages;
                if (!mbar_wait_bounded(smem_u32(&k_full[slot]), static_cast<uint32_t>(kt / kStages) & 1u,
                                       p.status, 322)) {
                    failed = true;
                    return;
                }
                tc_fence_after();
                const uint32_t q_addr = smem_base + kQOff + i * 2 * kAtomBytes;
                const uint32_t k_addr = smem_base + kKVOff + slot * kStageBytes;
                const uint32_t d = tmem_base + kColS + static_cast<uint32_t>(i) * 128u;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t off = (ks >> 2) * kAtomBytes + (ks & 3) * 32;
                    tc_mma_bf16(d, kmajor_sw128_desc(q_addr + off), kmajor_sw128_desc(k_addr + off), idesc_s,
                                ks > 0 ? 1u : 0u);
                }
                tc_commit(smem_u32(&s_full[i]));
                if (i == 1) tc_commit(smem_u32(&k_empty[slot]));   // both tiles have read this K tile
            };
            // O_i += P_i V of K/V tile kt; P_i sits in the first half of each 64-column half of S_i
            auto issue_pv = [&](int i, int kt) {
                const uint32_t slot = kt % kStages;
                if (!mbar_wait_bounded(smem_u32(&v_full[slot]), static_cast<uint32_t>(kt / kStages) & 1u, p.status, 326) ||
                    !mbar_wait_bounded(smem_u32(&p_full[i]), static_cast<uint32_t>(kt) & 1u, p.status, 323)) {
                    failed = true;
                    return;
                }
                tc_fence_after();
                const uint32_t v_addr = smem_base + kKVOff + slot * kStageBytes + 2 * kAtomBytes;
                const uint32_t s_base = tmem_base + kColS + static_cast<uint32_t>(i) * 128u;
                const uint32_t d = tmem_base + kColO + static_cast<uint32_t>(i) * 128u;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    // keys ks*16 .. +15: eight packed columns; keys 64-127 start at column 64
                    const uint32_t a = s_base + static_cast<uint32_t>((ks >> 2) * 64 + (ks & 3) * 8);
                    tc_mma_bf16_ts(d, a, mnmajor_sw128_desc2(v_addr + ks * 2048), idesc_pv, (kt > 0 || ks > 0) ? 1u : 0u);
                }
                tc_commit(smem_u32(&pv_done[i]));
                if (i == 1) tc_commit(smem_u32(&v_empty[slot]));   // both tiles have read this V tile
            };
            issue_s(0, 0);
            if (!failed) issue_s(1, 0);
            for (int kt = 0; kt < ntiles && !failed; ++kt) {
                for (int i = 0; i < 2 && !failed; ++i) {
                    issue_pv(i, kt);
                    if (failed || kt + 1 >= ntiles) continue;
                    // S_i of the next tile overwrites the columns P_i was read from: wait for that product
                    // (issuing straight away and trusting the MMAs to run in issue order measured the same)
                    if (!mbar_wait_bounded(smem_u32(&pv_done[i]), static_cast<uint32_t>(kt) & 1u, p.status, 327)) {
                        failed = true;
                        break;
                    }
                    issue_s(i, kt + 1);
                }
            }
        }
    } else {
        // ================= softmax / output rows =================
        const int sw = warp - 2;                  // 0..15
        const int tile = sw >> 3;                 // query tile of this warp
        const int qtr = warp & 3;                 // TMEM lane quarter this warp may read
        const int half = (sw & 7) >> 2;           // keys / head-dim columns [64*half, 64*half + 64)
        const int r = qtr * 32 + lane;            // query row = TMEM lane
        const int tok = t0 + tile * QB + r / G;
        const int head = h * G + r % G;
        const int limit = min(pos0 + tok, len - 1);   // last visible key of this row
        const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(qtr * 32) << 16);
        const uint32_t s_addr = lane_addr + kColS + static_cast<uint32_t>(tile) * 128u + static_cast<uint32_t>(half * 64);
        const uint32_t o_addr = lane_addr + kColO + static_cast<uint32_t>(tile) * 128u + static_cast<uint32_t>(half * 64);
        const float sc = p.scale_log2;
        float m_ref = -INFINITY;   // the maximum the exponentials refer to, in units of the raw scores
        float l_run = 0.f;
        bool failed = false;
        const int bar_id = 1 + tile * 4 + (sw & 3);
        auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory"); };
        auto ex2 = [](float x) {
            float y;
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
            return y;
        };

        for (int kt = 0; kt < ntiles; ++kt) {
            if (!failed && !mbar_wait_bounded(smem_u32(&s_full[tile]), static_cast<uint32_t>(kt) & 1u, p.status, 324))
                failed = true;
            tc_fence_after();
            const int k0 = kt * kTile + half * 64;    // first key of this thread's columns
            // (masking is decided per warp, so that the common case carries no per-element tests at all)
            const bool need_mask = __any_sync(0xffffffffu, k0 + 63 > limit);
            // pass 1: the maximum of this thread's 64 scores (both loads in flight before the first wait)
            float mx = -INFINITY;
            {
                uint32_t sa[32], sb[32];
                tmem_ld_32x32b_x32(s_addr, sa);
                tmem_ld_32x32b_x32(s_addr + 32, sb);
                tmem_ld_wait();
                if (need_mask) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (k0 + i <= limit) mx = fmaxf(mx, __uint_as_float(sa[i]));
                        if (k0 + 32 + i <= limit) mx = fmaxf(mx, __uint_as_float(sb[i]));
                    }
                } else {
                    float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        m0 = fmaxf(m0, __uint_as_float(sa[i]));
                        m1 = fmaxf(m1, __uint_as_float(sa[i + 1]));
                        m2 = fmaxf(m2, __uint_as_float(sb[i]));
                        m3 = fmaxf(m3, __uint_as_float(sb[i + 1]));
                    }
                    mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
                }
            }
            s_max[kt & 1][tile][half][r] = mx;   // two buffers: the partner may still be reading the last tile's
            pair_sync();
            mx = fmaxf(mx, s_max[kt & 1][tile][half ^ 1][r]);
            // Move the reference only when the row's maximum has outgrown it by 2^8 (both threads of the
            // row decide alike); O and the running sum shrink by the same factor.  The TMEM accesses are
            // warp-wide instructions, so a warp rescales all of its rows (by 1 where nothing moved) as soon
            // as one of them has to.
            float alpha = 1.f;
            if (mx != -INFINITY && (m_ref == -INFINITY || (mx - m_ref) * sc > kLazyLog2)) {
                if (m_ref != -INFINITY) alpha = ex2((m_ref - mx) * sc);
                m_ref = mx;
            }
            if (__any_sync(0xffffffffu, alpha != 1.f)) {
                l_run *= alpha;
                // no product of this query tile is in flight: S of this K/V tile was issued after the
                // previous P V had completed
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t ov[32];
                    tmem_ld_32x32b_x32(o_addr + c * 32, ov);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
                    tmem_st_32x32b_x32(o_addr + c * 32, ov);
                }
            }
            // a row that has seen no key yet: every exponent becomes -inf, every probability 0
            const float mb = m_ref == -INFINITY ? INFINITY : m_ref * sc;
            // pass 2: probabilities, 32 scores at a time, written over the first 32 columns of this
            // thread's 64 (which it has finished reading)
            float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t sv[32];
                tmem_ld_32x32b_x32(s_addr + c * 32, sv);
                tmem_ld_wait();
                uint32_t packed[16];
                if (need_mask) {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        float p0 = ex2(fmaf(__uint_as_float(sv[i]), sc, -mb));
                        float p1 = ex2(fmaf(__uint_as_float(sv[i + 1]), sc, -mb));
                        if (k0 + c * 32 + i > limit) p0 = 0.f;
                        if (k0 + c * 32 + i + 1 > limit) p1 = 0.f;
                        sum0 += p0;
                        sum1 += p1;
                        packed[i >> 1] = pack_bf16(p0, p1);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float p0 = ex2(fmaf(__uint_as_float(sv[i]), sc, -mb));
                        const float p1 = ex2(fmaf(__uint_as_float(sv[i + 1]), sc, -mb));
                        sum0 += p0;
                        sum1 += p1;
                        packed[i >> 1] = pack_bf16(p0, p1);
                    }
                }
                tmem_st_32x32b_x16(s_addr + c * 16, packed);
            }
            const float sum = sum0 + sum1;
            l_run += sum;
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&p_full[tile]));
        }
        // the last product, then O / (sum of the two halves' partial sums)
        if (!failed && !mbar_wait_bounded(smem_u32(&pv_done[tile]), static_cast<uint32_t>(ntiles - 1) & 1u, p.status, 325))
            failed = true;
        tc_fence_after();
        s_sum[tile][half][r] = l_run;
        pair_sync();
        const float l_tot = l_run + s_sum[tile][half ^ 1][r];
        {
            // (the TMEM loads are warp-wide: every lane takes part, only the stores are per row)
            const bool store = !failed && tok < t_end;
            const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
            uint4* dst = reinterpret_cast<uint4*>(p.out + (static_cast<int64_t>(q_begin + (store ? tok : 0)) * p.q_heads + head) * kD +
                                                  half * 64);
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t ov[32];
                tmem_ld_32x32b_x32(o_addr + c * 32, ov);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint4 w;
                    w.x = pack_bf16(__uint_as_float(ov[j * 8 + 0]) * inv, __uint_as_float(ov[j * 8 + 1]) * inv);
                    w.y = pack_bf16(__uint_as_float(ov[j * 8 + 2]) * inv, __uint_as_float(ov[j * 8 + 3]) * inv);
                    w.z = pack_bf16(__uint_as_float(ov[j * 8 + 4]) * inv, __uint_as_float(ov[j * 8 + 5]) * inv);
                    w.w = pack_bf16(__uint_as_float(ov[j * 8 + 6]) * inv, __uint_as_float(ov[j * 8 + 7]) * inv);
                    if (store) dst[c * 4 + j] = w;
                }
            }
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

int make_kv_tmap_3d_tc2(CUtensorMap* out, const void* cache, int64_t num_slots, int kv_heads, int kpc) {
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

int launch_attention_prefill_tc2(void* out, const void* q, int64_t q_st, int64_t q_sh, const void* k_cache,
                                 const void* v_cache, int64_t num_slots, const int32_t* page_table,
                                 int64_t pt_stride, const int32_t* table_idx, const int32_t* seq_lens,
                                 const int32_t* qo_indptr, int batch, int max_extend_len, int q_heads,
                                 int kv_heads, int page_size, float sm_scale, int* status,
                                 cudaStream_t stream) {
    if (batch == 0 || max_extend_len == 0) return B200_OK;
    PrefillTc2Params p;
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
    int err = make_kv_tmap_3d_tc2(&tk, k_cache, num_slots, kv_heads, p.kpc);
    if (err != B200_OK) return err;
    err = make_kv_tmap_3d_tc2(&tv, v_cache, num_slots, kv_heads, p.kpc);
    if (err != B200_OK) return err;
    CUtensorMap tk_tile, tv_tile;   // 128-key boxes for tiles whose pages are consecutive slots
    const int tile_box = num_slots >= kTile ? kTile : p.kpc;
    p.whole_tile_boxes = (tile_box == kTile && p.kpc < kTile) ? 1 : 0;
    err = make_kv_tmap_3d_tc2(&tk_tile, k_cache, num_slots, kv_heads, tile_box);
    if (err != B200_OK) return err;
    err = make_kv_tmap_3d_tc2(&tv_tile, v_cache, num_slots, kv_heads, tile_box);
    if (err != B200_OK) return err;
    const int QB = kTile / p.group;
    const int smem = kSmemBytes + 1024;
    B200_CHECK_CUDA(cudaFuncSetAttribute(attention_prefill_tc2_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    dim3 grid(div_ceil(max_extend_len, 2 * QB), kv_heads, batch);
    B200_CHECK_CUDA(launch_kernel(attention_prefill_tc2_kernel, grid, dim3(kThreads), smem, stream,
                                  dim3(1, 1, 1), tk, tv, tk_tile, tv_tile, p));
    return B200_OK;
}

}  // namespace b200
