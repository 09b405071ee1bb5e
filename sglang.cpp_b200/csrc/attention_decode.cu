// Paged-KV GQA decode attention: persistent split-KV flash-decode for sm_100a.
//
// The kernel is bound by streaming each request's K and V rows from HBM once.
// Design, in the order the bytes move:
//   * KV pool layout (one layer): [slots, kv_heads, 128] bf16, so all heads of a
//     slot are contiguous and a page of P consecutive slots is one dense block.
//     A 3-D TMA tensor map [head][slot][128] views it head-major; the producer warp copies
//     boxes of (all kv heads x keys-per-copy x 64 elements) with the 128-byte swizzle into a
//     3-stage ring of 64 KB stages (K lo/hi halves, V lo/hi halves), so the keys of one head
//     are adjacent 128-byte rows (conflict-free ldmatrix).
//   * a stage always holds 128 (key, head) rows: 128/kv_heads keys x kv_heads.
//     Eight consumer warps each own one (head, 16-key group) tile of a stage, so a
//     warp keeps the same KV head for the whole kernel.
//   * per tile: S = Q K^T with mma.sync m16n8k16 (the G = q_heads/kv_heads query
//     heads of the group are rows of the 16-row A operand), online softmax in the
//     exp2 domain, O += P V.  Tensor throughput is irrelevant here; mma + ldmatrix
//     is used because it needs ~10x fewer issue slots than CUDA-core dot products,
//     which keeps the SM free to run the copy pipeline.
//   * all stages of all requests form one global sequence that is cut into equal contiguous
//     runs, one per CTA (computed on the device from seq_lens alone: no host plan, graph-replay
//     safe), so every CTA streams the same number of bytes; a run is split into items at
//     request boundaries and the stage ring runs across item boundaries.
//   * every warp writes an (m, l, O) partial (or, for a request that is a single partial, bf16
//     outputs at once); a second, tiny kernel merges the partials of every request, one warp per
//     (request, query head), so the streaming kernel ends with its last stage.
#include <mutex>

#include "common.cuh"
#include "kernels.h"
#include "tensormap.cuh"

namespace b200 {
namespace {

constexpr int kD = 128;
constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;
constexpr int kStageRows = 128;                      // (key, head) rows per stage
constexpr uint32_t kHalfBytes = kStageRows * 128;    // one 64-element half tile
constexpr uint32_t kStageBytes = 4 * kHalfBytes;     // K lo, K hi, V lo, V hi
constexpr int kStages = 3;
constexpr int kMaxBatch = 1024;
constexpr int kSlotTab = 1024;
constexpr int kMinStagesPerCta = 2;   // do not split below two stages (128 KB) per CTA
constexpr int kMergeWarps = 4;    // merge kernel: one warp per (request, query head)

struct DecodeParams {
    __nv_bfloat16* out;
    const __nv_bfloat16* q;
    int64_t q_st, q_sh;
    const int32_t* page_table;
    int64_t pt_stride;
    const int32_t* table_idx;
    const int32_t* seq_lens;
    int batch, q_heads, kv_heads, group;
    int stage_keys;     // 128 / kv_heads
    int kpc;            // keys per TMA copy = min(page_size, stage_keys)
    int64_t num_slots;
    float scale_log2;
    float* ws_o;        // [max_items * KG, q_heads, 128]
    float* ws_ml;       // [max_items * KG, q_heads, 2]
    int max_items;
    int* status;
    int kv_evict_first;   // stream K/V through L2 with the evict-first policy (read once per step)
};

struct ItemInfo {
    int b, len, s_begin, s_end, nchunks, item, first_slot;
};

__device__ __forceinline__ void consumer_bar() {
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
attention_decode_kernel(const __grid_constant__ CUtensorMap tmap_k,
                        const __grid_constant__ CUtensorMap tmap_v, const DecodeParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kStages];
    __shared__ __align__(8) uint64_t empty_bar[kStages];
    __shared__ int s_prefix[kMaxBatch + 1];  // exclusive scan of items per request
    __shared__ int s_len[kMaxBatch];         // seq_lens, read once
    __shared__ int s_slot_tab[kSlotTab];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int B = p.batch;
    const int SK = p.stage_keys;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), kConsumerWarps);
        }
        fence_mbar_init();
    }
    if (warp == kConsumerWarps && lane == 0) {
        tma_prefetch_desc(&tmap_k);
        tma_prefetch_desc(&tmap_v);
    }

    // Programmatic dependent launch: what the kernel before this one (the K/V store of the same
    // layer) writes is only q and the newest token's K/V.  seq_lens, the page table and every older
    // K/V row were complete before that kernel could start, so the split and most K/V loads run
    // ahead of griddepcontrol.wait; consumers wait before reading q, the producer before the first
    // stage that holds a request's newest key.
    pdl_launch_dependents();

    // ---- device-side split ----
    // All stages of all requests form one global sequence; CTA i takes the contiguous run
    // [i*per, (i+1)*per) of it, so every CTA streams the same number of bytes (+-1 stage).
    // A run is cut into items at request boundaries.  s_prefix[b] = first global stage of
    // request b.  Request b is covered by the CTAs c0 = s_prefix[b]/per .. and its partials
    // live in the consecutive workspace slots b + c (unique because b and c grow together).
    if (warp == 0) {
        int carry = 0;
        for (int base = 0; base < B; base += 32) {
            const int b = base + lane;
            const int n = b < B ? (max(p.seq_lens[b], 0) + SK - 1) / SK : 0;
            int incl = n;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            if (b < B) {
                s_prefix[b] = carry + incl - n;
                s_len[b] = p.seq_lens[b];
            }
            carry += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) s_prefix[B] = carry;
    }
    __syncthreads();
    const int total_stages = s_prefix[B];
    const int per = max((total_stages + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x),
                        kMinStagesPerCta);
    const int g_begin = static_cast<int>(blockIdx.x) * per;
    const int g_end = min(total_stages, g_begin + per);
    if (static_cast<int>(gridDim.x) + B > p.max_items) {
        if (threadIdx.x == 0) atomicExch(&p.status[kStatusBadIndex], static_cast<int>(gridDim.x) + B + 1);
        return;
    }

    // The item that starts at global stage gpos (gpos < g_end).
    auto locate = [&](int gpos) {
        ItemInfo it;
        int lo = 0, hi = B;  // largest b with s_prefix[b] <= gpos (requests without stages are skipped)
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (s_prefix[mid] <= gpos) lo = mid; else hi = mid;
        }
        it.b = lo;
        it.len = s_len[lo];
        const int first = s_prefix[lo];
        const int st = s_prefix[lo + 1] - first;
        it.s_begin = gpos - first;
        it.s_end = min(st, it.s_begin + (g_end - gpos));
        const int c0 = first / per;
        it.nchunks = (first + st - 1) / per - c0 + 1;   // CTAs that share this request
        it.first_slot = lo + c0;
        it.item = lo + static_cast<int>(blockIdx.x);
        return it;
    };

    const int Hkv = p.kv_heads;
    const int KG = kConsumerWarps / Hkv;  // 16-key groups per stage
    bool failed = false;
    uint32_t it_count = 0;  // stages consumed / produced so far by this CTA

    if (warp == kConsumerWarps) {
        // ================= producer warp =================
        const uint32_t copy_bytes = static_cast<uint32_t>(p.kpc) * Hkv * 128u;  // one half-tile box
        const uint64_t kv_policy = l2_policy_evict_first();
        bool waited = false;
        for (int gpos = g_begin; gpos < g_end && !failed;) {
            const ItemInfo it = locate(gpos);
            gpos += it.s_end - it.s_begin;
            const int32_t* pt_row = p.page_table + static_cast<int64_t>(p.table_idx[it.b]) * p.pt_stride;
            const int first_key = it.s_begin * SK;
            const int item_keys = min(it.len, it.s_end * SK) - first_key;
            const int item_copies = (item_keys + p.kpc - 1) / p.kpc;
            // Slot of the first key of every copy of this item (the previous item's
            // table is no longer needed: all of its copies have been issued).
            __syncwarp();
            for (int c = lane; c < min(item_copies, kSlotTab); c += 32)
                s_slot_tab[c] = pt_row[first_key + c * p.kpc];
            __syncwarp();
            for (int st = it.s_begin; st < it.s_end; ++st, ++it_count) {
                const uint32_t slot = it_count % kStages;
                const uint32_t parity = ((it_count / kStages) & 1u) ^ 1u;
                if (!mbar_wait_bounded(smem_u32(&empty_bar[slot]), parity, p.status, 201)) {
                    failed = true;
                    break;
                }
                const int k0 = st * SK;
                const int valid = min(SK, it.len - k0);
                const int ncopies = (valid + p.kpc - 1) / p.kpc;
                if (!waited && k0 + valid >= it.len) {  // this stage holds the key written just now
                    pdl_wait_prior();
                    waited = true;
                }
                const uint32_t bar = smem_u32(&full_bar[slot]);
                if (lane == 0) mbar_arrive_expect_tx(bar, static_cast<uint32_t>(ncopies) * 4u * copy_bytes);
                __syncwarp();
                const uint32_t stage_base = smem_base + slot * kStageBytes;
                for (int ci = lane; ci < ncopies * 4; ci += 32) {
                    const int copy = ci >> 2, which = ci & 3;
                    const int tab = (k0 - first_key) / p.kpc + copy;
                    int64_t sl = tab < kSlotTab ? s_slot_tab[tab] : pt_row[k0 + copy * p.kpc];
                    if (sl < 0 || sl + p.kpc > p.num_slots) {
                        atomicExch(&p.status[kStatusBadIndex], static_cast<int>(sl) + 1);
                        sl = 0;
                    }
                    const uint32_t dst = stage_base + which * kHalfBytes + copy * copy_bytes;
                    if (p.kv_evict_first)
                        tma_load_3d_hint(dst, which < 2 ? &tmap_k : &tmap_v, (which & 1) * 64,
                                         static_cast<int>(sl), 0, bar, kv_policy);
                    else
                        tma_load_3d(dst, which < 2 ? &tmap_k : &tmap_v, (which & 1) * 64,
                                    static_cast<int>(sl), 0, bar);
                }
            }
        }
        return;
    }

    // ================= consumer warps =================
    const int h = warp % Hkv;       // KV head of this warp
    const int kg = warp / Hkv;      // 16-key group inside a stage
    const int G = p.group;
    const int g = lane >> 2, t = lane & 3;
    const int mi = lane >> 3, r8 = lane & 7;

    // Query fragments: rows of the A operand are the G heads of this KV group.
    uint32_t qa[8][4];
    auto load_q = [&](int b) {
        const __nv_bfloat16* q0 = p.q + b * p.q_st + static_cast<int64_t>(h * G + g) * p.q_sh;
        const __nv_bfloat16* q1 = q0 + 8 * p.q_sh;
        const bool r0 = g < G, r1 = (g + 8) < G;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            const int d0 = ks * 16 + 2 * t;
            qa[ks][0] = r0 ? *reinterpret_cast<const uint32_t*>(q0 + d0) : 0u;
            qa[ks][2] = r0 ? *reinterpret_cast<const uint32_t*>(q0 + d0 + 8) : 0u;
            qa[ks][1] = r1 ? *reinterpret_cast<const uint32_t*>(q1 + d0) : 0u;
            qa[ks][3] = r1 ? *reinterpret_cast<const uint32_t*>(q1 + d0 + 8) : 0u;
        }
    };
    const int Hq = p.q_heads;

    pdl_wait_prior();  // q comes from the kernel before this one
    int gpos = g_begin;
    bool have = gpos < g_end;
    ItemInfo it = {};
    if (have) {
        it = locate(gpos);
        load_q(it.b);
    }
    while (have) {
        gpos += it.s_end - it.s_begin;
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
        float o[16][4];
#pragma unroll
        for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

        for (int st = it.s_begin; st < it.s_end; ++st, ++it_count) {
            const uint32_t slot = it_count % kStages;
            const uint32_t parity = (it_count / kStages) & 1u;
            if (!failed && !mbar_wait_bounded(smem_u32(&full_bar[slot]), parity, p.status, 202))
                failed = true;
            const int nvalid = it.len - (st * SK + kg * 16);  // valid keys in this warp's tile
            if (!failed && nvalid > 0) {
                const uint32_t stage_base = smem_base + slot * kStageBytes;
                // Row of key j (0..15 of this warp's tile) inside a half tile.  A copy of
                // kpc keys lands as [head][key] rows, so the keys of one head are adjacent
                // 128-byte rows and the swizzle spreads an 8-key ldmatrix over all banks.
                const int kpc = p.kpc;
                auto tile_row = [&](int j) -> uint32_t {
                    const int js = kg * 16 + j;
                    return static_cast<uint32_t>((js & ~(kpc - 1)) * Hkv + h * kpc + (js & (kpc - 1)));
                };
                if (nvalid < 16) {
                    // Rows past the end of the sequence hold stale bytes: clear V so
                    // that 0 * garbage cannot poison the accumulator.
                    for (int i = lane; i < (16 - nvalid) * 16; i += 32) {
                        const int j = nvalid + (i >> 4), c16 = i & 15;
                        const uint32_t a = stage_base + (2 + (c16 >> 3)) * kHalfBytes +
                                           tile_row(j) * 128u + (c16 & 7) * 16u;
                        asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(a), "r"(0u) : "memory");
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                }
                // ---- S = Q K^T for 16 keys ----
                float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
                {
                    const int j = (mi >> 1) * 8 + r8;
                    const uint32_t rowoff = tile_row(j) * 128u;
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks) {
                        const int c16 = ks * 2 + (mi & 1);
                        const uint32_t row_addr = stage_base + (c16 >> 3) * kHalfBytes + rowoff;
                        uint32_t b00, b01, b10, b11;
                        ldmatrix_x4(swz128(row_addr, c16 & 7), b00, b01, b10, b11);
                        mma_bf16_16816(s0, qa[ks], b00, b01);
                        mma_bf16_16816(s1, qa[ks], b10, b11);
                    }
                }
                // ---- online softmax (exp2 domain) ----
                float x[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float v = (e < 4 ? s0[e] : s1[e - 4]) * p.scale_log2;
                    const int key = (e >> 2) * 8 + 2 * t + (e & 1);
                    x[e] = key < nvalid ? v : -INFINITY;
                }
                float mx0 = fmaxf(fmaxf(x[0], x[1]), fmaxf(x[4], x[5]));
                float mx1 = fmaxf(fmaxf(x[2], x[3]), fmaxf(x[6], x[7]));
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
                const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);  // finite: key 0 is valid
                const float al0 = exp2f(m0 - mn0), al1 = exp2f(m1 - mn1);
                m0 = mn0;
                m1 = mn1;
                const float p00 = exp2f(x[0] - mn0), p01 = exp2f(x[1] - mn0);
                const float p02 = exp2f(x[4] - mn0), p03 = exp2f(x[5] - mn0);
                const float p10 = exp2f(x[2] - mn1), p11 = exp2f(x[3] - mn1);
                const float p12 = exp2f(x[6] - mn1), p13 = exp2f(x[7] - mn1);
                l0 = l0 * al0 + (p00 + p01 + p02 + p03);
                l1 = l1 * al1 + (p10 + p11 + p12 + p13);
                uint32_t pa[4];
                pa[0] = pack_bf16(p00, p01);
                pa[1] = pack_bf16(p10, p11);
                pa[2] = pack_bf16(p02, p03);
                pa[3] = pack_bf16(p12, p13);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    o[i][0] *= al0;
                    o[i][1] *= al0;
                    o[i][2] *= al1;
                    o[i][3] *= al1;
                }
                // ---- O += P V ----
                {
                    const int j = (mi & 1) * 8 + r8;
                    const uint32_t rowoff = tile_row(j) * 128u;
#pragma unroll
                    for (int np = 0; np < 8; ++np) {
                        const int c16 = np * 2 + (mi >> 1);
                        const uint32_t row_addr = stage_base + (2 + (c16 >> 3)) * kHalfBytes + rowoff;
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

        // The next item's queries are requested now, so their latency hides behind this
        // item's epilogue (the fragments of the finished item are no longer needed).
        const bool has_next = gpos < g_end;
        ItemInfo nx = it;
        if (has_next) {
            nx = locate(gpos);
            load_q(nx.b);
        }

        // ---- item epilogue ----
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
        l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
        const int nparts = it.nchunks * KG;
        if (nparts == 1) {
            // Single partial: normalise and store bf16 directly.
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                const int row = g + rr * 8;
                if (row < G) {
                    const float l = rr ? l1 : l0;
                    const float inv = l > 0.f ? 1.f / l : 0.f;
                    __nv_bfloat16* dst = p.out + (static_cast<int64_t>(it.b) * Hq + h * G + row) * kD;
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t) =
                            pack_bf16(o[i][2 * rr] * inv, o[i][2 * rr + 1] * inv);
                }
            }
        } else {
            const int64_t part = static_cast<int64_t>(it.item) * KG + kg;
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                const int row = g + rr * 8;
                if (row < G) {
                    const int64_t ph = part * Hq + h * G + row;
                    float* dst = p.ws_o + ph * kD;
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        *reinterpret_cast<float2*>(dst + i * 8 + 2 * t) =
                            make_float2(o[i][2 * rr], o[i][2 * rr + 1]);
                    if (t == 0)
                        *reinterpret_cast<float2*>(p.ws_ml + ph * 2) =
                            make_float2(rr ? m1 : m0, rr ? l1 : l0);
                }
            }
        }
        have = has_next;
        it = nx;
    }
}

// Second kernel of a decode attention call: the partial results of every request that was cut over
// several CTAs (or several key groups of a stage) are combined and written as bf16.  One warp per
// (request, query head): it repeats the split arithmetic of the kernel above for its request, reads the
// (max, sum) pairs and the fp32 partial rows in one round trip to L2 and writes 128 outputs.  Kept out
// of the streaming kernel on purpose: there the CTA that happened to deliver a request's last partial
// merged it behind its own last stage, a chain of fences, a ticket and three dependent trips to L2 that
// left the other 147 SMs and HBM idle for about 12 us per launch.
__global__ void __launch_bounds__(kMergeWarps * 32)
attention_decode_merge_kernel(const DecodeParams p, int attn_grid) {
    __shared__ int s_first, s_stages, s_total;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_per_cta = kMergeWarps;
    const int ctas_per_req = (p.q_heads + heads_per_cta - 1) / heads_per_cta;
    const int b = static_cast<int>(blockIdx.x) / ctas_per_req;
    const int head = (static_cast<int>(blockIdx.x) % ctas_per_req) * heads_per_cta + warp;
    const int SK = p.stage_keys;
    pdl_launch_dependents();
    // seq_lens were complete before the attention kernel started: the split runs ahead of the wait
    if (warp == 0) {
        int carry = 0, first = 0, mine = 0;
        for (int base = 0; base < p.batch; base += 32) {
            const int r = base + lane;
            const int n = r < p.batch ? (max(p.seq_lens[r], 0) + SK - 1) / SK : 0;
            int incl = n;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            if (b >= base && b < base + 32) {
                first = carry + __shfl_sync(0xffffffffu, incl - n, b - base);
                mine = __shfl_sync(0xffffffffu, n, b - base);
            }
            carry += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) {
            s_first = first;
            s_stages = mine;
            s_total = carry;
        }
    }
    __syncthreads();
    const int first = s_first, st = s_stages;
    const int per = max((s_total + attn_grid - 1) / attn_grid, kMinStagesPerCta);
    const int KG = kConsumerWarps / p.kv_heads;
    const int c0 = first / per;
    const int nparts = st > 0 ? ((first + st - 1) / per - c0 + 1) * KG : 0;
    pdl_wait_prior();
    if (nparts <= 1 || head >= p.q_heads) return;   // a single partial was written as bf16 by the kernel above
    const int Hq = p.q_heads;
    const int64_t part0 = static_cast<int64_t>(b + c0) * KG;
    const float* ml = p.ws_ml + (part0 * Hq + head) * 2;
    const float* po = p.ws_o + (part0 * Hq + head) * kD + lane * 4;
    const int64_t ml_stride = static_cast<int64_t>(Hq) * 2, o_stride = static_cast<int64_t>(Hq) * kD;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float M = -INFINITY, Lsum = 0.f;
    for (int base = 0; base < nparts; base += 32) {
        const int n = min(32, nparts - base);
        // this chunk's (max, sum) pairs, one per lane, and its rows: all loads are independent
        float2 mine = make_float2(-INFINITY, 0.f);
        if (lane < n) mine = __ldcg(reinterpret_cast<const float2*>(ml + (base + lane) * ml_stride));
        float4 rows[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            rows[j] = j < n ? __ldcg(reinterpret_cast<const float4*>(po + (base + j) * o_stride))
                            : make_float4(0.f, 0.f, 0.f, 0.f);
        const float Mc = fmaxf(M, warp_max(mine.x));   // finite: a request's first partial holds key 0
        const float rescale = exp2f(M - Mc);           // 0 on the first chunk (M = -inf)
        acc.x *= rescale;
        acc.y *= rescale;
        acc.z *= rescale;
        acc.w *= rescale;
        const float w_mine = exp2f(mine.x - Mc);
        Lsum = Lsum * rescale + warp_sum(mine.y * w_mine);
        M = Mc;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (j < n) {   // n is the same on every lane
                const float w = __shfl_sync(0xffffffffu, w_mine, j);
                acc.x += rows[j].x * w;
                acc.y += rows[j].y * w;
                acc.z += rows[j].z * w;
                acc.w += rows[j].w * w;
            }
        }
        for (int j = 8; j < n; ++j) {
            const float w = __shfl_sync(0xffffffffu, w_mine, j);
            const float4 r = __ldcg(reinterpret_cast<const float4*>(po + (base + j) * o_stride));
            acc.x += r.x * w;
            acc.y += r.y * w;
            acc.z += r.z * w;
            acc.w += r.w * w;
        }
    }
    const float inv = Lsum > 0.f ? 1.f / Lsum : 0.f;
    uint2 packed;
    packed.x = pack_bf16(acc.x * inv, acc.y * inv);
    packed.y = pack_bf16(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(p.out + (static_cast<int64_t>(b) * Hq + head) * kD + lane * 4) = packed;
}

}  // namespace

int64_t decode_workspace_bytes(int max_batch, int q_heads, int kv_heads) {
    const int kg = kConsumerWarps / kv_heads;
    const int64_t items = static_cast<int64_t>(sm_count()) + max_batch;
    const int64_t parts = items * kg;
    return parts * q_heads * (kD + 2) * 4 + 256;
}

int launch_attention_decode(void* out, const void* q, int64_t q_st, int64_t q_sh,
                            const CUtensorMap& tmap_k, const CUtensorMap& tmap_v, int64_t num_slots,
                            const int32_t* page_table, int64_t pt_stride, const int32_t* table_idx,
                            const int32_t* seq_lens, int batch, int q_heads, int kv_heads,
                            int page_size, float sm_scale, void* workspace, int64_t workspace_bytes,
                            int* status, cudaStream_t stream, bool kv_evict_first) {
    const int kg = kConsumerWarps / kv_heads;
    const int grid = sm_count();
    // Workspace layout: ws_ml | ws_o
    const int64_t avail = workspace_bytes - 256;
    const int64_t per_item = static_cast<int64_t>(kg) * q_heads * (kD + 2) * 4;
    const int64_t max_items = avail / per_item;
    if (max_items < static_cast<int64_t>(grid) + batch) {
        set_last_error("attention_decode: workspace of %lld bytes is too small (need %lld)",
                       static_cast<long long>(workspace_bytes),
                       static_cast<long long>(decode_workspace_bytes(batch, q_heads, kv_heads)));
        return B200_ERR_INVALID_ARGUMENT;
    }
    DecodeParams p;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.q_st = q_st;
    p.q_sh = q_sh;
    p.page_table = page_table;
    p.pt_stride = pt_stride;
    p.table_idx = table_idx;
    p.seq_lens = seq_lens;
    p.batch = batch;
    p.q_heads = q_heads;
    p.kv_heads = kv_heads;
    p.group = q_heads / kv_heads;
    p.stage_keys = kStageRows / kv_heads;
    p.kpc = page_size < p.stage_keys ? page_size : p.stage_keys;
    p.num_slots = num_slots;
    p.scale_log2 = sm_scale * 1.4426950408889634f;
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    uint8_t* f = ws;
    f = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(f) + 255) & ~uintptr_t(255));
    p.ws_ml = reinterpret_cast<float*>(f);
    p.ws_o = p.ws_ml + max_items * kg * q_heads * 2;
    p.max_items = static_cast<int>(max_items < (1 << 30) ? max_items : (1 << 30));
    p.status = status;
    p.kv_evict_first = kv_evict_first ? 1 : 0;

    const int smem = kStages * kStageBytes + 1024;
    // The attribute belongs to (function, device): set it on every launch, as the other launchers do.
    B200_CHECK_CUDA(cudaFuncSetAttribute(attention_decode_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    B200_CHECK_CUDA(launch_kernel(attention_decode_kernel, dim3(grid), dim3(kThreads), smem, stream,
                                  dim3(1, 1, 1), tmap_k, tmap_v, p));
    const int merge_ctas = batch * ((q_heads + kMergeWarps - 1) / kMergeWarps);
    B200_CHECK_CUDA(launch_kernel(attention_decode_merge_kernel, dim3(merge_ctas), dim3(kMergeWarps * 32), 0, stream,
                                  dim3(1, 1, 1), p, grid));
    return B200_OK;
}

int make_kv_tmap(CUtensorMap* out, const void* cache, int64_t num_slots, int kv_heads, int page_size) {
    // 3-D view [heads][slots][128] of the pool's [slots][heads][128] memory (the head
    // stride is smaller than the slot stride), so that a box of kpc slots x all heads
    // arrives in shared memory head-major.
    const int stage_keys = kStageRows / kv_heads;
    const int kpc = page_size < stage_keys ? page_size : stage_keys;
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) {
        set_last_error("cuTensorMapEncodeTiled is not available from this driver");
        return B200_ERR_CUDA;
    }
    if ((reinterpret_cast<uintptr_t>(cache) & 15u) != 0) {
        set_last_error("attention_decode: the KV cache must be 16-byte aligned");
        return B200_ERR_INVALID_ARGUMENT;
    }
    const cuuint64_t dims[3] = {kD, static_cast<cuuint64_t>(num_slots), static_cast<cuuint64_t>(kv_heads)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(kv_heads) * kD * 2, kD * 2};
    const cuuint32_t box[3] = {64, static_cast<cuuint32_t>(kpc), static_cast<cuuint32_t>(kv_heads)};
    const cuuint32_t es[3] = {1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(cache), dims, strides,
                    box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_last_error("cuTensorMapEncodeTiled (KV map) failed with CUresult %d", static_cast<int>(r));
        return B200_ERR_CUDA;
    }
    return B200_OK;
}

}  // namespace b200

extern "C" {

int64_t b200_attention_decode_workspace_bytes(int max_batch, int q_heads, int kv_heads, int head_dim) {
    if (max_batch <= 0 || q_heads <= 0 || kv_heads <= 0 || head_dim != b200::kD) return -1;
    if (kv_heads > 8 || (8 % kv_heads) != 0) return -1;
    return b200::decode_workspace_bytes(max_batch, q_heads, kv_heads);
}

int b200_attention_decode(void* out, const void* q, int64_t q_stride_token, int64_t q_stride_head,
                          const void* k_cache, const void* v_cache, int64_t num_slots,
                          const int32_t* page_table, int64_t page_table_stride,
                          const int32_t* table_idx, const int32_t* seq_lens, int batch, int q_heads,
                          int kv_heads, int head_dim, int page_size, float sm_scale, void* workspace,
                          int64_t workspace_bytes, b200_stream_t stream) {
    B200_CHECK_ARG(batch == 0 || (out && q && k_cache && v_cache && page_table && table_idx && seq_lens && workspace),
                   "attention_decode: NULL tensor");
    B200_CHECK_ARG(head_dim == b200::kD, "attention_decode: head_dim must be 128");
    B200_CHECK_ARG(batch >= 0 && batch <= b200::kMaxBatch, "attention_decode: batch must be in [0, 1024]");
    B200_CHECK_ARG(kv_heads >= 1 && kv_heads <= 8 && (8 % kv_heads) == 0,
                   "attention_decode: kv_heads (per rank) must be 1, 2, 4 or 8");
    B200_CHECK_ARG(q_heads % kv_heads == 0 && q_heads / kv_heads <= 16,
                   "attention_decode: q_heads must be a multiple of kv_heads with group size <= 16");
    B200_CHECK_ARG(page_size >= 1 && (page_size & (page_size - 1)) == 0,
                   "attention_decode: page_size must be a power of two");
    B200_CHECK_ARG(q_stride_token % 2 == 0 && q_stride_head % 2 == 0,
                   "attention_decode: q strides must be even");
    B200_CHECK_ARG(num_slots > 0, "attention_decode: num_slots must be positive");
    if (batch == 0) return B200_OK;
    int err = B200_OK;
    int* status = b200::device_status_words(&err);
    if (err != B200_OK) return err;
    CUtensorMap tk, tv;
    err = b200::make_kv_tmap(&tk, k_cache, num_slots, kv_heads, page_size);
    if (err != B200_OK) return err;
    err = b200::make_kv_tmap(&tv, v_cache, num_slots, kv_heads, page_size);
    if (err != B200_OK) return err;
    return b200::launch_attention_decode(out, q, q_stride_token, q_stride_head, tk, tv, num_slots,
                                         page_table, page_table_stride, table_idx, seq_lens, batch,
                                         q_heads, kv_heads, page_size, sm_scale, workspace,
                                         workspace_bytes, status, static_cast<cudaStream_t>(stream));
}

}  // extern "C"

// ============================================================================
// Decode attention for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need
// attention: a serving process whose whole device-memory budget has already been
// handed to one pool (the reference sizes its KV pool from cudaMemGetInfo and lets
// LibTorch's caching allocator own the rest), or a step loop that must not meet
// cudaMalloc's device-wide synchronisation.  For them the split-KV scratch of the
// decode kernel lives in the library image itself: a file-scope __device__ array of
// kNoAllocScratchBytes that every GPU which loads the library carries until exit.
// ============================================================================
namespace b200 {
namespace {

constexpr int64_t kNoAllocScratchBytes = 8ll << 20;  // the stated maximum: 8 MiB per GPU
constexpr int64_t kNoAllocStatusBytes = 256;         // tail of the array: the kernel's status words
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

constexpr int kNoAllocMaxDevices = 64;
std::mutex g_noalloc_mu;
void* g_noalloc_ptr[kNoAllocMaxDevices] = {};  // device address of the array, per device

}  // namespace
}  // namespace b200

extern "C" {

int b200_attention_decode_noalloc(void* out, const void* q, int64_t q_stride_token,
                                  int64_t q_stride_head, const void* k_cache, const void* v_cache,
                                  int64_t num_slots, const int32_t* page_table,
                                  int64_t page_table_stride, const int32_t* table_idx,
                                  const int32_t* seq_lens, int batch, int q_heads, int kv_heads,
                                  int head_dim, int page_size, float sm_scale, b200_stream_t stream) {
    using namespace b200;
    B200_CHECK_ARG(batch == 0 || (out && q && k_cache && v_cache && page_table && table_idx && seq_lens),
                   "attention_decode_noalloc: NULL tensor");
    B200_CHECK_ARG(head_dim == kD, "attention_decode_noalloc: head_dim must be 128");
    B200_CHECK_ARG(batch >= 0 && batch <= kMaxBatch, "attention_decode_noalloc: batch must be in [0, 1024]");
    B200_CHECK_ARG(kv_heads >= 1 && kv_heads <= 8 && (8 % kv_heads) == 0,
                   "attention_decode_noalloc: kv_heads (per rank) must be 1, 2, 4 or 8");
    B200_CHECK_ARG(q_heads % kv_heads == 0 && q_heads / kv_heads <= 16,
                   "attention_decode_noalloc: q_heads must be a multiple of kv_heads with group size <= 16");
    B200_CHECK_ARG(page_size >= 1 && (page_size & (page_size - 1)) == 0,
                   "attention_decode_noalloc: page_size must be a power of two");
    B200_CHECK_ARG(q_stride_token % 2 == 0 && q_stride_head % 2 == 0,
                   "attention_decode_noalloc: q strides must be even");
    B200_CHECK_ARG(num_slots > 0, "attention_decode_noalloc: num_slots must be positive");
    if (batch == 0) return B200_OK;

    // The built-in scratch has a fixed size: refuse shapes whose partials do not fit.
    const int64_t usable = kNoAllocScratchBytes - kNoAllocStatusBytes;
    const int64_t need = decode_workspace_bytes(batch, q_heads, kv_heads);
    if (need > usable) {
        set_last_error("attention_decode_noalloc: batch %d with %d q heads / %d kv heads needs %lld bytes of "
                       "scratch, the built-in array holds %lld; use b200_attention_decode with a caller "
                       "workspace instead",
                       batch, q_heads, kv_heads, static_cast<long long>(need), static_cast<long long>(usable));
        return B200_ERR_UNSUPPORTED;
    }

    // Set-up, once per device, with that device current: the array's name is only a host-side
    // handle, so ask the runtime for its device address and hand THAT to the kernel.
    int dev = 0;
    B200_CHECK_CUDA(cudaGetDevice(&dev));
    B200_CHECK_ARG(dev >= 0 && dev < kNoAllocMaxDevices, "attention_decode_noalloc: device index out of range");
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mu);
        if (!g_noalloc_ptr[dev]) {
            void* ptr = nullptr;
            B200_CHECK_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
            g_noalloc_ptr[dev] = ptr;
        }
        scratch = g_noalloc_ptr[dev];
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned char* base = static_cast<unsigned char*>(scratch);
    int* status = reinterpret_cast<int*>(base + usable);
    // The array keeps whatever the previous call left: partial sums are always written before they
    // are read.  The status words in the array's tail are NOT cleared here: they keep the first
    // report until b200_attention_decode_noalloc_status reads it.

    CUtensorMap tk, tv;
    int err = make_kv_tmap(&tk, k_cache, num_slots, kv_heads, page_size);
    if (err != B200_OK) return err;
    err = make_kv_tmap(&tv, v_cache, num_slots, kv_heads, page_size);
    if (err != B200_OK) return err;
    return launch_attention_decode(out, q, q_stride_token, q_stride_head, tk, tv, num_slots, page_table,
                                   page_table_stride, table_idx, seq_lens, batch, q_heads, kv_heads,
                                   page_size, sm_scale, base, usable, status, s);
}

int b200_attention_decode_noalloc_status(int32_t out[2], b200_stream_t stream) {
    using namespace b200;
    B200_CHECK_ARG(out != nullptr, "attention_decode_noalloc_status: out must not be NULL");
    out[0] = out[1] = 0;
    int dev = 0;
    B200_CHECK_CUDA(cudaGetDevice(&dev));
    B200_CHECK_ARG(dev >= 0 && dev < kNoAllocMaxDevices, "attention_decode_noalloc_status: device index out of range");
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mu);
        scratch = g_noalloc_ptr[dev];
    }
    if (!scratch) return B200_OK;  // no call was made on this device yet
    int* status = reinterpret_cast<int*>(static_cast<unsigned char*>(scratch) + kNoAllocScratchBytes - kNoAllocStatusBytes);
    B200_CHECK_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    int host[2] = {0, 0};
    B200_CHECK_CUDA(cudaMemcpy(host, status, sizeof(host), cudaMemcpyDeviceToHost));
    out[0] = host[0];
    out[1] = host[1];
    if (host[0] != 0 || host[1] != 0) B200_CHECK_CUDA(cudaMemset(status, 0, sizeof(host)));
    return B200_OK;
}

}  // extern "C"
