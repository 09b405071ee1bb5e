// Decode-step layer chain: everything between two attention launches as ONE persistent kernel.
//
// For a decode batch (at most 64 tokens) the reference runs, between the attention of layer l and
// the attention of layer l + 1 (src/models/qwen3.cc:21-35, src/models/utils.cc:41-57,
// src/layers/attention_layer.cc:17-51):
//     o_proj -> fused add + RMSNorm -> gate_up_proj -> SwiGLU -> down_proj
//            -> fused add + RMSNorm -> qkv_proj -> QK-norm -> RoPE -> KV store.
// Run as seven launches these are latency chains: each streams a few MB of weights in well under
// the time it takes a kernel to start, exchange its split-K partials and drain.  Here they are
// four PHASES of one launch:
//   * the grid is a set of 8-CTA clusters, one CTA per SM; a cluster takes a 128-feature tile of a
//     phase's weight matrix and splits its K range eight ways (swap-AB tcgen05: the weight tile is
//     the M operand, the tokens are N = 64, the accumulator lives in TMEM);
//   * a producer warp streams the CTA's weight tiles with TMA through a ring of 16 KB slots in the
//     order the phases will use them.  Weights depend on nothing, so the stream runs ahead across
//     phase boundaries and the dependent chain only sees shared-memory latency;
//   * the activation operand of a phase comes from what the previous phase left in global memory:
//     by TMA where that is bf16 already (attention output, activated gate_up output), and for the
//     projections that follow a norm the CTA builds it in shared memory itself as
//     bf16(sum * rstd * norm_weight) from the fp32 sums, which is exactly what the reference's
//     fused add + RMSNorm stores (src/layers/normalization.cu:27-43), so no separate norm pass and
//     no extra barrier is needed;
//   * split-K partials go to the tile's owners through distributed shared memory: the CTA lays
//     its partial tile out per owner in its own shared memory and one thread sends each owner its
//     4 KB with a bulk copy that counts bytes on the owner's mbarrier.  Rank r of the cluster owns
//     tokens 8r..8r+7 of the tile, reduces the eight partials in rank order and runs the phase's
//     epilogue on whole 128-feature rows: residual add (+ partial sums of squares), SwiGLU, or — a qkv tile being
//     exactly one head — QK-norm, RoPE and the store into the paged KV pool;
//   * phases are separated by a grid barrier (one atomic per CTA; bounded wait).
// Every wait is bounded: when one runs out the kernel records the site in the status word, stops
// waiting for anything else and runs to its end on whatever it has (all indices stay in range), so
// nothing hangs and nobody exits while a peer may still write to it.
#include "common.cuh"
#include "kernels.h"
#include "tensormap.cuh"
#include "tcgen05.cuh"

namespace b200 {
namespace {

constexpr int kCluster = 8;     // CTAs per cluster = K split
constexpr int kTile = 128;      // features per unit (UMMA M)
constexpr int kBK = 64;         // elements per k-block (one 128-byte swizzle row)
constexpr int kNT = 64;         // token columns (UMMA N)
constexpr int kTokPerRank = kNT / kCluster;  // 8 tokens owned by each rank
constexpr int kWSlots = 5;
constexpr int kBSlots = 4;
constexpr int kThreads = 192;   // warp 0: weight TMA, warp 1: MMA + TMEM owner, warps 2-5: operand builders / epilogue
constexpr uint32_t kWBytes = kTile * kBK * 2;   // 16 KB
constexpr uint32_t kBBytes = kNT * kBK * 2;     // 8 KB
constexpr uint32_t kXPart = kTile * kTokPerRank * 4;          // one (source rank, accumulator) block: 4 KB
constexpr uint32_t kXchgBytes = kCluster * 2 * kXPart;        // 64 KB
constexpr uint32_t kSendBytes = kCluster * kXPart;             // 32 KB: one accumulator's partial tile, owner-major
constexpr uint32_t kStageBytes = 2 * kTokPerRank * kTile * 4; // 8 KB: reduced sums, token-major
constexpr uint32_t kSmemBytes =
    kWSlots * kWBytes + kBSlots * kBBytes + kXchgBytes + kSendBytes + kStageBytes + 1024;
constexpr uint32_t kTmemCols = 256;  // two accumulator buffers of 2 x 64 columns

enum PhaseKind : int {
    kPhaseNone = 0,
    kPhaseResidual = 1,  // y = W x; residual <- bf16(y) + residual; fp32 sums + partial sums of squares out
    kPhaseGated = 2,     // h = act(W_gate x) * (W_up x)
    kPhaseQkv = 3,       // qkv tile = one head: QK-norm, RoPE, q to the qkv buffer, k / v to the KV pool
    kPhasePlain = 4,     // y = W x
};

struct ChainPhase {
    int kind;
    int units;            // 128-feature tiles (gated: 128 gate rows + the 128 matching up rows)
    int kb_total;         // K / 64
    int b_norm;           // 1: operand = bf16(sums * rstd * norm_w); 0: bf16 rows of b_src
    int up_row_offset;    // gated: row of W where the up half starts
    int64_t ldb;          // row stride of b_src (elements)
    int64_t ldo;          // row stride of out (elements)
    const __nv_bfloat16* b_src;
    const __nv_bfloat16* norm_w;
    __nv_bfloat16* out;   // gated: h; plain: y; qkv: the qkv activation buffer (q heads are written)
};

struct ChainParams {
    ChainPhase ph[4];
    int T;                // tokens (<= 64)
    int hidden;
    float eps;
    int round_first;      // normalise the bf16-rounded sum (Llama wiring) instead of the fp32 sum
    int act;              // 0 SiLU, 1 tanh-GELU
    __nv_bfloat16* residual;  // [T, hidden]
    float* sums;          // [64, hidden] fp32: the values the norm is taken of
    float* ssq;           // [hidden / 128][64] partial sums of squares per tile
    const __nv_bfloat16* q_norm_w;
    const __nv_bfloat16* k_norm_w;
    const float* cos_t;
    const float* sin_t;
    const int32_t* positions;
    const int32_t* out_loc;
    __nv_bfloat16* k_cache;
    __nv_bfloat16* v_cache;
    int q_heads, kv_heads, max_pos;
    int64_t num_slots;
    unsigned* grid_bar;   // [4][2]: arrival count and generation per phase boundary
    int* status;
    unsigned long long wait_limit_ns;
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    return remote;
}
// `bytes` of this CTA's shared memory into a peer's, counted on the peer's mbarrier when they land.
__device__ __forceinline__ void bulk_copy_to_peer(uint32_t remote_dst, uint32_t local_src, uint32_t bytes,
                                                  uint32_t remote_bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(remote_dst),
        "r"(local_src), "r"(bytes), "r"(remote_bar)
        : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the bulk copies issued by this thread have finished READING their source
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_remote(uint32_t remote_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bar_epilogue() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One bounded wait.  After the first time-out of a CTA every later wait gives up at once, so a
// broken launch costs one wait limit, not one per barrier.
struct Waiter {
    volatile int* failed;
    int* status;
    unsigned long long limit;
    __device__ __forceinline__ void wait(uint32_t bar, uint32_t parity, int site, bool cluster_scope = false) const {
        if (cluster_scope ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity)) return;
        const uint64_t t0 = global_timer_ns();
        uint32_t spins = 0;
        while (!(cluster_scope ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity))) {
            if (*failed) return;
            if ((++spins & 0xffu) == 0 && global_timer_ns() - t0 > limit) {
                *failed = 1;
                atomicExch(&status[kStatusTimeout], site);
                return;
            }
        }
    }
};

template <int ACT>
__device__ __forceinline__ float gate_act(float g) {
    if (ACT == 0) return __fdividef(g, 1.0f + __expf(-g));
    return 0.5f * g * (1.0f + tanhf(0.7978845608f * (g + 0.044715f * g * g * g)));
}

template <int ACT>
__global__ void __launch_bounds__(kThreads, 1)
decode_chain_kernel(const __grid_constant__ CUtensorMap tm0, const __grid_constant__ CUtensorMap tm1,
                    const __grid_constant__ CUtensorMap tm2, const __grid_constant__ CUtensorMap tm3,
                    const __grid_constant__ CUtensorMap tmb0, const __grid_constant__ CUtensorMap tmb2,
                    const ChainParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t w_full[kWSlots], w_empty[kWSlots];
    __shared__ __align__(8) uint64_t b_full[kBSlots], b_empty[kBSlots];
    __shared__ __align__(8) uint64_t acc_full[2], acc_empty[2];
    __shared__ __align__(8) uint64_t xchg_full, xchg_free;
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int s_failed;
    __shared__ float s_rstd[kNT];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t w_base = smem_base;
    const uint32_t b_base = w_base + kWSlots * kWBytes;
    const uint32_t x_base = b_base + kBSlots * kBBytes;
    const uint32_t send_base = x_base + kXchgBytes;
    const uint32_t stage_base = send_base + kSendBytes;
    uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
    const float* xbuf = reinterpret_cast<const float*>(smem_al + (x_base - smem_base));
    float* stage = reinterpret_cast<float*>(smem_al + (stage_base - smem_base));

    const uint32_t rank = cluster_rank();
    const int cid = static_cast<int>(blockIdx.x) / kCluster;
    const int nclusters = static_cast<int>(gridDim.x) / kCluster;
    const CUtensorMap* tms[4] = {&tm0, &tm1, &tm2, &tm3};
    const CUtensorMap* tmbs[4] = {&tmb0, nullptr, &tmb2, nullptr};   // bf16 activation operands (phases 0 and 2)

    // K range of this rank in a phase
    auto kb_range = [&](const ChainPhase& ph, int& kb0, int& nkb) {
        const int per = (ph.kb_total + kCluster - 1) / kCluster;
        kb0 = static_cast<int>(rank) * per;
        nkb = max(0, min(kb0 + per, ph.kb_total) - kb0);
    };
    auto accs_of = [](const ChainPhase& ph) { return ph.kind == kPhaseGated ? 2 : 1; };
    // bytes the owners of one unit receive
    auto xchg_tx = [&](const ChainPhase& ph) -> uint32_t { return static_cast<uint32_t>(accs_of(ph)) * kCluster * kXPart; };

    if (threadIdx.x == 0) {
        for (int s = 0; s < kWSlots; ++s) {
            mbar_init(smem_u32(&w_full[s]), 1);
            mbar_init(smem_u32(&w_empty[s]), 1);
        }
        for (int s = 0; s < kBSlots; ++s) {
            mbar_init(smem_u32(&b_full[s]), 1);
            mbar_init(smem_u32(&b_empty[s]), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&acc_full[s]), 1);
            mbar_init(smem_u32(&acc_empty[s]), 128);
        }
        mbar_init(smem_u32(&xchg_full), 1);
        mbar_init(smem_u32(&xchg_free), kCluster);
        s_failed = 0;
        fence_mbar_init();
        // arm the exchange barrier for this cluster's first unit, before any peer can send
        for (int q = 0; q < 4; ++q) {
            if (p.ph[q].kind != kPhaseNone && cid < p.ph[q].units) {
                mbar_arrive_expect_tx(smem_u32(&xchg_full), xchg_tx(p.ph[q]));
                break;
            }
        }
        for (int q = 0; q < 4; ++q) tma_prefetch_desc(tms[q]);
        tma_prefetch_desc(&tmb0);
        tma_prefetch_desc(&tmb2);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();   // every peer's barriers exist before anybody pushes or signals
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    const Waiter W{&s_failed, p.status, p.wait_limit_ns};
    pdl_launch_dependents();

    if (warp == 0) {
        // ---------------- weight producer: runs ahead of the chain, bounded only by the ring ----------
        if (lane == 0) {
            uint32_t it = 0;
            for (int q = 0; q < 4; ++q) {
                const ChainPhase& ph = p.ph[q];
                if (ph.kind == kPhaseNone) continue;
                int kb0, nkb;
                kb_range(ph, kb0, nkb);
                const int na = accs_of(ph);
                for (int u = cid; u < ph.units; u += nclusters) {
                    for (int i = 0; i < nkb; ++i) {
                        for (int a = 0; a < na; ++a, ++it) {
                            const uint32_t s = it % kWSlots;
                            if (it >= kWSlots) W.wait(smem_u32(&w_empty[s]), ((it / kWSlots) - 1) & 1u, 501);
                            const uint32_t bar = smem_u32(&w_full[s]);
                            mbar_arrive_expect_tx(bar, kWBytes);
                            tma_load_2d(w_base + s * kWBytes, tms[q], (kb0 + i) * kBK,
                                        u * kTile + (a ? ph.up_row_offset : 0), bar);
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ------------------------------------------------------------------
        if (lane == 0) {
            const uint32_t idesc = idesc_bf16_m128(kNT);
            uint32_t wit = 0, bit = 0, un = 0;
            for (int q = 0; q < 4; ++q) {
                const ChainPhase& ph = p.ph[q];
                if (ph.kind == kPhaseNone) continue;
                int kb0, nkb;
                kb_range(ph, kb0, nkb);
                const int na = accs_of(ph);
                for (int u = cid; u < ph.units; u += nclusters, ++un) {
                    const uint32_t buf = un & 1u;
                    if (un >= 2) W.wait(smem_u32(&acc_empty[buf]), ((un >> 1) - 1) & 1u, 502);
                    tc_fence_after();
                    const uint32_t acc = tmem_base + buf * 128u;
                    for (int i = 0; i < nkb; ++i, ++bit) {
                        const uint32_t bs = bit % kBSlots;
                        W.wait(smem_u32(&b_full[bs]), (bit / kBSlots) & 1u, 503);
                        const uint32_t ws0 = wit % kWSlots, ws1 = (wit + 1) % kWSlots;
                        W.wait(smem_u32(&w_full[ws0]), (wit / kWSlots) & 1u, 504);
                        if (na == 2) W.wait(smem_u32(&w_full[ws1]), ((wit + 1) / kWSlots) & 1u, 504);
                        tc_fence_after();
                        const uint32_t b0 = b_base + bs * kBBytes;
#pragma unroll
                        for (int k = 0; k < kBK / 16; ++k) {
                            const uint32_t accum = (i > 0 || k > 0) ? 1u : 0u;
                            const uint64_t bdesc = kmajor_sw128_desc(b0 + k * 32);
                            tc_mma_bf16(acc, kmajor_sw128_desc(w_base + ws0 * kWBytes + k * 32), bdesc, idesc, accum);
                            if (na == 2)
                                tc_mma_bf16(acc + kNT, kmajor_sw128_desc(w_base + ws1 * kWBytes + k * 32), bdesc,
                                            idesc, accum);
                        }
                        tc_commit(smem_u32(&w_empty[ws0]));
                        if (na == 2) tc_commit(smem_u32(&w_empty[ws1]));
                        tc_commit(smem_u32(&b_empty[bs]));
                        wit += na;
                    }
                    if (nkb > 0)
                        tc_commit(smem_u32(&acc_full[buf]));
                    else
                        mbar_arrive(smem_u32(&acc_full[buf]));
                }
            }
        }
    } else {
        // ---------------- operand builders + epilogue (128 threads) -------------------------------------
        const int et = threadIdx.x - 64;            // 0..127
        const int qtr = warp & 3;                   // TMEM lane quarter this warp may read
        const int feat = qtr * 32 + lane;           // feature row this thread reads from TMEM
        const int tl = et >> 4;                     // token of this rank this thread finishes (0..7)
        const int fg = et & 15;                     // it finishes features fg*4.. and 64 + fg*4..
        const int tok = static_cast<int>(rank) * kTokPerRank + tl;
        const unsigned half_mask = 0xffffu << (lane & 16);
        const bool tok_valid = tok < p.T;
        const uint32_t xfull_addr = smem_u32(&xchg_full), xfree_addr = smem_u32(&xchg_free);
        uint32_t bit = 0, un = 0;
        unsigned my_gen = 0;        // (thread 0) generation of the boundary it last arrived at
        int prev_phase = -1;
        pdl_wait_prior();           // everything below reads or writes what other kernels own

        for (int q = 0; q < 4; ++q) {
            const ChainPhase& ph = p.ph[q];
            if (ph.kind == kPhaseNone) continue;
            int kb0, nkb;
            kb_range(ph, kb0, nkb);
            const int na = accs_of(ph);
            const bool has_units = cid < ph.units;

            // ---- the phase before this one must be complete on every CTA ----
            if (prev_phase >= 0 && has_units) {
                if (et == 0) {
                    const unsigned* gen = p.grid_bar + 2 * prev_phase + 1;
                    const uint64_t t0 = global_timer_ns();
                    uint32_t spins = 0;
                    while (ld_acquire_gpu(gen) == my_gen) {
                        if (s_failed) break;
                        if ((++spins & 0xffu) == 0 && global_timer_ns() - t0 > p.wait_limit_ns) {
                            s_failed = 1;
                            atomicExch(&p.status[kStatusTimeout], 505);
                            break;
                        }
                    }
                }
                bar_epilogue();
            }

            if (has_units && ph.b_norm) {
                // rstd of every token from the per-tile partial sums of squares, in tile order
                if (et < kNT) {
                    float tot = 0.f;
                    const int tiles = p.hidden / kTile;
                    for (int t = 0; t < tiles; ++t) tot += __ldcg(p.ssq + t * kNT + et);
                    s_rstd[et] = rsqrtf(tot / static_cast<float>(p.hidden) + p.eps);
                }
                bar_epilogue();
            }

            for (int u = cid; u < ph.units; u += nclusters, ++un) {
                // ---- this rank's slice of the activation operand: [64 tokens][64 k] per k-block ----
                if (!ph.b_norm) {
                    // bf16 rows in global memory: TMA (rows past T read as zero).  What an earlier phase of
                    // this launch wrote with ordinary stores is ordered before these reads by the grid
                    // barrier plus a proxy fence on either side.
                    if (et == 0) {
                        fence_proxy_async_all();
                        for (int i = 0; i < nkb; ++i) {
                            const uint32_t bs = (bit + i) % kBSlots;
                            if (bit + i >= kBSlots) W.wait(smem_u32(&b_empty[bs]), (((bit + i) / kBSlots) - 1) & 1u, 506);
                            const uint32_t bar = smem_u32(&b_full[bs]);
                            mbar_arrive_expect_tx(bar, kBBytes);
                            tma_load_2d(b_base + bs * kBBytes, tmbs[q], (kb0 + i) * kBK, 0, bar);
                        }
                    }
                    bit += nkb;
                } else {
                    // normalised operand, two k-blocks of loads in flight per thread
                    const int c = et & 7;
                    for (int i0 = 0; i0 < nkb; i0 += 2) {
                        const int ni = min(2, nkb - i0);
                        float4 lo[2][4], hi[2][4];
                        uint4 w4[2];
#pragma unroll
                        for (int ii = 0; ii < 2; ++ii) {
                            if (ii >= ni) continue;
                            const int k0 = (kb0 + i0 + ii) * kBK;
                            w4[ii] = __ldg(reinterpret_cast<const uint4*>(ph.norm_w + k0 + c * 8));
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const int t = (et >> 3) + 16 * j;
                                if (t < p.T) {
                                    const float4* sp = reinterpret_cast<const float4*>(p.sums + static_cast<int64_t>(t) * p.hidden + k0 + c * 8);
                                    lo[ii][j] = __ldcg(sp);
                                    hi[ii][j] = __ldcg(sp + 1);
                                }
                            }
                        }
#pragma unroll
                        for (int ii = 0; ii < 2; ++ii) {
                            if (ii >= ni) continue;
                            const uint32_t bs = (bit + ii) % kBSlots;
                            if (bit + ii >= kBSlots) W.wait(smem_u32(&b_empty[bs]), (((bit + ii) / kBSlots) - 1) & 1u, 506);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const int t = (et >> 3) + 16 * j;
                                uint4 packed = make_uint4(0u, 0u, 0u, 0u);
                                if (t < p.T) {
                                    const float rs = s_rstd[t];
                                    const float4 l = lo[ii][j], h = hi[ii][j];
                                    packed.x = pack_bf16(l.x * rs * bf16_lo(w4[ii].x), l.y * rs * bf16_hi(w4[ii].x));
                                    packed.y = pack_bf16(l.z * rs * bf16_lo(w4[ii].y), l.w * rs * bf16_hi(w4[ii].y));
                                    packed.z = pack_bf16(h.x * rs * bf16_lo(w4[ii].z), h.y * rs * bf16_hi(w4[ii].z));
                                    packed.w = pack_bf16(h.z * rs * bf16_lo(w4[ii].w), h.w * rs * bf16_hi(w4[ii].w));
                                }
                                const uint32_t dst = b_base + bs * kBBytes + static_cast<uint32_t>(t) * 128u +
                                                     (static_cast<uint32_t>(c ^ (t & 7)) << 4);
                                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(packed.x),
                                             "r"(packed.y), "r"(packed.z), "r"(packed.w)
                                             : "memory");
                            }
                        }
                        fence_proxy_async_smem();
                        bar_epilogue();
                        if (et == 0)
                            for (int ii = 0; ii < ni; ++ii) mbar_arrive(smem_u32(&b_full[(bit + ii) % kBSlots]));
                        bit += ni;
                    }
                }

                // ---- partial sums: TMEM -> own shared memory, owner-major -> bulk copies to the owners ----
                const uint32_t buf = un & 1u;
                W.wait(smem_u32(&acc_full[buf]), (un >> 1) & 1u, 507);
                tc_fence_after();
                for (int a = 0; a < na; ++a) {
                    uint32_t v0[32], v1[32];
                    if (nkb > 0) {
                        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(qtr * 32) << 16) + buf * 128u +
                                               static_cast<uint32_t>(a) * kNT;
                        tmem_ld_32x32b_x32(taddr, v0);
                        tmem_ld_32x32b_x32(taddr + 32, v1);
                        tmem_ld_wait();
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v0[j] = v1[j] = 0u;
                    }
                    // the send buffer is free once the previous bulk copies have read it (thread 0 issued them)
                    if (et == 0) bulk_wait_read();
                    bar_epilogue();
#pragma unroll
                    for (int o = 0; o < kCluster; ++o) {
                        const uint32_t dst = send_base + (static_cast<uint32_t>(o) * kTile + static_cast<uint32_t>(feat)) * 32u;
                        const uint32_t* src = o < 4 ? &v0[8 * o] : &v1[8 * (o - 4)];
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(src[0]), "r"(src[1]),
                                     "r"(src[2]), "r"(src[3])
                                     : "memory");
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + 16), "r"(src[4]), "r"(src[5]),
                                     "r"(src[6]), "r"(src[7])
                                     : "memory");
                    }
                    fence_proxy_async_smem();
                    bar_epilogue();
                    if (et == 0) {
                        // every owner's buffer must be free of the previous unit (each said so when it was done)
                        if (a == 0 && un >= 1) W.wait(xfree_addr, (un - 1) & 1u, 508, true);
                        const uint32_t off = x_base + (rank * 2u + static_cast<uint32_t>(a)) * kXPart;
                        for (int o = 0; o < kCluster; ++o)
                            bulk_copy_to_peer(map_to_rank(off, o), send_base + static_cast<uint32_t>(o) * kXPart, kXPart,
                                              map_to_rank(xfull_addr, o));
                        bulk_commit();
                    }
                }
                tc_fence_before();
                mbar_arrive(smem_u32(&acc_empty[buf]));

                // ---- owner: sum the eight partials in rank order, hand the sums over token-major ----
                W.wait(xfull_addr, un & 1u, 509);
                for (int a = 0; a < na; ++a) {
                    float s8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int r = 0; r < kCluster; ++r) {
                        const float4* xp = reinterpret_cast<const float4*>(xbuf + ((r * 2 + a) * kTile + feat) * 8);
                        const float4 lo = xp[0], hi = xp[1];
                        s8[0] += lo.x; s8[1] += lo.y; s8[2] += lo.z; s8[3] += lo.w;
                        s8[4] += hi.x; s8[5] += hi.y; s8[6] += hi.z; s8[7] += hi.w;
                    }
#pragma unroll
                    for (int t = 0; t < 8; ++t) stage[(a * 8 + t) * kTile + feat] = s8[t];
                }
                bar_epilogue();

                // ---- epilogue on whole rows: token `tok`, features fg*4.. and 64 + fg*4.. of tile u ----
                const float4 xa4 = *reinterpret_cast<const float4*>(stage + tl * kTile + fg * 4);
                const float4 xb4 = *reinterpret_cast<const float4*>(stage + tl * kTile + 64 + fg * 4);
                float xa[4] = {xa4.x, xa4.y, xa4.z, xa4.w}, xb[4] = {xb4.x, xb4.y, xb4.z, xb4.w};
                const int nA = u * kTile + fg * 4, nB = nA + 64;
                if (ph.kind == kPhaseResidual) {
                    float ss = 0.f;
                    if (tok_valid) {
                        __nv_bfloat16* rrow = p.residual + static_cast<int64_t>(tok) * p.hidden;
                        const uint2 ra = __ldcg(reinterpret_cast<const uint2*>(rrow + nA));
                        const uint2 rb = __ldcg(reinterpret_cast<const uint2*>(rrow + nB));
                        const float resa[4] = {bf16_lo(ra.x), bf16_hi(ra.x), bf16_lo(ra.y), bf16_hi(ra.y)};
                        const float resb[4] = {bf16_lo(rb.x), bf16_hi(rb.x), bf16_lo(rb.y), bf16_hi(rb.y)};
                        float va[4], vb[4];
                        uint32_t pa[2], pb[2];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            va[e] = round_bf16(xa[e]) + resa[e];   // the projection's bf16 output + residual, in fp32
                            vb[e] = round_bf16(xb[e]) + resb[e];
                        }
                        pa[0] = pack_bf16(va[0], va[1]); pa[1] = pack_bf16(va[2], va[3]);
                        pb[0] = pack_bf16(vb[0], vb[1]); pb[1] = pack_bf16(vb[2], vb[3]);
                        if (p.round_first) {
                            va[0] = bf16_lo(pa[0]); va[1] = bf16_hi(pa[0]); va[2] = bf16_lo(pa[1]); va[3] = bf16_hi(pa[1]);
                            vb[0] = bf16_lo(pb[0]); vb[1] = bf16_hi(pb[0]); vb[2] = bf16_lo(pb[1]); vb[3] = bf16_hi(pb[1]);
                        }
                        *reinterpret_cast<uint2*>(rrow + nA) = make_uint2(pa[0], pa[1]);
                        *reinterpret_cast<uint2*>(rrow + nB) = make_uint2(pb[0], pb[1]);
                        float* srow = p.sums + static_cast<int64_t>(tok) * p.hidden;
                        *reinterpret_cast<float4*>(srow + nA) = make_float4(va[0], va[1], va[2], va[3]);
                        *reinterpret_cast<float4*>(srow + nB) = make_float4(vb[0], vb[1], vb[2], vb[3]);
#pragma unroll
                        for (int e = 0; e < 4; ++e) ss += va[e] * va[e] + vb[e] * vb[e];
                    }
#pragma unroll
                    for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(half_mask, ss, o);
                    if (fg == 0) p.ssq[u * kNT + tok] = ss;
                } else if (ph.kind == kPhasePlain) {
                    if (tok_valid) {
                        __nv_bfloat16* orow = ph.out + static_cast<int64_t>(tok) * ph.ldo;
                        *reinterpret_cast<uint2*>(orow + nA) = make_uint2(pack_bf16(xa[0], xa[1]), pack_bf16(xa[2], xa[3]));
                        *reinterpret_cast<uint2*>(orow + nB) = make_uint2(pack_bf16(xb[0], xb[1]), pack_bf16(xb[2], xb[3]));
                    }
                } else if (ph.kind == kPhaseGated) {
                    const float4 ua4 = *reinterpret_cast<const float4*>(stage + (8 + tl) * kTile + fg * 4);
                    const float4 ub4 = *reinterpret_cast<const float4*>(stage + (8 + tl) * kTile + 64 + fg * 4);
                    const float ua[4] = {ua4.x, ua4.y, ua4.z, ua4.w}, ub[4] = {ub4.x, ub4.y, ub4.z, ub4.w};
                    if (tok_valid) {
                        float ha[4], hb[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            // both halves are rounded to bf16 where the unfused projection stores them
                            ha[e] = gate_act<ACT>(round_bf16(xa[e])) * round_bf16(ua[e]);
                            hb[e] = gate_act<ACT>(round_bf16(xb[e])) * round_bf16(ub[e]);
                        }
                        __nv_bfloat16* orow = ph.out + static_cast<int64_t>(tok) * ph.ldo;
                        *reinterpret_cast<uint2*>(orow + nA) = make_uint2(pack_bf16(ha[0], ha[1]), pack_bf16(ha[2], ha[3]));
                        *reinterpret_cast<uint2*>(orow + nB) = make_uint2(pack_bf16(hb[0], hb[1]), pack_bf16(hb[2], hb[3]));
                    }
                } else {  // kPhaseQkv: tile u is head u of the packed [q heads | k heads | v heads] projection
                    const bool is_q = u < p.q_heads;
                    const bool is_k = !is_q && u < p.q_heads + p.kv_heads;
                    const int kvh = is_q ? 0 : (is_k ? u - p.q_heads : u - p.q_heads - p.kv_heads);
                    float x1[4], x2[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        x1[e] = round_bf16(xa[e]);
                        x2[e] = round_bf16(xb[e]);
                    }
                    int64_t slot = -1;
                    if (!is_q && tok_valid) {
                        slot = p.out_loc[tok];
                        if (slot < 0 || slot >= p.num_slots) {
                            if (fg == 0) atomicExch(&p.status[kStatusBadIndex], static_cast<int>(slot) + 1);
                            slot = -1;
                        }
                    }
                    if (!is_q && !is_k) {
                        if (slot >= 0) {
                            __nv_bfloat16* dst = p.v_cache + (slot * p.kv_heads + kvh) * kTile;
                            *reinterpret_cast<uint2*>(dst + fg * 4) = make_uint2(pack_bf16(x1[0], x1[1]), pack_bf16(x1[2], x1[3]));
                            *reinterpret_cast<uint2*>(dst + 64 + fg * 4) = make_uint2(pack_bf16(x2[0], x2[1]), pack_bf16(x2[2], x2[3]));
                        }
                    } else {
                        const __nv_bfloat16* nw = is_q ? p.q_norm_w : p.k_norm_w;
                        if (nw != nullptr) {   // per-head RMSNorm (uniform over the block: no divergence at the shuffles)
                            float ss = 0.f;
#pragma unroll
                            for (int e = 0; e < 4; ++e) ss += x1[e] * x1[e] + x2[e] * x2[e];
#pragma unroll
                            for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(half_mask, ss, o);
                            const float scale = rsqrtf(ss / static_cast<float>(kTile) + p.eps);
                            const uint2 wa = __ldg(reinterpret_cast<const uint2*>(nw + fg * 4));
                            const uint2 wb = __ldg(reinterpret_cast<const uint2*>(nw + 64 + fg * 4));
                            const float wfa[4] = {bf16_lo(wa.x), bf16_hi(wa.x), bf16_lo(wa.y), bf16_hi(wa.y)};
                            const float wfb[4] = {bf16_lo(wb.x), bf16_hi(wb.x), bf16_lo(wb.y), bf16_hi(wb.y)};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                x1[e] = round_bf16(x1[e] * scale * wfa[e]);   // where the unfused norm stores its result
                                x2[e] = round_bf16(x2[e] * scale * wfb[e]);
                            }
                        }
                        if (tok_valid) {
                            int pos = p.positions[tok];
                            if (pos < 0 || pos >= p.max_pos) {
                                if (fg == 0) atomicExch(&p.status[kStatusBadIndex], pos + 1);
                                pos = min(max(pos, 0), p.max_pos - 1);
                            }
                            const float4 c4 = __ldg(reinterpret_cast<const float4*>(p.cos_t + static_cast<int64_t>(pos) * 64 + fg * 4));
                            const float4 s4 = __ldg(reinterpret_cast<const float4*>(p.sin_t + static_cast<int64_t>(pos) * 64 + fg * 4));
                            const float cs[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
                            float oa[4], ob[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                oa[e] = x1[e] * cs[e] - x2[e] * sn[e];
                                ob[e] = x2[e] * cs[e] + x1[e] * sn[e];
                            }
                            const uint2 pa = make_uint2(pack_bf16(oa[0], oa[1]), pack_bf16(oa[2], oa[3]));
                            const uint2 pb = make_uint2(pack_bf16(ob[0], ob[1]), pack_bf16(ob[2], ob[3]));
                            if (is_q) {
                                __nv_bfloat16* dst = ph.out + static_cast<int64_t>(tok) * ph.ldo + u * kTile;
                                *reinterpret_cast<uint2*>(dst + fg * 4) = pa;
                                *reinterpret_cast<uint2*>(dst + 64 + fg * 4) = pb;
                            } else if (slot >= 0) {
                                __nv_bfloat16* dst = p.k_cache + (slot * p.kv_heads + kvh) * kTile;
                                *reinterpret_cast<uint2*>(dst + fg * 4) = pa;
                                *reinterpret_cast<uint2*>(dst + 64 + fg * 4) = pb;
                            }
                        }
                    }
                }

                // ---- this CTA's exchange buffer is free again: arm it for the next unit, then tell the cluster ----
                bar_epilogue();
                if (et == 0) {
                    int nq = q;
                    if (u + nclusters >= ph.units) {
                        for (nq = q + 1; nq < 4; ++nq)
                            if (p.ph[nq].kind != kPhaseNone && cid < p.ph[nq].units) break;
                    }
                    if (nq < 4) mbar_arrive_expect_tx(xfull_addr, xchg_tx(p.ph[nq]));
                    for (int o = 0; o < kCluster; ++o) mbar_arrive_remote(map_to_rank(xfree_addr, o));
                }
            }

            // ---- end of the phase: arrive at its grid barrier (unless it is the last phase) ----
            bool more = false;
            for (int nq = q + 1; nq < 4; ++nq) more = more || p.ph[nq].kind != kPhaseNone;
            if (more) {
                fence_proxy_async_all();   // this phase's global stores may be read by TMA in the next one
                bar_epilogue();
                if (et == 0) {
                    unsigned* cnt = p.grid_bar + 2 * q;
                    unsigned* gen = cnt + 1;
                    my_gen = *reinterpret_cast<volatile unsigned*>(gen);
                    __threadfence();
                    const unsigned old = atomicAdd(cnt, 1u);
                    if (old == gridDim.x - 1) {
                        *reinterpret_cast<volatile unsigned*>(cnt) = 0u;
                        __threadfence();
                        atomicAdd(gen, 1u);
                    }
                }
            }
            prev_phase = q;
        }
    }

    // ---------------- teardown: nobody leaves while a peer may still write to it ----------------------
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace

int decode_chain_max_grid() {
    // Every CTA of the grid must be resident at once (the phases are separated by grid barriers):
    // ask how many 8-CTA clusters of this kernel the device can hold.
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (cached[dev] != 0) return cached[dev] > 0 ? cached[dev] : 0;
    auto kernel = decode_chain_kernel<0>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemBytes)) !=
        cudaSuccess) {
        cudaGetLastError();
        cached[dev] = -1;
        return 0;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count() / kCluster * kCluster);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = kCluster;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess) {
        cudaGetLastError();
        clusters = 0;
    }
    const int cap = sm_count() / kCluster;
    if (clusters > cap) clusters = cap;
    cached[dev] = clusters >= 8 ? clusters * kCluster : -1;   // fewer than 8 clusters: not worth it
    return cached[dev] > 0 ? cached[dev] : 0;
}

int64_t decode_chain_scratch_bytes(int hidden) {
    // fp32 sums [64, hidden] | partial sums of squares [hidden / 128][64] | grid barrier words
    return static_cast<int64_t>(kNT) * hidden * 4 + static_cast<int64_t>(hidden / kTile) * kNT * 4 + 256;
}

bool decode_chain_supported(int tokens, int hidden, int q_heads, int kv_heads, int head_dim, int inter,
                            bool has_bias) {
    return tokens >= 1 && tokens <= kNT && head_dim == kTile && hidden % kTile == 0 && hidden % kBK == 0 &&
           inter % kTile == 0 && q_heads >= 1 && kv_heads >= 1 && !has_bias && decode_chain_max_grid() > 0;
}

int launch_decode_chain(const DecodeChainArgs& a, cudaStream_t stream) {
    const int grid = decode_chain_max_grid();
    if (grid <= 0) {
        set_last_error("decode chain: the device cannot hold eight resident clusters of the kernel");
        return B200_ERR_UNSUPPORTED;
    }
    if (!decode_chain_supported(a.tokens, a.hidden, a.q_heads, a.kv_heads, 128, a.inter, false)) {
        set_last_error("decode chain: unsupported shape (tokens %d, hidden %d, intermediate %d)", a.tokens, a.hidden,
                       a.inter);
        return B200_ERR_UNSUPPORTED;
    }
    ChainParams p = {};
    CUtensorMap tm[4];
    const int qd = a.q_heads * kTile, qkv_dim = (a.q_heads + 2 * a.kv_heads) * kTile;
    auto wmap = [&](int i, const void* w, int N, int K) {
        return cached_tmap(&tm[i], w, static_cast<uint64_t>(K), static_cast<uint64_t>(N),
                           static_cast<uint64_t>(K) * 2, kBK, kTile);
    };
    uint8_t* scratch = static_cast<uint8_t*>(a.scratch);
    p.sums = reinterpret_cast<float*>(scratch);
    p.ssq = p.sums + static_cast<int64_t>(kNT) * a.hidden;
    p.grid_bar = reinterpret_cast<unsigned*>(p.ssq + static_cast<int64_t>(a.hidden / kTile) * kNT);
    int err;
    // phase 0: o_proj (+ residual)
    if ((err = wmap(0, a.w_o, a.hidden, qd)) != B200_OK) return err;
    p.ph[0].kind = kPhaseResidual;
    p.ph[0].units = a.hidden / kTile;
    p.ph[0].kb_total = qd / kBK;
    p.ph[0].b_src = static_cast<const __nv_bfloat16*>(a.attn_out);
    p.ph[0].ldb = qd;
    CUtensorMap tmb[2];
    if ((err = cached_tmap(&tmb[0], a.attn_out, static_cast<uint64_t>(qd), static_cast<uint64_t>(a.tokens),
                           static_cast<uint64_t>(qd) * 2, kBK, kNT)) != B200_OK)
        return err;
    if ((err = cached_tmap(&tmb[1], a.mlp_act, static_cast<uint64_t>(a.inter), static_cast<uint64_t>(a.tokens),
                           static_cast<uint64_t>(a.inter) * 2, kBK, kNT)) != B200_OK)
        return err;
    // phase 1: gate_up of normalised sums
    if ((err = wmap(1, a.w_gate_up, 2 * a.inter, a.hidden)) != B200_OK) return err;
    p.ph[1].kind = kPhaseGated;
    p.ph[1].units = a.inter / kTile;
    p.ph[1].kb_total = a.hidden / kBK;
    p.ph[1].b_norm = 1;
    p.ph[1].norm_w = static_cast<const __nv_bfloat16*>(a.post_norm_w);
    p.ph[1].up_row_offset = a.inter;
    p.ph[1].out = static_cast<__nv_bfloat16*>(a.mlp_act);
    p.ph[1].ldo = a.inter;
    // phase 2: down (+ residual, or plain for the last layer)
    if ((err = wmap(2, a.w_down, a.hidden, a.inter)) != B200_OK) return err;
    p.ph[2].kind = a.w_qkv_next ? kPhaseResidual : kPhasePlain;
    p.ph[2].units = a.hidden / kTile;
    p.ph[2].kb_total = a.inter / kBK;
    p.ph[2].b_src = static_cast<const __nv_bfloat16*>(a.mlp_act);
    p.ph[2].ldb = a.inter;
    p.ph[2].out = static_cast<__nv_bfloat16*>(a.x_out);
    p.ph[2].ldo = a.hidden;
    // phase 3: the next layer's qkv of normalised sums, QK-norm, RoPE, KV store
    if (a.w_qkv_next) {
        if ((err = wmap(3, a.w_qkv_next, qkv_dim, a.hidden)) != B200_OK) return err;
        p.ph[3].kind = kPhaseQkv;
        p.ph[3].units = qkv_dim / kTile;
        p.ph[3].kb_total = a.hidden / kBK;
        p.ph[3].b_norm = 1;
        p.ph[3].norm_w = static_cast<const __nv_bfloat16*>(a.next_input_norm_w);
        p.ph[3].out = static_cast<__nv_bfloat16*>(a.qkv_out);
        p.ph[3].ldo = qkv_dim;
    } else {
        tm[3] = tm[0];
    }
    p.T = a.tokens;
    p.hidden = a.hidden;
    p.eps = a.eps;
    p.round_first = a.round_first ? 1 : 0;
    p.act = a.gelu ? 1 : 0;
    p.residual = static_cast<__nv_bfloat16*>(a.residual);
    p.q_norm_w = static_cast<const __nv_bfloat16*>(a.q_norm_w);
    p.k_norm_w = static_cast<const __nv_bfloat16*>(a.k_norm_w);
    p.cos_t = a.cos_t;
    p.sin_t = a.sin_t;
    p.positions = a.positions;
    p.out_loc = a.out_loc;
    p.k_cache = static_cast<__nv_bfloat16*>(a.k_cache_next);
    p.v_cache = static_cast<__nv_bfloat16*>(a.v_cache_next);
    p.q_heads = a.q_heads;
    p.kv_heads = a.kv_heads;
    p.max_pos = a.max_pos;
    p.num_slots = a.num_slots;
    p.status = a.status;
    p.wait_limit_ns = 2000000000ull;
    auto kernel = a.gelu ? decode_chain_kernel<1> : decode_chain_kernel<0>;
    B200_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kSmemBytes)));
    B200_CHECK_CUDA(launch_kernel(kernel, dim3(grid), dim3(kThreads), kSmemBytes, stream, dim3(kCluster, 1, 1), tm[0],
                                  tm[1], tm[2], tm[3], tmb[0], tmb[1], p));
    return B200_OK;
}

}  // namespace b200

extern "C" {

int b200_decode_chain_grid(void) { return b200::decode_chain_max_grid(); }

}  // extern "C"
