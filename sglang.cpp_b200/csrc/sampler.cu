// Token selection from logits: greedy argmax and the sort-free temperature / top-k / top-p sampler
// (a full-resolution count histogram of the 16-bit keys in shared memory).
#include "common.cuh"
#include "kernels.h"

namespace b200 {
namespace {

struct MaxIdx {
    float v;
    int i;
};

__device__ __forceinline__ MaxIdx better(MaxIdx a, MaxIdx b) {
    // Larger value wins; on equal values the smaller index wins (first occurrence).
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

// A cluster of kArgmaxCluster CTAs per row (one CTA for short rows), each scanning a slice with
// 16-byte loads; the slices' winners meet in the first CTA's shared memory.  Larger value wins,
// first index on ties, so the result does not depend on how the row is cut.
constexpr int kArgmaxCluster = 8;

__device__ __forceinline__ void emit_token(int32_t* out, const TokenWriteBack& wb, int row, int tok) {
    out[row] = tok;
    if (wb.pool != nullptr && row < wb.count) {
        const int64_t r = wb.table_idx[row], p = wb.write_pos[row];
        if (r >= 0 && r < wb.rows && p >= 0 && p < wb.cols) wb.pool[r * wb.stride + p] = tok;
    }
}

__global__ void __launch_bounds__(512)
argmax_bf16_kernel(int32_t* __restrict__ out, const __nv_bfloat16* __restrict__ logits, int vocab,
                   int64_t ld, int ncta, const TokenWriteBack wb) {
    __shared__ float s_v[16];
    __shared__ int s_i[16];
    __shared__ float s_cv[kArgmaxCluster];
    __shared__ int s_ci[kArgmaxCluster];
    pdl_launch_dependents();
    pdl_wait_prior();
    const int row_id = blockIdx.x / ncta, rank = blockIdx.x % ncta;
    const __nv_bfloat16* row = logits + static_cast<int64_t>(row_id) * ld;
    MaxIdx best{-INFINITY, 0x7fffffff};
    const int nvec = vocab >> 3;
    const int per = (nvec + ncta - 1) / ncta;
    const int v_begin = rank * per, v_end = min(nvec, v_begin + per);
    const uint4* rv = reinterpret_cast<const uint4*>(row);
    for (int v = v_begin + threadIdx.x; v < v_end; v += blockDim.x) {
        const uint4 a = rv[v];
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            best = better(best, MaxIdx{bf16_lo(w[j]), v * 8 + 2 * j});
            best = better(best, MaxIdx{bf16_hi(w[j]), v * 8 + 2 * j + 1});
        }
    }
    if (rank == ncta - 1)
        for (int i = nvec * 8 + threadIdx.x; i < vocab; i += blockDim.x)
            best = better(best, MaxIdx{__bfloat162float(row[i]), i});
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        MaxIdx other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
        s_v[warp] = best.v;
        s_i[warp] = best.i;
    }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        best = lane < nw ? MaxIdx{s_v[lane], s_i[lane]} : MaxIdx{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            MaxIdx other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
            best = better(best, other);
        }
        if (ncta == 1) {
            if (lane == 0) emit_token(out, wb, row_id, best.i == 0x7fffffff ? 0 : best.i);
        } else if (lane == 0) {
            // hand this slice's winner to the first CTA of the cluster
            uint32_t rv_addr, ri_addr;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rv_addr) : "r"(smem_u32(&s_cv[rank])), "r"(0));
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ri_addr) : "r"(smem_u32(&s_ci[rank])), "r"(0));
            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(rv_addr), "f"(best.v) : "memory");
            asm volatile("st.shared::cluster.s32 [%0], %1;" ::"r"(ri_addr), "r"(best.i) : "memory");
        }
    }
    if (ncta > 1) {
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (rank == 0 && threadIdx.x == 0) {
            MaxIdx b0{-INFINITY, 0x7fffffff};
            for (int r = 0; r < ncta; ++r) b0 = better(b0, MaxIdx{s_cv[r], s_ci[r]});
            emit_token(out, wb, row_id, b0.i == 0x7fffffff ? 0 : b0.i);
        }
    }
}

}  // namespace

int launch_argmax(int32_t* out, const void* logits, int rows, int vocab, int64_t ld,
                  cudaStream_t stream, const TokenWriteBack* write_back) {
    if (rows == 0) return B200_OK;
    const int ncta = vocab >= 32768 ? kArgmaxCluster : 1;
    B200_CHECK_CUDA(launch_kernel(argmax_bf16_kernel, dim3(rows * ncta), dim3(512), 0, stream, dim3(ncta, 1, 1),
                                  out, static_cast<const __nv_bfloat16*>(logits), vocab, ld, ncta,
                                  write_back ? *write_back : TokenWriteBack{}));
    return B200_OK;
}

}  // namespace b200

extern "C" {

int b200_argmax(int32_t* out, const void* logits, int rows, int vocab, int64_t ld,
                b200_stream_t stream) {
    B200_CHECK_ARG(rows >= 0 && vocab > 0 && ld >= vocab, "argmax: bad shape");
    B200_CHECK_ARG(rows == 0 || (out && logits), "argmax: NULL tensor");
    B200_CHECK_ARG(ld % 8 == 0, "argmax: row stride must be a multiple of 8 (16-byte rows)");
    return b200::launch_argmax(out, logits, rows, vocab, ld, static_cast<cudaStream_t>(stream));
}

}  // extern "C"

// ============================================================================
// Temperature / top-k / top-p sampling without a sort.
//
// The logits are bf16, so their order-preserving 16-bit keys take at most 65536 values and equal
// keys are exact ties: a histogram of COUNTS at full key resolution holds everything the filters
// need, because the softmax weight is a function of the key alone,
//     w(key) = exp2((value(key) - max) / T * log2 e)   in 40-bit fixed point,
// so the mass at or above any key is sum(count[key'] * w(key')) and never depends on the order of
// the atomic adds.  The kept set is therefore exact, reproducible and the same on every rank of a
// tensor-parallel group.  It always has the form
//     key > thr   or   (key == thr and it is among the first n_eq such by index),
// which is how sample_row's sort-based definition (src/engine/engine.cc:126-158) reads when ties
// are ordered by index.
//
// A cluster of two CTAs owns a row.  Both read the whole row once (the second read hits L2); the
// first CTA counts the upper half of the key space (non-negative logits), the second the lower
// half, each into a 32768-bin shared-memory histogram - the halves are disjoint, so nothing is
// merged.  Counting at full resolution also spreads the adds: logits crowd into a handful of
// exponents, but into hundreds of distinct bf16 values, so lanes of one warp rarely meet in a bin.
// Every thread then owns 32 consecutive bins in descending key order; one block-wide scan of
// (count, mass) plus the other half's totals tells each thread what lies above its bins, and the one
// thread whose bins hold the k-th largest key (then the one whose bins cross p * Z) walks them and
// posts the threshold to both CTAs.  A last pass in index order, each CTA over half of the row,
// draws from the kept set with a Philox uniform.
// ============================================================================
namespace b200 {
namespace {

constexpr int kSampleThreads = 1024;
constexpr int kSampleWarps = kSampleThreads / 32;
constexpr int kSampleCluster = 2;
constexpr int kHalfBins = 32768;                               // keys per half of the key space
constexpr int kBinsPerThread = kHalfBins / kSampleThreads;     // 32
constexpr int kHistWords = kHalfBins + kHalfBins / 32;         // one pad word per 32 bins: a thread's run of
                                                               // 32 bins starts in a different bank than its neighbour's
constexpr float kFixedOne = 1099511627776.0f;  // 2^40
static_assert(kBinsPerThread == 32, "bin ownership assumes 32 bins per thread");

__device__ __forceinline__ uint32_t order_key(uint32_t bits16) {
    return (bits16 & 0x8000u) ? (~bits16 & 0xffffu) : (bits16 | 0x8000u);
}
__device__ __forceinline__ float key_to_float(uint32_t key) {
    const uint32_t bits = (key & 0x8000u) ? (key & 0x7fffu) : (~key & 0xffffu);
    return __uint_as_float(bits << 16);
}

// Philox4x32-10 (Salmon et al., SC'11); returns 4 x 32 random bits.
__device__ __forceinline__ uint4 philox4x32(uint4 ctr, uint2 key) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, ctr.x), lo0 = 0xD2511F53u * ctr.x;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, ctr.z), lo1 = 0xCD9E8D57u * ctr.z;
        ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
        key.x += 0x9E3779B9u;
        key.y += 0xBB67AE85u;
    }
    return ctr;
}

typedef unsigned long long u64;

// One per CTA; the peer writes its halves of the arrays, the deciding threads write the thresholds
// into both copies, and every read after a cluster barrier is local.
struct SampleMeet {
    uint32_t cnt_total[kSampleCluster];   // keys counted by each half of the key space
    u64 mass_total[kSampleCluster];
    uint32_t thr_k;                       // top-k: threshold key, kept ties, mass of the kept set
    int n_eq_k;
    u64 z_k;
    uint32_t thr_p;                       // after top-p
    int n_eq_p;
    int eqs[kSampleCluster];              // index halves: keys equal to thr, mass above thr
    u64 gts[kSampleCluster];
};

__device__ __forceinline__ uint32_t map_to_rank(const void* p, int r) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_u32(p)), "r"(r));
    return a;
}
__device__ __forceinline__ void post_u32(const void* p, uint32_t v) {   // into both CTAs' copies
#pragma unroll
    for (int r = 0; r < kSampleCluster; ++r)
        asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(map_to_rank(p, r)), "r"(v) : "memory");
}
__device__ __forceinline__ void post_u64(const void* p, u64 v) {
#pragma unroll
    for (int r = 0; r < kSampleCluster; ++r)
        asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(map_to_rank(p, r)), "l"(v) : "memory");
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__global__ void __launch_bounds__(kSampleThreads, 1)
sample_kernel(int32_t* __restrict__ out, const __nv_bfloat16* __restrict__ logits, int vocab,
              int64_t ld, const float* __restrict__ temps, const int32_t* __restrict__ top_k,
              const float* __restrict__ top_p, const uint64_t* __restrict__ seeds,
              const uint64_t* __restrict__ step_index_ptr, uint64_t step_index_arg,
              uint8_t* __restrict__ mask, const TokenWriteBack wb) {
    extern __shared__ __align__(16) uint32_t s_hist[];   // kHistWords counters; bin b lives at b + b / 32
    __shared__ SampleMeet meet;
    __shared__ u64 s_wm[kSampleWarps];
    __shared__ uint32_t s_wc[kSampleWarps];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row = blockIdx.x / kSampleCluster, rank = blockIdx.x % kSampleCluster;
    const uint32_t own_half = rank == 0 ? 1u : 0u;       // the first CTA counts keys >= 0x8000
    for (int i = tid; i < kHistWords / 4; i += kSampleThreads)
        reinterpret_cast<uint4*>(s_hist)[i] = make_uint4(0u, 0u, 0u, 0u);
    pdl_launch_dependents();
    pdl_wait_prior();
    const __nv_bfloat16* rowp = logits + static_cast<int64_t>(row) * ld;
    uint8_t* mrow = mask ? mask + static_cast<int64_t>(row) * vocab : nullptr;
    const float T = temps[row];
    const bool greedy = T <= 1.0000001e-6f;
    const int nvec = vocab >> 3;                          // the row is whole 16-byte vectors
    const uint4* rv = reinterpret_cast<const uint4*>(rowp);

    // Exclusive scan over the block, in thread order, of a (count, mass) pair; totals on every thread.
    auto block_scan = [&](uint32_t c, u64 m, uint32_t& c_excl, u64& m_excl, uint32_t& c_tot, u64& m_tot) {
        uint32_t ic = c;
        u64 im = m;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t tc = __shfl_up_sync(0xffffffffu, ic, o);
            const u64 tm = __shfl_up_sync(0xffffffffu, im, o);
            if (lane >= o) {
                ic += tc;
                im += tm;
            }
        }
        __syncthreads();   // the arrays may still be read from an earlier scan
        if (lane == 31) {
            s_wc[warp] = ic;
            s_wm[warp] = im;
        }
        __syncthreads();
        const uint32_t wc = s_wc[lane];
        const u64 wm = s_wm[lane];
        uint32_t pc = wc;
        u64 pm = wm;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t tc = __shfl_up_sync(0xffffffffu, pc, o);
            const u64 tm = __shfl_up_sync(0xffffffffu, pm, o);
            if (lane >= o) {
                pc += tc;
                pm += tm;
            }
        }
        c_tot = __shfl_sync(0xffffffffu, pc, 31);
        m_tot = __shfl_sync(0xffffffffu, pm, 31);
        c_excl = __shfl_sync(0xffffffffu, pc - wc, warp) + ic - c;
        m_excl = __shfl_sync(0xffffffffu, pm - wm, warp) + im - m;
    };

    if (greedy) {
        // Greedy request inside a sampled batch (Sampler::prepare clamps its temperature to 1e-6): the
        // distribution is one-hot on the first maximum.  The first CTA does it alone.
        if (rank != 0) return;
        uint32_t bk = 0;
        int bi = 0x7fffffff;
        for (int v = tid; v < nvec; v += kSampleThreads) {
            const uint4 a = __ldg(rv + v);
            const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t k = order_key((w[j >> 1] >> ((j & 1) * 16)) & 0xffffu);
                if (k > bk) {          // indices grow along a thread's walk: ">" keeps the first maximum
                    bk = k;
                    bi = v * 8 + j;
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const uint32_t ok = __shfl_xor_sync(0xffffffffu, bk, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ok > bk || (ok == bk && oi < bi)) {
                bk = ok;
                bi = oi;
            }
        }
        if (lane == 0) {
            s_wc[warp] = bk;
            s_wm[warp] = static_cast<u64>(bi);
        }
        __syncthreads();
        uint32_t k = s_wc[0];
        int idx = static_cast<int>(s_wm[0]);
        for (int w = 1; w < kSampleWarps; ++w) {
            const uint32_t ok = s_wc[w];
            const int oi = static_cast<int>(s_wm[w]);
            if (ok > k || (ok == k && oi < idx)) {
                k = ok;
                idx = oi;
            }
        }
        if (idx == 0x7fffffff) idx = 0;
        if (tid == 0) emit_token(out, wb, row, idx);
        if (mrow)
            for (int i = tid; i < vocab; i += kSampleThreads) mrow[i] = i == idx ? 1 : 0;
        return;
    }
    __syncthreads();   // the histogram is cleared

    // ---- the whole row once: count this CTA's half of the key space, take the row maximum ----
    uint32_t kmax = 0;
    for (int v0 = tid; v0 < nvec; v0 += 4 * kSampleThreads) {
        uint4 a[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int v = v0 + u * kSampleThreads;
            a[u] = v < nvec ? __ldg(rv + v) : make_uint4(0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu);   // key 0
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint32_t w[4] = {a[u].x, a[u].y, a[u].z, a[u].w};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t k = order_key((w[j >> 1] >> ((j & 1) * 16)) & 0xffffu);
                kmax = max(kmax, k);
                // key 0 is the bf16 pattern 0xFFFF (a NaN), never a logit: it is neither counted nor kept
                if ((k >> 15) == own_half && k != 0u) {
                    const uint32_t b = k & 0x7fffu;
                    atomicAdd(&s_hist[b + (b >> 5)], 1u);
                }
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) kmax = max(kmax, __shfl_xor_sync(0xffffffffu, kmax, o));
    if (lane == 0) s_wc[warp] = kmax;
    __syncthreads();   // the histogram is complete
    kmax = s_wc[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) kmax = max(kmax, __shfl_xor_sync(0xffffffffu, kmax, o));
    const float lmax = key_to_float(kmax);
    const float scale = 1.4426950408889634f / T;
    auto fixed_w = [&](uint32_t key) -> u64 {
        return static_cast<u64>(exp2f((key_to_float(key) - lmax) * scale) * kFixedOne);
    };

    // ---- every thread owns 32 bins in descending key order: thread 0 the largest keys of the half ----
    const uint32_t key_top = (own_half << 15) | static_cast<uint32_t>(kHalfBins - 1 - kBinsPerThread * tid);
    const uint32_t* my_bins = s_hist + 33 * (kSampleThreads - 1 - tid) + 31;   // my_bins[-i]: count of key_top - i
    uint32_t my_cnt = 0;
    u64 my_mass = 0;
#pragma unroll 8
    for (int i = 0; i < kBinsPerThread; ++i) {
        const uint32_t c = *(my_bins - i);
        if (c) {
            my_cnt += c;
            my_mass += static_cast<u64>(c) * fixed_w(key_top - i);
        }
    }
    uint32_t cnt_excl, cnt_tot;
    u64 mass_excl, mass_tot;
    block_scan(my_cnt, my_mass, cnt_excl, mass_excl, cnt_tot, mass_tot);
    if (tid == 0) {
        post_u32(&meet.cnt_total[rank], cnt_tot);
        post_u64(&meet.mass_total[rank], mass_tot);
    }
    cluster_barrier();   // (1) both halves' totals are in both CTAs
    const uint32_t all_cnt = meet.cnt_total[0] + meet.cnt_total[1];
    const u64 all_mass = meet.mass_total[0] + meet.mass_total[1];
    // what lies above this thread's bins: the upper half comes first
    const uint32_t cnt_above = (rank == 0 ? 0u : meet.cnt_total[0]) + cnt_excl;
    const u64 mass_above = (rank == 0 ? 0ull : meet.mass_total[0]) + mass_excl;

    // ---- top-k: the thread whose bins hold the K-th largest key walks them ----
    int K = top_k ? top_k[row] : vocab;
    if (K < 1 || K > vocab) K = vocab;
    const float P = top_p ? top_p[row] : 1.0f;
    const bool want_k = static_cast<uint32_t>(K) < all_cnt;
    uint32_t thr = 0;        // no filter: every counted key is above 0
    int n_eq = 0;
    u64 Z = all_mass;
    if (want_k) {
        if (cnt_above < static_cast<uint32_t>(K) && static_cast<uint32_t>(K) <= cnt_above + my_cnt) {
            uint32_t run_c = cnt_above;
            u64 run_m = mass_above;
            for (int i = 0; i < kBinsPerThread; ++i) {
                const uint32_t c = *(my_bins - i);
                if (!c) continue;
                const uint32_t key = key_top - i;
                const u64 w = fixed_w(key);
                if (run_c + c >= static_cast<uint32_t>(K)) {
                    const uint32_t keep = static_cast<uint32_t>(K) - run_c;
                    post_u32(&meet.thr_k, key);
                    post_u32(&meet.n_eq_k, keep);
                    post_u64(&meet.z_k, run_m + static_cast<u64>(keep) * w);
                    break;
                }
                run_c += c;
                run_m += static_cast<u64>(c) * w;
            }
        }
        cluster_barrier();   // (2)
        thr = meet.thr_k;
        n_eq = meet.n_eq_k;
        Z = meet.z_k;
    }

    // ---- top-p inside the top-k set: the largest key t whose "t and above" mass exceeds P * Z; of the
    //      keys equal to t, as many as still fit under the budget (at least one entry is always kept) ----
    if (P < 1.0f) {
        const u64 budget = static_cast<u64>(static_cast<double>(P) * static_cast<double>(Z));
        // this thread's mass inside the top-k set; the bins above it are untouched by the top-k cut
        const uint32_t key_bottom = key_top - (kBinsPerThread - 1);
        u64 in_set = my_mass;
        if (want_k) {
            if (key_top < thr) {
                in_set = 0;
            } else if (key_bottom <= thr) {
                in_set = 0;
                for (int i = 0; i < kBinsPerThread; ++i) {
                    const uint32_t c = *(my_bins - i), key = key_top - i;
                    if (!c || key < thr) continue;
                    in_set += static_cast<u64>(key == thr ? static_cast<uint32_t>(n_eq) : c) * fixed_w(key);
                }
            }
        }
        if (in_set > 0 && mass_above <= budget && budget < mass_above + in_set) {
            u64 run = mass_above;
            for (int i = 0; i < kBinsPerThread; ++i) {
                const uint32_t c = *(my_bins - i), key = key_top - i;
                if (!c || key < thr) continue;
                const uint32_t c_t = (want_k && key == thr) ? static_cast<uint32_t>(n_eq) : c;
                const u64 w_t = fixed_w(key);
                if (run + static_cast<u64>(c_t) * w_t > budget) {
                    u64 j = w_t > 0 ? (budget - run) / w_t : 0ull;
                    if (j > c_t) j = c_t;
                    if (run == 0ull && j == 0ull) j = 1;   // the first sorted entry is never dropped
                    post_u32(&meet.thr_p, key);
                    post_u32(&meet.n_eq_p, static_cast<uint32_t>(j));
                    break;
                }
                run += static_cast<u64>(c_t) * w_t;
            }
        }
        cluster_barrier();   // (3)
        thr = meet.thr_p;
        n_eq = meet.n_eq_p;
    }

    // ---- one pass in index order, each CTA over half of the row: every thread owns a contiguous run of
    //      whole 8-key vectors and takes, of its run, the mass above thr and the number of keys equal
    //      to thr.  Ties are kept in index order, so with the tie counts of everything before it a
    //      thread knows its kept mass without a second look: gt + w(thr) * clamp(n_eq - ties before, 0, own ties) ----
    const u64 w_thr = fixed_w(thr);
    const int vper = (nvec + kSampleCluster - 1) / kSampleCluster;
    const int s_begin = min(rank * vper, nvec), s_end = min(s_begin + vper, nvec);   // this CTA's vectors
    const int per_thread = (s_end - s_begin + kSampleThreads - 1) / kSampleThreads;
    const int v_begin = min(s_begin + tid * per_thread, s_end), v_end = min(v_begin + per_thread, s_end);
    uint32_t my_eq = 0;
    u64 my_gt = 0;
#pragma unroll 4
    for (int v = v_begin; v < v_end; ++v) {
        const uint4 a = __ldg(rv + v);
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t k = order_key((w[j >> 1] >> ((j & 1) * 16)) & 0xffffu);
            my_eq += k == thr ? 1u : 0u;
            if (k > thr) my_gt += fixed_w(k);
        }
    }
    uint32_t eq_in_cta, eq_total;
    u64 gt_in_cta, gt_total;
    block_scan(my_eq, my_gt, eq_in_cta, gt_in_cta, eq_total, gt_total);
    if (tid == 0) {
        post_u32(&meet.eqs[rank], eq_total);
        post_u64(&meet.gts[rank], gt_total);
    }
    cluster_barrier();   // (4) both index halves' totals are in both CTAs; nothing remote is touched after this
    int eq_before = 0;
    u64 mass_before = 0, Zf = 0;
    {
        int eq_run = 0;
#pragma unroll
        for (int r = 0; r < kSampleCluster; ++r) {
            const int e = meet.eqs[r];
            const int kept_ties = max(0, min(n_eq - eq_run, e));
            const u64 m = meet.gts[r] + static_cast<u64>(kept_ties) * w_thr;
            if (r < rank) {
                mass_before += m;
                eq_before += e;
            }
            Zf += m;
            eq_run += e;
        }
    }
    const int eq_rank = eq_before + static_cast<int>(eq_in_cta);                                  // ties before my run
    const int ties_before_in_cta = max(0, min(n_eq - eq_before, static_cast<int>(eq_in_cta)));   // kept ones of this CTA
    const int my_kept_ties = max(0, min(n_eq - eq_rank, static_cast<int>(my_eq)));
    const u64 my_kept = my_gt + static_cast<u64>(my_kept_ties) * w_thr;
    const u64 lo = mass_before + gt_in_cta + static_cast<u64>(ties_before_in_cta) * w_thr;

    // ---- draw ----
    const uint64_t seed = seeds ? seeds[row] : static_cast<uint64_t>(row);
    const uint64_t step_index = step_index_ptr ? *step_index_ptr : step_index_arg;
    const uint4 rnd = philox4x32(make_uint4(static_cast<uint32_t>(step_index), static_cast<uint32_t>(step_index >> 32), 0u, 0u),
                                 make_uint2(static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32)));
    const double u01 = static_cast<double>(rnd.x >> 8) * (1.0 / 16777216.0);  // [0, 1)
    const u64 target = static_cast<u64>(u01 * static_cast<double>(Zf));       // < Zf: u01 <= 1 - 2^-24
    if (Zf == 0ull && rank == 0 && tid == 0) emit_token(out, wb, row, 0);                    // a row of NaNs: nothing to draw from
    if (my_kept > 0 && target >= lo && target < lo + my_kept) {
        // this thread's run holds the target: walk it
        u64 c = lo;
        int er = eq_rank, pick = -1;
        for (int v = v_begin; v < v_end && pick < 0; ++v) {
            const uint4 a = __ldg(rv + v);
            const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t k = order_key((w[j >> 1] >> ((j & 1) * 16)) & 0xffffu);
                bool kept = k > thr;
                if (k == thr) kept = er++ < n_eq;
                if (kept && pick < 0) {
                    c += fixed_w(k);
                    if (target < c) pick = v * 8 + j;
                }
            }
        }
        if (pick >= 0) emit_token(out, wb, row, pick);
    }
    if (mrow) {   // candidate mask (tests): membership of every key of the run
        int er = eq_rank;
        for (int i = v_begin * 8; i < v_end * 8; ++i) {
            const uint32_t k = order_key(__bfloat16_as_ushort(rowp[i]));
            bool kept = k > thr;
            if (k == thr) kept = er++ < n_eq;
            mrow[i] = kept ? 1 : 0;
        }
    }
}

}  // namespace

int launch_sample(int32_t* out, const void* logits, int rows, int vocab, int64_t ld,
                  const float* temperatures, const int32_t* top_k, const float* top_p,
                  const uint64_t* seeds, uint64_t step_index, uint8_t* mask, cudaStream_t stream,
                  const uint64_t* step_index_dev, const TokenWriteBack* write_back) {
    if (rows == 0) return B200_OK;
    const size_t smem = kHistWords * sizeof(uint32_t);
    B200_CHECK_CUDA(cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem)));
    B200_CHECK_CUDA(launch_kernel(sample_kernel, dim3(rows * kSampleCluster), dim3(kSampleThreads), smem, stream,
                                  dim3(kSampleCluster, 1, 1), out, static_cast<const __nv_bfloat16*>(logits), vocab,
                                  ld, temperatures, top_k, top_p, seeds, step_index_dev, step_index, mask,
                                  write_back ? *write_back : TokenWriteBack{}));
    return B200_OK;
}

}  // namespace b200

extern "C" {

int b200_sample(int32_t* out, const void* logits, int rows, int vocab, int64_t ld,
                const float* temperatures, const int32_t* top_k, const float* top_p,
                const uint64_t* seeds, uint64_t step_index, uint8_t* candidate_mask,
                b200_stream_t stream) {
    B200_CHECK_ARG(rows >= 0 && vocab > 0 && ld >= vocab, "sample: bad shape");
    B200_CHECK_ARG(vocab % 8 == 0 && ld % 8 == 0, "sample: vocab and row stride must be multiples of 8");
    B200_CHECK_ARG(vocab <= (1 << 27), "sample: vocab too large");
    if (rows == 0) return B200_OK;
    B200_CHECK_ARG(out && logits && temperatures, "sample: NULL tensor");
    return b200::launch_sample(out, logits, rows, vocab, ld, temperatures, top_k, top_p, seeds,
                               step_index, candidate_mask, static_cast<cudaStream_t>(stream), nullptr);
}

}  // extern "C"
