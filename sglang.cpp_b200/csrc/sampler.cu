// Token selection from logits: greedy argmax and the single-pass
// temperature / top-k / top-p sampler.
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

__global__ void __launch_bounds__(512)
argmax_bf16_kernel(int32_t* __restrict__ out, const __nv_bfloat16* __restrict__ logits, int vocab,
                   int64_t ld, int ncta) {
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
            if (lane == 0) out[row_id] = best.i == 0x7fffffff ? 0 : best.i;
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
            out[row_id] = b0.i == 0x7fffffff ? 0 : b0.i;
        }
    }
}

}  // namespace

int launch_argmax(int32_t* out, const void* logits, int rows, int vocab, int64_t ld,
                  cudaStream_t stream) {
    if (rows == 0) return B200_OK;
    const int ncta = vocab >= 32768 ? kArgmaxCluster : 1;
    B200_CHECK_CUDA(launch_kernel(argmax_bf16_kernel, dim3(rows * ncta), dim3(512), 0, stream, dim3(ncta, 1, 1),
                                  out, static_cast<const __nv_bfloat16*>(logits), vocab, ld, ncta));
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
// The logits are bf16, so their order-preserving 16-bit keys take at most 65536
// values and equal keys are exact ties.  Top-k is "the k-th largest key" and
// top-p is "the key below which the cumulative mass first exceeds p"; both are
// found by a 16-step bitwise search whose probe is one pass over the row (which
// stays in L2) with a fixed-order block reduction, so the result is exact and
// deterministic.  The kept set always has the form
//     key > thr   or   (key == thr and it is among the first n_eq such by index),
// which is how sample_row's sort-based definition reads when ties are ordered by
// index.  One last pass in index order draws from the kept set with a Philox
// uniform.  One CTA of 1024 threads per row.
// ============================================================================
namespace b200 {
namespace {

constexpr int kSampleThreads = 1024;

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

struct SampleSmem {
    float f[32];
    int i[32];
    float bcast_f;
    int bcast_i;
};

__device__ __forceinline__ float block_sum_f(float v, SampleSmem& sm) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) sm.f[warp] = v;
    __syncthreads();
    float t = sm.f[lane];
    t = warp_sum(t);
    return t;
}
__device__ __forceinline__ int block_sum_i(int v, SampleSmem& sm) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) sm.i[warp] = v;
    __syncthreads();
    int t = sm.i[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}
__device__ __forceinline__ int block_max_i(int v, SampleSmem& sm) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) sm.i[warp] = v;
    __syncthreads();
    int t = sm.i[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t = max(t, __shfl_xor_sync(0xffffffffu, t, o));
    return t;
}

// Exclusive prefix over the block in thread order; `total` gets the block sum.
__device__ __forceinline__ float block_excl_scan_f(float v, float& total, SampleSmem& sm) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    __syncthreads();
    if (lane == 31) sm.f[warp] = incl;
    __syncthreads();
    float wsum = sm.f[lane], wincl = wsum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, wincl, o);
        if (lane >= o) wincl += t;
    }
    total = __shfl_sync(0xffffffffu, wincl, 31);
    const float warp_off = __shfl_sync(0xffffffffu, wincl - wsum, warp);
    return warp_off + incl - v;
}
__device__ __forceinline__ int block_excl_scan_i(int v, int& total, SampleSmem& sm) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    __syncthreads();
    if (lane == 31) sm.i[warp] = incl;
    __syncthreads();
    int wsum = sm.i[lane], wincl = wsum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, wincl, o);
        if (lane >= o) wincl += t;
    }
    total = __shfl_sync(0xffffffffu, wincl, 31);
    const int warp_off = __shfl_sync(0xffffffffu, wincl - wsum, warp);
    return warp_off + incl - v;
}

__device__ __forceinline__ void unpack_keys(const uint4& a, uint32_t (&k)[8]) {
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        k[2 * j] = order_key(w[j] & 0xffffu);
        k[2 * j + 1] = order_key(w[j] >> 16);
    }
}

__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(int32_t* __restrict__ out, const __nv_bfloat16* __restrict__ logits, int vocab,
              int64_t ld, const float* __restrict__ temps, const int32_t* __restrict__ top_k,
              const float* __restrict__ top_p, const uint64_t* __restrict__ seeds,
              uint64_t step_index, uint8_t* __restrict__ mask) {
    __shared__ SampleSmem sm;
    __shared__ int s_chosen;
    pdl_launch_dependents();
    pdl_wait_prior();
    const int row = blockIdx.x;
    const uint4* rv = reinterpret_cast<const uint4*>(logits + static_cast<int64_t>(row) * ld);
    const int nvec = vocab >> 3;
    uint8_t* mrow = mask ? mask + static_cast<int64_t>(row) * vocab : nullptr;

    auto count_ge = [&](uint32_t c) {
        int n = 0;
        for (int v = threadIdx.x; v < nvec; v += kSampleThreads) {
            uint32_t k[8];
            unpack_keys(rv[v], k);
#pragma unroll
            for (int e = 0; e < 8; ++e) n += k[e] >= c ? 1 : 0;
        }
        return block_sum_i(n, sm);
    };
    auto count_eq = [&](uint32_t c) {
        int n = 0;
        for (int v = threadIdx.x; v < nvec; v += kSampleThreads) {
            uint32_t k[8];
            unpack_keys(rv[v], k);
#pragma unroll
            for (int e = 0; e < 8; ++e) n += k[e] == c ? 1 : 0;
        }
        return block_sum_i(n, sm);
    };

    // ---- row maximum ----
    int kmax_local = 0;
    for (int v = threadIdx.x; v < nvec; v += kSampleThreads) {
        uint32_t k[8];
        unpack_keys(rv[v], k);
#pragma unroll
        for (int e = 0; e < 8; ++e) kmax_local = max(kmax_local, static_cast<int>(k[e]));
    }
    const uint32_t kmax = static_cast<uint32_t>(block_max_i(kmax_local, sm));
    const float lmax = key_to_float(kmax);

    const float T = temps[row];
    if (threadIdx.x == 0) s_chosen = -1;
    __syncthreads();
    if (T <= 1.0000001e-6f) {
        // Greedy request inside a sampled batch (Sampler::prepare clamps its temperature to
        // 1e-6): the distribution is one-hot on the first maximum.
        int best = -0x7fffffff;
        for (int v = threadIdx.x; v < nvec; v += kSampleThreads) {
            uint32_t k[8];
            unpack_keys(rv[v], k);
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if (k[e] == kmax) best = max(best, -(v * 8 + e));
        }
        const int idx = -block_max_i(best, sm);
        if (threadIdx.x == 0) out[row] = idx;
        if (mrow)
            for (int i = threadIdx.x; i < vocab; i += kSampleThreads) mrow[i] = i == idx ? 1 : 0;
        return;
    }
    const float scale = 1.4426950408889634f / T;
    auto weight = [&](uint32_t key) { return exp2f((key_to_float(key) - lmax) * scale); };
    // Mass of n tied entries (n may be 0, and then the key may be one no entry has).
    auto tie_mass = [&](int n, uint32_t key) { return n > 0 ? static_cast<float>(n) * weight(key) : 0.f; };
    auto mass_ge = [&](uint32_t c) {
        float s = 0.f;
        for (int v = threadIdx.x; v < nvec; v += kSampleThreads) {
            uint32_t k[8];
            unpack_keys(rv[v], k);
#pragma unroll
            for (int e = 0; e < 8; ++e) s += k[e] >= c ? weight(k[e]) : 0.f;
        }
        return block_sum_f(s, sm);
    };

    // ---- top-k: thr = k-th largest key, n_eq = how many of the keys equal to it are kept ----
    int K = top_k ? top_k[row] : vocab;
    if (K < 1 || K > vocab) K = vocab;
    uint32_t thr = 0;
    int n_eq;
    if (K < vocab) {
        uint32_t v = 0;
        for (int bit = 15; bit >= 0; --bit) {
            const uint32_t cand = v | (1u << bit);
            if (cand <= kmax && count_ge(cand) >= K) v = cand;
        }
        thr = v;
        n_eq = min(K - count_ge(thr + 1), count_eq(thr));
    } else {
        n_eq = count_eq(0);
    }
    // ---- top-p over the top-k set ----
    float P = top_p ? top_p[row] : 1.0f;
    if (P < 1.0f) {
        const float Z = mass_ge(thr + 1) + tie_mass(n_eq, thr);
        const float budget = P * Z;
        uint32_t t = 0;  // largest key whose "this key and above" mass exceeds the budget
        for (int bit = 15; bit >= 0; --bit) {
            const uint32_t cand = t | (1u << bit);
            if (cand > kmax) continue;
            const float m = cand <= thr ? Z : mass_ge(cand);
            if (m > budget) t = cand;
        }
        if (t < thr) t = thr;
        const float m_full = t + 1 > kmax ? 0.f : mass_ge(t + 1);
        const int c_t = t == thr ? n_eq : count_eq(t);
        int j = c_t > 0 ? static_cast<int>(floorf((budget - m_full) / weight(t))) : 0;
        j = max(0, min(j, c_t));
        if (m_full == 0.f && j == 0) j = 1;  // the first sorted entry is never dropped
        thr = t;
        n_eq = j;
    }
    const float Zf = mass_ge(thr + 1) + tie_mass(n_eq, thr);

    // ---- draw ----
    const uint64_t seed = seeds ? seeds[row] : static_cast<uint64_t>(row);
    const uint4 rnd = philox4x32(make_uint4(static_cast<uint32_t>(step_index), static_cast<uint32_t>(step_index >> 32), 0u, 0u),
                                 make_uint2(static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32)));
    const float u01 = static_cast<float>(rnd.x >> 8) * (1.0f / 16777216.0f);  // [0, 1)
    const float target = u01 * Zf;

    // ---- one pass in index order: membership, optional mask, and the draw ----
    int run_eq = 0, last_kept = -1;
    float run_w = 0.f;
    for (int base = 0; base < nvec; base += kSampleThreads) {
        const int v = base + threadIdx.x;
        uint32_t k[8];
        if (v < nvec) {
            unpack_keys(rv[v], k);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) k[e] = 0xffffffffu;  // matches nothing
        }
        int eq_local = 0;
#pragma unroll
        for (int e = 0; e < 8; ++e) eq_local += (k[e] == thr) ? 1 : 0;
        int eq_total;
        int eq_rank = run_eq + block_excl_scan_i(eq_local, eq_total, sm);
        float w[8], w_local = 0.f;
        int my_last = -1;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            bool kept = false;
            if (v < nvec) {
                if (k[e] > thr && k[e] != 0xffffffffu) kept = true;
                else if (k[e] == thr) kept = eq_rank++ < n_eq;
            }
            w[e] = kept ? weight(k[e]) : 0.f;
            w_local += w[e];
            if (kept) my_last = v * 8 + e;
            if (mrow && v < nvec) mrow[v * 8 + e] = kept ? 1 : 0;
        }
        float w_total;
        const float w_before = run_w + block_excl_scan_f(w_local, w_total, sm);
        if (my_last >= 0 && target >= w_before && target < w_before + w_local) {
            float c = w_before;
            int pick = my_last;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                if (w[e] > 0.f) {
                    c += w[e];
                    if (target < c) {
                        pick = v * 8 + e;
                        break;
                    }
                }
            }
            atomicMax(&s_chosen, pick);  // intervals are disjoint: at most one thread gets here
        }
        last_kept = max(last_kept, my_last);
        run_eq += eq_total;
        run_w += w_total;
    }
    const int last_all = block_max_i(last_kept, sm);
    __syncthreads();
    if (threadIdx.x == 0) out[row] = s_chosen >= 0 ? s_chosen : max(last_all, 0);
}

}  // namespace

int launch_sample(int32_t* out, const void* logits, int rows, int vocab, int64_t ld,
                  const float* temperatures, const int32_t* top_k, const float* top_p,
                  const uint64_t* seeds, uint64_t step_index, uint8_t* mask, cudaStream_t stream) {
    if (rows == 0) return B200_OK;
    B200_CHECK_CUDA(launch_kernel(sample_kernel, dim3(rows), dim3(kSampleThreads), 0, stream, dim3(1, 1, 1),
                                  out, static_cast<const __nv_bfloat16*>(logits), vocab, ld, temperatures,
                                  top_k, top_p, seeds, step_index, mask));
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
                               step_index, candidate_mask, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
