// Sampling from a probability matrix with given uniform numbers: what the reference's device
// sampling path asks FlashInfer for (flashinfer_*_sample_from_probs, src/engine/sampling.cu:65-192,
// called from Sampler::sample, src/engine/engine.cc:299-338).
//
// FlashInfer v0.2 draws by rejection: a token is accepted when it is among the top_k largest
// probabilities and the probabilities strictly larger than its own sum to less than top_p.  The
// accepted tokens are therefore "every token whose probability is >= max(v_k, v_p)", with v_k the
// k-th largest value and v_p the smallest value whose strictly-larger mass is below top_p, and the
// draw follows the probabilities restricted to that set.  This kernel finds the two values with a
// most-significant-byte-first radix select over the fp32 bit patterns (probabilities are
// non-negative, so the bit patterns order like the values): four passes over the row, each building
// a 256-bin count histogram for the top-k prefix and a 256-bin mass histogram for the top-p prefix.
// Masses are accumulated in 64-bit fixed point (2^-52 units), so the sums do not depend on the order
// of the atomic adds and the result is reproducible.  A last pass in index order picks the token at
// uniform * (mass of the set) by inverse CDF.  One CTA of 1024 threads per row; the row stays in L2.
#include "common.cuh"
#include "kernels.h"

namespace b200 {
namespace {

constexpr int kThreads = 1024;
constexpr double kFixedScale = 4503599627370496.0;  // 2^52

__device__ __forceinline__ uint32_t prob_key(float p) {
    // negative, NaN: treated as 0 (never sampled unless everything is)
    return p > 0.f ? __float_as_uint(p) : 0u;
}
__device__ __forceinline__ unsigned long long prob_fixed(float p) {
    return p > 0.f ? static_cast<unsigned long long>(static_cast<double>(p) * kFixedScale) : 0ull;
}

__device__ __forceinline__ unsigned long long warp_incl_scan_u64(unsigned long long v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
    }
    return v;
}

__global__ void __launch_bounds__(kThreads)
sample_probs_kernel(int32_t* __restrict__ out, const float* __restrict__ probs, int vocab,
                    const int32_t* __restrict__ top_k, int top_k_value, const float* __restrict__ top_p,
                    float top_p_value, const float* __restrict__ uniform) {
    __shared__ unsigned int h_cnt[256];
    __shared__ unsigned long long h_mass[256];
    __shared__ unsigned long long s_warp[32];
    __shared__ uint32_t s_prefix_k, s_prefix_p;
    __shared__ unsigned int s_cnt_above;
    __shared__ unsigned long long s_mass_above;
    __shared__ int s_done_k, s_done_p, s_chosen, s_last;
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* pr = probs + static_cast<int64_t>(row) * vocab;

    int K = top_k ? top_k[row] : top_k_value;
    if (K < 1 || K > vocab) K = vocab;
    float P = top_p ? top_p[row] : top_p_value;
    if (!(P > 0.f) || P > 1.f) P = 1.f;
    const bool want_k = K < vocab, want_p = P < 1.f;
    const unsigned long long p_fixed = static_cast<unsigned long long>(static_cast<double>(P) * kFixedScale);

    if (tid == 0) {
        s_prefix_k = s_prefix_p = 0u;
        s_cnt_above = 0u;
        s_mass_above = 0ull;
        s_done_k = want_k ? 0 : 1;   // "done": the value is known (0 when the filter is off)
        s_done_p = want_p ? 0 : 1;
        s_chosen = -1;
        s_last = -1;
    }
    __syncthreads();

    // ---- radix select, most significant byte first ----
    for (int level = 0; level < 4 && (want_k || want_p); ++level) {
        const int shift = 24 - 8 * level;
        const uint32_t hi_mask = level == 0 ? 0u : (0xffffffffu << (shift + 8));
        for (int i = tid; i < 256; i += kThreads) {
            h_cnt[i] = 0u;
            h_mass[i] = 0ull;
        }
        __syncthreads();
        const uint32_t pk = s_prefix_k, pp = s_prefix_p;
        const bool do_k = !s_done_k, do_p = !s_done_p;
        for (int i = tid; i < vocab; i += kThreads) {
            const float p = pr[i];
            const uint32_t key = prob_key(p);
            const uint32_t bin = (key >> shift) & 0xffu;
            if (do_k && (key & hi_mask) == pk) atomicAdd(&h_cnt[bin], 1u);
            if (do_p && (key & hi_mask) == pp) atomicAdd(&h_mass[bin], prob_fixed(p));
        }
        __syncthreads();
        if (tid == 0) {
            if (do_k) {
                unsigned int c = s_cnt_above;
                int b = 255;
                for (; b > 0; --b) {
                    if (c + h_cnt[b] >= static_cast<unsigned int>(K)) break;
                    c += h_cnt[b];
                }
                s_cnt_above = c;
                s_prefix_k = pk | (static_cast<uint32_t>(b) << shift);
            }
            if (do_p) {
                unsigned long long m = s_mass_above;
                int b = 255;
                for (; b > 0; --b) {
                    if (m + h_mass[b] >= p_fixed) break;
                    m += h_mass[b];
                }
                s_mass_above = m;
                s_prefix_p = pp | (static_cast<uint32_t>(b) << shift);
            }
        }
        __syncthreads();
    }
    // keys >= thr form the accepted set (a filter that is off contributes 0)
    const uint32_t thr = max(want_k ? s_prefix_k : 0u, want_p ? s_prefix_p : 0u);

    // ---- mass of the accepted set ----
    unsigned long long local = 0ull;
    for (int i = tid; i < vocab; i += kThreads) {
        const float p = pr[i];
        if (prob_key(p) >= thr) local += prob_fixed(p);
    }
    local = warp_incl_scan_u64(local, lane);
    if (lane == 31) s_warp[warp] = local;
    __syncthreads();
    unsigned long long Z = 0ull;
    for (int w = 0; w < kThreads / 32; ++w) Z += s_warp[w];
    __syncthreads();

    // ---- inverse CDF in index order ----
    float u = uniform[row];
    u = u < 0.f ? 0.f : (u >= 1.f ? 0.99999994f : u);
    const unsigned long long target = static_cast<unsigned long long>(static_cast<double>(u) * static_cast<double>(Z));
    unsigned long long run = 0ull;
    for (int base = 0; base < vocab; base += kThreads) {
        const int i = base + tid;
        unsigned long long w = 0ull;
        if (i < vocab) {
            const float p = pr[i];
            if (prob_key(p) >= thr) w = prob_fixed(p);
        }
        const unsigned long long incl = warp_incl_scan_u64(w, lane);
        if (lane == 31) s_warp[warp] = incl;
        __syncthreads();
        unsigned long long off = run, total = 0ull;
        for (int q = 0; q < kThreads / 32; ++q) {
            if (q < warp) off += s_warp[q];
            total += s_warp[q];
        }
        const unsigned long long before = off + incl - w;
        if (w > 0ull) {
            if (target >= before && target < before + w) atomicMax(&s_chosen, i);   // intervals are disjoint
            atomicMax(&s_last, i);
        }
        run += total;
        __syncthreads();
        if (s_chosen >= 0) break;   // uniform over the block: read after the barrier
    }
    __syncthreads();
    if (tid == 0) out[row] = s_chosen >= 0 ? s_chosen : max(s_last, 0);
}

}  // namespace
}  // namespace b200

extern "C" {

int b200_sample_from_probs(int32_t* out, const float* probs, int rows, int vocab, const int32_t* top_k,
                           int top_k_value, const float* top_p, float top_p_value, const float* uniform,
                           b200_stream_t stream) {
    B200_CHECK_ARG(rows >= 0 && vocab > 0, "sample_from_probs: bad shape");
    if (rows == 0) return B200_OK;
    B200_CHECK_ARG(out && probs && uniform, "sample_from_probs: NULL tensor");
    B200_CHECK_CUDA(b200::launch_kernel(b200::sample_probs_kernel, dim3(rows), dim3(b200::kThreads), 0,
                                        static_cast<cudaStream_t>(stream), dim3(1, 1, 1), out, probs, vocab, top_k,
                                        top_k_value, top_p, top_p_value, uniform));
    return B200_OK;
}

}  // extern "C"
