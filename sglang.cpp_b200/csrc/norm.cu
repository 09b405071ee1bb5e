// RMSNorm family: plain, fused residual-add, and strided per-head (QK) norm.
//
// All three are HBM-bound row reductions: one 16-byte load per thread per
// 8 bf16, values kept in registers between the reduction and the scaling pass
// so every element is read once, warp-shuffle + one shared-memory hop for the
// block reduction, fp32 arithmetic, bf16 storage.
#include "common.cuh"
#include "kernels.h"

namespace b200 {
namespace {

constexpr int kNormVecPerThread = 4;  // register-cached 16-byte vectors per thread

__device__ __forceinline__ float block_sum(float v, float* smem) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwarps = blockDim.x >> 5;
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? smem[lane] : 0.f;
    t = warp_sum(t);
    return t;
}

// One CTA per row.  FUSED_ADD: residual <- x + residual; x <- norm(sum) * w.
// Otherwise out <- norm(x) * w.  hidden % 8 == 0.
template <bool FUSED_ADD, bool ROUND_FIRST>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(__nv_bfloat16* out, const __nv_bfloat16* x_in,
               __nv_bfloat16* residual, const __nv_bfloat16* __restrict__ weight, int hidden,
               float eps) {
    __shared__ float red[32];
    const int64_t row = blockIdx.x;
    const int nvec = hidden >> 3;
    const uint4* xv = reinterpret_cast<const uint4*>(x_in + row * hidden);
    uint4* rv = FUSED_ADD ? reinterpret_cast<uint4*>(residual + row * hidden) : nullptr;
    uint4* ov = reinterpret_cast<uint4*>(out + row * hidden);
    const uint4* wv = reinterpret_cast<const uint4*>(weight);

    pdl_launch_dependents();
    // The norm weights do not come from the kernel before this one: fetch them ahead of the wait, so
    // that only the row itself is loaded behind it (one trip to L2 instead of two).
    uint4 wreg[kNormVecPerThread];
#pragma unroll
    for (int i = 0; i < kNormVecPerThread; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        wreg[i] = v < nvec ? __ldg(wv + v) : make_uint4(0u, 0u, 0u, 0u);
    }
    pdl_wait_prior();

    float vals[kNormVecPerThread][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kNormVecPerThread; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nvec) {
            uint4 a = xv[v];
            const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
            if (FUSED_ADD) {
                uint4 r = rv[v];
                const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
                uint32_t packed[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float lo = bf16_lo(aw[j]) + bf16_lo(rw[j]);
                    const float hi = bf16_hi(aw[j]) + bf16_hi(rw[j]);
                    packed[j] = pack_bf16(lo, hi);
                    vals[i][2 * j] = ROUND_FIRST ? bf16_lo(packed[j]) : lo;
                    vals[i][2 * j + 1] = ROUND_FIRST ? bf16_hi(packed[j]) : hi;
                }
                rv[v] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    vals[i][2 * j] = bf16_lo(aw[j]);
                    vals[i][2 * j + 1] = bf16_hi(aw[j]);
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
        }
    }
    // Rows wider than the register cache: accumulate the tail without caching.
    for (int v = threadIdx.x + kNormVecPerThread * blockDim.x; v < nvec; v += blockDim.x) {
        uint4 a = xv[v];
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
        float f[8];
        if (FUSED_ADD) {
            uint4 r = rv[v];
            const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
            uint32_t packed[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                f[2 * j] = bf16_lo(aw[j]) + bf16_lo(rw[j]);
                f[2 * j + 1] = bf16_hi(aw[j]) + bf16_hi(rw[j]);
                packed[j] = pack_bf16(f[2 * j], f[2 * j + 1]);
                if (ROUND_FIRST) {
                    f[2 * j] = bf16_lo(packed[j]);
                    f[2 * j + 1] = bf16_hi(packed[j]);
                }
            }
            rv[v] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                f[2 * j] = bf16_lo(aw[j]);
                f[2 * j + 1] = bf16_hi(aw[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }

    ss = block_sum(ss, red);
    const float scale = rsqrtf(ss / static_cast<float>(hidden) + eps);

#pragma unroll
    for (int i = 0; i < kNormVecPerThread; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nvec) {
            const uint4 w = wreg[i];
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
            uint32_t packed[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                packed[j] = pack_bf16(vals[i][2 * j] * scale * bf16_lo(ww[j]),
                                      vals[i][2 * j + 1] * scale * bf16_hi(ww[j]));
            }
            ov[v] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
    }
    for (int v = threadIdx.x + kNormVecPerThread * blockDim.x; v < nvec; v += blockDim.x) {
        // The fused variant re-reads the sum it stored (bf16-rounded) for this
        // tail; rows this wide (> 8192 at 256 threads) do not occur in the
        // supported model shapes.
        uint4 a = FUSED_ADD ? rv[v] : xv[v];
        uint4 w = wv[v];
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
        uint32_t packed[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            packed[j] = pack_bf16(bf16_lo(aw[j]) * scale * bf16_lo(ww[j]),
                                  bf16_hi(aw[j]) * scale * bf16_hi(ww[j]));
        }
        ov[v] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
}

// One warp per (token, head) row of q or k; head_dim = 32 * EPL * 2 ... handled
// generically: each lane walks the row in 4-byte (2 x bf16) steps.
__global__ void __launch_bounds__(128)
qk_rmsnorm_kernel(__nv_bfloat16* q, __nv_bfloat16* k, const __nv_bfloat16* __restrict__ qw,
                  const __nv_bfloat16* __restrict__ kw, int64_t q_rows, int64_t total_rows,
                  int q_heads, int k_heads, int head_dim, int64_t qst, int64_t qsh, int64_t kst,
                  int64_t ksh, float eps) {
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= total_rows) return;
    __nv_bfloat16* p;
    const __nv_bfloat16* w;
    if (row < q_rows) {
        const int64_t t = row / q_heads, h = row - t * q_heads;
        p = q + t * qst + h * qsh;
        w = qw;
    } else {
        const int64_t r = row - q_rows;
        const int64_t t = r / k_heads, h = r - t * k_heads;
        p = k + t * kst + h * ksh;
        w = kw;
    }
    uint32_t* p2 = reinterpret_cast<uint32_t*>(p);
    const uint32_t* w2 = reinterpret_cast<const uint32_t*>(w);
    const int npair = head_dim >> 1;
    float ss = 0.f;
    for (int i = lane; i < npair; i += 32) {
        const uint32_t v = p2[i];
        const float lo = bf16_lo(v), hi = bf16_hi(v);
        ss += lo * lo + hi * hi;
    }
    ss = warp_sum(ss);
    const float scale = rsqrtf(ss / static_cast<float>(head_dim) + eps);
    for (int i = lane; i < npair; i += 32) {
        const uint32_t v = p2[i];
        const uint32_t ww = w2[i];
        p2[i] = pack_bf16(bf16_lo(v) * scale * bf16_lo(ww), bf16_hi(v) * scale * bf16_hi(ww));
    }
}

}  // namespace

// Launch helpers shared with the model runner.
int launch_rmsnorm(void* out, const void* x, const void* weight, int rows, int hidden, float eps,
                   cudaStream_t stream) {
    if (rows == 0) return B200_OK;
    const int threads = hidden >= 2048 ? 256 : 128;
    B200_CHECK_CUDA(launch_kernel(rmsnorm_kernel<false, false>, dim3(rows), dim3(threads), 0, stream, dim3(1, 1, 1),
                                  static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(x),
                                  static_cast<__nv_bfloat16*>(nullptr),
                                  static_cast<const __nv_bfloat16*>(weight), hidden, eps));
    return B200_OK;
}

int launch_fused_add_rmsnorm(void* x, void* residual, const void* weight, int rows, int hidden,
                             float eps, bool round_sum_first, cudaStream_t stream) {
    if (rows == 0) return B200_OK;
    const int threads = hidden >= 2048 ? 256 : 128;
    auto kernel = round_sum_first ? rmsnorm_kernel<true, true> : rmsnorm_kernel<true, false>;
    B200_CHECK_CUDA(launch_kernel(kernel, dim3(rows), dim3(threads), 0, stream, dim3(1, 1, 1),
                                  static_cast<__nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(x),
                                  static_cast<__nv_bfloat16*>(residual),
                                  static_cast<const __nv_bfloat16*>(weight), hidden, eps));
    return B200_OK;
}

}  // namespace b200

extern "C" {

int b200_rmsnorm(void* out, const void* x, const void* weight, int rows, int hidden, float eps,
                 b200_stream_t stream) {
    B200_CHECK_ARG(rows >= 0, "rmsnorm: rows must be >= 0");
    B200_CHECK_ARG(rows == 0 || (out && x && weight), "rmsnorm: NULL tensor");
    B200_CHECK_ARG(hidden > 0, "RMSNorm last dimension must be positive");
    B200_CHECK_ARG(hidden % 8 == 0, "rmsnorm: hidden must be a multiple of 8 (16-byte rows)");
    return b200::launch_rmsnorm(out, x, weight, rows, hidden, eps, static_cast<cudaStream_t>(stream));
}

int b200_fused_add_rmsnorm(void* x, void* residual, const void* weight, int rows, int hidden,
                           float eps, b200_stream_t stream) {
    B200_CHECK_ARG(rows >= 0, "fused_add_rmsnorm: rows must be >= 0");
    B200_CHECK_ARG(rows == 0 || (x && residual && weight), "fused_add_rmsnorm: NULL tensor");
    B200_CHECK_ARG(hidden > 0, "RMSNorm last dimension must be positive");
    B200_CHECK_ARG(hidden % 8 == 0, "fused_add_rmsnorm: hidden must be a multiple of 8");
    return b200::launch_fused_add_rmsnorm(x, residual, weight, rows, hidden, eps, false,
                                          static_cast<cudaStream_t>(stream));
}

int b200_qk_rmsnorm_strided(void* q, void* k, const void* q_weight, const void* k_weight,
                            int tokens, int q_heads, int k_heads, int head_dim,
                            int64_t q_stride_token, int64_t q_stride_head, int64_t k_stride_token,
                            int64_t k_stride_head, float eps, b200_stream_t stream) {
    B200_CHECK_ARG(tokens >= 0 && q_heads >= 0 && k_heads >= 0, "qk_rmsnorm: negative size");
    B200_CHECK_ARG(head_dim > 0 && head_dim % 2 == 0, "qk_rmsnorm: head_dim must be even");
    B200_CHECK_ARG(tokens == 0 || q_heads == 0 || (q && q_weight), "qk_rmsnorm: q / q_weight is NULL");
    B200_CHECK_ARG(tokens == 0 || k_heads == 0 || (k && k_weight), "qk_rmsnorm: k / k_weight is NULL");
    B200_CHECK_ARG((q_stride_token % 2 == 0) && (q_stride_head % 2 == 0) &&
                       (k_stride_token % 2 == 0) && (k_stride_head % 2 == 0),
                   "qk_rmsnorm: strides must be even (4-byte aligned rows)");
    const int64_t q_rows = static_cast<int64_t>(tokens) * q_heads;
    const int64_t total = q_rows + static_cast<int64_t>(tokens) * k_heads;
    if (total == 0) return B200_OK;
    const int warps = 4;
    const unsigned blocks = static_cast<unsigned>((total + warps - 1) / warps);
    b200::qk_rmsnorm_kernel<<<blocks, warps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k),
        static_cast<const __nv_bfloat16*>(q_weight), static_cast<const __nv_bfloat16*>(k_weight),
        q_rows, total, q_heads, k_heads, head_dim, q_stride_token, q_stride_head, k_stride_token,
        k_stride_head, eps);
    B200_CHECK_LAUNCH();
    return B200_OK;
}

}  // extern "C"
