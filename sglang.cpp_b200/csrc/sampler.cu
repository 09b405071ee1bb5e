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

// One CTA per row; 16-byte loads; first index on ties.
__global__ void __launch_bounds__(512)
argmax_bf16_kernel(int32_t* __restrict__ out, const __nv_bfloat16* __restrict__ logits, int vocab,
                   int64_t ld) {
    __shared__ float s_v[16];
    __shared__ int s_i[16];
    pdl_wait_prior();
    const __nv_bfloat16* row = logits + static_cast<int64_t>(blockIdx.x) * ld;
    MaxIdx best{-INFINITY, 0x7fffffff};
    const int nvec = vocab >> 3;
    const uint4* rv = reinterpret_cast<const uint4*>(row);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
        const uint4 a = rv[v];
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            best = better(best, MaxIdx{bf16_lo(w[j]), v * 8 + 2 * j});
            best = better(best, MaxIdx{bf16_hi(w[j]), v * 8 + 2 * j + 1});
        }
    }
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
        if (lane == 0) out[blockIdx.x] = best.i == 0x7fffffff ? 0 : best.i;
    }
}

}  // namespace

int launch_argmax(int32_t* out, const void* logits, int rows, int vocab, int64_t ld,
                  cudaStream_t stream) {
    if (rows == 0) return B200_OK;
    B200_CHECK_CUDA(launch_kernel(argmax_bf16_kernel, dim3(rows), dim3(512), 0, stream, dim3(1, 1, 1), out,
                                  static_cast<const __nv_bfloat16*>(logits), vocab, ld));
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
