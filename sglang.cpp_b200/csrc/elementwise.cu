// Gated activations, embedding row gather, and the int32 index-table kernels.
#include "common.cuh"
#include "kernels.h"

namespace b200 {
namespace {

__device__ __forceinline__ float act_silu(float x) { return x / (1.0f + __expf(-x)); }
__device__ __forceinline__ float act_gelu_tanh(float x) {
    return 0.5f * x * (1.0f + tanhf(0.7978845608f * (x + 0.044715f * x * x * x)));
}

// out[t, j] = act(in[t, j]) * in[t, d + j]; 16-byte vectors, grid-stride over
// (token, vector) pairs so that the grid can be sized to the SM count.
template <bool GELU>
__global__ void __launch_bounds__(256)
act_and_mul_kernel(uint4* __restrict__ out, const uint4* __restrict__ in, int64_t tokens,
                   int vec_per_row) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int64_t total = tokens * vec_per_row;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t t = i / vec_per_row;
        const int v = static_cast<int>(i - t * vec_per_row);
        const uint4 g = in[t * 2 * vec_per_row + v];
        const uint4 u = in[t * 2 * vec_per_row + vec_per_row + v];
        const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
        const uint32_t uw[4] = {u.x, u.y, u.z, u.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float glo = bf16_lo(gw[j]), ghi = bf16_hi(gw[j]);
            const float alo = GELU ? act_gelu_tanh(glo) : act_silu(glo);
            const float ahi = GELU ? act_gelu_tanh(ghi) : act_silu(ghi);
            o[j] = pack_bf16(alo * bf16_lo(uw[j]), ahi * bf16_hi(uw[j]));
        }
        out[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

__global__ void __launch_bounds__(128)
embedding_kernel(uint4* __restrict__ out, const uint4* __restrict__ table,
                 const int32_t* __restrict__ ids, int vec_per_row, int vocab, int* status,
                 unsigned long long* __restrict__ ssq, int ssq_slots, int ssq_stride) {
    __shared__ float warp_part[4];
    pdl_launch_dependents();
    pdl_wait_prior();
    const int64_t t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    if (!ok && threadIdx.x == 0) atomicExch(&status[kStatusBadIndex], id + 1);
    const uint4* src = table + static_cast<int64_t>(ok ? id : 0) * vec_per_row;
    uint4* dst = out + t * vec_per_row;
    float part = 0.f;
    for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) {
        const uint4 u = ok ? src[v] : make_uint4(0, 0, 0, 0);
        dst[v] = u;
        const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) part += bf16_lo(w4[j]) * bf16_lo(w4[j]) + bf16_hi(w4[j]) * bf16_hi(w4[j]);
    }
    if (ssq == nullptr) return;
    // start of a step's residual stream: this row's statistic, and a clean slate for the GEMMs that add to the others
    for (int s = 1 + threadIdx.x; s < ssq_slots; s += blockDim.x) ssq[static_cast<int64_t>(s) * ssq_stride + t] = 0ull;
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = part;
    __syncthreads();
    if (threadIdx.x == 0)
        ssq[t] = static_cast<unsigned long long>((warp_part[0] + warp_part[1] + warp_part[2] + warp_part[3]) * 16777216.0f);
}

__global__ void scale_columns_kernel(uint4* __restrict__ out, const uint4* __restrict__ w,
                                     const uint4* __restrict__ scale, int64_t total_vec, int vec_per_row) {
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total_vec;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const uint4 a = w[i], b = scale[i % vec_per_row];
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = pack_bf16(bf16_lo(aw[j]) * bf16_lo(bw[j]), bf16_hi(aw[j]) * bf16_hi(bw[j]));
        out[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

__global__ void gather_int32_2d_kernel(int32_t* __restrict__ out, const int32_t* __restrict__ table,
                                       int64_t rows, int64_t stride, int64_t cols,
                                       const int32_t* __restrict__ req, const int32_t* __restrict__ pos,
                                       int64_t count) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const int64_t r = req[i], p = pos[i];
    out[i] = (r >= 0 && r < rows && p >= 0 && p < cols) ? table[r * stride + p] : 0;
}

__global__ void write_token_pool_kernel(int32_t* __restrict__ table, int64_t rows, int64_t stride,
                                        int64_t cols, const int32_t* __restrict__ req,
                                        const int32_t* __restrict__ pos,
                                        const int32_t* __restrict__ tokens, int64_t count) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const int64_t r = req[i], p = pos[i];
    if (r < 0 || r >= rows || p < 0 || p >= cols) return;
    table[r * stride + p] = tokens[i];
}

}  // namespace

int launch_act_and_mul(void* out, const void* in, int tokens, int d, bool gelu,
                       cudaStream_t stream) {
    if (tokens == 0) return B200_OK;
    const int vec = d / 8;
    const int64_t total = static_cast<int64_t>(tokens) * vec;
    const int64_t want = div_ceil64(total, 256);
    const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
    const unsigned blocks = static_cast<unsigned>(want < cap ? want : cap);
    auto kernel = gelu ? act_and_mul_kernel<true> : act_and_mul_kernel<false>;
    B200_CHECK_CUDA(launch_kernel(kernel, dim3(blocks), dim3(256), 0, stream, dim3(1, 1, 1),
                                  static_cast<uint4*>(out), static_cast<const uint4*>(in),
                                  static_cast<int64_t>(tokens), vec));
    return B200_OK;
}

int launch_embedding(void* out, const void* table, const int32_t* ids, int tokens, int hidden,
                     int vocab, int* status, cudaStream_t stream, unsigned long long* ssq, int ssq_slots,
                     int ssq_stride) {
    if (tokens == 0) return B200_OK;
    B200_CHECK_CUDA(launch_kernel(embedding_kernel, dim3(tokens), dim3(128), 0, stream, dim3(1, 1, 1),
                                  static_cast<uint4*>(out), static_cast<const uint4*>(table), ids,
                                  hidden / 8, vocab, status, ssq, ssq_slots, ssq_stride));
    return B200_OK;
}

int launch_scale_columns(void* out, const void* w, const void* scale, int64_t rows, int K, cudaStream_t stream) {
    const int64_t total = rows * (K / 8);
    if (total == 0) return B200_OK;
    const int64_t want = div_ceil64(total, 256);
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    scale_columns_kernel<<<static_cast<unsigned>(want < cap ? want : cap), 256, 0, stream>>>(
        static_cast<uint4*>(out), static_cast<const uint4*>(w), static_cast<const uint4*>(scale), total, K / 8);
    B200_CHECK_LAUNCH();
    return B200_OK;
}

}  // namespace b200

extern "C" {

int b200_silu_and_mul(void* out, const void* in, int tokens, int d, b200_stream_t stream) {
    B200_CHECK_ARG(tokens >= 0 && d > 0 && d % 8 == 0, "silu_and_mul: d must be a positive multiple of 8");
    B200_CHECK_ARG(tokens == 0 || (out && in), "silu_and_mul: NULL tensor");
    return b200::launch_act_and_mul(out, in, tokens, d, false, static_cast<cudaStream_t>(stream));
}

int b200_gelu_and_mul(void* out, const void* in, int tokens, int d, b200_stream_t stream) {
    B200_CHECK_ARG(tokens >= 0 && d > 0 && d % 8 == 0, "gelu_and_mul: d must be a positive multiple of 8");
    B200_CHECK_ARG(tokens == 0 || (out && in), "gelu_and_mul: NULL tensor");
    return b200::launch_act_and_mul(out, in, tokens, d, true, static_cast<cudaStream_t>(stream));
}

int b200_embedding(void* out, const void* table, const int32_t* ids, int tokens, int hidden,
                   int vocab, b200_stream_t stream) {
    B200_CHECK_ARG(tokens >= 0 && hidden > 0 && hidden % 8 == 0 && vocab > 0, "embedding: bad size");
    B200_CHECK_ARG(tokens == 0 || (out && table && ids), "embedding: NULL tensor");
    int err = B200_OK;
    int* status = b200::device_status_words(&err);
    if (err != B200_OK) return err;
    return b200::launch_embedding(out, table, ids, tokens, hidden, vocab, status,
                                  static_cast<cudaStream_t>(stream));
}

int b200_gather_int32_2d(int32_t* out, const int32_t* table, int64_t rows, int64_t stride,
                         int64_t cols, const int32_t* req_indices, const int32_t* positions,
                         int64_t count, b200_stream_t stream) {
    B200_CHECK_ARG(count >= 0 && rows >= 0 && cols >= 0, "gather_int32_2d: negative size");
    if (count == 0) return B200_OK;
    B200_CHECK_ARG(out && table && req_indices && positions, "gather_int32_2d: NULL tensor");
    const unsigned blocks = static_cast<unsigned>((count + 255) / 256);
    b200::gather_int32_2d_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        out, table, rows, stride, cols, req_indices, positions, count);
    B200_CHECK_LAUNCH();
    return B200_OK;
}

int b200_write_token_pool(int32_t* table, int64_t rows, int64_t stride, int64_t cols,
                          const int32_t* req_indices, const int32_t* positions,
                          const int32_t* tokens, int64_t count, b200_stream_t stream) {
    B200_CHECK_ARG(count >= 0 && rows >= 0 && cols >= 0, "write_token_pool: negative size");
    if (count == 0) return B200_OK;
    B200_CHECK_ARG(table && req_indices && positions && tokens, "write_token_pool: NULL tensor");
    const unsigned blocks = static_cast<unsigned>((count + 255) / 256);
    b200::write_token_pool_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        table, rows, stride, cols, req_indices, positions, tokens, count);
    B200_CHECK_LAUNCH();
    return B200_OK;
}

}  // extern "C"
