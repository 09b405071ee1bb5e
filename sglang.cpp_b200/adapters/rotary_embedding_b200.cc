// sglang::RotaryEmbedding (include/sglang/layers/rotary_embedding.h:11-22) on the C ABI.  Replaces
// src/layers/rotary_embedding.cu, whose forward calls FlashInfer's BatchQKApplyRotaryPosIdsCosSinCache.
// The tables are built here exactly as the reference builds them (src/layers/rotary_embedding.cu:75-94:
// fp32 torch ops on the CPU), so a model built on these adapters sees the reference's bit pattern.
#include "sglang/layers/rotary_embedding.h"

#include "adapter_common.h"

namespace sglang {

using b200_adapters::check;
using b200_adapters::current_stream;
using b200_adapters::require_bf16;

RotaryEmbedding::RotaryEmbedding(int head_size, int rotary_dim, int max_position_embeddings, float base)
    : head_size_(head_size), rotary_dim_(rotary_dim), max_position_embeddings_(max_position_embeddings), base_(base) {
    auto inv_freq = 1.0 / torch::pow(base, torch::arange(0, rotary_dim, 2, torch::kFloat32) /
                                               static_cast<float>(rotary_dim));
    auto t = torch::arange(max_position_embeddings, torch::kFloat32);
    auto freqs = torch::einsum("i,j->ij", {t, inv_freq});
    cos_cache_ = freqs.cos().contiguous();
    sin_cache_ = freqs.sin().contiguous();
}

void RotaryEmbedding::forward_inplace(torch::Tensor& positions, torch::Tensor& query, torch::Tensor& key,
                                      const torch::Tensor& cos_cache, const torch::Tensor& sin_cache) {
    TORCH_CHECK(query.is_cuda() && key.is_cuda() && positions.is_cuda(), "Inputs must be CUDA tensors");
    TORCH_CHECK(rotary_dim_ % 2 == 0, "rotary_dim must be even");
    TORCH_CHECK(cos_cache.dim() == 2 && sin_cache.dim() == 2, "cos/sin cache must be rank-2");
    TORCH_CHECK(cos_cache.size(1) == rotary_dim_ / 2 && sin_cache.size(1) == rotary_dim_ / 2,
                "cos / sin cache width must be rotary_dim / 2");
    TORCH_CHECK(cos_cache.is_cuda() && sin_cache.is_cuda() && cos_cache.is_contiguous() && sin_cache.is_contiguous() &&
                    cos_cache.scalar_type() == torch::kFloat32 && sin_cache.scalar_type() == torch::kFloat32,
                "cos / sin cache must be contiguous float32 CUDA tensors");
    TORCH_CHECK(query.dim() == 3 && key.dim() == 3 && query.stride(2) == 1 && key.stride(2) == 1,
                "query and key must be [tokens, heads, head_dim] with a contiguous last dimension");
    TORCH_CHECK(positions.scalar_type() == torch::kInt32 && positions.is_contiguous(), "positions must be int32");
    require_bf16(query, "query");
    require_bf16(key, "key");
    check(b200_rope_neox_inplace(query.data_ptr(), key.data_ptr(), cos_cache.data_ptr<float>(),
                                 sin_cache.data_ptr<float>(), positions.data_ptr<int32_t>(),
                                 static_cast<int>(positions.size(0)), static_cast<int>(query.size(1)),
                                 static_cast<int>(key.size(1)), static_cast<int>(query.size(2)), rotary_dim_,
                                 static_cast<int>(cos_cache.size(0)), query.stride(0), query.stride(1), key.stride(0),
                                 key.stride(1), current_stream()),
          "b200_rope_neox_inplace");
}

void RotaryEmbedding::forward_inplace(torch::Tensor& positions, torch::Tensor& query, torch::Tensor& key) {
    if (!cos_cache_.is_cuda() && query.is_cuda()) {   // lazy move, as the reference does
        cos_cache_ = cos_cache_.to(query.device());
        sin_cache_ = sin_cache_.to(query.device());
    }
    forward_inplace(positions, query, key, cos_cache_, sin_cache_);
}

}  // namespace sglang
