// sglang::RMSNorm and fused_qk_rmsnorm_inplace_3d_strided (include/sglang/layers/normalization.h:6-22)
// on the C ABI.  Replaces src/layers/normalization.cu, whose bodies call FlashInfer's norm kernels.
// Same argument checks and messages as the reference (src/layers/normalization.cu:229-416).
#include "sglang/layers/normalization.h"

#include "adapter_common.h"

namespace sglang {

using b200_adapters::check;
using b200_adapters::current_stream;
using b200_adapters::require_bf16;

RMSNorm::RMSNorm(int size, float eps) : eps_(eps) {
    // the reference registers an fp16 CUDA parameter; Module::to(device, dtype) converts it with the model
    weight = register_parameter("weight", torch::ones({size}, torch::device(torch::kCUDA).dtype(torch::kFloat16)));
}

torch::Tensor RMSNorm::forward(const torch::Tensor& x) {
    auto out = torch::empty_like(x);
    out.copy_(x);
    forward_inplace(out);
    return out;
}

void RMSNorm::forward_inplace(torch::Tensor& x) {
    TORCH_CHECK(x.is_cuda(), "x must be a CUDA tensor");
    TORCH_CHECK(x.dim() >= 2, "RMSNorm expects tensor rank >= 2");
    TORCH_CHECK(x.size(-1) > 0, "RMSNorm last dimension must be positive");
    const int64_t d = x.size(-1);
    TORCH_CHECK(weight.size(0) == d, "RMSNorm weight size must match last dimension");
    TORCH_CHECK(x.is_contiguous(), "RMSNorm expects contiguous rows");
    require_bf16(x, "x");
    require_bf16(weight, "RMSNorm weight");
    check(b200_rmsnorm(x.data_ptr(), x.data_ptr(), weight.data_ptr(), static_cast<int>(x.numel() / d),
                       static_cast<int>(d), eps_, current_stream()),
          "b200_rmsnorm");
}

void RMSNorm::forward_inplace_3d_strided(torch::Tensor& x) {
    TORCH_CHECK(x.is_cuda(), "x must be a CUDA tensor");
    TORCH_CHECK(x.dim() == 3, "Strided RMSNorm expects rank-3 tensor");
    TORCH_CHECK(x.stride(2) == 1, "Last dimension must be contiguous");
    TORCH_CHECK(weight.size(0) == x.size(2), "RMSNorm weight size must match last dimension");
    if (x.size(0) * x.size(1) == 0) return;
    require_bf16(x, "x");
    require_bf16(weight, "RMSNorm weight");
    check(b200_qk_rmsnorm_strided(x.data_ptr(), nullptr, weight.data_ptr(), nullptr, static_cast<int>(x.size(0)),
                                  static_cast<int>(x.size(1)), 0, static_cast<int>(x.size(2)), x.stride(0),
                                  x.stride(1), 0, 0, eps_, current_stream()),
          "b200_qk_rmsnorm_strided");
}

void RMSNorm::fused_add_forward_inplace(torch::Tensor& x, torch::Tensor& residual) {
    TORCH_CHECK(x.is_cuda() && residual.is_cuda(), "x and residual must be CUDA tensors");
    TORCH_CHECK(x.dim() == 2 && residual.dim() == 2, "FusedAddRMSNorm expects rank-2 tensors");
    TORCH_CHECK(x.sizes() == residual.sizes(), "x and residual shapes must match");
    TORCH_CHECK(x.size(-1) > 0, "RMSNorm last dimension must be positive");
    TORCH_CHECK(weight.size(0) == x.size(-1), "RMSNorm weight size must match last dimension");
    TORCH_CHECK(x.is_contiguous() && residual.is_contiguous(), "FusedAddRMSNorm expects contiguous rows");
    require_bf16(x, "x");
    require_bf16(residual, "residual");
    require_bf16(weight, "RMSNorm weight");
    check(b200_fused_add_rmsnorm(x.data_ptr(), residual.data_ptr(), weight.data_ptr(), static_cast<int>(x.size(0)),
                                 static_cast<int>(x.size(1)), eps_, current_stream()),
          "b200_fused_add_rmsnorm");
}

void fused_qk_rmsnorm_inplace_3d_strided(torch::Tensor& q, torch::Tensor& k, const RMSNorm& q_norm,
                                         const RMSNorm& k_norm) {
    TORCH_CHECK(q.is_cuda() && k.is_cuda(), "q and k must be CUDA tensors");
    TORCH_CHECK(q.dim() == 3 && k.dim() == 3, "Fused QK RMSNorm expects rank-3 tensors");
    TORCH_CHECK(q.stride(2) == 1 && k.stride(2) == 1, "Last dimension must be contiguous");
    TORCH_CHECK(q.scalar_type() == k.scalar_type(), "q and k dtypes must match");
    TORCH_CHECK(q.size(0) == k.size(0), "q and k token dimensions must match");
    TORCH_CHECK(q.size(2) == k.size(2), "q and k head dimensions must match");
    const int64_t d = q.size(2);
    TORCH_CHECK(q_norm.weight.size(0) == d && k_norm.weight.size(0) == d,
                "RMSNorm weight size must match last dimension");
    if (q.size(0) * (q.size(1) + k.size(1)) == 0) return;
    TORCH_CHECK(q_norm.eps() == k_norm.eps(), "Q and K RMSNorm eps must match");
    require_bf16(q, "q");
    require_bf16(q_norm.weight, "RMSNorm weight");
    require_bf16(k_norm.weight, "RMSNorm weight");
    check(b200_qk_rmsnorm_strided(q.data_ptr(), k.data_ptr(), q_norm.weight.data_ptr(), k_norm.weight.data_ptr(),
                                  static_cast<int>(q.size(0)), static_cast<int>(q.size(1)),
                                  static_cast<int>(k.size(1)), static_cast<int>(d), q.stride(0), q.stride(1),
                                  k.stride(0), k.stride(1), q_norm.eps(), current_stream()),
          "b200_qk_rmsnorm_strided");
}

}  // namespace sglang
