// The four sampling entry points of include/sglang/engine/sampling.h:12-34 on the C ABI.  Replaces
// src/engine/sampling.cu, whose bodies call FlashInfer's rejection samplers.  Argument checks and
// messages follow the reference (src/engine/sampling.cu:15-61).  b200_sample_from_probs draws by
// inverse CDF over the tokens those samplers accept, with the FIRST round's uniform number of each
// row, and never fails, so `success` is all true and Sampler::sample never needs its CPU fallback.
#include "sglang/engine/sampling.h"

#include <c10/cuda/CUDAGuard.h>

#include "adapter_common.h"

namespace sglang {
namespace {

using b200_adapters::check;
using b200_adapters::current_stream;

void check_probs(const torch::Tensor& probs) {
    TORCH_CHECK(probs.defined(), "probs must be defined");
    TORCH_CHECK(probs.is_cuda(), "FlashInfer sampling requires CUDA probs");
    TORCH_CHECK(probs.is_contiguous(), "FlashInfer sampling requires contiguous probs");
    TORCH_CHECK(probs.scalar_type() == torch::kFloat32, "FlashInfer sampling currently expects float32 probs");
    TORCH_CHECK(probs.dim() == 2, "probs must have shape [batch, vocab]");
}

void check_uniform(const torch::Tensor& probs, const torch::Tensor& u, int64_t dims) {
    TORCH_CHECK(u.defined(), "uniform_samples must be defined");
    TORCH_CHECK(u.is_cuda(), "FlashInfer sampling requires CUDA uniform_samples");
    TORCH_CHECK(u.is_contiguous(), "FlashInfer sampling requires contiguous uniform_samples");
    TORCH_CHECK(u.scalar_type() == torch::kFloat32, "FlashInfer sampling currently expects float32 uniform_samples");
    TORCH_CHECK(u.device() == probs.device(), "uniform_samples must be on the same device as probs");
    TORCH_CHECK(u.dim() == dims, "uniform_samples has unexpected dimensions");
    if (dims == 1) {
        TORCH_CHECK(u.size(0) == probs.size(0), "uniform_samples must have shape [batch]");
    } else {
        TORCH_CHECK(u.size(1) == probs.size(0), "uniform_samples must have shape [max_rounds, batch]");
    }
}

void check_filter(const torch::Tensor& t, const torch::Tensor& probs, torch::ScalarType type, const char* msg) {
    TORCH_CHECK(!t.defined() || (t.is_cuda() && t.is_contiguous() && t.scalar_type() == type &&
                                 t.device() == probs.device() && t.numel() == probs.size(0)),
                msg);
}

FlashInferSamplingResult run(const torch::Tensor& probs, const torch::Tensor& uniform, const torch::Tensor& top_k_i32,
                             int top_k_value, const torch::Tensor& top_p, float top_p_value) {
    c10::cuda::CUDAGuard guard(probs.device());
    auto samples = torch::empty({probs.size(0)}, torch::TensorOptions().dtype(torch::kInt32).device(probs.device()));
    // row 0 of [max_rounds, batch] (or the whole [batch] tensor): the first round's numbers
    check(b200_sample_from_probs(samples.data_ptr<int32_t>(), probs.data_ptr<float>(), static_cast<int>(probs.size(0)),
                                 static_cast<int>(probs.size(1)),
                                 top_k_i32.defined() ? top_k_i32.data_ptr<int32_t>() : nullptr, top_k_value,
                                 top_p.defined() ? top_p.data_ptr<float>() : nullptr, top_p_value,
                                 uniform.data_ptr<float>(), current_stream()),
          "b200_sample_from_probs");
    auto success = torch::ones({probs.size(0)}, torch::TensorOptions().dtype(torch::kBool).device(probs.device()));
    return {samples, success};
}

}  // namespace

torch::Tensor flashinfer_sample_from_probs(const torch::Tensor& probs, const torch::Tensor& uniform_samples,
                                           bool /*deterministic*/) {
    check_probs(probs);
    check_uniform(probs, uniform_samples, 1);
    return run(probs, uniform_samples, torch::Tensor(), 0, torch::Tensor(), 1.0f).samples;
}

FlashInferSamplingResult flashinfer_top_k_sample_from_probs(const torch::Tensor& probs,
                                                            const torch::Tensor& uniform_samples,
                                                            const torch::Tensor& top_k, int64_t top_k_value,
                                                            bool /*deterministic*/) {
    check_probs(probs);
    check_uniform(probs, uniform_samples, 2);
    check_filter(top_k, probs, torch::kFloat32, "top_k must be a contiguous CUDA float32 tensor with shape [batch]");
    // this entry point takes top_k as float32 (src/engine/engine.cc:322-323)
    auto k = top_k.defined() ? top_k.to(torch::kInt32).contiguous() : torch::Tensor();
    return run(probs, uniform_samples, k, static_cast<int>(top_k_value), torch::Tensor(), 1.0f);
}

FlashInferSamplingResult flashinfer_top_p_sample_from_probs(const torch::Tensor& probs,
                                                            const torch::Tensor& uniform_samples,
                                                            const torch::Tensor& top_p, double top_p_value,
                                                            bool /*deterministic*/) {
    check_probs(probs);
    check_uniform(probs, uniform_samples, 2);
    check_filter(top_p, probs, torch::kFloat32, "top_p must be a contiguous CUDA float32 tensor with shape [batch]");
    return run(probs, uniform_samples, torch::Tensor(), 0, top_p, top_p.defined() ? 1.0f : static_cast<float>(top_p_value));
}

FlashInferSamplingResult flashinfer_top_k_top_p_sample_from_probs(const torch::Tensor& probs,
                                                                  const torch::Tensor& uniform_samples,
                                                                  const torch::Tensor& top_k, double top_k_value,
                                                                  const torch::Tensor& top_p, double top_p_value,
                                                                  bool /*deterministic*/) {
    check_probs(probs);
    check_uniform(probs, uniform_samples, 2);
    check_filter(top_k, probs, torch::kInt32, "top_k must be a contiguous CUDA int32 tensor with shape [batch]");
    check_filter(top_p, probs, torch::kFloat32, "top_p must be a contiguous CUDA float32 tensor with shape [batch]");
    return run(probs, uniform_samples, top_k, static_cast<int>(top_k_value), top_p,
               top_p.defined() ? 1.0f : static_cast<float>(top_p_value));
}

}  // namespace sglang
