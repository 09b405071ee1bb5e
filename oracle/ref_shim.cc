// C wrapper around the reference's own CPU-capable MoE layer — TEST INFRASTRUCTURE ONLY.
//
// build_ref.py compiles this file together with the reference's src/moe/moe.cc (taken from the
// reference tree where it lies, never copied) against the LibTorch that ships inside the torch
// wheel.  The three tensor-parallel helpers moe.cc calls are defined here for the single-rank
// case (the reference's own definitions live in src/distributed/distributed.cc, which needs NCCL):
// tp_size() == 1, divide_even checks divisibility, and the all-reduce is the identity, exactly
// what the reference does when tp_size() == 1 (src/distributed/distributed.cc:205-226).
#include <cstdint>
#include <cstring>
#include <string>

#include <torch/torch.h>

#include "sglang/distributed/distributed.h"
#include "sglang/moe/moe.h"

namespace sglang {
int tp_size() { return 1; }
int tp_rank() { return 0; }
int divide_even(int value, int divisor, const char* name) {
    TORCH_CHECK(divisor > 0 && value % divisor == 0, name, " must be divisible by ", divisor);
    return value / divisor;
}
torch::Tensor tensor_model_parallel_all_reduce(const torch::Tensor& x) { return x; }
}  // namespace sglang

extern "C" {

// out[T, H] = MoELayer(E, top_k, H, I, renormalize, activation).forward(hidden, router_logits)
// with gate_up [E, 2I, H] and down [E, H, I]; all fp32, row-major.  Returns 0, or 1 on a
// c10::Error (message copied to err, if given).
int ref_moe_forward(const float* hidden, const float* router_logits, const float* gate_up,
                    const float* down, int T, int E, int top_k, int H, int I, int renormalize,
                    const char* activation, float* out, char* err, int err_len) {
    try {
        torch::NoGradGuard no_grad;
        sglang::MoELayer moe(E, top_k, H, I, renormalize != 0, std::string(activation));
        auto opts = torch::TensorOptions().dtype(torch::kFloat32);
        moe.gate_up_proj.copy_(torch::from_blob(const_cast<float*>(gate_up), {E, 2 * I, H}, opts));
        moe.down_proj.copy_(torch::from_blob(const_cast<float*>(down), {E, H, I}, opts));
        auto h = torch::from_blob(const_cast<float*>(hidden), {T, H}, opts).clone();
        auto r = torch::from_blob(const_cast<float*>(router_logits), {T, E}, opts).clone();
        auto y = moe.forward(h, r).contiguous();
        std::memcpy(out, y.data_ptr<float>(), sizeof(float) * static_cast<size_t>(T) * H);
        return 0;
    } catch (const std::exception& e) {
        if (err && err_len > 0) {
            std::strncpy(err, e.what(), static_cast<size_t>(err_len) - 1);
            err[err_len - 1] = 0;
        }
        return 1;
    }
}

}  // extern "C"
