// Shared by the adapter translation units: LibTorch on one side, the C ABI on the other.
//
// The adapters define the reference's own C++ symbols (same class declarations, taken from the
// reference's headers at build time) on top of libb200_token_loop.so.  They are the only place
// where torch::Tensor appears; below them everything is raw pointers, sizes, strides and a stream.
#pragma once

#include <ATen/cuda/CUDAContext.h>
#include <torch/torch.h>

#include "b200_token_loop.h"

namespace b200_adapters {

// The reference raises c10::Error through TORCH_CHECK; the C ABI returns a status and keeps the
// message in b200_last_error().
inline void check(int status, const char* what) {
    TORCH_CHECK(status == B200_OK, what, " failed: ", b200_last_error());
}

inline b200_stream_t current_stream() {
    return static_cast<b200_stream_t>(at::cuda::getCurrentCUDAStream().stream());
}

inline void require_bf16(const torch::Tensor& t, const char* name) {
    TORCH_CHECK(t.scalar_type() == torch::kBFloat16, name,
                " must be bfloat16: the sm_100a kernels behind these adapters compute in bf16 "
                "(set EngineConfig::dtype = torch::kBFloat16)");
}

}  // namespace b200_adapters
