"""Host-side mirror of sglang.cpp's operator interface, over the C ABI.

Each class / function keeps the reference's name, argument meaning and error
behaviour (a failed check raises, as ``TORCH_CHECK`` does) and unwraps torch CUDA
tensors into the raw pointers, sizes and strides the C ABI takes.  torch is used
for device memory and streams only; all arithmetic happens in the sm_100a
kernels.  Reference locations are given per item.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import _lib
from ._lib import B200Error, call

bf16 = torch.bfloat16


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise B200Error(1, msg)


def _cuda_bf16(t: torch.Tensor, name: str) -> None:
    _check(t.is_cuda, f"{name} must be a CUDA tensor")
    _check(t.dtype == bf16, f"{name} must be bfloat16")


# --------------------------------------------------------------------------- norm
class RMSNorm:
    """include/sglang/layers/normalization.h:6-22 (src/layers/normalization.cu:229-416)."""

    def __init__(self, size: int, eps: float, device="cuda"):
        self.eps_ = float(eps)
        self.weight = torch.ones(size, dtype=bf16, device=device)

    def eps(self) -> float:
        return self.eps_

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(x)
        self._run(out, x)
        return out

    def forward_inplace(self, x: torch.Tensor) -> None:
        self._run(x, x)

    def _run(self, out: torch.Tensor, x: torch.Tensor) -> None:
        _cuda_bf16(x, "x")
        _check(x.dim() >= 2, "RMSNorm expects tensor rank >= 2")
        _check(x.size(-1) > 0, "RMSNorm last dimension must be positive")
        _check(self.weight.size(0) == x.size(-1), "RMSNorm weight size must match last dimension")
        _check(x.is_contiguous() and out.is_contiguous(), "RMSNorm expects contiguous rows")
        d = x.size(-1)
        call("b200_rmsnorm", out.data_ptr(), x.data_ptr(), self.weight.data_ptr(), x.numel() // d, d,
             self.eps_, _stream())

    def fused_add_forward_inplace(self, x: torch.Tensor, residual: torch.Tensor) -> None:
        _cuda_bf16(x, "x")
        _cuda_bf16(residual, "residual")
        _check(x.dim() == 2 and residual.dim() == 2, "FusedAddRMSNorm expects rank-2 tensors")
        _check(x.shape == residual.shape, "x and residual shapes must match")
        _check(x.size(-1) > 0, "RMSNorm last dimension must be positive")
        _check(self.weight.size(0) == x.size(-1), "RMSNorm weight size must match last dimension")
        _check(x.is_contiguous() and residual.is_contiguous(), "FusedAddRMSNorm expects contiguous rows")
        call("b200_fused_add_rmsnorm", x.data_ptr(), residual.data_ptr(), self.weight.data_ptr(),
             x.size(0), x.size(1), self.eps_, _stream())

    def forward_inplace_3d_strided(self, x: torch.Tensor) -> None:
        _cuda_bf16(x, "x")
        _check(x.dim() == 3, "Strided RMSNorm expects rank-3 tensor")
        _check(x.stride(2) == 1, "Last dimension must be contiguous")
        _check(self.weight.size(0) == x.size(2), "RMSNorm weight size must match last dimension")
        call("b200_qk_rmsnorm_strided", x.data_ptr(), None, self.weight.data_ptr(), None, x.size(0),
             x.size(1), 0, x.size(2), x.stride(0), x.stride(1), 0, 0, self.eps_, _stream())


def fused_qk_rmsnorm_inplace_3d_strided(q: torch.Tensor, k: torch.Tensor, q_norm: RMSNorm,
                                        k_norm: RMSNorm) -> None:
    """src/layers/normalization.cu:322-384."""
    _check(q.is_cuda and k.is_cuda, "q and k must be CUDA tensors")
    _check(q.dim() == 3 and k.dim() == 3, "Fused QK RMSNorm expects rank-3 tensors")
    _check(q.stride(2) == 1 and k.stride(2) == 1, "Last dimension must be contiguous")
    _check(q.dtype == k.dtype == bf16, "q and k dtypes must match (bfloat16)")
    _check(q.size(0) == k.size(0), "q and k token dimensions must match")
    _check(q.size(2) == k.size(2), "q and k head dimensions must match")
    d = q.size(2)
    _check(q_norm.weight.size(0) == d and k_norm.weight.size(0) == d,
           "RMSNorm weight size must match last dimension")
    _check(q_norm.eps() == k_norm.eps(), "Q and K RMSNorm eps must match")
    call("b200_qk_rmsnorm_strided", q.data_ptr(), k.data_ptr(), q_norm.weight.data_ptr(),
         k_norm.weight.data_ptr(), q.size(0), q.size(1), k.size(1), d, q.stride(0), q.stride(1),
         k.stride(0), k.stride(1), q_norm.eps(), _stream())


# --------------------------------------------------------------------------- rope
def rope_tables(rotary_dim: int, max_position: int, base: float):
    """cos/sin tables exactly as RotaryEmbedding's constructor builds them on the CPU
    (src/layers/rotary_embedding.cu:75-94): fp32 throughout."""
    inv_freq = 1.0 / torch.pow(
        torch.tensor(base, dtype=torch.float32),
        torch.arange(0, rotary_dim, 2, dtype=torch.float32) / float(rotary_dim))
    t = torch.arange(max_position, dtype=torch.float32)
    freqs = torch.einsum("i,j->ij", t, inv_freq)
    return freqs.cos().contiguous(), freqs.sin().contiguous()


class RotaryEmbedding:
    """include/sglang/layers/rotary_embedding.h:11-22 (src/layers/rotary_embedding.cu:75-190)."""

    def __init__(self, head_size: int, rotary_dim: int, max_position_embeddings: int, base: float):
        self.head_size_ = head_size
        self.rotary_dim_ = rotary_dim
        self.max_position_embeddings_ = max_position_embeddings
        self.base_ = base
        self.cos_cache_, self.sin_cache_ = rope_tables(rotary_dim, max_position_embeddings, base)

    def forward_inplace(self, positions: torch.Tensor, query: torch.Tensor, key: torch.Tensor,
                        cos_cache: Optional[torch.Tensor] = None,
                        sin_cache: Optional[torch.Tensor] = None) -> None:
        _check(query.is_cuda and key.is_cuda and positions.is_cuda, "Inputs must be CUDA tensors")
        if cos_cache is None:
            if not self.cos_cache_.is_cuda:  # lazy move, as the reference does
                self.cos_cache_ = self.cos_cache_.to(query.device)
                self.sin_cache_ = self.sin_cache_.to(query.device)
            cos_cache, sin_cache = self.cos_cache_, self.sin_cache_
        _check(self.rotary_dim_ % 2 == 0, "rotary_dim must be even")
        _check(cos_cache.dim() == 2 and sin_cache.dim() == 2, "cos/sin cache must be rank-2")
        _check(cos_cache.size(1) == self.rotary_dim_ // 2 and sin_cache.size(1) == self.rotary_dim_ // 2,
               "cos/sin cache width must be rotary_dim / 2")
        _check(positions.dtype == torch.int32, "positions must be int32")
        _check(query.dtype == bf16 and key.dtype == bf16, "query and key must be bfloat16")
        _check(query.stride(2) == 1 and key.stride(2) == 1, "Last dimension must be contiguous")
        call("b200_rope_neox_inplace", query.data_ptr(), key.data_ptr(), cos_cache.data_ptr(),
             sin_cache.data_ptr(), positions.data_ptr(), positions.size(0), query.size(1), key.size(1),
             query.size(2), self.rotary_dim_, cos_cache.size(0), query.stride(0), query.stride(1),
             key.stride(0), key.stride(1), _stream())


# --------------------------------------------------------------------------- activation
def silu_and_mul(out: torch.Tensor, input: torch.Tensor) -> None:
    """src/layers/activation.cu:15-44."""
    _check(input.is_cuda and out.is_cuda, "Inputs must be CUDA tensors")
    _check(input.dtype == bf16, "Inputs must be BF16")
    call("b200_silu_and_mul", out.data_ptr(), input.data_ptr(), input.size(0), input.size(1) // 2, _stream())


def gelu_and_mul(out: torch.Tensor, input: torch.Tensor) -> None:
    """src/layers/activation.cu:46-75."""
    _check(input.is_cuda and out.is_cuda, "Inputs must be CUDA tensors")
    _check(input.dtype == bf16, "Inputs must be BF16")
    call("b200_gelu_and_mul", out.data_ptr(), input.data_ptr(), input.size(0), input.size(1) // 2, _stream())


# --------------------------------------------------------------------------- index tables
def write_token_pool(token_pool: torch.Tensor, req_indices: torch.Tensor, positions: torch.Tensor,
                     tokens: torch.Tensor) -> None:
    """src/kernels/token_pool.cu:53-91."""
    for name, t in (("token_pool", token_pool), ("req_indices", req_indices),
                    ("positions", positions), ("tokens", tokens)):
        _check(t.is_cuda, f"{name} must be a CUDA tensor")
        _check(t.dtype == torch.int32, f"{name} must be int32")
    _check(token_pool.dim() == 2, "token_pool must be rank 2")
    _check(req_indices.numel() == positions.numel() == tokens.numel(), "index tensors must have equal length")
    call("b200_write_token_pool", token_pool.data_ptr(), token_pool.size(0), token_pool.stride(0),
         token_pool.size(1), req_indices.data_ptr(), positions.data_ptr(), tokens.data_ptr(),
         req_indices.numel(), _stream())


def gather_int32_2d(table: torch.Tensor, req_indices: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """src/kernels/token_pool.cu:93-133."""
    for name, t in (("table", table), ("req_indices", req_indices), ("positions", positions)):
        _check(t.is_cuda, f"{name} must be a CUDA tensor")
        _check(t.dtype == torch.int32, f"{name} must be int32")
    _check(table.dim() == 2, "table must be rank 2")
    _check(req_indices.numel() == positions.numel(), "index tensors must have equal length")
    out = torch.empty(req_indices.numel(), dtype=torch.int32, device=table.device)
    call("b200_gather_int32_2d", out.data_ptr(), table.data_ptr(), table.size(0), table.stride(0),
         table.size(1), req_indices.data_ptr(), positions.data_ptr(), req_indices.numel(), _stream())
    return out


def embedding(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """torch::nn::Embedding as the models use it (src/models/qwen3.cc:38-43,56); ids int32."""
    _cuda_bf16(table, "table")
    _check(ids.dtype == torch.int32 and ids.is_cuda, "ids must be a CUDA int32 tensor")
    out = torch.empty(ids.numel(), table.size(1), dtype=bf16, device=table.device)
    call("b200_embedding", out.data_ptr(), table.data_ptr(), ids.data_ptr(), ids.numel(), table.size(1),
         table.size(0), _stream())
    return out


# --------------------------------------------------------------------------- linear
def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           epilogue: int = _lib.EPILOGUE_NONE) -> torch.Tensor:
    """torch::nn::functional::linear as LinearBase::forward calls it (src/layers/linear.cc:24-26),
    optionally with the gated activation of GatedMLP::forward folded in (src/models/utils.cc:41-57)."""
    _cuda_bf16(x, "x")
    _cuda_bf16(weight, "weight")
    _check(x.dim() == 2 and weight.dim() == 2, "linear expects rank-2 x and weight")
    _check(x.size(1) == weight.size(1), "linear: inner dimensions must match")
    _check(x.stride(1) == 1 and weight.is_contiguous(), "linear: rows must be contiguous")
    n_out = weight.size(0) if epilogue == _lib.EPILOGUE_NONE else weight.size(0) // 2
    y = torch.empty(x.size(0), n_out, dtype=bf16, device=x.device)
    call("b200_linear", y.data_ptr(), x.data_ptr(), weight.data_ptr(), _ptr(bias), x.size(0),
         weight.size(0), weight.size(1), x.stride(0), epilogue, _stream())
    return y


class LinearBase:
    """include/sglang/layers/linear.h:7-20: weight [local_osize, local_isize], optional bias."""

    def __init__(self, full_isize: int, full_osize: int, local_isize: int, local_osize: int,
                 has_bias: bool, device="cuda"):
        self.full_input_size_ = full_isize
        self.full_output_size_ = full_osize
        self.local_input_size_ = local_isize
        self.local_output_size_ = local_osize
        self.has_bias_ = has_bias
        self.weight = torch.empty(local_osize, local_isize, dtype=bf16, device=device)
        self.bias = torch.empty(local_osize, dtype=bf16, device=device) if has_bias else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return linear(x, self.weight, self.bias if self.has_bias_ else None)


# --------------------------------------------------------------------------- KV pool
class MHAKVCache:
    """include/sglang/kvcache/base.h:78-90, src/kvcache/mha_kvcache.cu:88-155.
    Buffer layout [2, layers, slots, kv_heads, head_dim] bf16."""

    def __init__(self, num_kv_heads: int, num_layers: int, head_dim: int, num_pages: int,
                 page_size: int, device="cuda"):
        self.num_layers_ = num_layers
        self.num_pages_ = num_pages
        self.page_size_ = page_size
        self.kv_heads_ = num_kv_heads
        self.head_dim_ = head_dim
        self.total_slots = num_pages * page_size
        self.kv_buffer_ = torch.zeros(2, num_layers, self.total_slots, num_kv_heads, head_dim,
                                      dtype=bf16, device=device)
        self.k_buffer_ = self.kv_buffer_[0]
        self.v_buffer_ = self.kv_buffer_[1]

    def k_cache(self, layer_id: int) -> torch.Tensor:
        return self.k_buffer_[layer_id]

    def v_cache(self, layer_id: int) -> torch.Tensor:
        return self.v_buffer_[layer_id]

    def num_layers(self) -> int:
        return self.num_layers_

    def store_kv(self, key: torch.Tensor, val: torch.Tensor, out_loc: torch.Tensor, layer_id: int) -> None:
        _check(key.is_cuda and val.is_cuda and out_loc.is_cuda, "key, val and out_loc must be CUDA tensors")
        _check(key.dtype == val.dtype == bf16, "key and val dtype must match (bfloat16)")
        _check(key.stride(-1) == 1 and val.stride(-1) == 1, "key and val last dimension must be contiguous")
        _check(out_loc.dim() == 1 and out_loc.dtype == torch.int32, "out_loc must be rank 1 int32")
        k = key if key.dim() == 2 else key.reshape(key.size(0), -1)
        v = val if val.dim() == 2 else val.reshape(val.size(0), -1)
        _check(k.size(0) == v.size(0) == out_loc.size(0), "key, val and out_loc token counts must match")
        _check(k.size(1) == self.kv_heads_ * self.head_dim_ == v.size(1),
               "key and val shape must match KV cache layout")
        call("b200_store_kv", self.k_cache(layer_id).data_ptr(), self.v_cache(layer_id).data_ptr(),
             k.data_ptr(), v.data_ptr(), out_loc.data_ptr(), k.size(0), self.kv_heads_, self.head_dim_,
             k.stride(0), v.stride(0), self.total_slots, _stream())


# --------------------------------------------------------------------------- attention
class PagedAttention:
    """Stands where FlashInferBackend::forward does (src/attention/flashinfer_backend.cu:522-682),
    without its host-side planning: the kernels read page_table rows directly."""

    def __init__(self, kv_cache: MHAKVCache, num_qo_heads: int, num_kv_heads: int, head_dim: int,
                 max_batch: int = 256):
        self.kv_cache_ = kv_cache
        self.num_qo_heads_ = num_qo_heads
        self.num_kv_heads_ = num_kv_heads
        self.head_dim_ = head_dim
        self.sm_scale = 1.0 / math.sqrt(head_dim)
        nbytes = _lib.load().b200_attention_decode_workspace_bytes(max_batch, num_qo_heads, num_kv_heads, head_dim)
        _check(nbytes > 0, "unsupported head configuration for decode attention")
        self.workspace = torch.zeros(nbytes, dtype=torch.uint8, device=kv_cache.kv_buffer_.device)

    def decode(self, q: torch.Tensor, layer_id: int, page_table: torch.Tensor, table_idx: torch.Tensor,
               seq_lens: torch.Tensor) -> torch.Tensor:
        kc = self.kv_cache_
        out = torch.empty(q.size(0), self.num_qo_heads_ * self.head_dim_, dtype=bf16, device=q.device)
        call("b200_attention_decode", out.data_ptr(), q.data_ptr(), q.stride(0), q.stride(1),
             kc.k_cache(layer_id).data_ptr(), kc.v_cache(layer_id).data_ptr(), kc.total_slots,
             page_table.data_ptr(), page_table.stride(0), table_idx.data_ptr(), seq_lens.data_ptr(),
             q.size(0), self.num_qo_heads_, self.num_kv_heads_, self.head_dim_, kc.page_size_,
             self.sm_scale, self.workspace.data_ptr(), self.workspace.numel(), _stream())
        return out

    def prefill(self, q: torch.Tensor, layer_id: int, page_table: torch.Tensor, table_idx: torch.Tensor,
                seq_lens: torch.Tensor, qo_indptr: torch.Tensor, max_extend_len: int) -> torch.Tensor:
        kc = self.kv_cache_
        out = torch.empty(q.size(0), self.num_qo_heads_ * self.head_dim_, dtype=bf16, device=q.device)
        call("b200_attention_prefill", out.data_ptr(), q.data_ptr(), q.stride(0), q.stride(1),
             kc.k_cache(layer_id).data_ptr(), kc.v_cache(layer_id).data_ptr(), kc.total_slots,
             page_table.data_ptr(), page_table.stride(0), table_idx.data_ptr(), seq_lens.data_ptr(),
             qo_indptr.data_ptr(), table_idx.numel(), max_extend_len, self.num_qo_heads_,
             self.num_kv_heads_, self.head_dim_, kc.page_size_, self.sm_scale, _stream())
        return out


def qknorm_rope_store(qkv: torch.Tensor, q_norm: Optional[RMSNorm], k_norm: Optional[RMSNorm],
                      rotary: RotaryEmbedding, positions: torch.Tensor, out_loc: torch.Tensor,
                      kv_cache: MHAKVCache, layer_id: int, num_qo_heads: int, num_kv_heads: int,
                      write_k_back: bool = False) -> None:
    """The pre-attention steps of AttentionLayer::forward (src/layers/attention_layer.cc:17-47) and the
    backend's store_kv (src/attention/flashinfer_backend.cu:530-532) as one pass."""
    _cuda_bf16(qkv, "qkv")
    _check(qkv.is_contiguous(), "qkv must be contiguous")
    d = kv_cache.head_dim_
    _check(qkv.size(1) == (num_qo_heads + 2 * num_kv_heads) * d, "qkv width mismatch")
    if not rotary.cos_cache_.is_cuda:
        rotary.cos_cache_ = rotary.cos_cache_.to(qkv.device)
        rotary.sin_cache_ = rotary.sin_cache_.to(qkv.device)
    eps = q_norm.eps() if q_norm is not None else 0.0
    call("b200_qknorm_rope_store", qkv.data_ptr(), _ptr(q_norm.weight) if q_norm else None,
         _ptr(k_norm.weight) if k_norm else None, rotary.cos_cache_.data_ptr(),
         rotary.sin_cache_.data_ptr(), positions.data_ptr(), out_loc.data_ptr(),
         kv_cache.k_cache(layer_id).data_ptr(), kv_cache.v_cache(layer_id).data_ptr(), qkv.size(0),
         num_qo_heads, num_kv_heads, d, rotary.cos_cache_.size(0), kv_cache.total_slots, eps,
         1 if write_k_back else 0, _stream())


# --------------------------------------------------------------------------- MoE
class MoELayer:
    """include/sglang/moe/moe.h:9-35, src/moe/moe.cc:7-96 (tp_size 1)."""

    def __init__(self, num_experts: int, top_k: int, hidden_size: int, intermediate_size: int,
                 renormalize: bool = False, activation: str = "silu", device="cuda",
                 expert_begin: int = 0, num_local_experts: Optional[int] = None):
        """expert_begin / num_local_experts (not in the reference): hold only that slice of the
        router's experts; forward then returns this rank's partial sum."""
        _check(num_experts > 0, "MoELayer requires num_experts > 0")
        _check(top_k > 0, "MoELayer requires top_k > 0")
        _check(top_k <= num_experts, "MoELayer top_k must be <= num_experts")
        _check(hidden_size > 0, "MoELayer requires hidden_size > 0")
        _check(intermediate_size > 0, "MoELayer requires intermediate_size > 0")
        _check(activation in ("silu", "gelu"), f"Unsupported MoE activation function: {activation}")
        self.num_experts_, self.top_k_ = num_experts, top_k
        self.hidden_size_, self.intermediate_size_ = hidden_size, intermediate_size
        self.renormalize_, self.activation_ = renormalize, activation
        self.expert_begin_ = expert_begin
        self.num_local_ = num_experts if num_local_experts is None else num_local_experts
        self.gate_up_proj = torch.empty(self.num_local_, 2 * intermediate_size, hidden_size, dtype=bf16, device=device)
        self.down_proj = torch.empty(self.num_local_, hidden_size, intermediate_size, dtype=bf16, device=device)
        self.w1, self.w2 = self.gate_up_proj, self.down_proj
        self._ws = None

    def forward(self, hidden_states: torch.Tensor, router_logits: torch.Tensor) -> torch.Tensor:
        _check(hidden_states.dim() == 2, "MoELayer hidden_states must be [num_tokens, hidden_size]")
        _check(router_logits.dim() == 2, "MoELayer router_logits must be [num_tokens, num_experts]")
        _check(hidden_states.size(0) == router_logits.size(0), "MoELayer token count mismatch")
        _check(hidden_states.size(1) == self.hidden_size_, "MoELayer hidden size mismatch")
        _check(router_logits.size(1) == self.num_experts_, "MoELayer expert count mismatch")
        _cuda_bf16(hidden_states, "hidden_states")
        _cuda_bf16(router_logits, "router_logits")
        T = hidden_states.size(0)
        need = _lib.load().b200_moe_workspace_bytes(T, self.num_experts_, self.top_k_, self.hidden_size_,
                                                    self.intermediate_size_)
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(need, dtype=torch.uint8, device=hidden_states.device)
        out = torch.empty_like(hidden_states)
        call("b200_moe_forward_local", out.data_ptr(), hidden_states.contiguous().data_ptr(),
             router_logits.contiguous().data_ptr(), self.gate_up_proj.data_ptr(), self.down_proj.data_ptr(), T,
             self.num_experts_, self.top_k_, self.hidden_size_, self.intermediate_size_,
             1 if self.renormalize_ else 0, 1 if self.activation_ == "gelu" else 0, self.expert_begin_,
             self.num_local_, self._ws.data_ptr(), self._ws.numel(), _stream())
        return out


def moe_route(router_logits: torch.Tensor, top_k: int, renormalize: bool):
    """Routing of MoELayer::forward (src/moe/moe.cc:47-55): (ids int32, weights float32, counts int32)."""
    _cuda_bf16(router_logits, "router_logits")
    T, E = router_logits.shape
    ids = torch.empty(T, top_k, dtype=torch.int32, device=router_logits.device)
    w = torch.empty(T, top_k, dtype=torch.float32, device=router_logits.device)
    counts = torch.empty(E + 1, dtype=torch.int32, device=router_logits.device)
    call("b200_moe_route", ids.data_ptr(), w.data_ptr(), counts.data_ptr(), router_logits.contiguous().data_ptr(),
         T, E, top_k, 1 if renormalize else 0, _stream())
    return ids, w, counts[:E]


# --------------------------------------------------------------------------- sampler
def argmax(logits: torch.Tensor) -> torch.Tensor:
    """Sampler::sample, greedy branch (src/engine/engine.cc:294-298); returns int32."""
    _cuda_bf16(logits, "logits")
    _check(logits.dim() == 2 and logits.stride(1) == 1, "logits must be rank 2 with contiguous rows")
    out = torch.empty(logits.size(0), dtype=torch.int32, device=logits.device)
    call("b200_argmax", out.data_ptr(), logits.data_ptr(), logits.size(0), logits.size(1),
         logits.stride(0), _stream())
    return out


def sample(logits: torch.Tensor, temperatures: torch.Tensor, top_k: Optional[torch.Tensor] = None,
           top_p: Optional[torch.Tensor] = None, seeds: Optional[torch.Tensor] = None,
           step_index: int = 0, return_mask: bool = False):
    """Sampler::sample, stochastic branch (src/engine/engine.cc:299-338); args as BatchSamplingArgs
    (include/sglang/engine/engine.h:22-26) holds them: float32 temperatures, int32 top_k, float32
    top_p, all on the device.  Returns int32 tokens (and the uint8 candidate mask if asked)."""
    _cuda_bf16(logits, "logits")
    _check(logits.dim() == 2 and logits.stride(1) == 1, "logits must be rank 2 with contiguous rows")
    _check(temperatures.dtype == torch.float32 and temperatures.numel() == logits.size(0),
           "temperatures must be float32 [rows]")
    out = torch.empty(logits.size(0), dtype=torch.int32, device=logits.device)
    mask = torch.empty(logits.shape, dtype=torch.uint8, device=logits.device) if return_mask else None
    call("b200_sample", out.data_ptr(), logits.data_ptr(), logits.size(0), logits.size(1), logits.stride(0),
         temperatures.data_ptr(), _ptr(top_k), _ptr(top_p), _ptr(seeds), step_index, _ptr(mask), _stream())
    return (out, mask) if return_mask else out


def sample_from_probs(probs: torch.Tensor, uniform: torch.Tensor, top_k: Optional[torch.Tensor] = None,
                      top_p: Optional[torch.Tensor] = None, top_k_value: int = 0,
                      top_p_value: float = 1.0) -> torch.Tensor:
    """flashinfer_*_sample_from_probs (include/sglang/engine/sampling.h:12-34): fp32 probs
    [rows, vocab], one uniform number per row, optional per-row top_k (int32) / top_p (fp32)."""
    _check(probs.is_cuda and probs.dtype == torch.float32 and probs.dim() == 2 and probs.is_contiguous(),
           "probs must be a contiguous CUDA float32 tensor [batch, vocab]")
    _check(uniform.is_cuda and uniform.dtype == torch.float32 and uniform.numel() >= probs.size(0),
           "uniform_samples must be CUDA float32 with one number per row")
    out = torch.empty(probs.size(0), dtype=torch.int32, device=probs.device)
    call("b200_sample_from_probs", out.data_ptr(), probs.data_ptr(), probs.size(0), probs.size(1), _ptr(top_k),
         top_k_value, _ptr(top_p), top_p_value, uniform.data_ptr(), _stream())
    return out


def read_device_status() -> tuple[int, int]:
    import ctypes
    buf = (ctypes.c_int32 * 2)()
    call("b200_read_device_status", buf, _stream())
    return int(buf[0]), int(buf[1])
