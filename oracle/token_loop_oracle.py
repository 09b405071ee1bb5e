"""CPU oracle for the per-step token loop of sglang.cpp — TEST INFRASTRUCTURE ONLY.

This file restates, in plain torch-CPU fp32, the arithmetic the reference runs on
the GPU for one prefill or decode step (Engine::forward_batch,
src/engine/engine.cc:495-544).  Only tests, the smoke check and the CPU-baseline
leg of the benchmark may import it; the product path never does.

Parity status.  The reference has no CPU implementation of the dense forward
(its layers assert CUDA tensors) and its RMSNorm / RoPE / SiLU-mul / attention /
sampling kernels come from FlashInfer v0.2.0.post1, which is not part of the
reference tree; the GEMMs are cuBLAS.  The reference's tests hold no golden
vectors for those operators, so for them this oracle is a restatement of the
published math: "parity unpinned".  What IS pinned against the reference's own
known-answer tests (tests/golden/): the greedy / top-p sampler rows
(tests/engine/test_sampler.cpp:21-48), the MoE layer
(tests/moe/test_moe.cpp:69-99) and the int32 index-table kernels
(src/kernels/token_pool.cu:10-49).

Every function takes a `store` callable that is applied wherever the reference
writes a tensor back to bf16 memory: `store_bf16` reproduces the reference's
rounding points, `store_fp32` (identity) gives the exact-arithmetic answer.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Optional

import numpy as np
import torch

f32 = torch.float32


def store_bf16(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(f32)


def store_fp32(t: torch.Tensor) -> torch.Tensor:
    return t


Store = Callable[[torch.Tensor], torch.Tensor]


# --------------------------------------------------------------------------- operators
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, store: Store = store_bf16) -> torch.Tensor:
    """src/layers/normalization.cu:27-43 (the math every RMSNorm variant shares): fp32 sum of
    squares, rsqrt(ss / d + eps), val * scale * w."""
    x = x.to(f32)
    scale = torch.rsqrt((x * x).sum(-1, keepdim=True) / x.shape[-1] + eps)
    return store(x * scale * w.to(f32))


def fused_add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float,
                      store: Store = store_bf16):
    """RMSNorm::fused_add_forward_inplace (src/layers/normalization.cu:386-416 -> FlashInfer
    FusedAddRMSNorm): residual <- x + residual (stored), x <- norm(unrounded sum) * w.
    Returns (x_out, residual_out)."""
    s = x.to(f32) + residual.to(f32)
    scale = torch.rsqrt((s * s).sum(-1, keepdim=True) / s.shape[-1] + eps)
    return store(s * scale * w.to(f32)), store(s)


def rope_tables(rotary_dim: int, max_position: int, base: float):
    """RotaryEmbedding constructor (src/layers/rotary_embedding.cu:75-94)."""
    inv_freq = 1.0 / torch.pow(torch.tensor(base, dtype=f32),
                               torch.arange(0, rotary_dim, 2, dtype=f32) / float(rotary_dim))
    t = torch.arange(max_position, dtype=f32)
    freqs = torch.einsum("i,j->ij", t, inv_freq)
    return freqs.cos().contiguous(), freqs.sin().contiguous()


def rope_neox(x: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
              rotary_dim: Optional[int] = None, store: Store = store_bf16) -> torch.Tensor:
    """NeoX rotation of x [tokens, heads, d] (src/layers/rotary_embedding.cu:49-66)."""
    x = x.to(f32)
    d = x.shape[-1]
    rd = d if rotary_dim is None else rotary_dim
    half = rd // 2
    c = cos[positions.long()][:, None, :half]
    s = sin[positions.long()][:, None, :half]
    x1, x2 = x[..., :half], x[..., half:rd]
    out = x.clone()
    out[..., :half] = x1 * c - x2 * s
    out[..., half:rd] = x2 * c + x1 * s
    return store(out)


def silu_and_mul(x: torch.Tensor, store: Store = store_bf16) -> torch.Tensor:
    """src/layers/activation.cu:7-9,15-44: silu(x) = x / (1 + exp(-x))."""
    x = x.to(f32)
    d = x.shape[-1] // 2
    g, u = x[..., :d], x[..., d:]
    return store(g / (1.0 + torch.exp(-g)) * u)


def gelu_and_mul(x: torch.Tensor, store: Store = store_bf16) -> torch.Tensor:
    """src/layers/activation.cu:11-13,46-75: tanh-approximated GELU."""
    x = x.to(f32)
    d = x.shape[-1] // 2
    g, u = x[..., :d], x[..., d:]
    act = 0.5 * g * (1.0 + torch.tanh(0.7978845608 * (g + 0.044715 * g * g * g)))
    return store(act * u)


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
           store: Store = store_bf16) -> torch.Tensor:
    """LinearBase::forward (src/layers/linear.cc:24-26): y = x W^T + b, fp32 accumulate."""
    y = x.to(f32) @ w.to(f32).t()
    if bias is not None:
        y = y + bias.to(f32)
    return store(y)


def gather_int32_2d(table: np.ndarray, req: np.ndarray, pos: np.ndarray) -> np.ndarray:
    """src/kernels/token_pool.cu:31-49."""
    rows, cols = table.shape
    out = np.zeros(len(req), dtype=np.int32)
    for i, (r, p) in enumerate(zip(req.tolist(), pos.tolist())):
        if 0 <= r < rows and 0 <= p < cols:
            out[i] = table[r, p]
    return out


def write_token_pool(table: np.ndarray, req: np.ndarray, pos: np.ndarray, tokens: np.ndarray) -> None:
    """src/kernels/token_pool.cu:10-29 (in place)."""
    rows, cols = table.shape
    for r, p, t in zip(req.tolist(), pos.tolist(), tokens.tolist()):
        if 0 <= r < rows and 0 <= p < cols:
            table[r, p] = t


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    page_table: np.ndarray, table_idx, seq_lens, qo_indptr, sm_scale: float,
                    store: Store = store_bf16) -> torch.Tensor:
    """Causal GQA attention over paged keys (src/attention/flashinfer_backend.cu:553-678: scale
    1/sqrt(d), causal, no soft-cap / window).  q [tokens, Hq, d]; caches [slots, Hkv, d]; request b
    owns query rows qo_indptr[b]:qo_indptr[b+1], which are the last positions of its seq_lens[b]
    keys.  Decode is the case of one query row per request."""
    q = q.to(f32)
    tokens, hq, d = q.shape
    hkv = k_cache.shape[1]
    g = hq // hkv
    out = torch.zeros(tokens, hq, d, dtype=f32)
    for b in range(len(seq_lens)):
        n = int(seq_lens[b])
        q0, q1 = int(qo_indptr[b]), int(qo_indptr[b + 1])
        ext = q1 - q0
        if ext <= 0 or n <= 0:
            continue
        slots = torch.from_numpy(np.asarray(page_table[int(table_idx[b]), :n]).astype(np.int64))
        k = k_cache[slots].to(f32)  # [n, hkv, d]
        v = v_cache[slots].to(f32)
        k = k.repeat_interleave(g, dim=1)
        v = v.repeat_interleave(g, dim=1)
        s = torch.einsum("qhd,khd->hqk", q[q0:q1], k) * sm_scale
        pos = torch.arange(n - ext, n)[:, None]
        mask = torch.arange(n)[None, :] > pos
        s = s.masked_fill(mask[None], float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[q0:q1] = torch.einsum("hqk,khd->qhd", p, v)
    return store(out)


def moe_forward(hidden: torch.Tensor, router_logits: torch.Tensor, gate_up: torch.Tensor,
                down: torch.Tensor, top_k: int, renormalize: bool, activation: str = "silu",
                store: Store = store_bf16, expert_begin: int = 0) -> torch.Tensor:
    """MoELayer::forward (src/moe/moe.cc:36-96), loop order and rounding points included:
    fp32 softmax -> top-k -> optional renormalisation -> weights cast to the activation dtype ->
    for k, for expert: linear, act*up, linear, scale, index_add_.

    ``expert_begin`` (no counterpart in the reference, which shards every expert's intermediate
    dimension instead): gate_up / down hold only experts [expert_begin, expert_begin + len) of the
    router's range and only their contributions are summed — one rank's share under expert
    parallelism, to be summed over ranks by the all-reduce that follows."""
    h = hidden.to(f32)
    probs = torch.softmax(router_logits.to(f32), -1)
    tw, ti = probs.topk(top_k, -1)
    if renormalize:
        tw = tw / (tw.sum(-1, keepdim=True) + 1e-8)
    out = torch.zeros_like(h)
    E = gate_up.shape[0]
    for k in range(top_k):
        ids = ti[:, k] - expert_begin
        w = store(tw[:, k])
        for e in range(E):
            idx = torch.nonzero(ids == e).squeeze(1)
            if idx.numel() == 0:
                continue
            xin = h.index_select(0, idx)
            gu = store(xin @ gate_up[e].to(f32).t())
            inter = gu.shape[1] // 2
            g, u = gu[:, :inter], gu[:, inter:]
            if activation == "silu":
                act = store(store(g * torch.sigmoid(g)) * u)
            else:
                act = store(store(torch.nn.functional.gelu(g)) * u)
            eo = store(act @ down[e].to(f32).t())
            eo = store(eo * w.index_select(0, idx).unsqueeze(1))
            out.index_add_(0, idx, eo)
            out = store(out)
    return out


# --------------------------------------------------------------------------- sampler
def greedy(logits: torch.Tensor) -> torch.Tensor:
    """Sampler::sample with no temperatures (src/engine/engine.cc:294-298)."""
    return torch.argmax(logits, -1)


def prepare_sampling(temperature: float, top_k: int, top_p: float, vocab: int, is_greedy: bool):
    """Per-request clamping done by Sampler::prepare (src/engine/engine.cc:264-275)."""
    t = max(0.0 if is_greedy else temperature, 1e-6)
    k = top_k if top_k >= 1 else vocab
    p = min(max(top_p, 1e-6), 1.0)
    return t, k, p


def sample_row_distribution(logits: torch.Tensor, temperature: float, top_k: int, top_p: float) -> torch.Tensor:
    """The distribution sample_row draws from (src/engine/engine.cc:126-158): temperature, top-k
    mask, then top-p over the sorted softmax with the first entry always kept.  Returns probs
    [vocab] (zeros outside the candidate set)."""
    logits = logits.to(f32) / max(temperature, 1e-6)
    if 0 < top_k < logits.shape[0]:
        vals, idx = torch.topk(logits, top_k)
        filt = torch.full_like(logits, float("-inf"))
        filt[idx] = vals
        logits = filt
    if top_p < 1.0:
        sl, si = torch.sort(logits, -1, descending=True)
        probs = torch.softmax(sl, -1)
        cum = torch.cumsum(probs, -1)
        cutoff = cum > top_p
        cutoff[0] = False
        sl = sl.masked_fill(cutoff, float("-inf"))
        filt = torch.full_like(logits, float("-inf"))
        filt[si] = sl
        logits = filt
    return torch.softmax(logits, -1)


def sample_from_probs(probs: torch.Tensor, u: float, top_k: int = 0, top_p: float = 1.0):
    """What flashinfer_*_sample_from_probs return in distribution (src/engine/sampling.cu:65-192 call
    FlashInfer v0.2.0.post1's SamplingFromProb / TopK / TopP / TopKTopPSamplingFromProb, which is not
    under the reference tree; this restates its published rejection rule): a token is accepted when
    fewer than top_k probabilities are strictly larger than its own and those strictly larger
    probabilities sum to less than top_p; the draw is by inverse CDF over the accepted tokens in
    index order with the uniform number u.  Returns (token, accepted mask)."""
    p = probs.to(torch.float64)
    n = p.numel()
    order = torch.argsort(p, descending=True, stable=True)
    sp = p[order]
    # for each sorted entry: how many and how much mass is strictly larger (ties share the first rank)
    first_of_value = torch.searchsorted(-sp, -sp, right=False)
    csum = torch.cat([torch.zeros(1, dtype=torch.float64), torch.cumsum(sp, 0)])
    larger_count = first_of_value
    larger_mass = csum[first_of_value]
    ok = torch.ones(n, dtype=torch.bool)
    if 0 < top_k < n:
        ok &= larger_count < top_k
    if top_p < 1.0:
        ok &= larger_mass < top_p
    accepted = torch.zeros(n, dtype=torch.bool)
    accepted[order[ok]] = True
    w = torch.where(accepted, p, torch.zeros_like(p))
    c = torch.cumsum(w, 0)
    target = u * c[-1]
    token = int(torch.searchsorted(c, target, right=True).clamp(max=n - 1))
    return token, accepted


# --------------------------------------------------------------------------- model
@dataclass
class ModelConfig:
    """The fields of include/sglang/models/config.h:15-42 that the forward pass reads."""
    num_layers: int
    hidden_size: int
    num_qo_heads: int
    num_kv_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    max_position: int = 40960
    tie_word_embeddings: bool = True
    qk_norm: bool = True              # Qwen3 / Qwen3-MoE
    fused_residual: bool = True       # Qwen3 wiring (qwen3.cc:21-35) vs Llama wiring (llama.cc:15-29)
    hidden_act: str = "silu"
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    attention_bias: bool = False      # Qwen2


def qwen3_0_6b() -> ModelConfig:
    return ModelConfig(28, 1024, 16, 8, 128, 3072, 151936, 1e-6, 1e6, 40960, True, True, True)


def llama3_8b() -> ModelConfig:
    return ModelConfig(32, 4096, 32, 8, 128, 14336, 128256, 1e-5, 5e5, 8192, False, False, False)


def qwen3_30b_a3b() -> ModelConfig:
    return ModelConfig(48, 2048, 32, 4, 128, 6144, 151936, 1e-6, 1e6, 40960, False, True, True,
                       "silu", 128, 8, 768, True)


def init_weights(cfg: ModelConfig, seed: int = 0, std: float = 0.02, router_std: Optional[float] = None):
    """Seeded random-init weights in the reference's packed layouts (src/models/weight_loader.cc:
    27-33,455,497; src/moe/moe.cc:25-30): one CPU generator, parameters drawn in the order embed,
    then per layer qkv, o, gate_up, down (or router, experts.gate_up, experts.down), then lm_head
    when untied; fp32 N(0, std) rounded once to bf16; all norm weights 1."""
    gen = torch.Generator().manual_seed(seed)

    def rnd(*shape, s=std):
        return (torch.randn(*shape, generator=gen, dtype=f32) * s).to(torch.bfloat16)

    w = {"embed": rnd(cfg.vocab_size, cfg.hidden_size), "layers": []}
    qkv_out = (cfg.num_qo_heads + 2 * cfg.num_kv_heads) * cfg.head_dim
    for _ in range(cfg.num_layers):
        L = {"qkv": rnd(qkv_out, cfg.hidden_size),
             "o": rnd(cfg.hidden_size, cfg.num_qo_heads * cfg.head_dim)}
        if cfg.attention_bias:
            L["qkv_bias"] = rnd(qkv_out)
        if cfg.num_experts > 0:
            rs = router_std if router_std is not None else 1.0 / math.sqrt(cfg.hidden_size)
            L["router"] = rnd(cfg.num_experts, cfg.hidden_size, s=rs)
            L["experts_gate_up"] = rnd(cfg.num_experts, 2 * cfg.moe_intermediate_size, cfg.hidden_size)
            L["experts_down"] = rnd(cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size)
        else:
            L["gate_up"] = rnd(2 * cfg.intermediate_size, cfg.hidden_size)
            L["down"] = rnd(cfg.hidden_size, cfg.intermediate_size)
        ones = lambda n: torch.ones(n, dtype=torch.bfloat16)
        L["input_norm"] = ones(cfg.hidden_size)
        L["post_norm"] = ones(cfg.hidden_size)
        if cfg.qk_norm:
            L["q_norm"] = ones(cfg.head_dim)
            L["k_norm"] = ones(cfg.head_dim)
        w["layers"].append(L)
    w["final_norm"] = torch.ones(cfg.hidden_size, dtype=torch.bfloat16)
    w["lm_head"] = w["embed"] if cfg.tie_word_embeddings else rnd(cfg.vocab_size, cfg.hidden_size)
    return w


@dataclass
class KVState:
    """KV pool [2, L, slots, Hkv, d] (src/kvcache/mha_kvcache.cu:88-104) held in fp32 on the CPU."""
    k: torch.Tensor
    v: torch.Tensor

    @staticmethod
    def create(cfg: ModelConfig, num_slots: int) -> "KVState":
        shape = (cfg.num_layers, num_slots, cfg.num_kv_heads, cfg.head_dim)
        return KVState(torch.zeros(shape, dtype=f32), torch.zeros(shape, dtype=f32))


@dataclass
class StepBatch:
    """What Scheduler::prepare_batch hands the forward pass (src/scheduler/scheduler.cc:275-358;
    include/sglang/core/batch.h:16-37)."""
    input_ids: np.ndarray      # [T] int32
    positions: np.ndarray      # [T] int32
    out_loc: np.ndarray        # [T] int32 KV-pool slot of each token
    table_idx: np.ndarray      # [B] page-table row per request
    seq_lens: np.ndarray       # [B] device_len (keys incl. the tokens of this step)
    qo_indptr: np.ndarray      # [B+1]
    is_prefill: bool = False


class OracleModel:
    """Op-for-op restatement of Qwen3ForCausalLM / LlamaForCausalLM / Qwen3MoeForCausalLM::forward
    (src/models/qwen3.cc:21-35,55-66,84-87; llama.cc:15-29,49-55,74-77; qwen3_moe.cc:14-28;
    src/models/utils.cc:8-19,41-57,82-91,138-142; src/layers/attention_layer.cc:17-51)."""

    def __init__(self, cfg: ModelConfig, weights: dict, store: Store = store_bf16, all_reduce=None,
                 expert_begin: int = 0):
        """all_reduce: under tensor parallelism, a callable that sums a tensor over the ranks
        (tensor_model_parallel_all_reduce, src/distributed/distributed.cc:205-226); cfg then holds
        the per-rank head counts and intermediate size and weights the rank's shard.
        expert_begin: under expert parallelism, the first expert this rank holds."""
        self.all_reduce = all_reduce
        self.expert_begin = expert_begin
        self.cfg = cfg
        # Up-cast the (bf16-rounded) weights to fp32 once; tied tensors stay tied.
        cache: dict[int, torch.Tensor] = {}

        def up(t):
            if id(t) not in cache:
                cache[id(t)] = t.to(f32)
            return cache[id(t)]

        self.w = {k: (up(v) if torch.is_tensor(v) else v) for k, v in weights.items() if k != "layers"}
        self.w["layers"] = [{k: up(v) for k, v in L.items()} for L in weights["layers"]]
        self.store = store
        self.cos, self.sin = rope_tables(cfg.head_dim, cfg.max_position, cfg.rope_theta)
        self.sm_scale = 1.0 / math.sqrt(cfg.head_dim)
        # Set to a list to record, per decoder layer of the fused-residual wiring, the tensors that
        # enter it (x, residual) and leave it (x, residual): the per-layer parity test feeds the
        # former to the CUDA operators and compares with the latter.
        self.layer_trace: Optional[list] = None

    def _attn(self, L, li: int, x, batch: StepBatch, kv: KVState, page_table: np.ndarray):
        cfg, st = self.cfg, self.store
        T = x.shape[0]
        qkv = linear(x, L["qkv"], L.get("qkv_bias"), st)
        qd, kd = cfg.num_qo_heads * cfg.head_dim, cfg.num_kv_heads * cfg.head_dim
        q = qkv[:, :qd].reshape(T, cfg.num_qo_heads, cfg.head_dim)
        k = qkv[:, qd:qd + kd].reshape(T, cfg.num_kv_heads, cfg.head_dim)
        v = qkv[:, qd + kd:].reshape(T, cfg.num_kv_heads, cfg.head_dim)
        if cfg.qk_norm:
            q = rmsnorm(q, L["q_norm"], cfg.rms_norm_eps, st)
            k = rmsnorm(k, L["k_norm"], cfg.rms_norm_eps, st)
        pos = torch.from_numpy(batch.positions.astype(np.int64))
        q = rope_neox(q, pos, self.cos, self.sin, store=st)
        k = rope_neox(k, pos, self.cos, self.sin, store=st)
        loc = torch.from_numpy(batch.out_loc.astype(np.int64))
        kv.k[li][loc] = k.to(kv.k.dtype)
        kv.v[li][loc] = v.to(kv.v.dtype)
        o = paged_attention(q, kv.k[li], kv.v[li], page_table, batch.table_idx, batch.seq_lens,
                            batch.qo_indptr, self.sm_scale, st)
        return self._reduce(linear(o.reshape(T, qd), L["o"], None, st))

    def _reduce(self, y):
        """LinearRowParallel / LinearOProj::forward (src/layers/linear.cc:52-55,73-76)."""
        return y if self.all_reduce is None else self.store(self.all_reduce(y))

    def _mlp(self, L, x):
        cfg, st = self.cfg, self.store
        if cfg.num_experts > 0:
            logits = linear(x, L["router"], None, st)
            return self._reduce(moe_forward(x, logits, L["experts_gate_up"], L["experts_down"],
                                            cfg.num_experts_per_tok, cfg.norm_topk_prob, cfg.hidden_act, st,
                                            self.expert_begin))
        gu = linear(x, L["gate_up"], None, st)
        y = silu_and_mul(gu, st) if cfg.hidden_act == "silu" else gelu_and_mul(gu, st)
        return self._reduce(linear(y, L["down"], None, st))

    def fused_layer(self, li: int, x, residual, batch: StepBatch, kv: KVState, page_table: np.ndarray):
        """One decoder layer of the running-residual wiring (Qwen3DecoderLayer::forward,
        src/models/qwen3.cc:21-35): returns (x, residual) as they leave the layer."""
        cfg, st, L = self.cfg, self.store, self.w["layers"][li]
        if residual is None:
            residual = x
            x = rmsnorm(x, L["input_norm"], cfg.rms_norm_eps, st)
        else:
            x, residual = fused_add_rmsnorm(x, residual, L["input_norm"], cfg.rms_norm_eps, st)
        a = self._attn(L, li, x, batch, kv, page_table)
        a, residual = fused_add_rmsnorm(a, residual, L["post_norm"], cfg.rms_norm_eps, st)
        return self._mlp(L, a), residual

    def hidden_states(self, batch: StepBatch, kv: KVState, page_table: np.ndarray) -> torch.Tensor:
        cfg, st = self.cfg, self.store
        x = self.w["embed"][torch.from_numpy(batch.input_ids.astype(np.int64))].to(f32)
        residual = None
        for li, L in enumerate(self.w["layers"]):
            if cfg.fused_residual:
                entering = (x, residual)
                x, residual = self.fused_layer(li, x, residual, batch, kv, page_table)
                if self.layer_trace is not None:
                    self.layer_trace.append({"x_in": entering[0], "res_in": entering[1], "x_out": x, "res_out": residual})
            else:
                res = x
                a = self._attn(L, li, rmsnorm(x, L["input_norm"], cfg.rms_norm_eps, st), batch, kv, page_table)
                x = st(res + a)
                res = x
                m = self._mlp(L, rmsnorm(x, L["post_norm"], cfg.rms_norm_eps, st))
                x = st(res + m)
        if cfg.fused_residual and residual is not None:
            x, _ = fused_add_rmsnorm(x, residual, self.w["final_norm"], cfg.rms_norm_eps, st)
        else:
            x = rmsnorm(x, self.w["final_norm"], cfg.rms_norm_eps, st)
        return x

    def forward(self, batch: StepBatch, kv: KVState, page_table: np.ndarray) -> torch.Tensor:
        """Returns logits [B, vocab] (last row of each request for prefill:
        src/models/utils.cc:8-19; all rows for decode)."""
        h = self.hidden_states(batch, kv, page_table)
        if batch.is_prefill:
            last = torch.from_numpy((batch.qo_indptr[1:] - 1).astype(np.int64))
            h = h.index_select(0, last)
        return linear(h, self.w["lm_head"], None, self.store)
