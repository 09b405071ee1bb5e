"""Host-side mirror of sglang.cpp's ``Engine`` for the per-step path, over the C ABI.

``Engine`` here keeps the reference's method names where one exists
(``forward_batch``, ``page_table``; include/sglang/engine/engine.h:57-103) and
otherwise exposes what the scheduler does either side of the forward pass
(page-table / token-pool writes).  All device state lives in the C++ step runner
(``csrc/engine.cu``); this file only marshals host arrays into the C structs.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from . import _lib
from ._lib import B200Error, EngineConfigStruct, ModelConfigStruct, StepStruct, call

PHASE_PREFILL = 0
PHASE_DECODE = 1


@dataclass
class EngineConfig:
    """The sizing fields of include/sglang/engine/config.h:13-32."""
    page_size: int = 1
    num_pages: int = 1024
    max_running_req: int = 64
    max_seq_len: int = 4096
    max_extend_tokens: int = 8192
    tp_rank: int = 0
    tp_size: int = 1
    expert_parallel: bool = False   # MoE under TP: whole experts per rank instead of slices of each


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.int32))


class ForwardOutput:
    """include/sglang/engine/engine.h:28-34: tokens on the host after ``synchronize()``."""

    def __init__(self, engine: "Engine", next_tokens_cpu: torch.Tensor, num_reqs: int):
        self._engine = engine
        self.next_tokens_cpu = next_tokens_cpu[:num_reqs]

    def synchronize(self) -> None:
        self._engine.synchronize()


class StepTicket:
    """A step in flight in the engine's result ring (b200_engine_step_async / b200_engine_wait)."""

    def __init__(self, engine: "Engine", ticket: int, num_reqs: int):
        self._engine, self.ticket, self.num_reqs = engine, ticket, num_reqs

    def wait(self):
        return self._engine.wait(self.ticket, self.num_reqs)


class Engine:
    def __init__(self, model_config, config: EngineConfig):
        """model_config: any object with the forward-pass fields of the reference's ModelConfig
        (include/sglang/models/config.h:15-42), named as b200_model_config names them."""
        self.model_config = model_config
        self.config = config
        m = ModelConfigStruct(
            model_config.num_layers, model_config.hidden_size, model_config.num_qo_heads,
            model_config.num_kv_heads, model_config.head_dim, model_config.intermediate_size,
            model_config.vocab_size, model_config.rms_norm_eps, model_config.rope_theta,
            model_config.max_position, int(model_config.tie_word_embeddings), int(model_config.qk_norm),
            int(model_config.fused_residual), int(model_config.attention_bias),
            1 if model_config.hidden_act == "gelu" else 0, model_config.num_experts,
            model_config.num_experts_per_tok, model_config.moe_intermediate_size,
            int(model_config.norm_topk_prob))
        c = EngineConfigStruct(config.page_size, config.num_pages, config.max_running_req,
                               config.max_seq_len, config.max_extend_tokens, config.tp_rank,
                               config.tp_size, int(config.expert_parallel))
        self._h = ctypes.c_void_p()
        call("b200_engine_create", ctypes.byref(m), ctypes.byref(c), ctypes.byref(self._h))
        # A small ring of pinned token buffers, one per step in flight: a step enqueued before the
        # previous step's tokens were read must not overwrite them (the reference allocates a
        # pinned tensor per ForwardOutput, src/engine/engine.cc:526-531).
        self._token_ring = [torch.empty(config.max_running_req + 1, dtype=torch.int32).pin_memory()
                            for _ in range(4)]
        self.page_size = config.page_size
        self.dummy_table_idx = config.max_running_req
        self.pt_cols = (config.max_seq_len + 31) // 32 * 32   # page-table row length (src/engine/engine.cc:452-459)
        self._step_index = 0

    def close(self) -> None:
        if self._h:
            call("b200_engine_destroy", self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------------ tensors
    def tensor_info(self, name: str, layer: int = 0) -> tuple[int, int]:
        ptr, n = ctypes.c_void_p(), ctypes.c_int64()
        call("b200_engine_tensor", self._h, name.encode(), layer, ctypes.byref(ptr), ctypes.byref(n))
        return int(ptr.value), int(n.value)

    def load(self, name: str, layer: int, host: torch.Tensor) -> None:
        host = host.contiguous()
        call("b200_engine_load", self._h, name.encode(), layer, host.data_ptr(),
             host.numel() * host.element_size())

    def load_weights(self, w: dict, tp_rank: int = 0, tp_size: int = 1) -> None:
        """Upload weights given in the reference's packed layouts (full, unsharded tensors: a dict
        with "embed", "final_norm", optional "lm_head" and a list "layers" of per-layer dicts),
        cut with the reference's TP shard rules for this rank (sglang_cpp_b200.tp.shard_layer)."""
        from .tp import shard_layer

        cfg = self.model_config
        self.load("embed", 0, w["embed"])
        if not cfg.tie_word_embeddings:
            self.load("lm_head", 0, w["lm_head"])
        self.load("final_norm", 0, w["final_norm"])
        for l, L in enumerate(w["layers"]):
            for name, t in shard_layer(cfg, L, tp_rank, tp_size, self.config.expert_parallel).items():
                self.load(name, l, t)

    def connect_tp(self, group=None, symmetric: Optional[bool] = None) -> None:
        """Connect the all-reduce buffers of the ranks (what the reference's NCCL unique-id
        rendezvous does, src/distributed/distributed.cc:142-173).

        Two forms.  CUDA IPC handles of the engine's own buffers travel over torch.distributed and
        the kernels sum peer loads in rank order.  Or (``symmetric``) the buffers are a
        torch.distributed symmetric-memory allocation whose peer addresses and NVLink multicast
        address come from torch's rendezvous: the all-reduce is then summed inside the switch
        (Llama-3-8B decode at batch 128 on 8 GPUs: 21.7 us per call against 28.2, 3.32 ms per step
        against 4.00; no gain with two ranks).  Needs an NCCL process group.  Default: symmetric
        for four ranks or more over an NCCL group, IPC otherwise; B200_TP_SYMMETRIC=0/1 in the
        environment overrides."""
        import os

        if symmetric is None:
            env = os.environ.get("B200_TP_SYMMETRIC", "")
            if env in ("0", "1"):
                symmetric = env == "1"
            else:
                import torch.distributed as dist

                symmetric = (self.config.tp_size >= 4 and dist.is_available() and dist.is_initialized()
                             and "nccl" in str(dist.get_backend(group)))
        if symmetric:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm_mem

            nbytes = int(_lib.load().b200_engine_comm_region_bytes(self._h))
            dev = torch.device("cuda", torch.cuda.current_device())
            region = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
            region.zero_()
            torch.cuda.synchronize()
            name = (group or dist.group.WORLD).group_name
            handle = symm_mem.rendezvous(region, name)
            peers = (ctypes.c_void_p * self.config.tp_size)(*[int(p) for p in handle.buffer_ptrs])
            mc = int(handle.multicast_ptr) if handle.multicast_ptr else None
            call("b200_engine_comm_attach", self._h, region.data_ptr(), peers, mc)
            self._symmetric_region = (region, handle)   # the memory must outlive the engine
            dist.barrier(group=group)
            return
        from .tp import exchange_handles

        n = _lib.load().b200_comm_handle_bytes()
        buf = ctypes.create_string_buffer(n)
        call("b200_engine_comm_export", self._h, buf)
        allh = exchange_handles(buf.raw, self.config.tp_rank, self.config.tp_size, group)
        call("b200_engine_comm_connect", self._h, allh)

    def fill_random(self, seed: int = 0, std: float = 0.02) -> None:
        """Random-init weights generated on the device (benchmarks of models too large to draw on
        the host): N(0, std) for matrices, 1 for norm weights.  Replicated tensors (embedding,
        lm_head, norms, router) get the same values on every rank; sharded ones differ by rank."""
        cfg, rank = self.model_config, self.config.tp_rank
        dev = torch.device("cuda", torch.cuda.current_device())

        def fill(name, layer, gen_seed, ones=False):
            try:
                ptr, n = self.tensor_info(name, layer)
            except B200Error:
                return
            view = _as_cuda_tensor(ptr, n).view(torch.bfloat16)
            if ones:
                view.fill_(1.0)
                return
            g = torch.Generator(device=dev).manual_seed(gen_seed)
            chunk = 1 << 26
            for off in range(0, view.numel(), chunk):
                m = min(chunk, view.numel() - off)
                view[off:off + m] = (torch.randn(m, generator=g, device=dev, dtype=torch.float32) * std).to(torch.bfloat16)

        fill("embed", 0, seed * 1000 + 1)
        if not cfg.tie_word_embeddings:
            fill("lm_head", 0, seed * 1000 + 2)
        fill("final_norm", 0, 0, ones=True)
        for l in range(cfg.num_layers):
            for i, name in enumerate(("qkv", "qkv_bias", "o", "gate_up", "down", "experts_gate_up", "experts_down")):
                fill(name, l, seed * 1000 + 100 + l * 16 + i + 7919 * (rank + 1))
            fill("router", l, seed * 1000 + 100 + l * 16 + 15)
            for name in ("input_norm", "post_norm", "q_norm", "k_norm"):
                fill(name, l, 0, ones=True)
        torch.cuda.synchronize()

    def load_rope_tables(self, cos: torch.Tensor, sin: torch.Tensor) -> None:
        """Overwrite the RoPE tables with ones built elsewhere (e.g. bit-identical to torch's)."""
        self.load("rope_cos", 0, cos.float())
        self.load("rope_sin", 0, sin.float())

    # ------------------------------------------------------------------ tables
    def write_page_table(self, rows, positions, slots) -> None:
        r, p, v = _i32(rows), _i32(positions), _i32(slots)
        call("b200_engine_write_table", self._h, 0, r.ctypes.data, p.ctypes.data, v.ctypes.data, len(r))

    def write_token_pool(self, rows, positions, tokens) -> None:
        r, p, v = _i32(rows), _i32(positions), _i32(tokens)
        call("b200_engine_write_table", self._h, 1, r.ctypes.data, p.ctypes.data, v.ctypes.data, len(r))

    def read_table(self, which: str) -> np.ndarray:
        ptr, n = self.tensor_info(which)
        rows = self.config.max_running_req + 1
        self.synchronize()
        return _as_cuda_tensor(ptr, n).view(torch.int32).cpu().numpy().reshape(rows, -1)

    def device_view(self, name: str, layer: int = 0) -> torch.Tensor:
        """A uint8 torch view of a named device tensor (debugging and tests)."""
        ptr, n = self.tensor_info(name, layer)
        return _as_cuda_tensor(ptr, n)

    # ------------------------------------------------------------------ steps
    def capture_graphs(self, batch_sizes: Sequence[int]) -> None:
        bs = _i32(batch_sizes)
        call("b200_engine_capture_graphs", self._h, bs.ctypes.data, len(bs))

    def forward_batch(self, phase: int, table_idx, cached_lens, extend_lens, write_pos=None,
                      num_reqs: Optional[int] = None, temperatures=None, top_k=None, top_p=None,
                      seeds=None) -> ForwardOutput:
        """Engine::forward_batch (src/engine/engine.cc:495-544).  Arrays are per request over the
        padded batch; the first ``num_reqs`` are real.  ``temperatures`` (per real request) switches
        the step from greedy argmax to sampling, as BatchSamplingArgs does in the reference."""
        t, c, e = _i32(table_idx), _i32(cached_lens), _i32(extend_lens)
        bp = len(t)
        b = bp if num_reqs is None else num_reqs
        wp = _i32(write_pos) if write_pos is not None else None
        keep = []

        def opt(a, dtype):
            if a is None:
                return None
            arr = np.ascontiguousarray(np.asarray(a, dtype=dtype))
            keep.append(arr)
            return arr.ctypes.data

        st = StepStruct(phase, b, bp, t.ctypes.data, c.ctypes.data, e.ctypes.data,
                        wp.ctypes.data if wp is not None else None, opt(temperatures, np.float32),
                        opt(top_k, np.int32), opt(top_p, np.float32), opt(seeds, np.uint64),
                        self._step_index)
        self._step_index += 1
        buf = self.next_token_buffer()
        call("b200_engine_step", self._h, ctypes.byref(st), buf.data_ptr())
        return ForwardOutput(self, buf, b)

    def set_eos_token(self, eos_token_id: int) -> None:
        """Engine::eos_token_id (include/sglang/engine/engine.h:71) for the device-side finish flags."""
        call("b200_engine_set_eos_token", self._h, int(eos_token_id))

    def forward_batch_async(self, phase: int, table_idx, cached_lens, extend_lens, write_pos=None,
                            num_reqs: Optional[int] = None, temperatures=None, top_k=None, top_p=None,
                            seeds=None, ignore_eos=None) -> "StepTicket":
        """forward_batch reporting through the engine's pinned result ring: ``StepTicket.wait()``
        blocks on this step's own event and returns (tokens, finished flags) as numpy views of the
        ring slot (valid until ``b200_engine_result_slots()`` further steps have been enqueued)."""
        t, c, e = _i32(table_idx), _i32(cached_lens), _i32(extend_lens)
        bp = len(t)
        b = bp if num_reqs is None else num_reqs
        wp = _i32(write_pos) if write_pos is not None else None
        keep = []

        def opt(a, dtype):
            if a is None:
                return None
            arr = np.ascontiguousarray(np.asarray(a, dtype=dtype))
            keep.append(arr)
            return arr.ctypes.data

        st = StepStruct(phase, b, bp, t.ctypes.data, c.ctypes.data, e.ctypes.data,
                        wp.ctypes.data if wp is not None else None, opt(temperatures, np.float32),
                        opt(top_k, np.int32), opt(top_p, np.float32), opt(seeds, np.uint64),
                        self._step_index)
        self._step_index += 1
        ticket = ctypes.c_int64()
        call("b200_engine_step_async", self._h, ctypes.byref(st), opt(ignore_eos, np.uint8), ctypes.byref(ticket))
        return StepTicket(self, int(ticket.value), b)

    def wait(self, ticket: int, num_reqs: int):
        tok, fin = ctypes.c_void_p(), ctypes.c_void_p()
        call("b200_engine_wait", self._h, ticket, ctypes.byref(tok), ctypes.byref(fin))
        if num_reqs == 0:
            return np.zeros(0, np.int32), np.zeros(0, np.uint8)
        tokens = np.ctypeslib.as_array(ctypes.cast(tok, ctypes.POINTER(ctypes.c_int32)), shape=(num_reqs,))
        finished = np.ctypeslib.as_array(ctypes.cast(fin, ctypes.POINTER(ctypes.c_uint8)), shape=(num_reqs,))
        return tokens, finished

    def next_token_buffer(self) -> torch.Tensor:
        """The pinned buffer the next step's tokens go to (call once per step)."""
        self._ring_pos = (getattr(self, "_ring_pos", -1) + 1) % len(self._token_ring)
        return self._token_ring[self._ring_pos]

    def synchronize(self) -> None:
        call("b200_engine_synchronize", self._h)

    def logits(self, rows: int) -> torch.Tensor:
        out = torch.empty(rows, self.model_config.vocab_size, dtype=torch.bfloat16)
        call("b200_engine_read_logits", self._h, out.data_ptr(), rows)
        return out

    def set_profiling(self, on: bool) -> None:
        call("b200_engine_set_profiling", self._h, 1 if on else 0)

    def read_profile(self) -> tuple[float, int, int]:
        """(attention ms of the last profiled step, attention launches, kernels launched by the last step)."""
        ms, n, k = ctypes.c_float(), ctypes.c_int32(), ctypes.c_int32()
        call("b200_engine_read_profile", self._h, ctypes.byref(ms), ctypes.byref(n), ctypes.byref(k))
        return float(ms.value), int(n.value), int(k.value)

    def read_profile_allreduce(self) -> tuple[float, int]:
        ms, n = ctypes.c_float(), ctypes.c_int32()
        call("b200_engine_read_profile_allreduce", self._h, ctypes.byref(ms), ctypes.byref(n))
        return float(ms.value), int(n.value)

    def last_step_ms(self) -> float:
        ms = ctypes.c_float()
        call("b200_engine_last_step_ms", self._h, ctypes.byref(ms))
        return float(ms.value)


def _as_cuda_tensor(ptr: int, nbytes: int) -> torch.Tensor:
    """A uint8 torch view of device memory owned by the C++ engine."""
    class _Holder:
        pass
    h = _Holder()
    h.__cuda_array_interface__ = {
        "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None,
    }
    return torch.as_tensor(h, device="cuda")
