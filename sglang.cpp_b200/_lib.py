"""ctypes binding of ``libb200_token_loop.so`` (the C ABI in ``include/b200_token_loop.h``).

The binding is deliberately thin: every Python-visible operator in this package
ends in exactly one of the calls declared here, and there is no fallback of any
kind — if the shared library is missing the import fails with instructions to
build it.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_void_p, POINTER
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "lib" / "libb200_token_loop.so"

B200_OK = 0
ERROR_NAMES = {
    1: "B200_ERR_INVALID_ARGUMENT",
    2: "B200_ERR_CUDA",
    3: "B200_ERR_TIMEOUT",
    4: "B200_ERR_UNSUPPORTED",
    5: "B200_ERR_STATE",
}

EPILOGUE_NONE = 0
EPILOGUE_SWIGLU = 1
EPILOGUE_GEGLU = 2


class B200Error(RuntimeError):
    """Raised when a C-ABI call returns a non-zero status (the reference raises c10::Error)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"{ERROR_NAMES.get(code, code)}: {message}")
        self.code = code


_P = c_void_p
_I = c_int
_L = c_int64
_F = c_float

# name -> (restype, argtypes).  Every symbol include/b200_token_loop.h declares is listed.
PROTOTYPES: dict[str, tuple] = {
    "b200_last_error": (c_char_p, []),
    "b200_abi_version": (_I, []),
    "b200_read_device_status": (_I, [POINTER(c_int32), _P]),
    "b200_rmsnorm": (_I, [_P, _P, _P, _I, _I, _F, _P]),
    "b200_fused_add_rmsnorm": (_I, [_P, _P, _P, _I, _I, _F, _P]),
    "b200_qk_rmsnorm_strided": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _L, _F, _P]),
    "b200_rope_neox_inplace": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _L, _L, _L, _L, _P]),
    "b200_store_kv": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _L, _L, _L, _P]),
    "b200_qknorm_rope_store": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _L, _F, _I, _P]),
    "b200_silu_and_mul": (_I, [_P, _P, _I, _I, _P]),
    "b200_gelu_and_mul": (_I, [_P, _P, _I, _I, _P]),
    "b200_embedding": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "b200_gather_int32_2d": (_I, [_P, _P, _L, _L, _L, _P, _P, _L, _P]),
    "b200_write_token_pool": (_I, [_P, _L, _L, _L, _P, _P, _P, _L, _P]),
    "b200_linear": (_I, [_P, _P, _P, _P, _I, _I, _I, _L, _I, _P]),
    "b200_moe_workspace_bytes": (_L, [_I, _I, _I, _I, _I]),
    "b200_moe_route": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "b200_moe_forward": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _L, _P]),
    "b200_moe_forward_local": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _L, _P]),
    "b200_attention_decode_workspace_bytes": (_L, [_I, _I, _I, _I]),
    "b200_attention_decode": (_I, [_P, _P, _L, _L, _P, _P, _L, _P, _L, _P, _P, _I, _I, _I, _I, _I, _F, _P, _L, _P]),
    "b200_attention_decode_noalloc": (_I, [_P, _P, _L, _L, _P, _P, _L, _P, _L, _P, _P, _I, _I, _I, _I, _I, _F, _P]),
    "b200_attention_decode_noalloc_status": (_I, [POINTER(c_int32), _P]),
    "b200_attention_prefill": (_I, [_P, _P, _L, _L, _P, _P, _L, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P]),
    "b200_argmax": (_I, [_P, _P, _I, _I, _L, _P]),
    "b200_sample": (_I, [_P, _P, _I, _I, _L, _P, _P, _P, _P, ctypes.c_uint64, _P, _P]),
    "b200_sample_from_probs": (_I, [_P, _P, _I, _I, _P, _I, _P, _F, _P, _P]),
    "b200_comm_create": (_I, [_I, _I, _L, POINTER(c_void_p)]),
    "b200_comm_handle_bytes": (_I, []),
    "b200_comm_export": (_I, [_P, _P]),
    "b200_comm_connect": (_I, [_P, _P]),
    "b200_comm_buffer": (c_void_p, [_P, _I]),
    "b200_comm_destroy": (_I, [_P]),
    "b200_comm_set_wait_limit_ns": (_I, [_P, ctypes.c_uint64]),
    "b200_comm_connect_loopback": (_I, [_P]),
    "b200_comm_loopback_announce": (_I, [_P, ctypes.c_uint32, _P]),
    "b200_engine_comm": (c_void_p, [_P]),
    "b200_decode_chain_grid": (_I, []),
    "b200_allreduce": (_I, [_P, _I, _P, _I, _I, _P]),
    "b200_allreduce_fused_add_rmsnorm": (_I, [_P, _I, _P, _P, _P, _I, _I, _F, _I, _P]),
    "b200_comm_region_bytes": (c_int64, [c_int64]),
    "b200_comm_create_on": (_I, [_I, _I, c_int64, _P, POINTER(c_void_p)]),
    "b200_comm_connect_pointers": (_I, [_P, _P, _P]),
    "b200_comm_uses_multicast": (_I, [_P]),
    "b200_engine_comm_region_bytes": (c_int64, [_P]),
    "b200_engine_comm_attach": (_I, [_P, _P, _P, _P]),
    "b200_engine_comm_export": (_I, [_P, _P]),
    "b200_engine_comm_connect": (_I, [_P, _P]),
    "b200_engine_create": (_I, [_P, _P, POINTER(c_void_p)]),
    "b200_engine_destroy": (_I, [_P]),
    "b200_engine_tensor": (_I, [_P, c_char_p, _I, POINTER(c_void_p), POINTER(c_int64)]),
    "b200_engine_load": (_I, [_P, c_char_p, _I, _P, _L]),
    "b200_engine_write_table": (_I, [_P, _I, _P, _P, _P, _L]),
    "b200_engine_capture_graphs": (_I, [_P, _P, _I]),
    "b200_engine_step": (_I, [_P, _P, _P]),
    "b200_engine_synchronize": (_I, [_P]),
    "b200_engine_set_eos_token": (_I, [_P, c_int32]),
    "b200_engine_result_slots": (_I, []),
    "b200_engine_step_async": (_I, [_P, _P, _P, POINTER(c_int64)]),
    "b200_engine_wait": (_I, [_P, c_int64, POINTER(c_void_p), POINTER(c_void_p)]),
    "b200_engine_read_logits": (_I, [_P, _P, _I]),
    "b200_engine_stream": (c_void_p, [_P]),
    "b200_engine_last_step_ms": (_I, [_P, POINTER(c_float)]),
    "b200_engine_set_profiling": (_I, [_P, _I]),
    "b200_engine_read_profile_allreduce": (_I, [_P, POINTER(c_float), POINTER(c_int32)]),
    "b200_engine_read_profile": (_I, [_P, POINTER(c_float), POINTER(c_int32), POINTER(c_int32)]),
}


class ModelConfigStruct(ctypes.Structure):
    """b200_model_config."""
    _fields_ = [
        ("num_layers", c_int32), ("hidden_size", c_int32), ("num_qo_heads", c_int32),
        ("num_kv_heads", c_int32), ("head_dim", c_int32), ("intermediate_size", c_int32),
        ("vocab_size", c_int32), ("rms_norm_eps", c_float), ("rope_theta", c_float),
        ("max_position", c_int32), ("tie_word_embeddings", c_int32), ("qk_norm", c_int32),
        ("fused_residual", c_int32), ("attention_bias", c_int32), ("hidden_act", c_int32),
        ("num_experts", c_int32), ("num_experts_per_tok", c_int32),
        ("moe_intermediate_size", c_int32), ("norm_topk_prob", c_int32),
    ]


class EngineConfigStruct(ctypes.Structure):
    """b200_engine_config."""
    _fields_ = [
        ("page_size", c_int32), ("num_pages", c_int32), ("max_running_req", c_int32),
        ("max_seq_len", c_int32), ("max_extend_tokens", c_int32), ("tp_rank", c_int32),
        ("tp_size", c_int32), ("expert_parallel", c_int32),
    ]


class StepStruct(ctypes.Structure):
    """b200_step."""
    _fields_ = [
        ("phase", c_int32), ("num_reqs", c_int32), ("num_padded_reqs", c_int32),
        ("table_idx", c_void_p), ("cached_lens", c_void_p), ("extend_lens", c_void_p),
        ("write_pos", c_void_p), ("temperatures", c_void_p), ("top_k", c_void_p),
        ("top_p", c_void_p), ("seeds", c_void_p), ("step_index", ctypes.c_uint64),
    ]

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library (once) and attach the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    path = LIB_PATH
    if not path.exists():
        raise ImportError(
            f"{path} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
            "(nvcc, sm_100a).  There is no fallback path."
        )
    lib = ctypes.CDLL(str(path))
    for name, (restype, argtypes) in PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(code: int) -> None:
    if code != B200_OK:
        msg = load().b200_last_error()
        raise B200Error(code, msg.decode() if msg else "")


def call(name: str, *args) -> None:
    """Call an int-returning entry point and raise B200Error on a non-zero status."""
    check(getattr(load(), name)(*args))
