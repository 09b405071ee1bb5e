"""Checkpoint loading on the CPU: safetensors shards with Hugging Face names come back as the packed
layouts the engine holds (qkv / gate_up merged, experts stacked), bit for bit."""
import json
import struct

import pytest
import torch

from oracle import token_loop_oracle as O


def _cfg(kind):
    if kind == "qwen3":
        return O.ModelConfig(2, 256, 4, 2, 128, 512, 1024, 1e-6, 1e6, 512, True, True, True)
    if kind == "qwen2":
        return O.ModelConfig(2, 256, 8, 8, 128, 512, 1024, 1e-6, 1e6, 512, True, False, False, attention_bias=True)
    if kind == "llama":
        return O.ModelConfig(2, 256, 4, 1, 128, 448, 1536, 1e-5, 5e5, 512, False, False, False)
    return O.ModelConfig(2, 256, 4, 2, 128, 512, 1024, 1e-6, 1e6, 512, False, True, True, "silu", 8, 2, 128, True)


def _same(a, b):
    assert a.keys() == b.keys()
    for k in a:
        if k == "layers":
            assert len(a[k]) == len(b[k])
            for la, lb in zip(a[k], b[k]):
                assert la.keys() == lb.keys()
                for n in la:
                    assert torch.equal(la[n], lb[n]), n
        else:
            assert torch.equal(a[k], b[k]), k


@pytest.mark.parametrize("kind", ["qwen3", "qwen2", "llama", "qwen3moe"])
def test_sharded_checkpoint_round_trip(pkg, tmp_path, kind):
    from sglang_cpp_b200 import weights as W

    cfg = _cfg(kind)
    w = O.init_weights(cfg, seed=4)
    w["final_norm"] = (torch.randn(cfg.hidden_size) * 0.1 + 1).to(torch.bfloat16)
    flat = W.unpack_checkpoint(cfg, w)
    names = sorted(flat)
    # two shards, the second one with the multimodal prefix the reference strips
    W.write_safetensors(tmp_path / "model-00001-of-00002.safetensors", {n: flat[n] for n in names[::2]})
    W.write_safetensors(tmp_path / "model-00002-of-00002.safetensors",
                        {"language_model." + n: flat[n] for n in names[1::2]})
    got = W.load_checkpoint(cfg, tmp_path)
    _same(got, w)
    if cfg.tie_word_embeddings:
        assert got["lm_head"] is got["embed"]


def test_f32_and_f16_tensors_are_cast_to_bf16(pkg, tmp_path):
    from sglang_cpp_b200 import weights as W

    cfg = _cfg("llama")
    w = O.init_weights(cfg, seed=5)
    flat = W.unpack_checkpoint(cfg, w)
    mixed = {n: (t.float() if i % 3 == 0 else t.half() if i % 3 == 1 else t) for i, (n, t) in enumerate(sorted(flat.items()))}
    W.write_safetensors(tmp_path / "model.safetensors", mixed)
    got = W.load_checkpoint(cfg, tmp_path)
    back = W.unpack_checkpoint(cfg, got)
    for i, (n, t) in enumerate(sorted(flat.items())):
        assert back[n].dtype == torch.bfloat16
        if i % 3 != 1:
            assert torch.equal(back[n], t), n        # bf16 -> f32 -> bf16 is exact
        else:                                        # f16 has fewer exponent bits: tiny values lose precision
            assert torch.allclose(back[n].float(), t.float(), atol=1e-6, rtol=2 ** -8), n


def test_missing_and_unsupported_tensors_are_reported(pkg, tmp_path):
    from sglang_cpp_b200 import weights as W

    cfg = _cfg("qwen3")
    flat = W.unpack_checkpoint(cfg, O.init_weights(cfg, seed=6))
    del flat["model.layers.1.self_attn.k_norm.weight"]
    W.write_safetensors(tmp_path / "a.safetensors", flat)
    with pytest.raises(KeyError):
        W.load_checkpoint(cfg, tmp_path)
    # a dtype outside BF16 / F16 / F32 (the reference's FP8 checkpoints) is refused, not misread
    hdr = json.dumps({"x": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    (tmp_path / "b.safetensors").write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0\0\0\0")
    with pytest.raises(ValueError):
        W.read_safetensors(tmp_path / "b.safetensors")
    with pytest.raises(FileNotFoundError):
        W.load_checkpoint(cfg, tmp_path / "nothing_here")
