"""Tensor-parallel host logic on two gloo ranks (no GPU): the shard rules give, after the
all-reduces the reference performs, the unsharded model's logits."""
import socket

import pytest
import torch
import torch.multiprocessing as mp

from tests import tp_workers


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("kind", ["llama", "moe_ep", "moe_tp"])
def test_sharded_oracle_equals_unsharded_on_two_gloo_ranks(tmp_path, kind):
    """llama: heads and MLP columns split.  moe_ep: whole experts per rank (the router replicated)
    and one kv head replicated on both ranks, its query heads split between them.  moe_tp: the
    reference's own layout, every rank a slice of every expert's intermediate dimension
    (src/moe/moe.cc:22-30; tests/moe/test_moe.cpp:127-138)."""
    out = tmp_path / "tp_cpu.pt"
    mp.spawn(tp_workers.cpu_oracle_worker, args=(2, _free_port(), str(out), kind), nprocs=2, join=True)
    r = torch.load(out)
    assert torch.allclose(r["got"], r["want"], atol=2e-5, rtol=1e-5)


def test_kv_head_replication_and_expert_partition_shapes(pkg):
    from oracle import token_loop_oracle as O
    from sglang_cpp_b200 import tp

    cfg = O.ModelConfig(1, 256, 8, 2, 128, 512, 64, 1e-6, 1e6, 256, False, True, True, "silu", 8, 2, 128, True)
    w = O.init_weights(cfg, seed=1)
    L0 = w["layers"][0]
    assert [tp.kv_heads_of_rank(2, r, 4) for r in range(4)] == [(0, 1), (0, 1), (1, 1), (1, 1)]
    assert [tp.kv_heads_of_rank(8, r, 4) for r in range(4)] == [(0, 2), (2, 2), (4, 2), (6, 2)]
    for rank in range(4):
        S = tp.shard_layer(cfg, L0, rank, 4, expert_parallel=True)
        assert S["qkv"].shape == ((2 + 1 + 1) * 128, 256)
        # the rank's k rows are those of kv head rank // 2
        kv = rank // 2
        assert torch.equal(S["qkv"][2 * 128:3 * 128], L0["qkv"][8 * 128 + kv * 128:8 * 128 + (kv + 1) * 128])
        assert S["experts_gate_up"].shape == (2, 2 * 128, 256) and S["experts_down"].shape == (2, 256, 128)
        assert torch.equal(S["experts_down"], L0["experts_down"][2 * rank:2 * rank + 2])
    assert tp.local_config(cfg, 4, True).num_kv_heads == 1
    assert tp.local_config(cfg, 4, True).moe_intermediate_size == 128
    assert tp.local_config(cfg, 4, False).moe_intermediate_size == 32
    with pytest.raises(ValueError):
        tp.kv_heads_of_rank(2, 0, 3)


def test_shard_shapes_follow_the_reference_rules(pkg):
    """tests/layers/test_linear.cpp:101-123 (TP shard shapes) on the packed layouts."""
    from oracle import token_loop_oracle as O
    from sglang_cpp_b200 import tp

    cfg = O.ModelConfig(1, 256, 8, 4, 128, 512, 64, tie_word_embeddings=False)
    w = O.init_weights(cfg, seed=1)
    for size in (1, 2, 4):
        for rank in range(size):
            L = tp.shard_layer(cfg, w["layers"][0], rank, size)
            assert L["qkv"].shape == ((8 + 2 * 4) * 128 // size, 256)
            assert L["o"].shape == (256, 8 * 128 // size)
            assert L["gate_up"].shape == (2 * 512 // size, 256)
            assert L["down"].shape == (256, 512 // size)
    # the shards tile the full matrices
    full = w["layers"][0]["down"]
    assert torch.equal(torch.cat([tp.shard_layer(cfg, w["layers"][0], r, 4)["down"] for r in range(4)], 1), full)
    import pytest
    with pytest.raises(ValueError):
        tp.shard_layer(cfg, w["layers"][0], 0, 3)   # 8 q heads are not divisible by 3
