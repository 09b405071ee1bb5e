"""The CPU oracle against the known answers the reference's own tests hold, and against itself."""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import token_loop_oracle as O

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_greedy_known_answer():
    """tests/engine/test_sampler.cpp:21-33 (GreedySamplingUsesArgmax)."""
    logits = torch.tensor([[1.0, 3.0, 2.0, 0.5], [0.0, 2.0, 5.0, 1.0]])
    assert O.greedy(logits).tolist() == [1, 2]


def test_top_p_known_answer():
    """tests/engine/test_sampler.cpp:35-48 (TopPSamplingKeepsOnlyAllowedPrefix): temperature 0.8,
    top_p 0.6 on [10, 1, .5, -1] leaves only token 0."""
    t, k, p = O.prepare_sampling(0.8, -1, 0.6, 4, False)
    probs = O.sample_row_distribution(torch.tensor([10.0, 1.0, 0.5, -1.0]), t, k, p)
    assert probs.nonzero().flatten().tolist() == [0]
    assert float(probs[0]) == pytest.approx(1.0)


def test_prepare_sampling_clamps():
    """tests/engine/test_sampler.cpp:50-75 (PrepareMaterializesPerRequestSamplingArgs)."""
    assert O.prepare_sampling(0.7, 4, 0.9, 16, False) == (pytest.approx(0.7), 4, pytest.approx(0.9))
    assert O.prepare_sampling(1.0, -1, 1.0, 16, False) == (1.0, 16, 1.0)
    assert O.prepare_sampling(0.0, -1, 1.0, 16, True)[0] == pytest.approx(1e-6)


def test_top_k_one_is_argmax():
    """tests/engine/test_sampler.cpp:92-109 (FlashInferTopKOneSamplesArgmax)."""
    gen = torch.Generator().manual_seed(0)
    logits = torch.randn(4, 64, generator=gen)
    for row in logits:
        probs = O.sample_row_distribution(row, 1.0, 1, 1.0)
        assert probs.nonzero().flatten().tolist() == [int(row.argmax())]


def test_token_pool_semantics():
    """src/kernels/token_pool.cu:10-49: out-of-range reads give 0, out-of-range writes are dropped."""
    table = np.arange(12, dtype=np.int32).reshape(3, 4)
    got = O.gather_int32_2d(table, np.array([0, 2, 3, -1, 1]), np.array([1, 3, 0, 0, 4]))
    assert got.tolist() == [1, 11, 0, 0, 0]
    O.write_token_pool(table, np.array([1, 5, 0]), np.array([2, 0, -1]), np.array([99, 98, 97]))
    assert table[1, 2] == 99 and 98 not in table and 97 not in table


def test_rope_is_a_rotation_and_position_zero_is_identity():
    cos, sin = O.rope_tables(128, 64, 1e6)
    gen = torch.Generator().manual_seed(1)
    x = torch.randn(5, 3, 128, generator=gen)
    pos = torch.tensor([0, 1, 7, 33, 63])
    y = O.rope_neox(x, pos, cos, sin, store=O.store_fp32)
    assert torch.allclose(y[0], x[0])
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), rtol=1e-5)


def test_attention_decode_equals_last_prefill_row():
    gen = torch.Generator().manual_seed(2)
    n, hq, hkv, d = 37, 4, 2, 128
    k = torch.randn(64, hkv, d, generator=gen)
    v = torch.randn(64, hkv, d, generator=gen)
    q = torch.randn(n, hq, d, generator=gen)
    pt = np.arange(64, dtype=np.int32)[None, :]
    full = O.paged_attention(q, k, v, pt, [0], [n], [0, n], 0.1, O.store_fp32)
    last = O.paged_attention(q[-1:], k, v, pt, [0], [n], [0, 1], 0.1, O.store_fp32)
    assert torch.allclose(full[-1], last[0], atol=1e-6)
    first = O.paged_attention(q[:1], k, v, pt, [0], [1], [0, 1], 0.1, O.store_fp32)
    assert torch.allclose(full[0], first[0], atol=1e-6)


def test_moe_matches_reference_fixture():
    """Golden vectors produced by the reference's own MoELayer::forward (src/moe/moe.cc) compiled
    from source and run on the CPU in fp32; see tests/golden/make_moe_golden.py."""
    path = GOLDEN / "moe_ref_fp32.json"
    if not path.exists():
        pytest.skip("golden fixture not generated")
    fx = json.loads(path.read_text())
    for case in fx["cases"]:
        t = lambda key: torch.tensor(case[key], dtype=torch.float32)
        got = O.moe_forward(t("hidden"), t("router_logits"), t("gate_up"), t("down"), case["top_k"],
                            case["renormalize"], case["activation"], O.store_fp32)
        assert torch.allclose(got, t("out"), rtol=1e-5, atol=1e-5), case["name"]


def test_model_prefill_then_decode_consistency():
    """A decode step after a prefill gives the logits a one-longer prefill gives for its last row."""
    cfg = O.ModelConfig(2, 64, 4, 2, 16, 96, 50, max_position=64)
    w = O.init_weights(cfg, seed=0, std=0.2)
    m = O.OracleModel(cfg, w, O.store_fp32)
    ids = np.array([3, 7, 11, 2, 40], dtype=np.int32)
    pt = np.arange(32, dtype=np.int32)[None, :]
    kv = O.KVState.create(cfg, 32)
    full = O.StepBatch(ids, np.arange(5, dtype=np.int32), pt[0, :5].copy(), np.array([0]), np.array([5]),
                       np.array([0, 5]), True)
    want = m.forward(full, kv, pt)
    kv2 = O.KVState.create(cfg, 32)
    pre = O.StepBatch(ids[:4], np.arange(4, dtype=np.int32), pt[0, :4].copy(), np.array([0]), np.array([4]),
                      np.array([0, 4]), True)
    m.forward(pre, kv2, pt)
    dec = O.StepBatch(ids[4:], np.array([4], dtype=np.int32), pt[0, 4:5].copy(), np.array([0]), np.array([5]),
                      np.array([0, 1]), False)
    got = m.forward(dec, kv2, pt)
    assert torch.allclose(got, want, atol=1e-5)
