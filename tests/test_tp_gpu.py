"""Tensor parallelism on two GPUs: one process per GPU, the fused all-reduce + add + norm over
peer memory.  Needs two devices; skipped otherwise."""
import socket

import pytest
import torch
import torch.multiprocessing as mp

from tests import tp_workers

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("kind,two_shot", [("llama", False), ("moe_ep", False), ("moe_tp", False), ("llama", True),
                                           ("llama", "symmetric"), ("moe_ep", "symmetric")])
def test_tp2_engine_matches_unsharded_oracle(tmp_path, monkeypatch, kind, two_shot):
    """llama: heads and MLP columns split over the two GPUs.  moe_ep: experts partitioned over the
    GPUs (expert parallelism riding on the fused all-reduce) and the single kv head replicated.
    moe_tp: the reference's own MoE layout, a slice of every expert's intermediate dimension per rank.
    Prefill logits and the logits of three decode steps (fed the engine's own tokens) are compared.
    two_shot: the reduce-scatter + gather form of the all-reduce that larger groups use.
    "symmetric": the exchange buffers are a torch symmetric-memory allocation and the sums are formed
    inside the NVLink switch (multimem.ld_reduce / multimem.st) when it offers a multicast address."""
    symmetric = two_shot == "symmetric"
    if two_shot is True:
        monkeypatch.setenv("B200_AR_TWO_SHOT_MIN_WORLD", "2")   # read when the communicator is created
    out = tmp_path / "tp_gpu.pt"
    mp.spawn(tp_workers.gpu_engine_worker, args=(2, _free_port(), str(out), kind, symmetric), nprocs=2, join=True)
    r = torch.load(out)
    if symmetric:
        print("multicast address in use:", r.get("multicast"))
    assert r["ranks_agree"], "the two ranks produced different logits or tokens"
    d = (r["prefill"].float() - r["want_prefill"].float()).abs()
    rms = float(r["want_prefill"].float().pow(2).mean().sqrt())
    assert float(d.max()) <= 2e-2, f"max-abs {float(d.max()):.4g}"
    assert float(d.mean()) <= 1e-3 + rms * 2 ** -8, f"mean-abs {float(d.mean()):.4g}"
    for k in range(3):
        d = (r["decode_logits"][k].float() - r["want_decode"][k].float()).abs()
        assert float(d.max()) <= 2e-2, f"decode step {k}: max-abs {float(d.max()):.4g}"
        assert float(d.mean()) <= 1e-3 + rms * 2 ** -8, f"decode step {k}: mean-abs {float(d.mean()):.4g}"


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("two_shot", [False, True, "symmetric"])
def test_allreduce_calls_of_the_c_abi(tmp_path, monkeypatch, two_shot):
    """b200_allreduce is bit-exact (fp32 sum in rank order, one bf16 rounding; with in-switch sums -
    "symmetric" - within one bf16 step of that); the fused form
    leaves the same residual and the norm of it, over five calls alternating the buffer parity —
    then 2000 more calls back to back with no host synchronisation, every sum checked bit for bit on
    the device (the flag protocol must hold when one rank runs ahead of the other)."""
    symmetric = two_shot == "symmetric"   # in-switch sums: with two ranks a + b is still the rank-order sum
    if two_shot is True:
        monkeypatch.setenv("B200_AR_TWO_SHOT_MIN_WORLD", "2")
    out = tmp_path / "ar.pt"
    mp.spawn(tp_workers.gpu_allreduce_worker, args=(2, _free_port(), str(out), 2000, symmetric), nprocs=2, join=True)
    r = torch.load(out)
    if symmetric:
        print("multicast address in use:", r.get("multicast"))
    assert r["stress_calls"] == 2000 and r["stress_bad_all_ranks"] == [0, 0], r["stress_bad_all_ranks"]
    assert len(r["plain"]) == 3 and len(r["fused_x"]) == 2
    for got, want in zip(r["plain"] + r["fused_res"], r["want_plain"] + r["want_res"]):
        if symmetric:   # the switch rounds the fp32 sum its own way: a bf16 step per sum that went into the value
            assert torch.allclose(got.float(), want.float(), atol=2 ** -4, rtol=2 ** -6)
        else:
            assert torch.equal(got, want)
    for got, want in zip(r["fused_x"], r["want_x"]):
        if symmetric:
            d = (got.float() - want.float()).abs()
            assert float(d.max()) <= 0.1 and float(d.mean()) <= 5e-3, (float(d.max()), float(d.mean()))
        else:
            assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2 ** -7)
