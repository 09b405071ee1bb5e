"""Failure detection without a GPU fault: bounded waits that run out report through the device
status words, the kernel returns, its outputs stay untouched and the context stays usable.

The failure is made on the host: a loop-back communicator (every "peer" mapped onto this rank's own
buffers) in which nobody plays the peers' part, so their announcement never arrives and the
all-reduce kernel runs into its wait limit (set to 20 ms here; 2 s by default).  The reference's
only time-out on this path is the NCCL rendezvous (src/distributed/distributed.cc:106-120,145).
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import token_loop_oracle as O

pytestmark = pytest.mark.gpu
LIMIT_NS = 20_000_000


def _comm(pkg, world, rows, hidden):
    from sglang_cpp_b200._lib import call

    comm = ctypes.c_void_p()
    call("b200_comm_create", 0, world, rows * hidden * 2, ctypes.byref(comm))
    call("b200_comm_set_wait_limit_ns", comm, LIMIT_NS)
    call("b200_comm_connect_loopback", comm)
    return comm


def _buffer(pkg, comm, parity, rows, hidden):
    from sglang_cpp_b200.engine import _as_cuda_tensor

    ptr = pkg.load_library().b200_comm_buffer(comm, parity)
    return _as_cuda_tensor(ptr, rows * hidden * 2).view(torch.bfloat16).view(rows, hidden)


@pytest.mark.parametrize("two_shot", [False, True])
def test_allreduce_wait_runs_out_outputs_untouched_then_recovers(pkg, L, monkeypatch, two_shot):
    from sglang_cpp_b200._lib import call

    if two_shot:
        monkeypatch.setenv("B200_AR_TWO_SHOT_MIN_WORLD", "2")
    rows, hidden, world = 24, 1024, 2
    comm = _comm(pkg, world, rows, hidden)
    stream = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator().manual_seed(3)
    part = torch.randn(rows, hidden, generator=gen).to(torch.bfloat16).cuda()
    weight = torch.ones(hidden, dtype=torch.bfloat16, device="cuda")
    residual0 = torch.randn(rows, hidden, generator=gen).to(torch.bfloat16).cuda()
    residual = residual0.clone()
    out = torch.full((rows, hidden), 7.0, dtype=torch.bfloat16, device="cuda")
    _buffer(pkg, comm, 0, rows, hidden).copy_(part)
    # call 1: nobody announces -> the wait runs out, the kernel returns, nothing was written
    call("b200_allreduce_fused_add_rmsnorm", comm, 0, out.data_ptr(), residual.data_ptr(), weight.data_ptr(),
         rows, hidden, 1e-6, 0, stream)
    torch.cuda.synchronize()
    site, bad = L.read_device_status()
    assert site in ((402, 403) if two_shot else (401,)) and bad == 0
    assert torch.equal(residual, residual0), "residual must be left as it was"
    assert bool((out == 7.0).all()), "out must be left as it was"
    assert L.read_device_status() == (0, 0), "the read clears the report"
    # call 2: the host plays the peer (announces call 2); with every peer aliased to this rank the sum is
    # world x the partial — and the context is as usable as before
    _buffer(pkg, comm, 1, rows, hidden).copy_(part)
    torch.cuda.synchronize()
    call("b200_comm_loopback_announce", comm, 2, stream)
    if not two_shot:
        call("b200_allreduce", comm, 1, out.data_ptr(), rows, hidden, stream)
        torch.cuda.synchronize()
        assert L.read_device_status() == (0, 0)
        assert torch.equal(out, (part.float() * world).to(torch.bfloat16))
    # an unrelated kernel still runs and is right
    x = torch.randn(8, hidden, generator=gen).to(torch.bfloat16)
    y = L.RMSNorm(hidden, 1e-6)
    y.weight = weight
    got = y.forward(x.cuda())
    assert torch.allclose(got.float().cpu(), O.rmsnorm(x, weight.cpu(), 1e-6).float(), atol=2e-2, rtol=2e-2)
    call("b200_comm_destroy", comm)


def test_engine_step_reports_a_peer_that_never_arrives(pkg):
    """A 2-rank engine whose peer never joins: the step returns, b200_engine_synchronize reports
    B200_ERR_TIMEOUT with the wait site, and the next synchronize is clean again."""
    from sglang_cpp_b200._lib import call, load
    from sglang_cpp_b200.engine import Engine, EngineConfig
    from sglang_cpp_b200.host_batch import HostBatcher

    cfg = O.ModelConfig(2, 256, 4, 2, 128, 512, 512, 1e-6, 1e6, 512, True, True, True)
    eng = Engine(cfg, EngineConfig(16, 16, 2, 128, 256, 0, 2))
    eng.fill_random(seed=0)
    comm = load().b200_engine_comm(eng._h)
    assert comm
    call("b200_comm_set_wait_limit_ns", comm, LIMIT_NS)
    call("b200_comm_connect_loopback", comm)
    hb = HostBatcher(eng, 16, 16, 2, enable_prefix_cache=False)
    req = hb.add_request(np.arange(1, 20, dtype=np.int32), 4)
    out = hb.prefill([req])
    with pytest.raises(pkg.B200Error) as err:
        out.synchronize()
    assert err.value.code == 3 and "site 401" in str(err.value)
    eng.synchronize()   # the report was cleared; nothing hangs, the context still answers
    eng.close()
