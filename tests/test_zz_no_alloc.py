"""The allocation-free decode-attention entry point against the ordinary one and the oracle.

`b200_attention_decode_noalloc` exists for callers that cannot allocate device memory at the point
of the call (their device-memory budget already belongs to one pool, or their step loop must not
hit cudaMalloc's device-wide synchronisation); it keeps its split-KV scratch in an 8 MiB array
inside the library.  It runs the kernel `b200_attention_decode` runs with a caller-supplied
workspace, so the two must agree bit for bit — here on two calls in a row with different inputs, so
the second call runs on the contents the first one left in the shared array — and both must agree
with the CPU oracle within the tolerance of the decode-attention parity tests.  Shapes beyond the
array are refused, and what its kernel reports (here: a page-table slot outside the pool) is read
through `b200_attention_decode_noalloc_status`, not through the library's ordinary status words.

This file sorts last on purpose: if it fails, a run that stops at the first failure has already
run every other test.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

from oracle import token_loop_oracle as O
from tests.parity_cases import PagedSetup, assert_close_bf16, randn_bf16

pytestmark = pytest.mark.gpu
ATOL, RTOL = 2e-2, 2e-2   # the tolerance of the decode-attention parity tests


def _noalloc_status():
    from sglang_cpp_b200._lib import call

    buf = (ctypes.c_int32 * 2)()
    call("b200_attention_decode_noalloc_status", buf, torch.cuda.current_stream().cuda_stream)
    return buf[0], buf[1]


def _run_both(pkg, L, seq_lens, q_heads, kv_heads, page_size, seed, poison_slot=None):
    from sglang_cpp_b200._lib import call

    d, dev = 128, "cuda"
    ps = PagedSetup(seq_lens, page_size, kv_heads, d, seed)
    gen = torch.Generator().manual_seed(seed + 1)
    B = len(seq_lens)
    q = randn_bf16(gen, B, q_heads, d).to(dev)
    cache = L.MHAKVCache(kv_heads, 1, d, ps.num_slots // page_size, page_size, device=dev)
    cache.kv_buffer_[0, 0].copy_(ps.k_cache.to(dev))
    cache.kv_buffer_[1, 0].copy_(ps.v_cache.to(dev))
    table = ps.page_table.copy()
    if poison_slot is not None:
        table[ps.table_idx[0], 0:page_size] = poison_slot + np.arange(page_size)
    pt = torch.from_numpy(table).to(dev)
    ti = torch.from_numpy(ps.table_idx).to(dev)
    sl = torch.from_numpy(ps.seq_lens).to(dev)
    attn = L.PagedAttention(cache, q_heads, kv_heads, d, max_batch=B)
    want = attn.decode(q, 0, pt, ti, sl) if poison_slot is None else None
    got = torch.empty(B, q_heads * d, dtype=torch.bfloat16, device=dev)
    call("b200_attention_decode_noalloc", got.data_ptr(), q.data_ptr(), q.stride(0), q.stride(1),
         cache.k_cache(0).data_ptr(), cache.v_cache(0).data_ptr(), cache.total_slots, pt.data_ptr(),
         pt.stride(0), ti.data_ptr(), sl.data_ptr(), B, q_heads, kv_heads, d, page_size,
         1.0 / math.sqrt(d), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    oracle = O.paged_attention(q.cpu(), ps.k_cache, ps.v_cache, ps.page_table, ps.table_idx, ps.seq_lens,
                               np.arange(B + 1), 1.0 / math.sqrt(d), O.store_fp32).reshape(B, q_heads * d) \
        if poison_slot is None else None
    return got, want, oracle


def test_noalloc_matches_workspace_entry_point_and_oracle_twice(pkg, L):
    rng = np.random.default_rng(0)
    first = rng.integers(100, 1500, size=24).tolist()      # several partials per request
    got, want, oracle = _run_both(pkg, L, first, 16, 8, 16, seed=21)
    assert torch.equal(got, want.view_as(got)), "first call: the two entry points run the same kernel"
    assert_close_bf16(got.view_as(oracle), oracle, ATOL, RTOL, "first call against the oracle")
    # second call: other lengths, other head shape, on whatever the first call left in the array
    second = [3, 700, 64, 1, 2049, 333]
    got, want, oracle = _run_both(pkg, L, second, 32, 4, 16, seed=22)
    assert torch.equal(got, want.view_as(got)), "second call"
    assert_close_bf16(got.view_as(oracle), oracle, ATOL, RTOL, "second call against the oracle")
    assert _noalloc_status() == (0, 0)
    assert L.read_device_status() == (0, 0)


def test_noalloc_reports_a_slot_outside_the_pool_through_its_own_status_words(pkg, L):
    """The kernel checks every page-table entry before it becomes an address: a slot beyond the pool
    is recorded (slot + 1) and read as slot 0 instead — nothing faults.  The report waits in the
    built-in array until it is read, and the read clears it."""
    lens = [40, 70, 33]
    bad = 10 ** 6
    _run_both(pkg, L, lens, 16, 8, 16, seed=5, poison_slot=bad)
    # a later, healthy call does not wipe the report
    got, want, _ = _run_both(pkg, L, lens, 16, 8, 16, seed=6)
    assert torch.equal(got, want.view_as(got))
    timeout_site, bad_index = _noalloc_status()
    assert timeout_site == 0 and bad_index == bad + 1
    assert _noalloc_status() == (0, 0)
    assert L.read_device_status() == (0, 0), "the ordinary status words belong to the other entry points"


def test_noalloc_refuses_shapes_beyond_its_array(pkg, L):
    from sglang_cpp_b200._lib import load

    # 1024 requests x 128 query heads over one KV head per rank needs far more than 8 MiB.
    assert load().b200_attention_decode_workspace_bytes(1024, 128, 8, 128) > (8 << 20)
    with pytest.raises(pkg.B200Error, match="built-in array"):
        _run_both(pkg, L, [5] * 1024, 128, 8, 16, seed=1)
