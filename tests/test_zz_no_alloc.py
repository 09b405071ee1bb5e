"""The allocation-free decode-attention entry point against the ordinary one.

`b200_attention_decode_noalloc` exists for callers that cannot allocate device memory at the point
of the call (their device-memory budget already belongs to one pool, or their step loop must not
hit cudaMalloc's device-wide synchronisation); it keeps its split-KV scratch in an 8 MiB array
inside the library.  It must give what `b200_attention_decode` gives with a caller-supplied
workspace — here on two calls in a row with different inputs, so the second call runs on the
contents the first one left in the shared array — and refuse shapes beyond the array.

This file sorts last on purpose: if it fails, a run that stops at the first failure has already
run every other test.
"""
import math

import numpy as np
import pytest
import torch

from tests.parity_cases import PagedSetup, assert_close_bf16, randn_bf16

pytestmark = pytest.mark.gpu
ATOL, RTOL = 2e-2, 2e-2   # the tolerance of the decode-attention parity tests


def _run_both(pkg, L, seq_lens, q_heads, kv_heads, page_size, seed):
    from sglang_cpp_b200._lib import call

    d, dev = 128, "cuda"
    ps = PagedSetup(seq_lens, page_size, kv_heads, d, seed)
    gen = torch.Generator().manual_seed(seed + 1)
    B = len(seq_lens)
    q = randn_bf16(gen, B, q_heads, d).to(dev)
    cache = L.MHAKVCache(kv_heads, 1, d, ps.num_slots // page_size, page_size, device=dev)
    cache.kv_buffer_[0, 0].copy_(ps.k_cache.to(dev))
    cache.kv_buffer_[1, 0].copy_(ps.v_cache.to(dev))
    pt = torch.from_numpy(ps.page_table).to(dev)
    ti = torch.from_numpy(ps.table_idx).to(dev)
    sl = torch.from_numpy(ps.seq_lens).to(dev)
    attn = L.PagedAttention(cache, q_heads, kv_heads, d, max_batch=B)
    want = attn.decode(q, 0, pt, ti, sl)
    got = torch.empty_like(want)
    call("b200_attention_decode_noalloc", got.data_ptr(), q.data_ptr(), q.stride(0), q.stride(1),
         cache.k_cache(0).data_ptr(), cache.v_cache(0).data_ptr(), cache.total_slots, pt.data_ptr(),
         pt.stride(0), ti.data_ptr(), sl.data_ptr(), B, q_heads, kv_heads, d, page_size,
         1.0 / math.sqrt(d), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return got, want


def test_noalloc_matches_workspace_entry_point_twice(pkg, L):
    rng = np.random.default_rng(0)
    first = rng.integers(100, 1500, size=24).tolist()      # several partials per request
    got, want = _run_both(pkg, L, first, 16, 8, 16, seed=21)
    assert_close_bf16(got, want, ATOL, RTOL, "first call")
    # second call: other lengths, other head shape, on whatever the first call left in the array
    second = [3, 700, 64, 1, 2049, 333]
    got, want = _run_both(pkg, L, second, 32, 4, 16, seed=22)
    assert_close_bf16(got, want, ATOL, RTOL, "second call")
    assert L.read_device_status() == (0, 0)


def test_noalloc_refuses_shapes_beyond_its_array(pkg, L):
    from sglang_cpp_b200._lib import load

    # 1024 requests x 128 query heads over one KV head per rank needs far more than 8 MiB.
    assert load().b200_attention_decode_workspace_bytes(1024, 128, 8, 128) > (8 << 20)
    with pytest.raises(pkg.B200Error, match="built-in array"):
        _run_both(pkg, L, [5] * 1024, 128, 8, 16, seed=1)
