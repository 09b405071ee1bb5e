"""Shared builders for the parity tests: seeded inputs, paged-KV set-ups and comparisons.

Nothing here is collected by pytest; the GPU tests, the CPU tests and
``__graft_entry__.smoke()`` import it.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from oracle import token_loop_oracle as O

bf16 = torch.bfloat16


def randn_bf16(gen: torch.Generator, *shape, std: float = 1.0) -> torch.Tensor:
    return (torch.randn(*shape, generator=gen, dtype=torch.float32) * std).to(bf16)


def max_mean_err(got: torch.Tensor, want: torch.Tensor):
    d = (got.detach().float().cpu() - want.detach().float().cpu()).abs()
    return float(d.max()) if d.numel() else 0.0, float(d.mean()) if d.numel() else 0.0


def assert_close_bf16(got, want, atol, rtol, what=""):
    g = got.detach().float().cpu()
    w = want.detach().float().cpu()
    assert g.shape == w.shape, f"{what}: shape {tuple(g.shape)} vs {tuple(w.shape)}"
    err = (g - w).abs()
    tol = atol + rtol * w.abs()
    bad = err > tol
    assert not bool(bad.any()), (
        f"{what}: {int(bad.sum())} of {bad.numel()} elements out of tolerance; "
        f"max err {float(err.max()):.4g} at {np.unravel_index(int(err.argmax()), tuple(err.shape))}")


class PagedSetup:
    """A KV pool with random contents and a page table that scatters each request's pages over
    the pool (page_size-aligned, shuffled), the way CacheManager::allocate_paged +
    write_page_table lay them out (src/scheduler/prefill.cc:144-206)."""

    def __init__(self, seq_lens, page_size: int, kv_heads: int, head_dim: int = 128, seed: int = 0,
                 extra_pages: int = 3, shared_prefix: int = 0, std: float = 1.0, shuffle_pages: bool = True):
        gen = torch.Generator().manual_seed(seed)
        rng = np.random.default_rng(seed)
        B = len(seq_lens)
        self.page_size = page_size
        self.seq_lens = np.asarray(seq_lens, dtype=np.int32)
        pages_per_req = [math.ceil(max(int(n), 1) / page_size) for n in seq_lens]
        total_pages = sum(pages_per_req) + extra_pages
        self.num_slots = total_pages * page_size
        max_len = max(int(max(seq_lens)) if B else 1, 1)
        cols = (math.ceil(max_len / page_size) * page_size + 31) // 32 * 32
        self.page_table = np.zeros((B + 2, cols), dtype=np.int32)
        self.table_idx = rng.permutation(B + 2)[:B].astype(np.int32)
        # shuffle_pages=False: each request's pages are consecutive slots, as they are when a
        # prompt's pages are allocated in one go
        order = rng.permutation(total_pages) if shuffle_pages else np.arange(total_pages)
        cur = 0
        shared_pages = None
        for b in range(B):
            row = self.table_idx[b]
            for pg in range(pages_per_req[b]):
                if shared_prefix and (pg + 1) * page_size <= shared_prefix and shared_pages is not None \
                        and pg < len(shared_pages) and (pg + 1) * page_size <= int(seq_lens[b]):
                    page = shared_pages[pg]
                else:
                    page = int(order[cur])
                    cur += 1
                self.page_table[row, pg * page_size:(pg + 1) * page_size] = page * page_size + np.arange(page_size)
            if shared_prefix and shared_pages is None:
                shared_pages = [int(self.page_table[row, pg * page_size]) // page_size
                                for pg in range(pages_per_req[b])]
        self.k_cache = randn_bf16(gen, self.num_slots, kv_heads, head_dim, std=std)
        self.v_cache = randn_bf16(gen, self.num_slots, kv_heads, head_dim, std=std)


def decode_attention_case(L, seq_lens, page_size, q_heads, kv_heads, seed=0, poison_unused=False):
    """Runs the CUDA decode attention and the oracle on the same seeded inputs; returns (got, want)."""
    dev = "cuda"
    d = 128
    ps = PagedSetup(seq_lens, page_size, kv_heads, d, seed)
    gen = torch.Generator().manual_seed(seed + 1)
    B = len(seq_lens)
    qkv_width = (q_heads + 2 * kv_heads) * d
    qkv = randn_bf16(gen, B, qkv_width)
    k_cache, v_cache = ps.k_cache.clone(), ps.v_cache.clone()
    if poison_unused:
        # Slots no request owns hold NaN: the kernel must not let them reach the output.
        used = np.zeros(ps.num_slots, dtype=bool)
        for b in range(B):
            used[ps.page_table[ps.table_idx[b], :int(seq_lens[b])]] = True
        mask = torch.from_numpy(~used)
        k_cache[mask] = float("nan")
        v_cache[mask] = float("nan")
    cache = L.MHAKVCache(kv_heads, 1, d, ps.num_slots // page_size, page_size, device=dev)
    cache.kv_buffer_[0, 0].copy_(k_cache.to(dev))
    cache.kv_buffer_[1, 0].copy_(v_cache.to(dev))
    attn = L.PagedAttention(cache, q_heads, kv_heads, d, max_batch=max(B, 1))
    q_dev = qkv.to(dev)
    q_view = q_dev[:, :q_heads * d].view(B, q_heads, d)
    got = attn.decode(q_view, 0, torch.from_numpy(ps.page_table).to(dev),
                      torch.from_numpy(ps.table_idx).to(dev), torch.from_numpy(ps.seq_lens).to(dev))
    torch.cuda.synchronize()
    want = O.paged_attention(qkv[:, :q_heads * d].view(B, q_heads, d), ps.k_cache, ps.v_cache,
                             ps.page_table, ps.table_idx, ps.seq_lens, np.arange(B + 1),
                             1.0 / math.sqrt(d), O.store_fp32).reshape(B, q_heads * d)
    return got, want, attn


def prefill_attention_case(L, seq_lens, extend_lens, page_size, q_heads, kv_heads, seed=0, shuffle_pages=True):
    dev = "cuda"
    d = 128
    ps = PagedSetup(seq_lens, page_size, kv_heads, d, seed, shuffle_pages=shuffle_pages)
    gen = torch.Generator().manual_seed(seed + 1)
    B = len(seq_lens)
    qo = np.zeros(B + 1, dtype=np.int32)
    qo[1:] = np.cumsum(extend_lens)
    T = int(qo[-1])
    q = randn_bf16(gen, T, q_heads, d)
    cache = L.MHAKVCache(kv_heads, 1, d, ps.num_slots // page_size, page_size, device=dev)
    cache.kv_buffer_[0, 0].copy_(ps.k_cache.to(dev))
    cache.kv_buffer_[1, 0].copy_(ps.v_cache.to(dev))
    attn = L.PagedAttention(cache, q_heads, kv_heads, d, max_batch=max(B, 1))
    got = attn.prefill(q.to(dev), 0, torch.from_numpy(ps.page_table).to(dev),
                       torch.from_numpy(ps.table_idx).to(dev), torch.from_numpy(ps.seq_lens).to(dev),
                       torch.from_numpy(qo).to(dev), int(max(extend_lens)) if B else 0)
    torch.cuda.synchronize()
    want = O.paged_attention(q, ps.k_cache, ps.v_cache, ps.page_table, ps.table_idx, ps.seq_lens, qo,
                             1.0 / math.sqrt(d), O.store_fp32).reshape(T, q_heads * d)
    return got, want


def run_smoke_case(pkg) -> None:
    """One decode-shaped pass of the hot-path operators on cuda:0, each checked against the oracle."""
    L = pkg.layers
    gen = torch.Generator().manual_seed(7)
    x = randn_bf16(gen, 8, 1024)
    w = randn_bf16(gen, 256, 1024, std=0.05)
    y = L.linear(x.cuda(), w.cuda())
    assert_close_bf16(y, O.linear(x, w), 2e-2, 2e-2, "smoke linear")
    got, want, _ = decode_attention_case(L, [5, 37, 130], 16, 16, 8, seed=3)
    assert_close_bf16(got, want, 2e-2, 2e-2, "smoke decode attention")
    status = L.read_device_status()
    assert status == (0, 0), f"device status words {status}"
