"""The sampling kernel against the reference sampler's CPU definition (sample_row, via the oracle).

Candidate sets are compared bit-exactly on logits without ties; with ties (bf16 logits over a wide
vocabulary tie often) the boundary tie group may be ordered differently by a sort, so there the
set SIZE and every token strictly above the boundary value are compared.
"""
import numpy as np
import pytest
import torch

from oracle import token_loop_oracle as O

pytestmark = pytest.mark.gpu
bf16 = torch.bfloat16


def distinct_logits(rows, vocab, seed):
    """Rows of distinct bf16 values: a permutation of vocab distinct bf16 bit patterns in (-8, 8)."""
    gen = torch.Generator().manual_seed(seed)
    half = vocab // 2
    pos = (0x3D00 + 2 * np.arange(half)).astype(np.uint16)          # 0.03125 ... < 8.0
    neg = (pos | 0x8000).astype(np.uint16)
    bits = np.concatenate([pos, neg])
    base = torch.from_numpy(bits.view(np.int16).copy()).view(bf16)
    assert base.float().unique().numel() == vocab
    return torch.stack([base[torch.randperm(vocab, generator=gen)] for _ in range(rows)])


def run(L, logits, temps, top_k=None, top_p=None, seeds=None, step=0):
    dev = "cuda"
    t = torch.tensor(temps, dtype=torch.float32, device=dev)
    k = torch.tensor(top_k, dtype=torch.int32, device=dev) if top_k is not None else None
    p = torch.tensor(top_p, dtype=torch.float32, device=dev) if top_p is not None else None
    s = torch.tensor(seeds, dtype=torch.int64, device=dev) if seeds is not None else None
    tok, mask = L.sample(logits.to(dev), t, k, p, s, step, return_mask=True)
    torch.cuda.synchronize()
    return tok.cpu(), mask.cpu().bool()


def test_known_answers_of_the_reference_sampler(L):
    """tests/engine/test_sampler.cpp:35-48 (top_p 0.6 at temperature 0.8 keeps only token 0) and
    :92-109 (top_k = 1 is argmax), padded to the 8-wide rows the kernel takes."""
    logits = torch.full((1, 8), -30.0)
    logits[0, :4] = torch.tensor([10.0, 1.0, 0.5, -1.0])
    tok, mask = run(L, logits.to(bf16), [0.8], None, [0.6])
    assert tok.tolist() == [0] and mask[0].nonzero().flatten().tolist() == [0]
    gen = torch.Generator().manual_seed(0)
    lg = torch.randn(4, 64, generator=gen).to(bf16)
    tok, mask = run(L, lg, [1.0] * 4, [1] * 4, None)
    assert tok.tolist() == lg.float().argmax(-1).tolist()
    assert mask.sum(-1).tolist() == [1] * 4


@pytest.mark.parametrize("temp,k,p", [(0.7, 50, 0.9), (1.0, 50, 1.0), (1.3, -1, 0.9), (0.7, 5, 0.5), (1.0, -1, 1.0),
                                      (0.5, 1000, 0.95)])
def test_candidate_set_equals_sample_row(L, temp, k, p):
    rows, vocab = 6, 1024
    logits = distinct_logits(rows, vocab, seed=int(temp * 10) + max(k, 0))
    tk = k if k >= 1 else vocab
    tok, mask = run(L, logits, [temp] * rows, [tk] * rows, [p] * rows, list(range(rows)))
    for r in range(rows):
        t, kk, pp = O.prepare_sampling(temp, k, p, vocab, False)
        want = O.sample_row_distribution(logits[r].float(), t, kk, pp) > 0
        assert torch.equal(mask[r], want), f"row {r}: {int(mask[r].sum())} vs {int(want.sum())} candidates"
        assert bool(want[tok[r]]), "sampled token outside the candidate set"


def test_wide_vocabulary_with_ties(L):
    rows, vocab = 4, 151936
    gen = torch.Generator().manual_seed(3)
    logits = (torch.randn(rows, vocab, generator=gen) * 2.0).to(bf16)
    temp, k, p = 0.7, 50, 0.9
    tok, mask = run(L, logits, [temp] * rows, [k] * rows, [p] * rows, [11, 12, 13, 14])
    for r in range(rows):
        want = O.sample_row_distribution(logits[r].float(), temp, k, p) > 0
        assert int(mask[r].sum()) == int(want.sum())
        vals = logits[r].float()
        boundary = vals[want].min()
        assert torch.equal(mask[r] & (vals > boundary), want & (vals > boundary))
        assert bool(mask[r][tok[r]])


def test_draw_is_reproducible_and_follows_the_distribution(L):
    vocab = 64
    gen = torch.Generator().manual_seed(5)
    row = torch.randn(1, vocab, generator=gen).to(bf16)
    a, _ = run(L, row.repeat(8, 1), [1.0] * 8, None, None, list(range(8)), step=3)
    b, _ = run(L, row.repeat(8, 1), [1.0] * 8, None, None, list(range(8)), step=3)
    assert torch.equal(a, b)                       # same seeds and step: same tokens
    c, _ = run(L, row.repeat(8, 1), [1.0] * 8, None, None, list(range(8)), step=4)
    assert not torch.equal(a, c)                   # another step: another draw
    n = 4096
    toks, _ = run(L, row.repeat(n, 1), [1.0] * n, None, None, list(range(1000, 1000 + n)))
    freq = torch.bincount(toks.long(), minlength=vocab).float() / n
    want = torch.softmax(row[0].float(), -1)
    assert float((freq - want).abs().max()) < 0.03  # ~4 sigma at n = 4096


def test_greedy_rows_inside_a_sampled_batch(L):
    gen = torch.Generator().manual_seed(7)
    lg = torch.randn(3, 256, generator=gen).to(bf16)
    tok, mask = run(L, lg, [1e-6, 0.9, 1e-6], [256] * 3, [1.0] * 3)
    am = lg.float().argmax(-1)
    assert tok[0] == am[0] and tok[2] == am[2]
    assert mask[0].sum() == 1 and mask[2].sum() == 1


# ---- sampling from probabilities (the reference's device path: flashinfer_*_sample_from_probs) -----
def _probs(rows, vocab, seed, sharp=3.0):
    gen = torch.Generator().manual_seed(seed)
    return torch.softmax(torch.randn(rows, vocab, generator=gen) * sharp, -1).contiguous()


def test_sample_from_probs_known_answers(L):
    """tests/engine/test_sampler.cpp:92-109 (top_k = 1 samples the argmax whatever the uniform
    number) and the no-filter form on a one-hot row."""
    probs = _probs(5, 1000, 1)
    u = torch.tensor([0.0, 0.3, 0.5, 0.9, 0.999], device="cuda")
    k = torch.ones(5, dtype=torch.int32, device="cuda")
    got = L.sample_from_probs(probs.cuda(), u, top_k=k)
    assert got.cpu().tolist() == probs.argmax(-1).tolist()
    one_hot = torch.zeros(2, 64)
    one_hot[0, 17] = 1.0
    one_hot[1, 63] = 1.0
    got = L.sample_from_probs(one_hot.cuda(), torch.tensor([0.7, 0.2], device="cuda"))
    assert got.cpu().tolist() == [17, 63]


@pytest.mark.parametrize("vocab,k,p", [(1000, 0, 1.0), (1000, 50, 1.0), (1000, 0, 0.9), (1000, 20, 0.8),
                                       (151936, 50, 0.9), (4099, 3, 0.5)])
def test_sample_from_probs_matches_the_rejection_rule(L, vocab, k, p):
    rows = 6
    probs = _probs(rows, vocab, vocab + k)
    us = torch.tensor([0.0, 0.11, 0.37, 0.5, 0.83, 0.9999], dtype=torch.float32)
    tk = torch.full((rows,), k if k > 0 else vocab, dtype=torch.int32)
    tp = torch.full((rows,), p, dtype=torch.float32)
    got = L.sample_from_probs(probs.cuda(), us.cuda(), tk.cuda(), tp.cuda()).cpu().tolist()
    for r in range(rows):
        want, accepted = O.sample_from_probs(probs[r], float(us[r]), k, p)
        assert bool(accepted[got[r]]), f"row {r}: token {got[r]} is outside the accepted set"
        if got[r] != want:
            # the inverse CDF lands within rounding of a boundary between two neighbouring accepted tokens
            idx = accepted.nonzero().flatten().tolist()
            assert abs(idx.index(got[r]) - idx.index(want)) <= 1, (r, got[r], want)
    # scalar filter arguments give the same tokens as per-row arrays
    again = L.sample_from_probs(probs.cuda(), us.cuda(), None, None, k, p).cpu().tolist()
    assert again == got


def test_sample_from_probs_follows_the_distribution(L):
    probs = _probs(1, 32, 9, sharp=1.0)
    n = 8192
    gen = torch.Generator().manual_seed(0)
    u = torch.rand(n, generator=gen)
    got = L.sample_from_probs(probs.repeat(n, 1).contiguous().cuda(), u.cuda()).cpu()
    freq = torch.bincount(got.long(), minlength=32).float() / n
    assert float((freq - probs[0]).abs().max()) < 0.02


def test_sampler_time_per_call(L):
    """64 rows of a 151 936-word vocabulary (the decode batch of the benchmark): device time per call,
    printed with -s.  The bound only catches a regression to the multi-pass form (0.3 ms)."""
    rows, vocab = 64, 151936
    gen = torch.Generator().manual_seed(0)
    logits = (torch.randn(rows, vocab, generator=gen) * 0.64).to(torch.bfloat16).cuda()
    seeds = torch.arange(rows, dtype=torch.int64).cuda()
    for t, k, p in ((0.7, 50, 0.9), (1.0, -1, 1.0)):
        temps = torch.full((rows,), t).cuda()
        tk = torch.full((rows,), k, dtype=torch.int32).cuda()
        tp = torch.full((rows,), p).cuda()
        for _ in range(3):
            L.sample(logits, temps, tk, tp, seeds=seeds, step_index=3)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(20):
            L.sample(logits, temps, tk, tp, seeds=seeds, step_index=3)
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) * 1000 / 20
        print(f"sample_kernel, {rows} x {vocab}, temperature {t} top_k {k} top_p {p}: {us:.1f} us per call")
        assert us < 150.0
