"""Parity of the elementwise / norm / rope / index kernels against the CPU oracle (through the C ABI).

Tolerances: these operators compute in fp32 and store bf16, exactly as the oracle's `store_bf16`
mode does, so results may differ from the oracle by at most one bf16 rounding step of the value
(rtol 2^-7 = 7.8e-3) plus a small absolute term for values near zero.  Integer kernels are bit-exact.
"""
import numpy as np
import pytest
import torch

from oracle import token_loop_oracle as O
from tests.parity_cases import assert_close_bf16, randn_bf16

pytestmark = pytest.mark.gpu
bf16 = torch.bfloat16
RTOL = 2 ** -7
ATOL = 1e-3


@pytest.mark.parametrize("rows,hidden", [(1, 1024), (64, 1024), (130, 4096), (7, 2048), (3, 8192), (2, 16384), (0, 1024)])
def test_rmsnorm(L, rows, hidden):
    gen = torch.Generator().manual_seed(rows * 31 + hidden)
    x = randn_bf16(gen, rows, hidden)
    norm = L.RMSNorm(hidden, 1e-6)
    norm.weight = randn_bf16(gen, hidden).cuda()
    got = norm.forward(x.cuda())
    assert_close_bf16(got, O.rmsnorm(x, norm.weight.cpu(), 1e-6), ATOL, RTOL, "rmsnorm")
    xi = x.cuda()
    norm.forward_inplace(xi)
    assert torch.equal(xi, got)


@pytest.mark.parametrize("rows,hidden", [(64, 1024), (128, 4096), (5, 2048), (8192, 1024)])
def test_fused_add_rmsnorm(L, rows, hidden):
    gen = torch.Generator().manual_seed(rows + hidden)
    x = randn_bf16(gen, rows, hidden)
    r = randn_bf16(gen, rows, hidden)
    norm = L.RMSNorm(hidden, 1e-6)
    norm.weight = randn_bf16(gen, hidden).cuda()
    xd, rd = x.cuda(), r.cuda()
    norm.fused_add_forward_inplace(xd, rd)
    wx, wr = O.fused_add_rmsnorm(x, r, norm.weight.cpu(), 1e-6)
    assert_close_bf16(rd, wr, 0.0, 0.0, "residual (bit-exact: one fp32 add, one rounding)")
    assert_close_bf16(xd, wx, ATOL, RTOL, "normed")


def test_rmsnorm_rejects_bad_shapes(L, pkg):
    norm = L.RMSNorm(1024, 1e-6)
    with pytest.raises(pkg.B200Error):
        norm.forward(torch.zeros(1024, dtype=bf16, device="cuda"))  # rank 1
    with pytest.raises(pkg.B200Error):
        norm.forward(torch.zeros(4, 512, dtype=bf16, device="cuda"))  # weight mismatch


@pytest.mark.parametrize("tokens,hq,hkv,d", [(64, 16, 8, 128), (5, 32, 4, 128), (3, 4, 1, 64), (0, 16, 8, 128)])
def test_qk_rmsnorm_strided(L, tokens, hq, hkv, d):
    gen = torch.Generator().manual_seed(tokens + hq)
    qkv = randn_bf16(gen, tokens, (hq + 2 * hkv) * d)
    qn, kn = L.RMSNorm(d, 1e-6), L.RMSNorm(d, 1e-6)
    qn.weight, kn.weight = randn_bf16(gen, d).cuda(), randn_bf16(gen, d).cuda()
    dev = qkv.cuda()
    q = dev[:, :hq * d].view(tokens, hq, d)
    k = dev[:, hq * d:(hq + hkv) * d].view(tokens, hkv, d)
    L.fused_qk_rmsnorm_inplace_3d_strided(q, k, qn, kn)
    wq = O.rmsnorm(qkv[:, :hq * d].view(tokens, hq, d), qn.weight.cpu(), 1e-6)
    wk = O.rmsnorm(qkv[:, hq * d:(hq + hkv) * d].view(tokens, hkv, d), kn.weight.cpu(), 1e-6)
    assert_close_bf16(q, wq, ATOL, RTOL, "q norm")
    assert_close_bf16(k, wk, ATOL, RTOL, "k norm")
    # v must be untouched
    assert torch.equal(dev[:, (hq + hkv) * d:].cpu(), qkv[:, (hq + hkv) * d:])
    # The fused form equals two single-tensor calls (the reference's own self-consistency test,
    # tests/layers/test_normalization.cpp:21-53).
    dev2 = qkv.cuda()
    q2 = dev2[:, :hq * d].view(tokens, hq, d)
    k2 = dev2[:, hq * d:(hq + hkv) * d].view(tokens, hkv, d)
    qn.forward_inplace_3d_strided(q2)
    kn.forward_inplace_3d_strided(k2)
    assert torch.equal(dev, dev2)


@pytest.mark.parametrize("tokens,hq,hkv,d,rd", [(64, 16, 8, 128, 128), (9, 8, 2, 64, 64), (4, 4, 4, 128, 64)])
def test_rope(L, tokens, hq, hkv, d, rd):
    gen = torch.Generator().manual_seed(tokens * 7 + d)
    q = randn_bf16(gen, tokens, hq, d)
    k = randn_bf16(gen, tokens, hkv, d)
    pos = torch.randint(0, 4096, (tokens,), generator=gen, dtype=torch.int32)
    rot = L.RotaryEmbedding(d, rd, 4096, 1e6)
    qd, kd = q.cuda(), k.cuda()
    rot.forward_inplace(pos.cuda(), qd, kd)
    cos, sin = O.rope_tables(rd, 4096, 1e6)
    assert torch.equal(cos, rot.cos_cache_.cpu())
    assert_close_bf16(qd, O.rope_neox(q, pos, cos, sin, rd), ATOL, RTOL, "q rope")
    assert_close_bf16(kd, O.rope_neox(k, pos, cos, sin, rd), ATOL, RTOL, "k rope")


@pytest.mark.parametrize("tokens,hkv,d", [(64, 8, 128), (1, 1, 128), (33, 4, 128)])
def test_store_kv(L, tokens, hkv, d):
    gen = torch.Generator().manual_seed(tokens)
    cache = L.MHAKVCache(hkv, 2, d, 40, 4)
    width = 3 * hkv * d
    buf = randn_bf16(gen, tokens, width).cuda()
    k, v = buf[:, hkv * d:2 * hkv * d], buf[:, 2 * hkv * d:]
    loc = torch.randperm(cache.total_slots, generator=gen)[:tokens].to(torch.int32)
    cache.store_kv(k, v, loc.cuda(), 1)
    assert torch.equal(cache.k_cache(1)[loc.long().cuda()].reshape(tokens, -1), k)
    assert torch.equal(cache.v_cache(1)[loc.long().cuda()].reshape(tokens, -1), v)
    assert float(cache.k_cache(0).abs().sum()) == 0.0


@pytest.mark.parametrize("tokens,hq,hkv,qk_norm", [(64, 16, 8, True), (128, 32, 8, False), (7, 32, 4, True), (1, 4, 1, True),
                                                  (1401, 16, 8, True)])   # a prefill batch: several rows per warp
def test_qknorm_rope_store_matches_unfused_sequence(L, tokens, hq, hkv, qk_norm):
    d = 128
    gen = torch.Generator().manual_seed(tokens + hq * 3)
    qkv = randn_bf16(gen, tokens, (hq + 2 * hkv) * d)
    pos = torch.randint(0, 2048, (tokens,), generator=gen, dtype=torch.int32)
    cache = L.MHAKVCache(hkv, 1, d, max(64, tokens // 16 + 2), 16)
    loc = torch.randperm(cache.total_slots, generator=gen)[:tokens].to(torch.int32)
    rot = L.RotaryEmbedding(d, d, 2048, 1e6)
    qn = kn = None
    if qk_norm:
        qn, kn = L.RMSNorm(d, 1e-6), L.RMSNorm(d, 1e-6)
        qn.weight, kn.weight = randn_bf16(gen, d).cuda(), randn_bf16(gen, d).cuda()
    fused = qkv.cuda()
    L.qknorm_rope_store(fused, qn, kn, rot, pos.cuda(), loc.cuda(), cache, 0, hq, hkv, write_k_back=True)
    # Oracle with the reference's rounding points (norm -> bf16 -> rope -> bf16).
    q = qkv[:, :hq * d].view(tokens, hq, d)
    k = qkv[:, hq * d:(hq + hkv) * d].view(tokens, hkv, d)
    v = qkv[:, (hq + hkv) * d:].view(tokens, hkv, d)
    if qk_norm:
        q = O.rmsnorm(q, qn.weight.cpu(), 1e-6)
        k = O.rmsnorm(k, kn.weight.cpu(), 1e-6)
    cos, sin = O.rope_tables(d, 2048, 1e6)
    q = O.rope_neox(q, pos, cos, sin)
    k = O.rope_neox(k, pos, cos, sin)
    # Two roundings in sequence can each flip one bf16 step.
    assert_close_bf16(fused[:, :hq * d].view(tokens, hq, d), q, 2 * ATOL, 2 * RTOL, "q")
    assert_close_bf16(fused[:, hq * d:(hq + hkv) * d].view(tokens, hkv, d), k, 2 * ATOL, 2 * RTOL, "k back")
    assert_close_bf16(cache.k_cache(0)[loc.long().cuda()], k, 2 * ATOL, 2 * RTOL, "k cache")
    assert torch.equal(cache.v_cache(0)[loc.long().cuda()].cpu(), v)
    # ... and equal, to one bf16 step, to this library's own unfused kernels run in the reference's order.
    unf = qkv.cuda()
    qv = unf[:, :hq * d].view(tokens, hq, d)
    kv_ = unf[:, hq * d:(hq + hkv) * d].view(tokens, hkv, d)
    if qk_norm:
        L.fused_qk_rmsnorm_inplace_3d_strided(qv, kv_, qn, kn)
    rot.forward_inplace(pos.cuda(), qv, kv_)
    assert_close_bf16(fused, unf, ATOL, RTOL, "fused vs unfused kernels")


@pytest.mark.parametrize("tokens,d", [(64, 3072), (3, 768), (0, 64), (8192, 3072)])
def test_silu_and_gelu_and_mul(L, tokens, d):
    gen = torch.Generator().manual_seed(d)
    x = randn_bf16(gen, tokens, 2 * d, std=2.0)
    out = torch.empty(tokens, d, dtype=bf16, device="cuda")
    L.silu_and_mul(out, x.cuda())
    assert_close_bf16(out, O.silu_and_mul(x), ATOL, RTOL, "silu_and_mul")
    L.gelu_and_mul(out, x.cuda())
    assert_close_bf16(out, O.gelu_and_mul(x), ATOL, RTOL, "gelu_and_mul")


def test_embedding_and_bad_id(L):
    gen = torch.Generator().manual_seed(5)
    table = randn_bf16(gen, 1000, 1024)
    ids = torch.randint(0, 1000, (77,), generator=gen, dtype=torch.int32)
    got = L.embedding(table.cuda(), ids.cuda())
    assert torch.equal(got.cpu(), table[ids.long()])
    assert L.read_device_status() == (0, 0)
    ids[3] = 1000
    got = L.embedding(table.cuda(), ids.cuda())
    assert float(got[3].abs().sum()) == 0.0
    assert L.read_device_status() == (0, 1001)
    assert L.read_device_status() == (0, 0)  # reading clears


def test_token_pool_kernels_bit_exact(L):
    rng = np.random.default_rng(0)
    table = rng.integers(0, 1 << 30, size=(9, 64), dtype=np.int32)
    n = 500
    req = rng.integers(-2, 11, size=n).astype(np.int32)   # includes out-of-range rows
    pos = rng.integers(-3, 70, size=n).astype(np.int32)   # includes out-of-range columns
    got = L.gather_int32_2d(torch.from_numpy(table).cuda(), torch.from_numpy(req).cuda(), torch.from_numpy(pos).cuda())
    assert np.array_equal(got.cpu().numpy(), O.gather_int32_2d(table, req, pos))
    # scatter: unique targets so the result does not depend on write order
    flat = rng.permutation(9 * 64)[:200]
    req2 = np.concatenate([(flat // 64), [-1, 9, 3]]).astype(np.int32)
    pos2 = np.concatenate([(flat % 64), [0, 0, 64]]).astype(np.int32)
    tok = rng.integers(0, 151936, size=len(req2)).astype(np.int32)
    dev = torch.from_numpy(table).cuda()
    L.write_token_pool(dev, torch.from_numpy(req2).cuda(), torch.from_numpy(pos2).cuda(), torch.from_numpy(tok).cuda())
    want = table.copy()
    O.write_token_pool(want, req2, pos2, tok)
    assert np.array_equal(dev.cpu().numpy(), want)
    # empty input is a no-op
    e = torch.empty(0, dtype=torch.int32, device="cuda")
    assert L.gather_int32_2d(dev, e, e).numel() == 0
    L.write_token_pool(dev, e, e, e)


@pytest.mark.parametrize("rows,vocab", [(64, 151936), (1, 128256), (5, 1000), (3, 64)])
def test_argmax_first_index_on_ties(L, rows, vocab):
    gen = torch.Generator().manual_seed(vocab)
    logits = randn_bf16(gen, rows, vocab)
    got = L.argmax(logits.cuda())
    assert got.dtype == torch.int32
    assert torch.equal(got.cpu().long(), O.greedy(logits.float()))
    # exact ties: bf16 rounding makes them common on wide vocabularies
    logits[:, :] = 0.5
    logits[:, vocab // 2] = 1.0
    logits[:, vocab - 1] = 1.0
    assert torch.equal(L.argmax(logits.cuda()).cpu().long(), torch.full((rows,), vocab // 2))
