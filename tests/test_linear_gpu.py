"""Parity of the tcgen05 GEMMs against the CPU oracle (through the C ABI).

Tolerance: bf16 operands, fp32 accumulation on both sides; the only differences are the order of
the fp32 additions (K split across a cluster) and the final bf16 rounding: one bf16 step (rtol
2^-7) plus an absolute term that covers cancellation in long dot products.
"""
import pytest
import torch

from oracle import token_loop_oracle as O
from tests.parity_cases import assert_close_bf16, randn_bf16

pytestmark = pytest.mark.gpu
RTOL = 2 ** -7


@pytest.mark.parametrize("M,N,K", [
    (64, 4096, 1024),     # Qwen3-0.6B qkv at batch 64
    (64, 1024, 2048),     # o_proj
    (64, 1024, 3072),     # down_proj
    (1, 4096, 1024),      # batch 1
    (17, 256, 64),        # one k-block, partial rows
    (128, 6144, 4096),    # Llama qkv at batch 128
    (256, 128, 2048),     # Qwen3-MoE router
    (33, 1000, 192),      # N not a multiple of the 128-feature tile
    (300, 512, 256),      # more rows than one slab
    (70, 384, 512),       # row counts between two multiples of the 64-column exchange round:
    (96, 256, 128),       #   every row must be written (one round per 64 accumulator columns)
    (150, 1024, 384),
    (218, 1280, 384),
    (224, 384, 640),
    (64, 151936, 1024),   # Qwen3-0.6B lm_head (tied embedding): 311 MB of weights
    (0, 512, 256),
])
def test_linear_matches_oracle(L, M, N, K):
    gen = torch.Generator().manual_seed(M + N + K)
    x = randn_bf16(gen, M, K)
    w = randn_bf16(gen, N, K, std=0.05)
    y = L.linear(x.cuda(), w.cuda())
    assert y.shape == (M, N)
    assert_close_bf16(y, O.linear(x, w), 2e-3 * (K / 1024) ** 0.5 + 1e-3, RTOL, f"linear {M}x{N}x{K}")
    assert L.read_device_status() == (0, 0)


def test_linear_bias_and_strided_input(L):
    gen = torch.Generator().manual_seed(3)
    buf = randn_bf16(gen, 40, 2048)
    x = buf[:, 512:1536]           # row stride 2048, K = 1024
    w = randn_bf16(gen, 384, 1024, std=0.05)
    b = randn_bf16(gen, 384)
    y = L.linear(buf.cuda()[:, 512:1536], w.cuda(), b.cuda())
    assert_close_bf16(y, O.linear(x, w, b), 4e-3, RTOL, "linear + bias, strided rows")


@pytest.mark.parametrize("M,I,K", [(64, 3072, 1024), (5, 768, 2048), (128, 14336 // 8, 4096), (256, 256, 128),
                                   (90, 640, 384), (200, 256, 512)])
def test_gate_up_swiglu_epilogue(L, pkg, M, I, K):
    gen = torch.Generator().manual_seed(I)
    x = randn_bf16(gen, M, K)
    w = randn_bf16(gen, 2 * I, K, std=0.05)
    y = L.linear(x.cuda(), w.cuda(), epilogue=pkg.EPILOGUE_SWIGLU)
    assert y.shape == (M, I)
    want = O.silu_and_mul(O.linear(x, w))
    # The product of two rounded values: two bf16 steps.
    assert_close_bf16(y, want, 4e-3, 3 * RTOL, "gate_up + SwiGLU")
    # and equal to the unfused pair of kernels of this library, to one bf16 step
    gu = L.linear(x.cuda(), w.cuda())
    out = torch.empty(M, I, dtype=torch.bfloat16, device="cuda")
    L.silu_and_mul(out, gu)
    # (the two GEMMs split K differently, so gate or up may differ by one bf16 step before the
    # product is rounded again)
    assert_close_bf16(y, out, 4e-3, 3 * RTOL, "fused vs unfused SwiGLU")


@pytest.mark.parametrize("M,N,K", [
    (257, 256, 64),       # smallest prefill-path case: 3 token blocks, one k-block
    (1000, 1000, 192),    # ragged in M and N
    (2048, 4096, 1024),   # one full band, Qwen3-0.6B qkv
    (4500, 1024, 3072),   # more than two bands, down_proj
    (8192, 512, 128),     # more tiles per CTA than accumulators
    (8192, 4096, 1024),   # a full prefill batch of Qwen3-0.6B qkv: 1.7 tiles per CTA per band
])
def test_linear_prefill_tiles_match_oracle(L, M, N, K):
    """Batches of more than 256 rows take the persistent 128 x 256 tile kernel."""
    gen = torch.Generator().manual_seed(M + N + K)
    x = randn_bf16(gen, M, K)
    w = randn_bf16(gen, N, K, std=0.05)
    b = randn_bf16(gen, N)
    y = L.linear(x.cuda(), w.cuda(), b.cuda())
    assert y.shape == (M, N)
    assert_close_bf16(y, O.linear(x, w, b), 2e-3 * (K / 1024) ** 0.5 + 1e-3, RTOL, f"tile linear {M}x{N}x{K}")
    assert L.read_device_status() == (0, 0)


def test_linear_prefill_tiles_equal_slab_path(L, monkeypatch):
    """The tile kernel and the 256-row slab path agree (fp32 accumulation in k order on both)."""
    gen = torch.Generator().manual_seed(21)
    buf = randn_bf16(gen, 700, 1536)
    w = randn_bf16(gen, 1000, 1024, std=0.05)
    xs = buf.cuda()[:, 256:1280]                      # row stride 1536, K = 1024
    y_tile = L.linear(xs, w.cuda())
    monkeypatch.setenv("B200_GEMM_TILE_MIN_M", "1000000")
    monkeypatch.setenv("B200_GEMM_SPLIT", "1")
    y_slab = L.linear(xs, w.cuda())
    monkeypatch.delenv("B200_GEMM_TILE_MIN_M")
    monkeypatch.delenv("B200_GEMM_SPLIT")
    assert torch.equal(y_tile, y_slab)


@pytest.mark.parametrize("M,I,K", [(300, 768, 2048), (2048, 3072, 1024), (513, 200, 64)])
def test_gate_up_swiglu_prefill_tiles(L, pkg, M, I, K):
    gen = torch.Generator().manual_seed(M + I)
    x = randn_bf16(gen, M, K)
    w = randn_bf16(gen, 2 * I, K, std=0.05)
    y = L.linear(x.cuda(), w.cuda(), epilogue=pkg.EPILOGUE_SWIGLU)
    assert y.shape == (M, I)
    assert_close_bf16(y, O.silu_and_mul(O.linear(x, w)), 4e-3, 3 * RTOL, "tile gate_up + SwiGLU")
    assert L.read_device_status() == (0, 0)


def test_linear_split_k_variants_agree(L, monkeypatch):
    """Every cluster size gives the same result up to fp32 summation order."""
    import os
    gen = torch.Generator().manual_seed(8)
    x = randn_bf16(gen, 64, 2048)
    w = randn_bf16(gen, 256, 2048, std=0.05)
    want = O.linear(x, w)
    for split in (1, 2, 4, 8):
        monkeypatch.setenv("B200_GEMM_SPLIT", str(split))
        y = L.linear(x.cuda(), w.cuda())
        assert_close_bf16(y, want, 4e-3, RTOL, f"split {split}")
    monkeypatch.delenv("B200_GEMM_SPLIT")
    assert L.read_device_status() == (0, 0)


def test_linear_rejects_bad_shapes(L, pkg):
    x = torch.zeros(4, 100, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(64, 100, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(pkg.B200Error):
        L.linear(x, w)  # K not a multiple of 64
    with pytest.raises(pkg.B200Error):
        L.linear(torch.zeros(4, 128, dtype=torch.bfloat16, device="cuda"), w)  # inner mismatch
