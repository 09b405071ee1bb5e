"""The MoE kernels against the oracle (which is pinned to the reference's own MoELayer, see
tests/golden/moe_ref_fp32.json) and routing against torch.topk.

Tolerance: the oracle here reproduces the reference's bf16 rounding points (store_bf16); the CUDA
path rounds at the same points, so results differ by summation order inside the GEMMs only: one
bf16 step per stage, a few steps after the k-fold accumulation.
"""
import pytest
import torch

from oracle import token_loop_oracle as O
from tests.parity_cases import assert_close_bf16, randn_bf16

pytestmark = pytest.mark.gpu
bf16 = torch.bfloat16


def distinct_router_logits(gen, T, E):
    """Rows without ties (each a permutation of E distinct bf16-exact values in [-4, 4)): with equal
    probabilities at the k-th place torch.topk and any other top-k may pick different experts."""
    grid = (torch.arange(E, dtype=torch.float32) - E / 2) * (8.0 / E if E >= 8 else 1.0)
    assert torch.equal(grid.to(bf16).float(), grid) and grid.unique().numel() == E
    return torch.stack([grid[torch.randperm(E, generator=gen)] for _ in range(T)]).to(bf16)


@pytest.mark.parametrize("T,E,k,renorm", [(6, 3, 2, True), (256, 128, 8, True), (33, 16, 1, False), (64, 64, 4, True)])
def test_route_matches_torch_topk(L, T, E, k, renorm):
    gen = torch.Generator().manual_seed(T + E)
    logits = distinct_router_logits(gen, T, E)
    ids, w, counts = L.moe_route(logits.cuda(), k, renorm)
    probs = torch.softmax(logits.float(), -1)
    tw, ti = probs.topk(k, -1)
    if renorm:
        tw = tw / (tw.sum(-1, keepdim=True) + 1e-8)
    assert torch.equal(ids.cpu().long(), ti)          # bit-exact experts, in the same order
    assert_close_bf16(w.cpu(), tw.to(bf16).float(), 1e-6, 2 ** -7, "routing weights")
    assert torch.equal(counts.cpu().long(), torch.bincount(ti.flatten(), minlength=E))


@pytest.mark.parametrize("T,E,k,H,I,renorm,act", [
    (6, 3, 2, 64, 64, True, "silu"),            # the reference test's routing shape
    (64, 16, 4, 256, 128, True, "silu"),
    (256, 128, 8, 2048, 768, True, "silu"),     # Qwen3-30B-A3B decode step at batch 256
    (40, 8, 2, 128, 192, False, "gelu"),
    (300, 4, 2, 128, 64, True, "silu"),         # 150 rows per expert: the tile kernel's grouped mode
    (2048, 16, 4, 256, 128, True, "silu"),      # a prefill batch: ~512 rows per expert, ragged
    (1500, 6, 3, 128, 192, False, "gelu"),      # tile kernel, exact-GELU epilogue, k-loop of 3
    (1, 8, 8, 64, 64, True, "silu"),
])
def test_moe_forward_matches_oracle(L, T, E, k, H, I, renorm, act):
    gen = torch.Generator().manual_seed(T * 7 + E)
    hidden = randn_bf16(gen, T, H)
    logits = distinct_router_logits(gen, T, E)
    moe = L.MoELayer(E, k, H, I, renorm, act)
    gu = randn_bf16(gen, E, 2 * I, H, std=H ** -0.5)
    dn = randn_bf16(gen, E, H, I, std=I ** -0.5)
    moe.gate_up_proj.copy_(gu.cuda())
    moe.down_proj.copy_(dn.cuda())
    got = moe.forward(hidden.cuda(), logits.cuda())
    want = O.moe_forward(hidden, logits, gu, dn, k, renorm, act, O.store_bf16)
    assert_close_bf16(got, want, 2e-2, 4 * 2 ** -7, f"moe forward {T}x{E} top{k}")
    assert L.read_device_status() == (0, 0)


@pytest.mark.parametrize("T,E,k,H,I,parts", [(64, 16, 4, 256, 128, 4), (256, 128, 8, 2048, 768, 8), (5, 8, 2, 64, 64, 2),
                                             (900, 8, 2, 128, 64, 2)])   # tile kernel on a rank's experts
def test_moe_expert_partition_matches_oracle_share(L, T, E, k, H, I, parts):
    """Expert parallelism: a rank holding experts [b, b + E/parts) returns exactly the oracle's
    share for that range, rows whose experts all live elsewhere come back zero, and the shares
    add up (in fp32) to the whole layer within the rounding of the partial sums."""
    gen = torch.Generator().manual_seed(T + E + parts)
    hidden = randn_bf16(gen, T, H)
    logits = distinct_router_logits(gen, T, E)
    gu = randn_bf16(gen, E, 2 * I, H, std=H ** -0.5)
    dn = randn_bf16(gen, E, H, I, std=I ** -0.5)
    el = E // parts
    total = torch.zeros(T, H)
    for r in range(parts):
        moe = L.MoELayer(E, k, H, I, True, "silu", expert_begin=r * el, num_local_experts=el)
        moe.gate_up_proj.copy_(gu[r * el:(r + 1) * el].cuda())
        moe.down_proj.copy_(dn[r * el:(r + 1) * el].cuda())
        got = moe.forward(hidden.cuda(), logits.cuda())
        want = O.moe_forward(hidden, logits, gu[r * el:(r + 1) * el], dn[r * el:(r + 1) * el], k, True, "silu",
                             O.store_bf16, expert_begin=r * el)
        assert_close_bf16(got, want, 2e-2, 4 * 2 ** -7, f"moe share of rank {r}/{parts}")
        ids = torch.softmax(logits.float(), -1).topk(k, -1).indices
        nothing_here = ~((ids >= r * el) & (ids < (r + 1) * el)).any(-1)
        assert torch.all(got.cpu()[nothing_here] == 0)
        total += got.float().cpu()
    whole = O.moe_forward(hidden, logits, gu, dn, k, True, "silu", O.store_bf16)
    assert_close_bf16(total, whole, 3e-2, 8 * 2 ** -7, "sum of the shares")
    assert L.read_device_status() == (0, 0)


def test_moe_rejects_bad_arguments(L, pkg):
    with pytest.raises(pkg.B200Error):
        L.MoELayer(4, 5, 64, 64)            # top_k > num_experts
    moe = L.MoELayer(4, 2, 64, 64)
    with pytest.raises(pkg.B200Error):
        moe.forward(torch.zeros(3, 32, dtype=bf16, device="cuda"), torch.zeros(3, 4, dtype=bf16, device="cuda"))
    with pytest.raises(pkg.B200Error):
        moe.forward(torch.zeros(3, 64, dtype=bf16, device="cuda"), torch.zeros(2, 4, dtype=bf16, device="cuda"))
