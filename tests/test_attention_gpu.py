"""Parity of the paged-KV attention kernels against the CPU oracle (through the C ABI).

Tolerance: the kernels keep scores and accumulators in fp32 but, like every tensor-core flash
kernel (FlashInfer's prefill included), round the probabilities to bf16 before P.V and the output
to bf16.  Against the exact-arithmetic oracle on N(0,1) inputs that is at most a few 1e-3 absolute;
2e-2 is the bound the logits tolerance of the whole model is stated in.
"""
import numpy as np
import pytest
import torch

from tests.parity_cases import assert_close_bf16, decode_attention_case, prefill_attention_case

pytestmark = pytest.mark.gpu
ATOL, RTOL = 2e-2, 2e-2


@pytest.mark.parametrize("seq_lens,page_size,hq,hkv", [
    ([1], 16, 16, 8),                               # a single key (the padded dummy request)
    ([5, 37, 130, 16, 17, 1], 16, 16, 8),           # ragged, partial last pages
    ([200, 3, 64, 1000], 1, 16, 8),                 # page size 1, as the reference Engine runs
    ([33, 512, 77], 16, 32, 8),                     # Llama GQA group 4
    ([65, 129, 700], 16, 32, 4),                    # Qwen3-MoE group 8, two key groups per stage
    ([40, 900, 130], 16, 4, 1),                     # one KV head per rank (TP=8): eight key groups
    ([257, 31], 4, 8, 2),                           # pages smaller than a stage
    ([90, 45], 1, 4, 1),                            # page size 1 with a single KV head
    ([300, 20], 64, 16, 8),                         # pages larger than a stage
])
def test_decode_matches_oracle(L, seq_lens, page_size, hq, hkv):
    got, want, _ = decode_attention_case(L, seq_lens, page_size, hq, hkv, seed=len(seq_lens) + page_size)
    assert_close_bf16(got, want, ATOL, RTOL, "decode attention")
    assert L.read_device_status() == (0, 0)


def test_decode_config2_shape(L):
    """Batch 64, contexts uniform in [512, 2304) (the decode-throughput workload): every request is
    cut over two to four CTAs, so every output comes from the merge kernel."""
    rng = np.random.default_rng(2)
    seq_lens = rng.integers(512, 2304, size=64).tolist()
    got, want, attn = decode_attention_case(L, seq_lens, 16, 16, 8, seed=11)
    assert_close_bf16(got, want, ATOL, RTOL, "decode attention, batch 64")
    assert L.read_device_status() == (0, 0)


def test_decode_ignores_unowned_slots(L):
    """NaN in every slot that no request owns (including the tail of partially filled pages)."""
    got, want, _ = decode_attention_case(L, [5, 37, 130, 200], 16, 16, 8, seed=4, poison_unused=True)
    assert not bool(torch.isnan(got.float()).any())
    assert_close_bf16(got, want, ATOL, RTOL, "decode attention with poisoned pool")


def test_decode_empty_batch_and_bad_args(L, pkg):
    cache = L.MHAKVCache(8, 1, 128, 4, 16)
    attn = L.PagedAttention(cache, 16, 8, 128, max_batch=4)
    q = torch.zeros(0, 16, 128, dtype=torch.bfloat16, device="cuda")
    z = torch.zeros(0, dtype=torch.int32, device="cuda")
    pt = torch.zeros(2, 32, dtype=torch.int32, device="cuda")
    assert attn.decode(q, 0, pt, z, z).shape == (0, 2048)
    with pytest.raises(pkg.B200Error):
        L.PagedAttention(cache, 16, 3, 128)  # kv_heads must divide 8


@pytest.mark.parametrize("seq_lens,extend_lens,page_size,hq,hkv", [
    ([7], [7], 16, 16, 8),                                   # one short prompt, no prefix
    ([100, 64, 1], [100, 64, 1], 16, 16, 8),                 # full prefill, ragged
    ([300, 200], [44, 200], 16, 16, 8),                      # cached prefix + extension
    ([513, 70], [129, 3], 1, 16, 8),                         # page size 1
    ([260, 90], [100, 90], 16, 32, 8),                       # group 4
    ([150], [150], 16, 32, 4),                               # group 8
    ([190, 65], [64, 65], 16, 4, 1),                         # one KV head per rank
    ([130], [130], 4, 8, 2),
    ([2048, 1500], [2048, 1500], 16, 16, 8),                 # prompts of the decode benchmark's size
])
def test_prefill_matches_oracle(L, seq_lens, extend_lens, page_size, hq, hkv):
    got, want = prefill_attention_case(L, seq_lens, extend_lens, page_size, hq, hkv, seed=sum(seq_lens))
    assert_close_bf16(got, want, ATOL, RTOL, "prefill attention")
    assert L.read_device_status() == (0, 0)


@pytest.mark.parametrize("seq_lens,extend_lens,page_size", [
    ([700, 300], [700, 300], 16), ([513], [200], 4), ([260, 130], [260, 2], 1)])
def test_prefill_with_consecutive_pages(L, seq_lens, extend_lens, page_size):
    """Pages in consecutive slots take the whole-tile copies; the ragged last tile and the other
    requests still go page by page."""
    got, want = prefill_attention_case(L, seq_lens, extend_lens, page_size, 16, 8, seed=5, shuffle_pages=False)
    assert_close_bf16(got, want, ATOL, RTOL, "prefill attention, consecutive pages")
    assert L.read_device_status() == (0, 0)


def test_prefill_equals_decode_on_last_row(L):
    """The last query row of a prefill sees every key, as a decode step does: the same pool, page
    table and query row through both kernels, each against the oracle and against one another."""
    import math

    from tests.parity_cases import PagedSetup, randn_bf16
    from oracle import token_loop_oracle as O

    n, hq, hkv, d, page = 333, 16, 8, 128, 16
    ps = PagedSetup([n], page, hkv, d, seed=9)
    q = randn_bf16(torch.Generator().manual_seed(10), n, hq, d)
    cache = L.MHAKVCache(hkv, 1, d, ps.num_slots // page, page, device="cuda")
    cache.kv_buffer_[0, 0].copy_(ps.k_cache.cuda())
    cache.kv_buffer_[1, 0].copy_(ps.v_cache.cuda())
    attn = L.PagedAttention(cache, hq, hkv, d, max_batch=1)
    pt, ti, sl = (torch.from_numpy(a).cuda() for a in (ps.page_table, ps.table_idx, ps.seq_lens))
    qo = torch.tensor([0, n], dtype=torch.int32, device="cuda")
    got_p = attn.prefill(q.cuda(), 0, pt, ti, sl, qo, n)[-1:].clone()
    got_d = attn.decode(q[-1:].cuda(), 0, pt, ti, sl)
    torch.cuda.synchronize()
    want = O.paged_attention(q[-1:], ps.k_cache, ps.v_cache, ps.page_table, ps.table_idx, ps.seq_lens,
                             np.arange(2), 1.0 / math.sqrt(d), O.store_fp32).reshape(1, hq * d)
    assert_close_bf16(got_d, want, ATOL, RTOL, "decode")
    assert_close_bf16(got_p, want, ATOL, RTOL, "last prefill row")
    # the two kernels round the probabilities at different points: a few bf16 steps apart at most
    assert_close_bf16(got_p, got_d, 8e-3, 2e-2, "last prefill row against the decode step")
