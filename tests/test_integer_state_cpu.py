"""The integer side of the path — table rows, KV slots, prefix-match lengths, request lengths —
against the reference's own objects.

Two checkers: (a) the reference's TableManager / CacheManager / RadixPrefixCache / PrefillManager /
DecodeManager / Req compiled from the reference tree into oracle/_ref (skipped where that library
was not built), and (b) the known answers the reference's own unit tests hold
(tests/kvcache/test_cache_manager.cpp:13-146, tests/kvcache/test_radix_tree.cpp:73-135,
tests/core/test_req.cpp:7-78, tests/scheduler/test_managers.cpp:21-68, tests/kernels/test_radix.cpp:7-48),
replayed on both the compiled reference and the restatement in sglang_cpp_b200.host_batch.
Everything here is bit-exact.
"""
import json
from pathlib import Path

import numpy as np
import pytest

import __graft_entry__ as entry
from oracle import ref_sched

entry.load_package()
from sglang_cpp_b200 import host_batch as HB  # noqa: E402

GOLDEN = Path(__file__).parent / "golden" / "integer_state_trace.json"
needs_ref = pytest.mark.skipif(not ref_sched.available(), reason="oracle/_ref was not built (no reference tree)")
IMPLS = [pytest.param("reference", marks=needs_ref), "restated"]


class PyRadix:
    """RadixPrefixCache of host_batch behind the handle-id interface of oracle.ref_sched.RefRadixCache."""

    def __init__(self, page_size):
        self.c = HB.RadixPrefixCache(page_size)
        self.handles = []

    def insert_prefix(self, ids, indices):
        had, h = self.c.insert_prefix(ids, indices)
        self.handles.append(h)
        return had, h.cached_len, len(self.handles) - 1

    def match_prefix(self, ids):
        h = self.c.match_prefix(ids)
        self.handles.append(h)
        return h.cached_len, h.matched_indices(), len(self.handles) - 1

    def lock_handle(self, hid, unlock=False):
        self.c.lock_handle(self.handles[hid], unlock)

    def evict(self, size):
        return self.c.evict(size)

    def size_info(self):
        return self.c.evictable_size, self.c.protected_size


def radix(impl, page_size=1):
    return ref_sched.RefRadixCache(page_size) if impl == "reference" else PyRadix(page_size)


ERRORS = (ref_sched.RefError, ValueError)


# ---- known answers of tests/kvcache/test_cache_manager.cpp --------------------------------------
@pytest.mark.parametrize("impl", IMPLS)
def test_radix_cache_known_answers(impl):
    c = radix(impl)
    n, idx, _ = c.match_prefix([1, 2, 3])                         # EmptyMatchPrefix
    assert n == 0 and len(idx) == 0
    had, hlen, _ = c.insert_prefix([10, 20, 30, 40], [0, 1, 2, 3])  # InsertAndMatch
    assert (had, hlen) == (0, 4)
    n, idx, _ = c.match_prefix([10, 20, 30, 40])
    assert n == 4 and idx.tolist() == [0, 1, 2, 3]

    c = radix(impl)                                               # PartialMatch
    c.insert_prefix([1, 2, 3, 4, 5], [10, 20, 30, 40, 50])
    n, idx, _ = c.match_prefix([1, 2, 3, 9, 9])
    assert n == 3 and idx.tolist() == [10, 20, 30]

    c = radix(impl)                                               # SizeInfoAfterInsert, LockAndUnlock
    assert c.size_info() == (0, 0)
    _, _, h = c.insert_prefix([1, 2, 3], [0, 1, 2])
    assert c.size_info() == (3, 0)
    c.lock_handle(h)
    assert c.size_info() == (0, 3)
    with pytest.raises(ERRORS):                                   # EvictProtectedFails
        c.evict(1)
    c.lock_handle(h, unlock=True)
    assert c.size_info() == (3, 0)
    assert len(c.evict(0)) == 0                                   # EvictZero
    ev = c.evict(2)                                               # EvictBasic: the whole leaf goes
    assert sorted(ev.tolist()) == [0, 1, 2] and c.size_info() == (0, 0)

    c = radix(impl)                                               # InsertMatchEvictCycle
    c.insert_prefix([1, 2, 3], [10, 11, 12])
    c.insert_prefix([4, 5, 6], [20, 21, 22])
    assert c.size_info()[0] == 6
    ev = c.evict(3)
    assert ev.tolist() == [10, 11, 12]                            # least recently used first
    assert c.size_info()[0] == 3
    assert c.match_prefix([1, 2, 3])[0] == 0 and c.match_prefix([4, 5, 6])[0] == 3

    c = radix(impl)                                               # DuplicateInsert
    c.insert_prefix([1, 2, 3], [0, 1, 2])
    had, hlen, _ = c.insert_prefix([1, 2, 3], [7, 8, 9])
    assert (had, hlen) == (3, 3) and c.size_info() == (3, 0)
    assert c.match_prefix([1, 2, 3])[1].tolist() == [0, 1, 2]


# ---- known answers of tests/kvcache/test_radix_tree.cpp and tests/kernels/test_radix.cpp -------------
@pytest.mark.parametrize("impl", IMPLS)
def test_split_key_fn_and_compare_known_answers(impl):
    if impl == "reference":
        pk, pv, sk, sv, rc, ok = ref_sched.node_split([1, 2, 3, 4], [10, 20, 30, 40], 2, 2)
        key_fn, cmp = ref_sched.key_fn, ref_sched.fast_compare_key
    else:
        root = HB.RadixNode(1, 1)
        root.ref_count = 1
        child = HB.RadixNode(1, 2)
        child.set_key_value(np.array([1, 2, 3, 4], np.int32), np.array([10, 20, 30, 40], np.int32))
        child.set_parent(root)
        child.ref_count = 2
        head = child.split_at(2)
        pk, pv, sk, sv, rc = head.key, head.value, child.key, child.value, head.ref_count
        ok = head.parent is root and child.parent is head and not head.is_leaf()
        key_fn = lambda ps, ids: HB.page_key(np.asarray(ids, np.int32), ps)  # noqa: E731
        cmp = lambda a, b: HB.compare_key(np.asarray(a, np.int32), np.asarray(b, np.int32))  # noqa: E731
    assert (list(pk), list(pv), list(sk), list(sv), rc, ok) == ([1, 2], [10, 20], [3, 4], [30, 40], 2, True)
    assert key_fn(1, [42, 99, 7]) == 42                             # KeyFnTest.PageSizeOne
    assert key_fn(2, [1, 2, 3]) == key_fn(2, [1, 2, 9]) != key_fn(2, [1, 3, 3])
    assert cmp([1, 2, 3, 4, 5], [1, 2, 3, 4, 5]) == 5               # FastCompareKeyTest.*
    assert cmp([1, 2, 3], [9, 8, 7]) == 0
    assert cmp([1, 2, 3, 4, 5], [1, 2, 3, 9, 9]) == 3
    assert cmp([], []) == 0
    assert cmp([1, 2, 3, 4, 5], [1, 2, 3]) == 3
    assert cmp([1, 2, 9], [1, 2, 3, 4, 5]) == 2
    assert cmp([42], [42]) == 1 and cmp([42], [99]) == 0


@needs_ref
def test_page_hash_is_the_reference_hash():
    rng = np.random.default_rng(0)
    for ps in (2, 4, 16, 64):
        for _ in range(50):
            ids = rng.integers(0, 151936, size=int(rng.integers(1, 2 * ps))).astype(np.int32)
            assert HB.page_key(ids, ps) == ref_sched.key_fn(ps, ids)


# ---- known answers of tests/core/test_req.cpp ---------------------------------------------------------
class PyReq:
    def __init__(self, ids, cached_len=0, output_len=0, chunked=False, initialize=False):
        ids = np.asarray(ids, np.int32)
        self.r = HB.Req(ids, -1, cached_len, len(ids), len(ids) + output_len, 0, chunked)

    def state(self):
        r = self.r
        return {"device_len": r.device_len, "max_device_len": r.max_device_len, "remain_len": r.remain_len(),
                "extend_len": r.extend_len(), "can_decode": int(r.can_decode()), "cached_len": r.cached_len,
                "host_len": len(r.input_ids)}

    def complete_one(self):
        self.r.complete_one()

    def append_host(self, tok):
        self.r.append_host_token(tok)


@pytest.mark.parametrize("impl", IMPLS)
def test_req_known_answers(impl):
    Req = ref_sched.RefReq if impl == "reference" else PyReq
    s = Req([1, 2, 3, 4, 5], 0, 3).state()                           # BasicProperties
    assert (s["device_len"], s["max_device_len"], s["remain_len"], s["extend_len"], s["can_decode"]) == (5, 8, 3, 5, 1)
    r = Req([1, 2, 3], 0, 2, initialize=True)                        # CompleteOneAdvancesDeviceBeforeHostAppend
    r.complete_one()
    s = r.state()
    assert (s["cached_len"], s["device_len"], s["remain_len"]) == (3, 4, 1)
    r.append_host(10)
    s = r.state()
    assert (s["device_len"], s["cached_len"], s["remain_len"], s["extend_len"], s["can_decode"]) == (4, 3, 1, 1, 1)
    r = Req([1], 0, 1, initialize=True)                              # CanDecodeReturnsFalseWhenDone
    r.complete_one()
    r.append_host(2)
    assert r.state()["can_decode"] == 0
    r = Req([1, 2, 3], 0, 1, initialize=True)                        # AppendHostRequiresAdvancedDeviceLen
    with pytest.raises(ERRORS):
        r.append_host(4)
    r.complete_one()
    r.append_host(4)
    assert r.state()["host_len"] == 4
    assert Req([1, 2, 3], 1, 4, chunked=True, initialize=True).state()["can_decode"] == 0   # ChunkedPrefillNeverDecodes


# ---- whole-scheduler traces -------------------------------------------------------------------------
def scheduler(impl, **kw):
    if impl == "reference":
        return ref_sched.RefScheduler(kw["num_pages"], kw["page_size"], kw["max_running_req"], kw["max_seq_len"],
                                      kw["max_extend_tokens"])
    return HB.HostScheduler(None, kw["num_pages"], kw["page_size"], kw["max_running_req"], kw["max_seq_len"],
                            kw["max_extend_tokens"])


def next_batch(impl, s):
    if impl == "reference":
        return s.next_batch()
    b = s.next_batch()
    if b is None:
        return None
    s._cur = b
    r = b.reqs
    return {"phase": b.phase, "uid": np.array([q.uid for q in r], np.uint64),
            "table_idx": np.array([q.table_idx for q in r], np.int32),
            "cached_len": np.array([q.cached_len for q in r], np.int32),
            "device_len": np.array([q.device_len for q in r], np.int32),
            "chunked": np.array([int(q.is_chunked_prefill) for q in r], np.int32),
            "write_pos": np.array([q.write_pos() for q in r], np.int32)}


def finish(impl, s, toks):
    return s.finish_batch(toks) if impl == "reference" else s.finish_batch(s._cur, toks)


def tables(impl, s):
    if impl == "reference":
        return s.page_table(), s.token_pool()
    return s.tables.page_table, s.tables.token_pool


def sizes(impl, s):
    if impl == "reference":
        return s.sizes()
    cm = s.cache_manager
    if not s.running and not s.pending:
        cm.check_integrity()
    return {"evictable": cm.prefix_cache.evictable_size, "protected": cm.prefix_cache.protected_size,
            "available": cm.available_size(), "free_rows": s.table_manager.available_size(),
            "inflight": s.inflight_tokens(), "pending": len(s.pending)}


def token_for(uid, device_len):
    """The stand-in for the forward pass: any function of the request's state, the same for both sides."""
    return int((uid * 7919 + device_len * 104729) % 151936)


def run_trace(impl, prompts, max_new, waves, **kw):
    """Submits `prompts` in `waves` groups (the next group once the scheduler went idle) and returns a
    list of per-step records: everything the step runner is handed, plus the tables and sizes."""
    s = scheduler(impl, **kw)
    trace, uid = [], 0
    per = -(-len(prompts) // waves)
    for w in range(waves):
        for p in prompts[w * per:(w + 1) * per]:
            uid += 1
            s.submit(uid, p, max_new[uid - 1])
        for _ in range(100000):
            b = next_batch(impl, s)
            if b is None:
                break
            toks = [token_for(int(u), int(d)) for u, d in zip(b["uid"], b["device_len"])]
            fin = finish(impl, s, toks)
            pt, tp = tables(impl, s)
            trace.append({**{k: np.asarray(v).tolist() for k, v in b.items()}, "finished": [bool(f) for f in fin],
                          "page_table_sum": int(pt.astype(np.int64).sum()), "page_table": pt.copy(),
                          "token_pool": tp.copy(), "sizes": sizes(impl, s)})
        else:
            raise AssertionError("the scheduler never went idle")
    return trace


def compare(tr_a, tr_b):
    assert len(tr_a) == len(tr_b)
    for i, (a, b) in enumerate(zip(tr_a, tr_b)):
        for k in ("phase", "uid", "table_idx", "cached_len", "device_len", "chunked", "write_pos", "finished", "sizes"):
            assert a[k] == b[k], (i, k, a[k], b[k])
        assert np.array_equal(a["page_table"], b["page_table"]), f"step {i}: page tables differ"
        assert np.array_equal(a["token_pool"], b["token_pool"]), f"step {i}: token pools differ"


def config2_prompts(vocab=151936, batch=64, lo=512, hi=2048, shared=256, seed=2):
    rng = np.random.default_rng(seed)
    lens = rng.integers(lo, hi + 1, size=batch)
    out = []
    for b in range(batch):
        if b % 4 == 0:
            head = rng.integers(0, vocab, size=shared)
        out.append(np.concatenate([head, rng.integers(0, vocab, size=int(lens[b]) - shared)]).astype(np.int32))
    return out


@needs_ref
@pytest.mark.parametrize("page_size", [16, 1])
def test_config2_batch_rows_slots_and_prefix_lengths_equal_the_reference(page_size):
    """BASELINE config 2's 64 prompts (256-token prefix shared per group of 4), prefilled in
    8192-token batches and decoded for a few steps."""
    prompts = config2_prompts()
    pages = sum(-(-(len(p) + 8) // page_size) for p in prompts) + 8
    kw = dict(num_pages=pages, page_size=page_size, max_running_req=64, max_seq_len=2048 + 16, max_extend_tokens=8192)
    a = run_trace("reference", prompts, [6] * 64, 1, **kw)
    b = run_trace("restated", prompts, [6] * 64, 1, **kw)
    compare(a, b)
    assert any(sum(x["cached_len"]) > 0 for x in a if x["phase"] == 0), "no prefix hit in the whole run"
    assert sum(1 for x in a if x["phase"] == 1) >= 5


def small_prompts(rng, n, vocab=50):
    """Short prompts over a tiny vocabulary with shared heads of random length: splits, partial
    matches and re-use of finished requests' prefixes all happen."""
    heads = [rng.integers(0, vocab, size=int(rng.integers(2, 24))) for _ in range(4)]
    out = []
    for _ in range(n):
        h = heads[int(rng.integers(0, 4))]
        cut = int(rng.integers(1, len(h) + 1))
        out.append(np.concatenate([h[:cut], rng.integers(0, vocab, size=int(rng.integers(1, 20)))]).astype(np.int32))
    return out


SMALL_CASES = [
    # page size, pages, rows, extend budget, waves, seed
    (1, 400, 4, 64, 3, 0),      # rows recycle, requests finish and are matched later
    (1, 120, 6, 16, 4, 1),      # tight pool: eviction; small budget: chunked prefill
    (4, 60, 5, 24, 4, 2),       # page size 4: aligned matches, partially filled last pages
    (16, 24, 3, 40, 5, 3),
    (2, 90, 8, 7, 2, 4),
]


@needs_ref
@pytest.mark.parametrize("page_size,pages,rows,budget,waves,seed", SMALL_CASES)
def test_scheduler_traces_equal_the_reference(page_size, pages, rows, budget, waves, seed):
    rng = np.random.default_rng(seed)
    prompts = small_prompts(rng, 40)
    max_new = rng.integers(1, 9, size=len(prompts)).tolist()
    kw = dict(num_pages=pages, page_size=page_size, max_running_req=rows, max_seq_len=96, max_extend_tokens=budget)
    a = run_trace("reference", prompts, max_new, waves, **kw)
    b = run_trace("restated", prompts, max_new, waves, **kw)
    compare(a, b)
    assert any(any(x["chunked"]) for x in a) or budget > 30
    assert any(sum(x["cached_len"]) > 0 for x in a if x["phase"] == 0)


def _golden_record(trace):
    return [{k: v for k, v in step.items() if k not in ("page_table", "token_pool")} for step in trace]


def test_restated_scheduler_matches_the_committed_reference_trace():
    """The fixture was written by the compiled reference (tests/golden/make_integer_golden.py); it
    stands in where the reference tree is absent."""
    g = json.loads(GOLDEN.read_text())
    for case in g["cases"]:
        rng = np.random.default_rng(case["seed"])
        prompts = small_prompts(rng, 40)
        max_new = rng.integers(1, 9, size=len(prompts)).tolist()
        tr = run_trace("restated", prompts, max_new, case["waves"], **case["kw"])
        assert json.loads(json.dumps(_golden_record(tr))) == case["trace"]


def test_managers_known_answers():
    """tests/scheduler/test_managers.cpp:21-68 on the restatement."""
    tm = HB.TableManager(2)
    a, b = tm.allocate(), tm.allocate()
    assert a != b and tm.available_size() == 0
    tm.free(a)
    assert tm.available_size() == 1
    s = HB.HostScheduler(None, 32, 1, 3, 16, 2)                      # ChunksRequestWhenBudgetIsTooSmall
    s.submit(7, [10, 11, 12, 13], 3)
    batch = s.next_batch()
    assert len(batch.reqs) == 1 and batch.reqs[0].is_chunked_prefill and len(batch.reqs[0].input_ids) == 2
    assert len(s.pending) == 1
    live = HB.Req(np.arange(4, dtype=np.int32), 0, 4, 4, 6, 1)       # FiltersOnlyDecodableReqs
    done = HB.Req(np.arange(4, dtype=np.int32), 1, 4, 4, 4, 2)
    s2 = HB.HostScheduler(None, 32, 1, 3, 16, 8)
    s2.running = [r for r in (live, done) if r.can_decode()]
    assert [r.uid for r in s2.running] == [1] and s2.inflight_tokens() == 2
