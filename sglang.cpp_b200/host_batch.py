"""Host-side request bookkeeping that feeds the step runner.

The reference keeps this logic in its scheduler (TableManager, CacheManager,
RadixPrefixCache, Req), which stays unchanged behind the drop-in boundary.  This
module restates just enough of it, with the same allocation order, for the tests
and the benchmark to drive the engine the way the scheduler would:

* page-table rows are handed out from the BACK of ``[0, max_running_req)``
  (TableManager::allocate, src/scheduler/prefill.cc:25-30);
* pages are taken from the FRONT of the free list, which starts as
  ``0, page_size, 2*page_size, ...`` (CacheManager ctor and allocate_pages,
  src/scheduler/prefill.cc:55-101);
* a prompt is matched against cached prefixes on ``input_ids[:-1]``, page-aligned
  (CacheManager::match_req, src/scheduler/prefill.cc:69-72), and a finished
  prefill inserts its page-aligned prefix (CacheManager::cache_req, :231-252).
  The prefix index here is a dictionary keyed by page-aligned token prefixes — a
  stand-in for the radix tree that gives the same match lengths when no eviction
  happens (eviction is not modelled).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np


@dataclass
class Req:
    """include/sglang/core/req.h:13-58 (the length state machine of src/core/req.cc:5-53)."""
    input_ids: np.ndarray
    table_idx: int = -1
    cached_len: int = 0
    device_len: int = 0          # tokens whose KV will be in the pool after the current step
    max_device_len: int = 0
    output: list = field(default_factory=list)

    def extend_len(self) -> int:
        return self.device_len - self.cached_len

    def remain_len(self) -> int:
        return self.max_device_len - self.device_len

    def can_decode(self) -> bool:
        return self.remain_len() > 0

    def write_pos(self) -> int:
        """Where the sampled token goes in the token pool (src/scheduler/scheduler.cc:321-325)."""
        return self.device_len if self.can_decode() else -1

    def complete_one(self) -> None:
        """Req::complete_one (src/core/req.cc:47-53)."""
        self.cached_len = self.device_len
        if self.device_len < self.max_device_len:
            self.device_len += 1


class HostBatcher:
    def __init__(self, engine, num_pages: int, page_size: int, max_running_req: int,
                 enable_prefix_cache: bool = True):
        self.engine = engine
        self.page_size = page_size
        self.free_rows = list(range(max_running_req))
        self.free_pages = [i * page_size for i in range(num_pages)]
        self.enable_prefix_cache = enable_prefix_cache
        self.prefix_index: dict[bytes, int] = {}   # key: bytes of the token prefix ending at a page boundary -> page start slot
        self.page_table = np.zeros((max_running_req + 1, 0), dtype=np.int32)  # host mirror, grown lazily
        self._mirror: dict[int, list[int]] = {}   # table row -> slots per position
        self.prefix_hits = 0

    # ---- allocation ---------------------------------------------------------
    def _match_prefix(self, ids: np.ndarray) -> list[int]:
        """Slots of the longest cached page-aligned prefix of ids[:-1]."""
        if not self.enable_prefix_cache:
            return []
        P = self.page_size
        usable = (len(ids) - 1) // P * P
        slots: list[int] = []
        for end in range(P, usable + 1, P):
            start = self.prefix_index.get(ids[:end].tobytes())
            if start is None:
                break
            slots.extend(range(start, start + P))
        return slots

    def add_request(self, input_ids, max_new_tokens: int) -> Req:
        ids = np.ascontiguousarray(np.asarray(input_ids, dtype=np.int32))
        req = Req(ids)
        req.table_idx = self.free_rows.pop()
        req.max_device_len = len(ids) + max_new_tokens
        matched = self._match_prefix(ids)
        req.cached_len = len(matched)
        req.device_len = len(ids)
        self.prefix_hits += len(matched)
        self._mirror[req.table_idx] = list(matched)
        rows = np.full(len(ids), req.table_idx, dtype=np.int32)
        pos = np.arange(len(ids), dtype=np.int32)
        self.engine.write_token_pool(rows, pos, ids)
        if matched:
            self.engine.write_page_table(rows[:len(matched)], pos[:len(matched)], matched)
        return req

    def allocate(self, reqs) -> None:
        """CacheManager::allocate_paged: pages for positions [cached_len, device_len) of each request."""
        P = self.page_size
        rows, pos, slots = [], [], []
        for r in reqs:
            have = len(self._mirror[r.table_idx])
            first, last = -(-have // P), -(-r.device_len // P)
            for page in range(first, last):
                start = self.free_pages.pop(0)
                for i in range(P):
                    rows.append(r.table_idx)
                    pos.append(page * P + i)
                    slots.append(start + i)
                    self._mirror[r.table_idx].append(start + i)
        if rows:
            self.engine.write_page_table(rows, pos, slots)

    def cache_prefix(self, req: Req) -> None:
        """Insert the page-aligned prefix of a request whose prefill finished."""
        if not self.enable_prefix_cache:
            return
        P = self.page_size
        ids, slots = req.input_ids, self._mirror[req.table_idx]
        for end in range(P, min(req.cached_len, len(ids)) // P * P + 1, P):
            self.prefix_index.setdefault(ids[:end].tobytes(), slots[end - P])

    def slots_of(self, req: Req) -> list[int]:
        return self._mirror[req.table_idx]

    # ---- steps --------------------------------------------------------------
    def prefill(self, reqs, chunk_tokens: Optional[int] = None, sampling: Optional[dict] = None):
        """One prefill step over `reqs` (each runs positions [cached_len, device_len)).

        With ``chunk_tokens`` a request whose remaining prompt is longer runs only that many tokens
        this step (the chunked request of src/scheduler/prefill.cc:301-330,382-400): its sampled token is dropped
        (write position -1) and the next call continues where this one stopped.  ``sampling`` holds
        per-request ``temperatures / top_k / top_p / seeds`` (BatchSamplingArgs)."""
        partial = []
        for r in reqs:
            full = len(r.input_ids)
            if r.device_len < full:          # continuing a chunked request
                r.device_len = full
            cut = chunk_tokens is not None and r.extend_len() > chunk_tokens
            if cut:
                r.device_len = r.cached_len + chunk_tokens
            partial.append(cut)
        self.allocate(reqs)
        out = self.engine.forward_batch(
            0, [r.table_idx for r in reqs], [r.cached_len for r in reqs], [r.extend_len() for r in reqs],
            write_pos=[-1 if cut else r.write_pos() for r, cut in zip(reqs, partial)], **(sampling or {}))
        for r, cut in zip(reqs, partial):
            if cut:
                r.cached_len = r.device_len
            else:
                r.complete_one()
        return out

    def decode(self, reqs, padded_size: Optional[int] = None, sampling: Optional[dict] = None):
        """One decode step; pads with the dummy request up to `padded_size`."""
        self.allocate(reqs)
        n = len(reqs)
        bp = max(padded_size or n, n)
        dummy = self.engine.dummy_table_idx
        out = self.engine.forward_batch(
            1, [r.table_idx for r in reqs] + [dummy] * (bp - n),
            [r.cached_len for r in reqs] + [0] * (bp - n), [1] * bp,
            write_pos=[r.write_pos() for r in reqs], num_reqs=n, **(sampling or {}))
        for r in reqs:
            r.complete_one()
        return out


class DecodeSession:
    """A fixed set of running requests stepped many times: what the scheduler's decode loop does
    (src/scheduler/scheduler.cc:391-422, decode.cc:10-27) with the per-step host work kept to a few
    vector operations, as the reference's C++ loop keeps it.  The request lengths live in numpy
    arrays between ``step()`` calls; ``sync_back()`` writes them to the ``Req`` objects again."""

    def __init__(self, batcher: HostBatcher, reqs, padded_size: Optional[int] = None):
        import ctypes

        from ._lib import StepStruct

        self.hb, self.reqs, self.engine = batcher, list(reqs), batcher.engine
        n = len(self.reqs)
        bp = max(padded_size or n, n)
        dummy = self.engine.dummy_table_idx
        self.n = n
        self.table_idx = np.array([r.table_idx for r in self.reqs] + [dummy] * (bp - n), dtype=np.int32)
        self.cached = np.zeros(bp, dtype=np.int32)
        self.extend = np.ones(bp, dtype=np.int32)
        self.write_pos = np.full(max(n, 1), -1, dtype=np.int32)
        self.device_len = np.array([r.device_len for r in self.reqs], dtype=np.int64)
        self.max_len = np.array([r.max_device_len for r in self.reqs], dtype=np.int64)
        self.cached[:n] = [r.cached_len for r in self.reqs]
        self.pages_have = np.array([-(-len(batcher.slots_of(r)) // batcher.page_size) for r in self.reqs], dtype=np.int64)
        self._st = StepStruct(1, n, bp, self.table_idx.ctypes.data, self.cached.ctypes.data, self.extend.ctypes.data,
                              self.write_pos.ctypes.data, None, None, None, None, 0)
        self._st_ref = ctypes.byref(self._st)

    def step(self):
        """One decode step of every request (asynchronous, like Engine.forward_batch)."""
        from ._lib import call

        hb, P = self.hb, self.hb.page_size
        # pages for the position this step writes (CacheManager::allocate_paged): rare, so per request
        need = np.nonzero(-(-self.device_len // P) > self.pages_have)[0]
        for i in need:
            r = self.reqs[int(i)]
            r.device_len = int(self.device_len[i])
            hb.allocate([r])
            self.pages_have[i] = -(-len(hb.slots_of(r)) // P)
        can = self.device_len < self.max_len
        self.write_pos[:self.n] = np.where(can, self.device_len, -1)
        eng = self.engine
        self._st.step_index = eng._step_index
        eng._step_index += 1
        call("b200_engine_step", eng._h, self._st_ref, eng._next_tokens_cpu.data_ptr())
        # Req::complete_one for every request
        self.cached[:self.n] = self.device_len
        self.device_len += can
        return eng._next_tokens_cpu[:self.n]

    def sync_back(self) -> None:
        for i, r in enumerate(self.reqs):
            r.cached_len, r.device_len = int(self.cached[i]), int(self.device_len[i])
