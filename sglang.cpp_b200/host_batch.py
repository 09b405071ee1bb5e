"""Host-side request bookkeeping that feeds the step runner.

The reference keeps this logic in its scheduler (TableManager, CacheManager, RadixPrefixCache,
PrefillManager, DecodeManager, Req), which stays unchanged behind the drop-in boundary.  This
module restates its integer side — which table row, which KV slots, how long a cached prefix —
so the tests and the benchmark can drive the engine the way the scheduler would, and the parity
tests compare every page-table row, slot and prefix-match length it produces, bit for bit, with
the reference's own objects compiled from the reference tree:

* page-table rows are handed out from the BACK of ``[0, max_running_req)``
  (TableManager::allocate, src/scheduler/prefill.cc:25-30);
* pages are taken from the FRONT of the free list, which starts as ``0, page_size, ...``; freed
  pages go to its BACK (CacheManager ctor, allocate_pages, free_indices,
  src/scheduler/prefill.cc:55-101,200-222);
* a prompt is matched against the radix tree on ``input_ids[:-1]``, page-aligned
  (CacheManager::match_req :69-72; RadixPrefixCache::tree_walk, src/kvcache/cache_manager.cc:171-211),
  matched nodes are locked while a request uses them and a request's prefix is inserted when its
  prefill ends and again when it finishes (CacheManager::cache_req :231-252);
* eviction takes unlocked leaves, least recently used first (cache_manager.cc:110-158).  The
  reference stamps nodes with steady_clock readings; here a counter that advances at every point
  where the reference reads the clock gives the same order.
"""
from __future__ import annotations

import heapq
from dataclasses import dataclass, field
from typing import Optional

import numpy as np

_MASK64 = (1 << 64) - 1


def _to_signed64(v: int) -> int:
    v &= _MASK64
    return v - (1 << 64) if v >> 63 else v


def page_key(ids: np.ndarray, page_size: int) -> int:
    """get_key_fn (src/kvcache/radix_tree.cc:16-35): the first id, or a hash of the first page."""
    if page_size == 1:
        return int(ids[0])
    h = 0
    for v in ids[:page_size]:
        h ^= _to_signed64(int(v) + 0x9E3779B9 + _to_signed64(h << 6) + (h >> 2))
    return h


def compare_key(a: np.ndarray, b: np.ndarray) -> int:
    """fast_compare_key (src/kernels/radix.cc:5-25): length of the common prefix."""
    n = min(len(a), len(b))
    if n == 0:
        return 0
    diff = np.nonzero(a[:n] != b[:n])[0]
    return int(diff[0]) if len(diff) else n


class _Clock:
    def __init__(self):
        self.t = 0

    def now(self) -> int:
        self.t += 1
        return self.t


class RadixNode:
    """RadixTreeNode (include/sglang/kvcache/radix_tree.h; src/kvcache/radix_tree.cc:41-82)."""

    def __init__(self, page_size: int, timestamp: int):
        self.page_size = page_size
        self.key = np.zeros(0, dtype=np.int32)
        self.value = np.zeros(0, dtype=np.int32)
        self.parent: Optional["RadixNode"] = None
        self.children: dict[int, "RadixNode"] = {}
        self.ref_count = 0
        self.timestamp = timestamp

    def __len__(self) -> int:
        return len(self.key)

    def is_root(self) -> bool:
        return self.parent is None

    def is_leaf(self) -> bool:
        return not self.children

    def set_key_value(self, key, value) -> None:
        if len(key) != len(value):
            raise ValueError("set_key_value: key and value must have the same length")
        self.key, self.value = key, value

    def set_parent(self, parent: "RadixNode") -> None:
        self.parent = parent
        parent.children[page_key(self.key, self.page_size)] = self

    def split_at(self, pos: int) -> "RadixNode":
        if not 0 < pos < len(self.key):
            raise ValueError("split_at: pos must be in range (0, length)")
        if self.parent is None:
            raise ValueError("split_at: cannot split root node")
        head = RadixNode(self.page_size, self.timestamp)
        head.set_key_value(self.key[:pos], self.value[:pos])
        head.set_parent(self.parent)
        head.ref_count = self.ref_count
        self.set_key_value(self.key[pos:], self.value[pos:])
        self.set_parent(head)
        return head


@dataclass
class CacheHandle:
    """RadixCacheHandle (src/kvcache/cache_manager.cc:15-31)."""
    cached_len: int
    node: RadixNode

    def matched_indices(self) -> np.ndarray:
        parts, n = [], self.node
        while not n.is_root():
            parts.append(n.value)
            n = n.parent
        if not parts:
            return np.zeros(0, dtype=np.int32)
        return np.concatenate(parts[::-1]).astype(np.int32)


class RadixPrefixCache:
    """RadixPrefixCache (src/kvcache/cache_manager.cc:37-236)."""

    def __init__(self, page_size: int):
        self.page_size = page_size
        self.clock = _Clock()
        self.root = RadixNode(page_size, self.clock.now())
        self.root.ref_count = 1
        self.evictable_size = 0
        self.protected_size = 0

    def lock_handle(self, handle: CacheHandle, unlock: bool = False) -> None:
        node = handle.node
        while not node.is_root():
            if unlock:
                node.ref_count -= 1
                if node.ref_count < 0:
                    raise ValueError("lock_handle: ref_count went negative")
                if node.ref_count == 0:
                    self.evictable_size += len(node)
                    self.protected_size -= len(node)
            else:
                if node.ref_count == 0:
                    self.evictable_size -= len(node)
                    self.protected_size += len(node)
                node.ref_count += 1
            node = node.parent

    def _walk(self, ids: np.ndarray):
        P = self.page_size
        prefix, node, tic = 0, self.root, self.clock.now()
        while prefix < len(ids):
            child = node.children.get(page_key(ids[prefix:], P))
            if child is None:
                return node, prefix
            node = child
            m = compare_key(node.key, ids[prefix:]) // P * P
            prefix += m
            if m != len(node):
                return node.split_at(m), prefix
            node.timestamp = tic
        return node, prefix

    def match_prefix(self, ids) -> CacheHandle:
        node, n = self._walk(np.asarray(ids, dtype=np.int32))
        return CacheHandle(n, node)

    def insert_prefix(self, ids, indices):
        """Returns (length that was cached before, handle of the whole page-aligned prefix)."""
        ids, indices = np.asarray(ids, dtype=np.int32), np.asarray(indices, dtype=np.int32)
        n = len(ids) // self.page_size * self.page_size
        ids, indices = ids[:n], indices[:n]
        node, prefix = self._walk(ids)
        if prefix != n:
            leaf = RadixNode(self.page_size, self.clock.now())
            leaf.set_key_value(ids[prefix:].copy(), indices[prefix:].copy())
            leaf.set_parent(node)
            self.evictable_size += len(leaf)
            node = leaf
        return prefix, CacheHandle(n, node)

    def evict(self, size: int) -> np.ndarray:
        if size == 0:
            return np.zeros(0, dtype=np.int32)
        if size > self.evictable_size:
            raise ValueError(f"Cannot evict {size}, only {self.evictable_size} is evictable")
        heap, stack, order = [], [self.root], 0
        while stack:
            n = stack.pop()
            if n.is_leaf():
                if n.ref_count == 0 and not n.is_root():
                    heap.append((n.timestamp, order, n))
                    order += 1
            else:
                stack.extend(n.children.values())
        heapq.heapify(heap)
        out, got = [], 0
        while got < size:
            if not heap:
                raise ValueError(f"Cannot evict enough cache, need {size}, only {got} evicted")
            _, _, n = heapq.heappop(heap)
            got += len(n)
            out.append(n.value)
            self.evictable_size -= len(n)
            par = n.parent
            del par.children[page_key(n.key, self.page_size)]
            if par.is_leaf() and par.ref_count == 0 and not par.is_root():
                heapq.heappush(heap, (par.timestamp, order, par))
                order += 1
        return np.concatenate(out).astype(np.int32)


@dataclass
class Req:
    """include/sglang/core/req.h:13-58 (the length state machine of src/core/req.cc:5-53)."""
    input_ids: np.ndarray
    table_idx: int = -1
    cached_len: int = 0
    device_len: int = 0          # tokens whose KV will be in the pool after the current step
    max_device_len: int = 0
    uid: int = 0
    is_chunked_prefill: bool = False
    cache_handle: Optional[CacheHandle] = None
    output: list = field(default_factory=list)

    def extend_len(self) -> int:
        return self.device_len - self.cached_len

    def remain_len(self) -> int:
        return self.max_device_len - self.device_len

    def can_decode(self) -> bool:
        return not self.is_chunked_prefill and self.remain_len() > 0

    def write_pos(self) -> int:
        """Where the sampled token goes in the token pool (src/scheduler/scheduler.cc:321-325)."""
        return self.device_len if self.can_decode() else -1

    def complete_one(self) -> None:
        """Req::complete_one (src/core/req.cc:47-53)."""
        self.cached_len = self.device_len
        if self.device_len < self.max_device_len:
            self.device_len += 1

    def append_host_token(self, token: int) -> None:
        """Req::append_host_token (src/core/req.cc:70-82)."""
        if len(self.input_ids) + 1 > self.device_len:
            raise ValueError("append_host_token cannot advance beyond device_len")
        self.input_ids = np.append(self.input_ids, np.int32(token))


class _Tables:
    """The page table and token pool: a host mirror, forwarded to the engine's device tables when
    one is attached (the reference keeps only the device copies and reads rows back)."""

    def __init__(self, engine, rows: int, cols: int):
        self.engine = engine
        self.page_table = np.zeros((rows, cols), dtype=np.int32)
        self.token_pool = np.zeros((rows, cols), dtype=np.int32)

    def write_pages(self, rows, pos, slots) -> None:
        rows, pos, slots = (np.asarray(a, dtype=np.int32) for a in (rows, pos, slots))
        self.page_table[rows, pos] = slots
        if self.engine is not None and len(rows):
            self.engine.write_page_table(rows, pos, slots)

    def write_tokens(self, rows, pos, ids) -> None:
        rows, pos, ids = (np.asarray(a, dtype=np.int32) for a in (rows, pos, ids))
        ok = (pos >= 0) & (pos < self.token_pool.shape[1])
        self.token_pool[rows[ok], pos[ok]] = ids[ok]
        if self.engine is not None and len(rows):
            self.engine.write_token_pool(rows, pos, ids)


class TableManager:
    """src/scheduler/prefill.cc:12-34."""

    def __init__(self, max_running_req: int):
        self.free_rows = list(range(max_running_req))

    def available_size(self) -> int:
        return len(self.free_rows)

    def allocate(self) -> int:
        if not self.free_rows:
            raise ValueError("TableManager has no free slots")
        return self.free_rows.pop()

    def free(self, row: int) -> None:
        self.free_rows.append(row)


class CacheManager:
    """src/scheduler/prefill.cc:36-260."""

    def __init__(self, num_pages: int, page_size: int, tables: _Tables, enable_prefix_cache: bool = True):
        self.num_pages, self.page_size, self.tables = num_pages, page_size, tables
        self.prefix_cache = RadixPrefixCache(page_size)
        self.free_pages = [i * page_size for i in range(num_pages)]
        self.enabled = enable_prefix_cache
        self._lazy: Optional[list] = None

    def match_req(self, ids: np.ndarray) -> CacheHandle:
        if len(ids) <= 0:
            raise ValueError("Input length must be greater than 0")
        if not self.enabled:
            return CacheHandle(0, self.prefix_cache.root)
        return self.prefix_cache.match_prefix(ids[:len(ids) - 1])

    def available_size(self) -> int:
        return self.prefix_cache.evictable_size + len(self.free_pages) * self.page_size

    def lock(self, handle: CacheHandle) -> None:
        self.prefix_cache.lock_handle(handle, unlock=False)

    def unlock(self, handle: CacheHandle) -> None:
        self.prefix_cache.lock_handle(handle, unlock=True)

    def allocate_pages(self, needed: int) -> list:
        if needed <= 0:
            return []
        if needed > len(self.free_pages):
            self.free_indices(self.prefix_cache.evict((needed - len(self.free_pages)) * self.page_size))
        if needed > len(self.free_pages):
            raise ValueError("CacheManager failed to allocate enough pages")
        out, self.free_pages = self.free_pages[:needed], self.free_pages[needed:]
        return out

    def allocate_paged(self, reqs) -> None:
        """Pages for positions [cached_len, device_len) of each request, one allocation for the batch."""
        P = self.page_size
        info, needed = [], 0
        for r in reqs:
            first, last = -(-r.cached_len // P), -(-r.device_len // P)
            if last > first:
                needed += last - first
                info.append((r.table_idx, first, last))
        if needed == 0:
            return
        pages = iter(self.allocate_pages(needed))
        rows, pos, slots = [], [], []
        for row, first, last in info:
            for page in range(first, last):
                start = next(pages)
                rows.extend([row] * P)
                pos.extend(range(page * P, page * P + P))
                slots.extend(range(start, start + P))
        self.tables.write_pages(rows, pos, slots)

    def free_indices(self, indices) -> None:
        if indices is None or len(indices) == 0:
            return
        if self._lazy is not None:
            self._lazy.append(np.array(indices, dtype=np.int32))
            return
        self.free_pages.extend(int(v) for v in np.asarray(indices)[::self.page_size])

    def begin_lazy_free(self) -> None:
        if self._lazy is not None:
            raise ValueError("Nested lazy free regions are not allowed")
        self._lazy = []

    def end_lazy_free(self) -> None:
        pending, self._lazy = self._lazy, None
        for t in pending:
            self.free_indices(t)

    def cache_req(self, req: Req, finished: bool) -> None:
        if not self.enabled:
            if finished:
                self.free_indices(self.tables.page_table[req.table_idx, :req.cached_len])
            return
        ids = req.input_ids[:req.cached_len]
        slots = self.tables.page_table[req.table_idx, :req.cached_len]
        old = req.cache_handle
        had, handle = self.prefix_cache.insert_prefix(ids, slots)
        if old is not None:
            self.unlock(old)
            if had > old.cached_len:
                self.free_indices(slots[old.cached_len:had])
        if finished:
            if req.cached_len > handle.cached_len:
                self.free_indices(slots[handle.cached_len:req.cached_len])
        else:
            req.cache_handle = handle
            self.lock(handle)

    def check_integrity(self) -> None:
        cached = (self.prefix_cache.evictable_size + self.prefix_cache.protected_size) // self.page_size
        if len(self.free_pages) + cached != self.num_pages:
            raise ValueError("CacheManager integrity check failed")


@dataclass
class _Pending:
    uid: int
    input_ids: np.ndarray
    max_new_tokens: int
    chunked_req: Optional[Req] = None


@dataclass
class Batch:
    reqs: list
    phase: int   # 0 prefill, 1 decode


class HostScheduler:
    """The integer side of Scheduler::step_no_overlap (src/scheduler/scheduler.cc:365-389,424-470,
    574-580): PrefillManager / PrefillAdder (src/scheduler/prefill.cc:262-400), DecodeManager
    (src/scheduler/decode.cc:10-67) and the bookkeeping after a forward pass, with the forward pass
    left to the caller (``next_batch`` -> run it -> ``finish_batch`` with the sampled tokens)."""

    def __init__(self, engine, num_pages: int, page_size: int, max_running_req: int, max_seq_len: int,
                 max_extend_tokens: int, enable_prefix_cache: bool = True):
        cols = (max_seq_len + 31) // 32 * 32
        self.engine, self.page_size, self.max_extend_tokens = engine, page_size, max_extend_tokens
        self.tables = _Tables(engine, max_running_req + 1, cols)
        self.table_manager = TableManager(max_running_req)
        self.cache_manager = CacheManager(num_pages, page_size, self.tables, enable_prefix_cache)
        self.pending: list[_Pending] = []
        self.running: list[Req] = []
        self.prefix_hits = 0

    # ---- PrefillManager ------------------------------------------------------
    def submit(self, uid: int, input_ids, max_new_tokens: int) -> None:
        ids = np.ascontiguousarray(np.asarray(input_ids, dtype=np.int32))
        self.pending.append(_Pending(uid, ids, max_new_tokens))

    def inflight_tokens(self) -> int:
        return (self.page_size - 1) * len(self.running) + sum(r.remain_len() for r in self.running)

    def _schedule_prefill(self):
        if not self.pending:
            return None
        budget, reserved = self.max_extend_tokens, self.inflight_tokens()
        cm, tm = self.cache_manager, self.table_manager
        reqs, chunked = [], []
        for p in self.pending:
            if budget <= 0:
                break
            if p.chunked_req is not None:
                handle, row, cached = p.chunked_req.cache_handle, p.chunked_req.table_idx, p.chunked_req.cached_len
            else:
                if tm.available_size() == 0:
                    break
                handle = cm.match_req(p.input_ids)
                cached = handle.cached_len
                need = len(p.input_ids) - cached + p.max_new_tokens
                if need + reserved > cm.available_size():
                    break
                cm.lock(handle)
                if need + reserved > cm.available_size():
                    cm.unlock(handle)
                    break
                row = tm.allocate()
                self.prefix_hits += cached
                if cached > 0:
                    at = np.arange(cached, dtype=np.int32)
                    self.tables.write_tokens(np.full(cached, row, np.int32), at, p.input_ids[:cached])
                    self.tables.write_pages(np.full(cached, row, np.int32), at, handle.matched_indices())
            remain = len(p.input_ids) - cached
            chunk = min(budget, remain)
            budget -= chunk
            reserved += remain + p.max_new_tokens
            at = np.arange(cached, cached + chunk, dtype=np.int32)
            self.tables.write_tokens(np.full(chunk, row, np.int32), at, p.input_ids[cached:cached + chunk])
            r = Req(p.input_ids[:cached + chunk].copy(), row, cached, cached + chunk,
                    cached + chunk + p.max_new_tokens, p.uid, chunk < remain, handle)
            p.chunked_req = None
            if r.is_chunked_prefill:
                p.chunked_req = r
                chunked.append(p)
            reqs.append(r)
        if not reqs:
            return None
        self.pending = chunked + self.pending[len(reqs):]
        return Batch(reqs, 0)

    # ---- one scheduler step ----------------------------------------------------
    def next_batch(self) -> Optional[Batch]:
        batch = self._schedule_prefill()
        if batch is None and self.running:
            batch = Batch(list(self.running), 1)
        if batch is not None:
            self.cache_manager.allocate_paged(batch.reqs)
        return batch

    def finish_batch(self, batch: Batch, next_tokens) -> list:
        """Everything after the launch of a forward pass; returns the finished flag per request."""
        reqs = batch.reqs
        self.tables.write_tokens([r.table_idx for r in reqs], [r.write_pos() for r in reqs],
                                 np.asarray(next_tokens, dtype=np.int32)[:len(reqs)])
        for r in reqs:
            r.complete_one()
        # DecodeManager::filter_reqs: the running set, then the batch, keeping those that can decode
        seen, merged = set(), []
        for r in self.running + reqs:
            if r.can_decode() and r.uid not in seen:
                seen.add(r.uid)
                merged.append(r)
        self.running = merged
        finished = []
        cm = self.cache_manager
        cm.begin_lazy_free()
        for r, tok in zip(reqs, next_tokens):
            if r.is_chunked_prefill:
                finished.append(False)
                continue
            r.append_host_token(int(tok))
            r.output.append(int(tok))
            fin = not r.can_decode()
            if fin:
                self.running = [q for q in self.running if q.uid != r.uid]
                self.table_manager.free(r.table_idx)
                cm.cache_req(r, finished=True)
            elif batch.phase == 0:
                cm.cache_req(r, finished=False)
            finished.append(fin)
        cm.end_lazy_free()
        return finished


class HostBatcher:
    """Requests driven by hand (which requests prefill together, when they decode) on the same
    TableManager / CacheManager: what most tests and the benchmark use."""

    def __init__(self, engine, num_pages: int, page_size: int, max_running_req: int,
                 enable_prefix_cache: bool = True, max_seq_len: Optional[int] = None):
        self.engine = engine
        self.page_size = page_size
        cols = engine.pt_cols if engine is not None else (max_seq_len + 31) // 32 * 32
        self.tables = _Tables(engine, max_running_req + 1, cols)
        self.table_manager = TableManager(max_running_req)
        self.cache_manager = CacheManager(num_pages, page_size, self.tables, enable_prefix_cache)
        self.prefix_hits = 0
        self._next_uid = 0
        self._held: dict[int, int] = {}   # table row -> pages its positions already map to

    def add_request(self, input_ids, max_new_tokens: int) -> Req:
        """PrefillAdder::try_allocate_one + add_one_req (src/scheduler/prefill.cc:270-330), whole prompt."""
        ids = np.ascontiguousarray(np.asarray(input_ids, dtype=np.int32))
        handle = self.cache_manager.match_req(ids)
        self.cache_manager.lock(handle)
        row = self.table_manager.allocate()
        cached = handle.cached_len
        self.prefix_hits += cached
        at = np.arange(len(ids), dtype=np.int32)
        self.tables.write_tokens(np.full(len(ids), row, np.int32), at, ids)
        if cached:
            self.tables.write_pages(np.full(cached, row, np.int32), at[:cached], handle.matched_indices())
        self._next_uid += 1
        self._held[row] = cached // self.page_size
        return Req(ids, row, cached, len(ids), len(ids) + max_new_tokens, self._next_uid, False, handle)

    def allocate(self, reqs) -> None:
        """CacheManager::allocate_paged for the positions that have no page yet.  (A request whose
        lengths were wound back — the benchmark replays the same steps — keeps the pages it has.)"""
        from types import SimpleNamespace

        P, todo = self.page_size, []
        for r in reqs:
            held = self._held.get(r.table_idx, 0)
            need = -(-r.device_len // P)
            if need > held:
                todo.append(SimpleNamespace(table_idx=r.table_idx, device_len=r.device_len,
                                            cached_len=max(r.cached_len, held * P)))
                self._held[r.table_idx] = need
        if todo:
            self.cache_manager.allocate_paged(todo)

    def cache_prefix(self, req: Req) -> None:
        """Insert the page-aligned prefix of a request whose prefill finished (cache_req, not finished)."""
        self.cache_manager.cache_req(req, finished=False)

    def slots_of(self, req: Req) -> np.ndarray:
        """The request's page-table row (one slot per position; unallocated positions read 0)."""
        return self.tables.page_table[req.table_idx]

    def pages_held(self, req: Req) -> int:
        return self._held.get(req.table_idx, 0)

    # ---- steps --------------------------------------------------------------
    def prefill(self, reqs, chunk_tokens: Optional[int] = None, sampling: Optional[dict] = None):
        """One prefill step over `reqs` (each runs positions [cached_len, device_len)).

        With ``chunk_tokens`` a request whose remaining prompt is longer runs only that many tokens
        this step (the chunked request of src/scheduler/prefill.cc:301-330,382-400): its sampled token is dropped
        (write position -1) and the next call continues where this one stopped.  ``sampling`` holds
        per-request ``temperatures / top_k / top_p / seeds`` (BatchSamplingArgs)."""
        for r in reqs:
            full = len(r.input_ids)
            if r.device_len < full or r.is_chunked_prefill:   # continuing a chunked request
                r.device_len = full
            r.is_chunked_prefill = chunk_tokens is not None and r.extend_len() > chunk_tokens
            if r.is_chunked_prefill:
                r.device_len = r.cached_len + chunk_tokens
        self.allocate(reqs)
        out = self.engine.forward_batch(
            0, [r.table_idx for r in reqs], [r.cached_len for r in reqs], [r.extend_len() for r in reqs],
            write_pos=[r.write_pos() for r in reqs], **(sampling or {}))
        for r in reqs:
            if r.is_chunked_prefill:
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

    def __init__(self, batcher: HostBatcher, reqs, padded_size: Optional[int] = None, ring: bool = False):
        import ctypes

        self.ring = ring          # steps report through the engine's pinned result ring; step() returns a ticket
        self._ticket = ctypes.c_int64()
        self._ticket_ref = ctypes.byref(self._ticket)

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
        self.pages_have = np.array([batcher.pages_held(r) for r in self.reqs], dtype=np.int64)
        self._st = StepStruct(1, n, bp, self.table_idx.ctypes.data, self.cached.ctypes.data, self.extend.ctypes.data,
                              self.write_pos.ctypes.data, None, None, None, None, 0)
        self._st_ref = ctypes.byref(self._st)

    def step(self):
        """One decode step of every request (asynchronous, like Engine.forward_batch): returns the
        pinned token buffer, valid after ``engine.synchronize()`` (or the ticket for ``wait``)."""
        from ._lib import call

        hb, P = self.hb, self.hb.page_size
        # pages for the position this step writes (CacheManager::allocate_paged): rare, so per request
        need = np.nonzero(-(-self.device_len // P) > self.pages_have)[0]
        if len(need):
            batch = []
            for i in need:
                r = self.reqs[int(i)]
                r.cached_len, r.device_len = int(self.cached[i]), int(self.device_len[i])
                batch.append(r)
            hb.allocate(batch)
            self.pages_have[need] = [hb.pages_held(r) for r in batch]
        can = self.device_len < self.max_len
        self.write_pos[:self.n] = np.where(can, self.device_len, -1)
        eng = self.engine
        self._st.step_index = eng._step_index
        eng._step_index += 1
        if self.ring:
            call("b200_engine_step_async", eng._h, self._st_ref, None, self._ticket_ref)
            out = self._ticket.value
        else:
            buf = eng.next_token_buffer()
            call("b200_engine_step", eng._h, self._st_ref, buf.data_ptr())
            out = buf[:self.n]
        # Req::complete_one for every request
        self.cached[:self.n] = self.device_len
        self.device_len += can
        return out

    def wait(self, ticket: int):
        """(tokens, finish flags) of a step enqueued with ``ring=True``: blocks on that step only."""
        return self.engine.wait(ticket, self.n)

    def sync_back(self) -> None:
        for i, r in enumerate(self.reqs):
            r.cached_len, r.device_len = int(self.cached[i]), int(self.device_len[i])
