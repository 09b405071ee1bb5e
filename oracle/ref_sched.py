"""ctypes access to the reference's own integer-side objects — TEST INFRASTRUCTURE ONLY.

``oracle/_ref/libsglang_ref_cpu.so`` (see build_ref.py, ref_sched_shim.cc) holds the reference's
Req, RadixTreeNode, RadixPrefixCache, TableManager, CacheManager, PrefillManager and DecodeManager
compiled from the reference tree.  The classes below call them; nothing here computes.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import numpy as np

LIB_PATH = Path(__file__).resolve().parent / "_ref" / "libsglang_ref_cpu.so"
_lib = None

_i32p = ctypes.POINTER(ctypes.c_int32)
_i64p = ctypes.POINTER(ctypes.c_int64)
_u64p = ctypes.POINTER(ctypes.c_uint64)
_ip = ctypes.POINTER(ctypes.c_int)


def available() -> bool:
    return LIB_PATH.exists()


def lib():
    global _lib
    if _lib is None:
        import torch  # noqa: F401  (the library links against the wheel's LibTorch)

        L = ctypes.CDLL(str(LIB_PATH))
        L.ref_last_error.restype = ctypes.c_char_p
        L.ref_sched_create.restype = ctypes.c_void_p
        L.ref_sched_create.argtypes = [ctypes.c_int] * 5
        L.ref_sched_destroy.argtypes = [ctypes.c_void_p]
        L.ref_sched_submit.argtypes = [ctypes.c_void_p, ctypes.c_uint64, _i32p, ctypes.c_int, ctypes.c_int]
        L.ref_sched_next_batch.argtypes = [ctypes.c_void_p, _ip, ctypes.c_int, _u64p, _i32p, _i32p, _i32p, _i32p, _i32p]
        L.ref_sched_finish_batch.argtypes = [ctypes.c_void_p, _i32p, ctypes.c_int, _i32p]
        L.ref_sched_page_table.restype = _i32p
        L.ref_sched_page_table.argtypes = [ctypes.c_void_p, _ip, _ip]
        L.ref_sched_token_pool.restype = _i32p
        L.ref_sched_token_pool.argtypes = [ctypes.c_void_p]
        L.ref_sched_sizes.argtypes = [ctypes.c_void_p, _i64p, _i64p, _ip, _ip, _ip, _ip]
        L.ref_radix_create.restype = ctypes.c_void_p
        L.ref_radix_create.argtypes = [ctypes.c_int]
        L.ref_radix_destroy.argtypes = [ctypes.c_void_p]
        L.ref_radix_insert.restype = ctypes.c_int64
        L.ref_radix_insert.argtypes = [ctypes.c_void_p, _i32p, _i32p, ctypes.c_int, _i64p, _ip]
        L.ref_radix_match.restype = ctypes.c_int64
        L.ref_radix_match.argtypes = [ctypes.c_void_p, _i32p, ctypes.c_int, _ip, _i32p, ctypes.c_int]
        L.ref_radix_lock.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
        L.ref_radix_evict.restype = ctypes.c_int64
        L.ref_radix_evict.argtypes = [ctypes.c_void_p, ctypes.c_int64, _i32p, ctypes.c_int]
        L.ref_radix_size.argtypes = [ctypes.c_void_p, _i64p, _i64p]
        L.ref_fast_compare_key.restype = ctypes.c_int64
        L.ref_fast_compare_key.argtypes = [_i32p, ctypes.c_int, _i32p, ctypes.c_int]
        L.ref_key_fn.restype = ctypes.c_int64
        L.ref_key_fn.argtypes = [ctypes.c_int, _i32p, ctypes.c_int]
        L.ref_node_split.argtypes = [_i32p, _i32p, ctypes.c_int, ctypes.c_int, ctypes.c_int, _i32p, _i32p, _i32p, _i32p, _ip, _ip]
        L.ref_req_create.restype = ctypes.c_void_p
        L.ref_req_create.argtypes = [_i32p, ctypes.c_int] + [ctypes.c_int] * 4
        L.ref_req_destroy.argtypes = [ctypes.c_void_p]
        L.ref_req_state.argtypes = [ctypes.c_void_p, _i32p]
        L.ref_req_complete_one.argtypes = [ctypes.c_void_p]
        L.ref_req_append_host.argtypes = [ctypes.c_void_p, ctypes.c_int32]
        _lib = L
    return _lib


class RefError(RuntimeError):
    """A c10::Error raised inside the reference's code."""


def _arr(a):
    a = np.ascontiguousarray(np.asarray(a, dtype=np.int32))
    return a, a.ctypes.data_as(_i32p)


def _fail():
    raise RefError(lib().ref_last_error().decode(errors="replace").splitlines()[0])


class RefScheduler:
    """The reference's managers driven as Scheduler::step_no_overlap drives them."""

    def __init__(self, num_pages, page_size, max_running_req, max_seq_len, max_extend_tokens):
        self.h = lib().ref_sched_create(num_pages, page_size, max_running_req, max_seq_len, max_extend_tokens)
        if not self.h:
            _fail()
        self.cap = max_running_req + 1
        self._n = 0

    def __del__(self):
        if getattr(self, "h", None):
            lib().ref_sched_destroy(self.h)
            self.h = None

    def submit(self, uid, ids, max_new_tokens):
        a, p = _arr(ids)
        if lib().ref_sched_submit(self.h, uid, p, len(a), max_new_tokens):
            _fail()

    def next_batch(self):
        """None when idle, else a dict of per-request arrays and the phase (0 prefill, 1 decode)."""
        c = self.cap
        phase = ctypes.c_int(0)
        uids = np.zeros(c, dtype=np.uint64)
        cols = [np.zeros(c, dtype=np.int32) for _ in range(5)]
        n = lib().ref_sched_next_batch(self.h, ctypes.byref(phase), c, uids.ctypes.data_as(_u64p),
                                       *[x.ctypes.data_as(_i32p) for x in cols])
        if n < 0:
            _fail()
        if n == 0:
            return None
        self._n = n
        names = ("table_idx", "cached_len", "device_len", "chunked", "write_pos")
        out = {k: v[:n].copy() for k, v in zip(names, cols)}
        out["uid"] = uids[:n].copy()
        out["phase"] = phase.value
        return out

    def finish_batch(self, next_tokens):
        a, p = _arr(next_tokens)
        fin = np.zeros(self._n, dtype=np.int32)
        if lib().ref_sched_finish_batch(self.h, p, self._n, fin.ctypes.data_as(_i32p)):
            _fail()
        return fin.astype(bool).tolist()

    def page_table(self):
        r, c = ctypes.c_int(), ctypes.c_int()
        p = lib().ref_sched_page_table(self.h, ctypes.byref(r), ctypes.byref(c))
        return np.ctypeslib.as_array(p, shape=(r.value, c.value)).copy()

    def token_pool(self):
        shape = self.page_table().shape
        return np.ctypeslib.as_array(lib().ref_sched_token_pool(self.h), shape=shape).copy()

    def sizes(self):
        ev, pr = ctypes.c_int64(), ctypes.c_int64()
        a, f, i, p = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        if lib().ref_sched_sizes(self.h, ctypes.byref(ev), ctypes.byref(pr), ctypes.byref(a), ctypes.byref(f),
                                 ctypes.byref(i), ctypes.byref(p)):
            _fail()
        return {"evictable": ev.value, "protected": pr.value, "available": a.value, "free_rows": f.value,
                "inflight": i.value, "pending": p.value}


class RefRadixCache:
    """RadixPrefixCache of the reference; handles are small integers."""

    def __init__(self, page_size):
        self.h = lib().ref_radix_create(page_size)

    def __del__(self):
        if getattr(self, "h", None):
            lib().ref_radix_destroy(self.h)
            self.h = None

    def insert_prefix(self, ids, indices):
        a, pa = _arr(ids)
        b, pb = _arr(indices)
        hl, hid = ctypes.c_int64(), ctypes.c_int()
        had = lib().ref_radix_insert(self.h, pa, pb, len(a), ctypes.byref(hl), ctypes.byref(hid))
        if had < 0:
            _fail()
        return had, hl.value, hid.value

    def match_prefix(self, ids):
        a, pa = _arr(ids)
        out = np.zeros(max(len(a), 1), dtype=np.int32)
        hid = ctypes.c_int()
        n = lib().ref_radix_match(self.h, pa, len(a), ctypes.byref(hid), out.ctypes.data_as(_i32p), len(out))
        if n < 0:
            _fail()
        return n, out[:n].copy(), hid.value

    def lock_handle(self, handle_id, unlock=False):
        if lib().ref_radix_lock(self.h, handle_id, int(unlock)):
            _fail()

    def evict(self, size, cap=1 << 16):
        out = np.zeros(cap, dtype=np.int32)
        n = lib().ref_radix_evict(self.h, size, out.ctypes.data_as(_i32p), cap)
        if n < 0:
            _fail()
        return out[:n].copy()

    def size_info(self):
        ev, pr = ctypes.c_int64(), ctypes.c_int64()
        lib().ref_radix_size(self.h, ctypes.byref(ev), ctypes.byref(pr))
        return ev.value, pr.value


def fast_compare_key(a, b):
    x, px = _arr(a)
    y, py = _arr(b)
    return lib().ref_fast_compare_key(px, len(x), py, len(y))


def key_fn(page_size, ids):
    x, px = _arr(ids)
    return lib().ref_key_fn(page_size, px, len(x))


def node_split(key, value, pos, ref_count):
    k, pk = _arr(key)
    v, pv = _arr(value)
    n = len(k)
    outs = [np.zeros(n, dtype=np.int32) for _ in range(4)]
    rc, ok = ctypes.c_int(), ctypes.c_int()
    if lib().ref_node_split(pk, pv, n, pos, ref_count, *[o.ctypes.data_as(_i32p) for o in outs], ctypes.byref(rc),
                            ctypes.byref(ok)):
        _fail()
    return outs[0][:pos], outs[1][:pos], outs[2][:n - pos], outs[3][:n - pos], rc.value, bool(ok.value)


class RefReq:
    FIELDS = ("device_len", "max_device_len", "remain_len", "extend_len", "can_decode", "cached_len", "host_len")

    def __init__(self, ids, cached_len=0, output_len=0, chunked=False, initialize=False):
        a, p = _arr(ids)
        self.h = lib().ref_req_create(p, len(a), cached_len, output_len, int(chunked), int(initialize))
        if not self.h:
            _fail()

    def __del__(self):
        if getattr(self, "h", None):
            lib().ref_req_destroy(self.h)
            self.h = None

    def state(self):
        out = np.zeros(7, dtype=np.int32)
        lib().ref_req_state(self.h, out.ctypes.data_as(_i32p))
        return dict(zip(self.FIELDS, out.tolist()))

    def complete_one(self):
        if lib().ref_req_complete_one(self.h):
            _fail()

    def append_host(self, token):
        if lib().ref_req_append_host(self.h, token):
            _fail()
