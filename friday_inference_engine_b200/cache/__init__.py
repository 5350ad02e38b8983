"""The cache's book-keeping, reachable without a GPU (cache/cache.cpp, include/friday/cache.h).

CacheBook builds the library's Cache without device memory: slots, pages, tables and
lengths behave exactly as in an engine, which is what the tests of "no slot or page lost,
held twice or freed twice" drive.  An engine's own books are read with Engine.stats().
"""
import json
from ctypes import byref, c_int, c_void_p

from .. import native
from ..native import CacheError, CacheFull  # noqa: F401

PAGE = 64


def kv_request(n_kv_heads, head_dim, window=None):
    return {"kind": "kv", "n_kv_heads": int(n_kv_heads), "head_dim": int(head_dim), "window": int(window or 0)}


def state_request(shape, dtype="float32"):
    return {"kind": "state", "shape": [int(s) for s in shape], "dtype": dtype}


class CacheBook:
    def __init__(self, requests, max_tokens, max_seq_tokens, max_slots=0):
        """requests: cache entry id -> kv_request(...) | state_request(...)."""
        self._h = c_void_p()
        native.call("friday_cache_new", native.text(json.dumps({str(k): v for k, v in requests.items()})),
                    int(max_tokens), int(max_seq_tokens), int(max_slots), byref(self._h))

    def __del__(self):
        if getattr(self, "_h", None) and native._lib is not None:
            native._lib.friday_cache_free(self._h)
            self._h = None

    def alloc_slot(self):
        s = c_int()
        native.call("friday_cache_alloc_slot", self._h, byref(s))
        return s.value

    def free_slot(self, slot):
        native.call("friday_cache_free_slot", self._h, int(slot))

    def reserve(self, slots, q_lens):
        native.call("friday_cache_reserve", self._h, len(slots), native.ints(slots), native.ints(q_lens))

    def commit(self, slots, q_lens):
        native.call("friday_cache_commit", self._h, len(slots), native.ints(slots), native.ints(q_lens))

    def info(self):
        """lens, held, slots_held/free, groups (entries, window, n_pages, width, pages_held/free, pool_shape, table),
        states (entry -> shape), group_of."""
        return native.call_json("friday_cache_info", self._h)

    def held_pages(self, group, slot):
        return [p for p in self.info()["groups"][group]["table"][slot] if p >= 0]
