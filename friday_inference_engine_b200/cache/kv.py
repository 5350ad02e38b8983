"""Storage of keys and values for one group of cache entries, in pages.

Entries (one per layer call that keeps keys and values) with the same needs, that is
the same number of kv heads, head size and window, form a group.  A group owns

  k_pool, v_pool   [entries, pages, PAGE, kv_heads, head_dim] in the activation dtype
  a free list of page numbers (a page number means the same rows in every entry)
  table            host array [slots, width]: page of each logical page of each slot,
                   -1 where the slot holds none

A group without a window keeps every position of a live sequence.  A group with a
window W gives a page back as soon as every position in it is more than W-1 behind the
sequence's end: no later query can reach it.  So a long sequence holds about W/PAGE + 2
pages of such a group, whatever its length.

The reference keeps two flat buffers [layers][ctx][kv] for its one sequence
(transformer.h:145-149, transformer.cpp:483-497); pages and slots are this library's.
"""
import numpy as np
import torch

from .slots import CacheError, FreeList

PAGE = 64


class KVGroup:
    def __init__(self, request, entries, n_slots, n_pages, width, dtype, device):
        self.request = request
        self.entries = list(entries)                 # cache entry ids, in pool order
        self.index_of = {e: i for i, e in enumerate(self.entries)}
        self.window = request.window
        self.n_pages, self.width = int(n_pages), int(width)
        shape = (len(self.entries), self.n_pages, PAGE, request.n_kv_heads, request.head_dim)
        self.k_pool = torch.empty(shape, dtype=dtype, device=device)
        self.v_pool = torch.empty(shape, dtype=dtype, device=device)
        self.pages = FreeList(self.n_pages, "page")
        self.table = np.full((n_slots, self.width), -1, dtype=np.int32)

    def first_needed_page(self, start_pos):
        """Logical page of the earliest key that a query at `start_pos` or later can see."""
        if self.window is None:
            return 0
        return max(0, start_pos - self.window + 1) // PAGE

    def pages_missing(self, slot, start_pos, new_len):
        if new_len > self.width * PAGE:
            raise CacheError("a sequence of %d tokens does not fit the cache's %d tokens per sequence"
                             % (new_len, self.width * PAGE))
        row = self.table[slot]
        lo, hi = self.first_needed_page(start_pos), (new_len + PAGE - 1) // PAGE
        return [lp for lp in range(lo, hi) if row[lp] < 0]

    def reserve(self, slot, start_pos, new_len):
        for lp in self.pages_missing(slot, start_pos, new_len):
            self.table[slot, lp] = self.pages.take()

    def release_behind(self, slot, length):
        """Gives back the pages that no query at position >= length can reach."""
        if self.window is None:
            return
        row = self.table[slot]
        for lp in range(0, max(0, length - self.window + 1) // PAGE):
            if row[lp] >= 0:
                self.pages.give(int(row[lp]))
                row[lp] = -1

    def release_all(self, slot):
        row = self.table[slot]
        for lp in np.nonzero(row >= 0)[0]:
            self.pages.give(int(row[lp]))
        row[:] = -1

    def held_pages(self, slot):
        return [int(p) for p in self.table[slot] if p >= 0]


class KVView:
    """What an attention mixer gets for one layer call."""
    __slots__ = ("k_pool", "v_pool", "block_table", "page_size", "write", "window")

    def __init__(self, k_pool, v_pool, block_table, write, window):
        self.k_pool, self.v_pool, self.block_table = k_pool, v_pool, block_table
        self.page_size, self.write, self.window = PAGE, write, window


class StateView:
    """What a mixer with fixed-size state gets: state[slot] is the sequence's own tensor;
    seq_slots (device, int64) gives the slot of every sequence of the step, slots (host
    list) the same numbers."""
    __slots__ = ("state", "seq_slots", "slots", "write")

    def __init__(self, state, seq_slots, slots, write):
        self.state, self.seq_slots, self.slots, self.write = state, seq_slots, slots, write
