"""The cache of a model: slots, groups of paged keys and values, fixed-size states.

It is built from what the model's mixers ask for, entry by entry: KVRequests are
grouped by their needs and each group gets storage of its own; every StateRequest gets
a tensor [slots, *shape] that is zeroed when a slot is taken.  The cache also keeps
each slot's length.  Lengths, not contents, decide what is valid: slots and pages are
used again without being cleared.

Capacity is given in tokens: `max_tokens` is the most tokens that live sequences hold
together, each sequence counted in whole pages of 64; `max_seq_tokens` bounds one
sequence.
"""
import numpy as np
import torch

from ..parts.base import KVRequest, StateRequest
from .kv import PAGE, KVGroup, KVView, StateView
from .slots import CacheError, CacheFull, FreeList


class Cache:
    def __init__(self, requests, max_tokens, max_seq_tokens, dtype, device, max_slots=None):
        """requests: cache entry id -> KVRequest | StateRequest."""
        self.device = torch.device(device)
        n_pages = max(1, (int(max_tokens) + PAGE - 1) // PAGE)
        self.max_seq_tokens = int(max_seq_tokens)
        width = max(1, min(n_pages, (self.max_seq_tokens + PAGE - 1) // PAGE))
        self.max_slots = int(max_slots) if max_slots else min(n_pages, 4096)
        self.slots = FreeList(self.max_slots, "slot")
        self.lens = [0] * self.max_slots
        self.groups = []
        self.group_of = {}            # entry -> KVGroup
        self.states = {}              # entry -> tensor [slots, *shape]
        by_need = {}
        for entry, req in sorted(requests.items()):
            if isinstance(req, KVRequest):
                by_need.setdefault(req, []).append(entry)
            elif isinstance(req, StateRequest):
                self.states[entry] = torch.zeros((self.max_slots,) + tuple(req.shape), dtype=req.dtype,
                                                 device=self.device)
            elif req is not None:
                raise CacheError("cache entry %r asks for %r, which is neither keys and values nor a state"
                                 % (entry, req))
        for req, entries in by_need.items():
            g = KVGroup(req, entries, self.max_slots, n_pages, width, dtype, self.device)
            self.groups.append(g)
            for e in entries:
                self.group_of[e] = g

    # -- slots ------------------------------------------------------------
    def alloc_slot(self):
        slot = self.slots.take()
        self.lens[slot] = 0
        for state in self.states.values():
            state[slot].zero_()
        return slot

    def free_slot(self, slot):
        self.slots.give(slot)            # raises if the slot is not held
        for g in self.groups:
            g.release_all(slot)
        self.lens[slot] = 0

    # -- one pass of the step function ------------------------------------
    def reserve(self, slots, q_lens):
        """Pages for the tokens that each slot is about to take.  Either all of it
        succeeds or nothing is held afterwards that was not held before."""
        for g in self.groups:
            need = 0
            for slot, q in zip(slots, q_lens):
                if not self.slots.holds(slot):
                    raise CacheError("slot %r is not held" % (slot,))
                need += len(g.pages_missing(slot, self.lens[slot], self.lens[slot] + q))
            if need > g.pages.free_count:
                raise CacheFull("the cache is full: %d more pages of %d tokens are needed, %d are free "
                                "(capacity %d tokens)" % (need, PAGE, g.pages.free_count, g.n_pages * PAGE))
        for g in self.groups:
            for slot, q in zip(slots, q_lens):
                g.reserve(slot, self.lens[slot], self.lens[slot] + q)

    def commit(self, slots, q_lens):
        for slot, q in zip(slots, q_lens):
            self.lens[slot] += q
            for g in self.groups:
                g.release_behind(slot, self.lens[slot])

    def tables_for(self, slots, pad_to=None):
        """Per group, the block table rows of `slots` as one int32 array [n, width]
        (rows beyond len(slots), up to pad_to, are -1)."""
        n = pad_to or len(slots)
        out = []
        for g in self.groups:
            t = np.full((n, g.width), -1, dtype=np.int32)
            if slots:
                t[:len(slots)] = g.table[np.asarray(slots, dtype=np.int64)]
            out.append(t)
        return out

    def view(self, entry, write, step_tables, seq_slots_dev, slots):
        """The view of `entry` for one layer call; step_tables: per group, this step's
        block table on the device."""
        g = self.group_of.get(entry)
        if g is not None:
            i = g.index_of[entry]
            return KVView(g.k_pool[i], g.v_pool[i], step_tables[self.groups.index(g)], write, g.window)
        if entry in self.states:
            return StateView(self.states[entry], seq_slots_dev, slots, write)
        return None

    # -- accounting ----------------------------------------------------------
    def held_tokens(self):
        return sum(g.pages.held_count for g in self.groups[:1]) * PAGE if self.groups else 0

    def bytes(self):
        b = sum(g.k_pool.numel() * g.k_pool.element_size() * 2 for g in self.groups)
        return b + sum(s.numel() * s.element_size() for s in self.states.values())
