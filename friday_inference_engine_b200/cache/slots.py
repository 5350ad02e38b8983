"""Slots and pages: who holds what.  Pure bookkeeping on the host, no tensors.

A slot stands for one live sequence.  A page is PAGE consecutive positions of one
sequence's keys and values.  Both are handed out from free lists and given back when
the sequence ends; a freed slot or page is used again as it is, without being cleared:
what makes a row valid is the sequence's length, never the row's content.
"""


class CacheError(RuntimeError):
    pass


class CacheFull(CacheError):
    """No free slot or page is left."""


class FreeList:
    """Hands out the integers 0 .. n-1, lowest first among those given back last."""

    def __init__(self, n, what):
        self.n = int(n)
        self.what = what
        self._free = list(range(self.n - 1, -1, -1))   # pop() gives 0 first
        self._held = set()

    def take(self):
        if not self._free:
            raise CacheFull("no free %s (all %d are held)" % (self.what, self.n))
        i = self._free.pop()
        self._held.add(i)
        return i

    def take_many(self, count):
        if count > len(self._free):
            raise CacheFull("%d %ss wanted, %d free of %d" % (count, self.what, len(self._free), self.n))
        return [self.take() for _ in range(count)]

    def give(self, i):
        if i not in self._held:
            raise CacheError("%s %r is not held (freed twice, or never taken)" % (self.what, i))
        self._held.remove(i)
        self._free.append(i)

    def holds(self, i):
        return i in self._held

    @property
    def free_count(self):
        return len(self._free)

    @property
    def held_count(self):
        return len(self._held)
