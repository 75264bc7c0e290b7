"""Identity-keyed memo used by the operators for load-time conversions."""

from __future__ import annotations

import weakref
from collections import OrderedDict


class IdentityCache:
    """Memo of derived objects keyed by the IDENTITY and VERSION of their source tensors, so that operators
    called with the reference's own argument types (GroupQuantizedWeight, [A, K, r] LoRA tables) convert them
    once, not on every call.  An entry dies with its first source tensor; an in-place update of any source
    (an optimizer step on a LoRA table bumps `_version`) makes a new entry."""

    def __init__(self, capacity: int = 256):
        self.capacity = capacity
        self._items: OrderedDict = OrderedDict()
        self.hits = 0
        self.misses = 0

    @staticmethod
    def _key(tensors, extra):
        return tuple((id(t), t._version, t.data_ptr(), tuple(t.shape)) for t in tensors) + (extra,)

    def get(self, tensors, extra, build):
        key = self._key(tensors, extra)
        hit = self._items.get(key)
        if hit is not None and all(ref() is t for ref, t in zip(hit[0], tensors)):
            self._items.move_to_end(key)
            self.hits += 1
            return hit[1]
        self.misses += 1
        value = build()
        self._items[key] = ([weakref.ref(t) for t in tensors], value)
        # drop entries whose sources are gone, then the oldest beyond capacity
        for k_ in [k_ for k_, (refs, _) in self._items.items() if any(r() is None for r in refs)]:
            del self._items[k_]
        while len(self._items) > self.capacity:
            self._items.popitem(last=False)
        return value

    def clear(self):
        self._items.clear()
