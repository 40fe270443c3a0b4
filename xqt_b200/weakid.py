"""Identity-keyed weak mapping for tensors.

``weakref.WeakKeyDictionary`` compares keys with ``==``, which for tensors is element-wise and has
no truth value; caches of derived layouts are keyed on the tensor *object* instead: an entry is found
only through the very tensor it was stored under and disappears when that tensor is collected, so a
recycled device address can never hit a stale entry.
"""

from __future__ import annotations

import weakref
from typing import Any


class WeakIdDict:
    def __init__(self) -> None:
        self._items: dict[int, tuple[weakref.ref, Any]] = {}

    def get(self, key: Any, default: Any = None) -> Any:
        hit = self._items.get(id(key))
        if hit is None or hit[0]() is not key:
            return default
        return hit[1]

    def __setitem__(self, key: Any, value: Any) -> None:
        ident = id(key)

        def drop(_ref: weakref.ref, ident: int = ident, items: dict = self._items) -> None:
            hit = items.get(ident)
            if hit is not None and hit[0] is _ref:
                del items[ident]

        self._items[ident] = (weakref.ref(key, drop), value)

    def __contains__(self, key: Any) -> bool:
        return self.get(key, self) is not self

    def __len__(self) -> int:
        return sum(1 for ref, _ in self._items.values() if ref() is not None)


__all__ = ["WeakIdDict"]
