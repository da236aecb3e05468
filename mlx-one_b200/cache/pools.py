"""Host-side pools of page and slot numbers."""

from __future__ import annotations

from .errors import CacheCapacityError, CacheOwnershipError


class IndexPool:
    """Hands out the numbers 0..count-1. A number that was given back last is handed out
    first, so reuse happens as early as possible and stale contents would show."""

    def __init__(self, count: int, what: str = "page") -> None:
        if count < 1:
            raise ValueError(f"a pool needs at least one {what}")
        self.count = count
        self.what = what
        self._free = list(range(count - 1, -1, -1))
        self._held = [False] * count
        self.low_water = count

    @property
    def free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheCapacityError(f"no free {self.what}", retryable=True)
        index = self._free.pop()
        if self._held[index]:
            raise CacheOwnershipError(f"{self.what} {index} was handed out twice")
        self._held[index] = True
        self.low_water = min(self.low_water, len(self._free))
        return index

    def give_back(self, index: int) -> None:
        if not 0 <= index < self.count or not self._held[index]:
            raise CacheOwnershipError(f"{self.what} {index} is given back but not held")
        self._held[index] = False
        self._free.append(index)

    def held(self) -> set[int]:
        return {i for i, flag in enumerate(self._held) if flag}
