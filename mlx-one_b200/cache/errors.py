"""Errors of the cache manager (the reference's taxonomy,
src/mlx_one/engine/cache_errors.py)."""


class CacheError(RuntimeError):
    pass


class CacheCapacityError(CacheError):
    """Not enough pages or slots. ``retryable``: it may fit once other requests end;
    otherwise the request is larger than the whole pool and can never fit."""

    def __init__(self, message: str, *, retryable: bool) -> None:
        super().__init__(message)
        self.retryable = retryable


class CacheOwnershipError(CacheError):
    """A page, slot or request was used by someone who does not hold it: an unknown or
    closed request, a page freed twice, a slot handed out twice."""
