"""Kernel set of the engine. ``default_ops(device)`` builds and loads the CUDA extension;
there is no other implementation on the product path."""

from .build import KernelBuildError, library_path
from .cuda_ops import CudaOps, KernelError

_CACHE: dict[str, CudaOps] = {}


def default_ops(device="cuda:0", verbose: bool = True) -> CudaOps:
    key = str(device)
    if key not in _CACHE:
        _CACHE[key] = CudaOps(device, verbose=verbose)
    return _CACHE[key]


__all__ = ["CudaOps", "KernelBuildError", "KernelError", "default_ops", "library_path"]
