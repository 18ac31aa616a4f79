"""Loads the compiled CUDA libraries (ctypes) on first use.

There is no fallback: when a library cannot be built or loaded, or no CUDA
device is present, the call raises `KernelUnavailable`.
"""
from __future__ import annotations

import ctypes
from typing import Dict

from ..csrc import build as _build


class KernelUnavailable(RuntimeError):
    pass


class KernelError(RuntimeError):
    pass


_LIBS: Dict[str, ctypes.CDLL] = {}


def library(source: str) -> ctypes.CDLL:
    """The shared library compiled from csrc/<source>."""
    lib = _LIBS.get(source)
    if lib is None:
        try:
            path = _build.cuda_library(source)
            lib = ctypes.CDLL(path)
        except (_build.BuildError, OSError) as e:
            raise KernelUnavailable(
                f"the CUDA extension csrc/{source} is missing and could not be built: {e}") from None
        _LIBS[source] = lib
    return lib


def require_cuda() -> None:
    import torch

    if not torch.cuda.is_available():
        raise KernelUnavailable(
            "no CUDA device: this engine runs on sm_100a kernels only and has no CPU path")


LAUNCHES = [0]      # launches of this package's own kernels (library products not counted)


def check(code: int, what: str) -> None:
    if code == 0:
        LAUNCHES[0] += 1
        return
    if code == -1:
        raise KernelError(f"{what}: bad argument (dtype or shape combination not accepted)")
    if code == -2:
        raise KernelError(f"{what}: size not supported by this kernel")
    if code == -3:
        raise KernelError(f"{what}: size beyond the kernel's stated maximum")
    raise KernelError(f"{what}: CUDA error {code}")
