"""Kernel backend selection, kept for signature compatibility only.

The reference chooses between its JAX path and a Pallas kernel, with an environment override
and a silent fallback (kernels/backend.py:13-60).  Here there is one backend -- the sm_100a
CUDA library -- and no fallback, so every preference resolves to it.
"""

from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Optional


class KernelBackend(str, Enum):
    SM100 = "sm100"
    # Names the reference accepts; both resolve to the CUDA library.
    REFERENCE = "reference"
    PALLAS = "pallas"


@dataclass(frozen=True)
class BackendAvailability:
    sm100: bool
    pallas: bool = False


def backend_availability() -> BackendAvailability:
    from . import _lib
    return BackendAvailability(sm100=_lib.LIB_PATH.exists())


def select_kernel_backend(preferred: Optional[str] = None) -> KernelBackend:
    """Always ``KernelBackend.SM100``; unknown strings raise ValueError."""
    if preferred is not None and preferred.lower() not in {"", "auto", "reference", "pallas", "sm100", "cuda"}:
        raise ValueError(f"unknown kernel backend {preferred!r}")
    return KernelBackend.SM100
