"""Seeded synthetic inputs with the value distributions of the reference's own benchmarks.

q, k ~ N(0,1), l2-normalised over the last axis in fp32; v ~ N(0,1); beta = sigmoid(N(0,1));
g = logsigmoid(N(0,1) + 4) -- one scalar per token for "gated", one per key channel for "kda"
(benchmarks/bench_kda_kernels.py:120-129 of the reference draws the same families with the JAX PRNG, which
cannot be reproduced without JAX; numpy's ``default_rng`` stands in for it).

Every batch row is drawn from its own seed (``seed * 4096 + row``), so a rank of a multi-GPU run can build
just its rows of the global batch and gets exactly the tensors a single process would have cut out of it.
"""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np
import torch

Tensor = torch.Tensor


def _l2norm(x: Tensor) -> Tensor:
    return x / (x.norm(dim=-1, keepdim=True) + 1e-6)


def make_row(variant: str, H: int, T: int, K: int, V: int, seed: int, row: int, io_dtype=torch.float32,
             h0_std: Optional[float] = None, g_dtype=torch.float32) -> Dict[str, Optional[Tensor]]:
    """One batch row ``[1, H, ...]`` of the global batch defined by ``seed``."""
    rng = np.random.default_rng(int(seed) * 4096 + int(row))
    f = lambda *s: torch.from_numpy(rng.standard_normal(s, dtype=np.float32))
    q, k, v = _l2norm(f(1, H, T, K)), _l2norm(f(1, H, T, K)), f(1, H, T, V)
    beta = torch.sigmoid(f(1, H, T))
    g = None
    if variant == "gated":
        g = torch.nn.functional.logsigmoid(f(1, H, T) + 4.0).to(g_dtype)
    elif variant == "kda":
        g = torch.nn.functional.logsigmoid(f(1, H, T, K) + 4.0).to(g_dtype)
    elif variant != "delta":
        raise ValueError(f"unknown variant {variant!r}")
    h0 = None if h0_std is None else f(1, H, K, V) * h0_std
    return dict(q=q.to(io_dtype), k=k.to(io_dtype), v=v.to(io_dtype), g=g, beta=beta, h0=h0)


def make_rows(variant: str, lo: int, hi: int, H: int, T: int, K: int, V: int, seed: int, **kw) -> Dict[str, Optional[Tensor]]:
    """Rows ``lo .. hi-1`` of the global batch: ``{q, k, v, g, beta, h0}`` with leading size ``hi - lo``."""
    rows = [make_row(variant, H, T, K, V, seed, r, **kw) for r in range(lo, hi)]
    return {name: (None if rows[0][name] is None else torch.cat([r[name] for r in rows], dim=0)) for name in rows[0]}
