"""CPU oracle for the element-wise steps around the delta-rule op (TEST INFRASTRUCTURE ONLY).

torch-on-CPU restatements of
  * ``depthwise_conv1d_causal`` (``linearnexus/core/conv.py:13-68``) followed by ``jax.nn.silu``
    (``gated_deltanet.py:764-783``),
  * the gate activations of the Gated DeltaNet block (``gated_deltanet.py:804-815``) and ``kda_gate``
    (``kda.py:120-172``),
  * ``RMSNorm`` (``modules/common.py:42-53``) with the sigmoid gate of ``gated_deltanet.py:853-865`` and
    ``FusedRMSNormGated`` (``kda.py:664-700``).
It checks the CUDA kernels of ``dr_block_ops.cuh``; it is never the product path.  Only ``tests/``,
``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline legs may import it.

PINNED against the reference's own source for the conv, ``kda_gate``, ``RMSNorm`` and ``FusedRMSNormGated``
(``tests/golden/reference_vectors.npz``: the reference's files executed over a numpy stand-in for ``jax.numpy``,
``tests/golden/make_reference_vectors.py``; checked in ``tests/test_reference_vectors.py``).  The two gate lines of
the Gated DeltaNet block sit inside its ``__call__`` and are restated from the cited lines only.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

Tensor = torch.Tensor


def short_conv_silu(x: Tensor, weight: Tensor, bias: Optional[Tensor] = None, cache: Optional[Tensor] = None,
                    apply_silu: bool = True, compute_dtype=torch.float32) -> Tuple[Tensor, Tensor]:
    """x [B,T,C], weight [W,C], cache [B,W-1,C] -> (y [B,T,C], new_cache [B,W-1,C]) (conv.py:34-68)."""
    B, T, C = x.shape
    W = weight.shape[0]
    if W < 1:
        raise ValueError("kernel_size must be >= 1")
    xf = x.to(compute_dtype)
    if W == 1:   # conv.py:39-44: the input itself (+ bias); the weight is not applied
        y = xf if bias is None else xf + bias.to(compute_dtype)
        new_cache = torch.zeros(B, 0, C, dtype=x.dtype)
    else:
        if cache is None:
            cache = torch.zeros(B, W - 1, C, dtype=x.dtype)
        if cache.shape != (B, W - 1, C):
            raise ValueError("cache shape must be (batch, kernel-1, channels)")
        xx = torch.cat([cache.to(compute_dtype), xf], dim=1)            # conv.py:56
        wf = weight.to(compute_dtype)
        # VALID cross-correlation, feature_group_count = channels: out[t] = sum_j w[j] xx[t + j]   (conv.py:57-64)
        y = torch.zeros(B, T, C, dtype=compute_dtype)
        for j in range(W):
            y = y + wf[j] * xx[:, j:j + T]
        if bias is not None:
            y = y + bias.to(compute_dtype)
        new_cache = torch.cat([cache, x], dim=1)[:, -(W - 1):]          # conv.py:67
    if apply_silu:
        y = y * torch.sigmoid(y)
    return y, new_cache


def gdn_gate_activations(a: Tensor, b: Tensor, A_log: Tensor, dt_bias: Tensor, allow_neg_eigval: bool = False,
                         compute_dtype=torch.float32) -> Tuple[Tensor, Tensor]:
    """a, b [B,T,H] -> g, beta [B,T,H] fp32 (gated_deltanet.py:804-815, before the transposes)."""
    beta = torch.sigmoid(b.to(compute_dtype))
    if allow_neg_eigval:
        beta = beta * 2.0
    g = -torch.exp(A_log.to(compute_dtype)) * torch.nn.functional.softplus(
        a.to(compute_dtype) + dt_bias.to(compute_dtype), beta=1.0, threshold=1e9)
    return g, beta


def kda_gate(g: Tensor, A_log: Tensor, head_k_dim: int, g_bias: Optional[Tensor] = None,
             beta: Optional[Tensor] = None, threshold: float = 20.0, compute_dtype=torch.float32):
    """g [B,T,H*K] -> g_out [B,T,H,K], sigmoid(beta) (kda.py:146-172; the result is returned in compute_dtype)."""
    if g_bias is not None:
        g = g + g_bias
    B, T, _ = g.shape
    H = A_log.shape[0]
    gf = g.reshape(B, T, H, head_k_dim).to(compute_dtype)
    a_exp = -torch.exp(A_log.to(compute_dtype))
    sp = torch.where(gf > threshold, gf, torch.nn.functional.softplus(gf, beta=1.0, threshold=1e9))
    g_out = a_exp[None, None, :, None] * sp
    beta_out = None if beta is None else torch.sigmoid(beta.to(compute_dtype))
    return g_out, beta_out


def gated_rmsnorm(o: Tensor, weight: Tensor, gate: Optional[Tensor] = None, eps: float = 1e-6,
                  compute_dtype=torch.float32) -> Tensor:
    """o [..., V], gate [..., V] or None -> x / sqrt(mean(x^2) + eps) * weight * sigmoid(gate)
    (common.py:52-53; gated_deltanet.py:862)."""
    xf = o.to(compute_dtype)
    rms = torch.sqrt(torch.mean(xf * xf, dim=-1, keepdim=True) + eps)
    y = xf / rms * weight.to(compute_dtype)
    if gate is not None:
        y = y * torch.sigmoid(gate.to(compute_dtype))
    return y
