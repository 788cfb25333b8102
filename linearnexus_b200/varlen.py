"""Variable-length (packed) batches: the padding helpers of the reference and the chunkwise ops over a packed batch.

``compute_unpadded_indices`` / ``unpad`` / ``pad`` mirror ``linearnexus/core/padding.py:13-53`` on torch tensors.
``chunkwise_varlen`` runs the chunkwise op over the packed tokens: every sequence starts from its own state and
is chunked from its own first token, so the result equals the reference op applied to each sequence alone -- which
is what the reference obtains by padding each sequence with zeros (padded rows have k = 0, beta = 0, g = 0 and
leave the state untouched, gated_deltanet.py:288-294), without spending kernel time on the padding.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence, Tuple

import torch

from . import _lib, ops
from ._lib import DR_DELTA, DR_GATED, DR_KDA, DR_LAYOUT_BTHD

Tensor = torch.Tensor


def compute_unpadded_indices(mask: Tensor) -> Tuple[Tensor, Tensor]:
    """``mask`` [batch, seq] (1 = valid token) -> ``(indices, cu_seqlens)``: flat positions of the valid tokens and
    the int32 prefix sums of the per-row counts (core/padding.py:13-34)."""
    if mask.dim() != 2:
        raise ValueError("mask must be rank-2 [batch, seq]")
    flat = mask.reshape(-1).to(torch.bool)
    indices = torch.nonzero(flat, as_tuple=False).reshape(-1).to(torch.int32)
    counts = mask.to(torch.int32).sum(dim=1, dtype=torch.int32)
    cu = torch.cat([torch.zeros(1, dtype=torch.int32, device=mask.device), torch.cumsum(counts, 0, dtype=torch.int32)])
    return indices, cu


def unpad(x: Tensor, indices: Tensor) -> Tensor:
    """Gather the valid tokens of ``x`` [batch, seq, ...] (core/padding.py:37-44)."""
    if x.dim() < 2:
        raise ValueError("x must be at least 2D (batch, seq, ...)")
    return x.reshape(x.shape[0] * x.shape[1], *x.shape[2:])[indices.long()]


def pad(x_flat: Tensor, indices: Tensor, batch: int, seq: int) -> Tensor:
    """Scatter packed tokens back to the zero-padded [batch, seq, ...] layout (core/padding.py:47-57)."""
    if x_flat.shape[0] != indices.shape[0]:
        raise ValueError("x_flat length must match indices length")
    out = x_flat.new_zeros((batch * seq,) + tuple(x_flat.shape[1:]))
    out[indices.long()] = x_flat
    return out.reshape((batch, seq) + tuple(x_flat.shape[1:]))


_VAR = {"delta": DR_DELTA, "gated": DR_GATED, "kda": DR_KDA}


def chunkwise_varlen(variant: str, q: Tensor, k: Tensor, v: Tensor, g: Optional[Tensor], beta: Tensor,
                     cu_seqlens: Sequence[int], initial_state: Optional[Tensor] = None, scale: Optional[float] = None,
                     chunk_size: int = 64, use_qk_l2norm: Optional[bool] = None, out_dtype=None) -> Tuple[Tensor, Tensor]:
    """Chunkwise op over a packed batch.  q, k ``[total_T, Hq, K]``, v ``[total_T, H, V]``, beta ``[total_T, H]``,
    g ``[total_T, H]`` ("gated") / ``[total_T, H, K]`` ("kda") / None ("delta"); ``cu_seqlens``: n_seqs + 1 token
    offsets (a tensor or a list; read on the host); ``initial_state`` ``[n_seqs, H, K, V]`` or None.
    Returns ``(o [total_T, H, V], final_state [n_seqs, H, K, V] float32)`` with the output dtype rules of the
    per-sequence op (q's dtype; float32 for "kda").  Differentiable: when an input requires grad the sequences go
    one by one through the autograd-aware ops and the results are concatenated."""
    if variant not in _VAR:
        raise ValueError(f"unknown variant {variant!r}")
    if (g is None) != (variant == "delta"):
        raise ValueError("g must be given for 'gated' / 'kda' and omitted for 'delta'")
    cu = [int(c) for c in (cu_seqlens.tolist() if isinstance(cu_seqlens, Tensor) else cu_seqlens)]
    n = len(cu) - 1
    if n < 1 or cu[0] != 0 or cu[-1] != q.shape[0] or any(b <= a for a, b in zip(cu, cu[1:])):
        raise ValueError("cu_seqlens must rise strictly from 0 to the number of packed tokens")
    if use_qk_l2norm is None:
        use_qk_l2norm = variant != "delta"
    total, Hq, K = q.shape
    H, V = v.shape[1], v.shape[2]
    if initial_state is not None and tuple(initial_state.shape) != (n, H, K, V):
        raise ValueError(f"initial_state must be [n_seqs,H,K,V]={n, H, K, V}")
    if ops._wants_grad(q, k, v, g, beta, initial_state):
        outs, states = [], []
        for i in range(n):
            sl = slice(cu[i], cu[i + 1])
            view = lambda t: None if t is None else t[sl].unsqueeze(0).transpose(1, 2)   # [1, heads, T_i, ...], no copy
            h0 = None if initial_state is None else initial_state[i:i + 1]
            if variant == "delta":
                o, s = ops.delta_rule_chunkwise(view(q), view(k), view(v), view(beta), h0, chunk_size=chunk_size, scale=scale)
            elif variant == "gated":
                o, s = ops.gated_delta_rule_chunkwise(view(q), view(k), view(v), view(g), view(beta), scale=scale,
                                                      initial_state=h0, chunk_size=chunk_size, use_qk_l2norm=use_qk_l2norm)
            else:
                o, s = ops.kda_chunkwise(view(q), view(k), view(v), view(g), view(beta), scale=scale, initial_state=h0,
                                         chunk_size=chunk_size, use_qk_l2norm=use_qk_l2norm, out_dtype=out_dtype)
            outs.append(o[0].transpose(0, 1))
            states.append(s)
        return torch.cat(outs, dim=0), torch.cat(states, dim=0)
    ops._require_cuda(q, k, v, g, beta, initial_state)
    if scale is None:
        scale = K ** -0.5
    dev = q.device
    native = ops._NATIVE
    common = torch.float32 if any(t.dtype not in native for t in (q, k, v)) or len({q.dtype, k.dtype, v.dtype}) > 1 else q.dtype
    qn, kn, vn = (t.to(common).contiguous() for t in (q, k, v))
    gn = None if g is None else ops._native(g).contiguous()
    bn = beta.to(torch.float32).contiguous()
    h0 = None if initial_state is None else initial_state.to(device=dev, dtype=torch.float32).contiguous()
    if out_dtype is None:
        out_dtype = torch.float32 if variant == "kda" else q.dtype
    native_out = out_dtype if out_dtype in native else torch.float32
    o = torch.empty((total, H, V), dtype=native_out, device=dev)
    hT = torch.empty((n, H, K, V), dtype=torch.float32, device=dev)
    longest = max(b - a for a, b in zip(cu, cu[1:]))
    d = ops._desc(_VAR[variant], DR_LAYOUT_BTHD, 1, H, longest, K, V, chunk_size, qn, gn, native_out, use_qk_l2norm, scale)
    d.qk_heads = Hq
    lib = _lib.load()
    need = int(lib.dr_workspace_bytes(ctypes.byref(d), 0))
    if need == -7:
        raise ValueError(f"chunk_size (BT={chunk_size}) must be divisible by BC=16.")
    _lib.check(need if need < 0 else 0, "dr_workspace_bytes")
    ws = torch.empty(need, dtype=torch.uint8, device=dev) if need > 0 else None
    cu_arr = (ctypes.c_int32 * (n + 1))(*cu)
    with torch.cuda.device(dev):
        st = lib.dr_chunk_fwd_varlen(ctypes.byref(d), ops._ptr(qn), ops._ptr(kn), ops._ptr(vn), ops._ptr(gn), ops._ptr(bn),
                                     cu_arr, n, ops._ptr(h0), ops._ptr(o), ops._ptr(hT), ops._ptr(ws), max(need, 0),
                                     ops._ptr(ops._status(dev)), ops._stream(dev))
    if st == -7:
        raise ValueError(f"chunk_size (BT={chunk_size}) must be divisible by BC=16.")
    _lib.check(st, "dr_chunk_fwd_varlen")
    return (o if o.dtype == out_dtype else o.to(out_dtype)), hT


def chunk_backward_varlen(variant: str, q: Tensor, k: Tensor, v: Tensor, g: Optional[Tensor], beta: Tensor, d_o: Tensor,
                          cu_seqlens: Sequence[int], initial_state: Optional[Tensor] = None,
                          d_final_state: Optional[Tensor] = None, scale: Optional[float] = None, chunk_size: int = 64,
                          use_qk_l2norm: Optional[bool] = None) -> dict:
    """Gradients of ``sum(o * d_o) + sum(final_state * d_final_state)`` of :func:`chunkwise_varlen` over a packed
    batch, in one library call (``dr_chunk_bwd_varlen``).  Tensors as in :func:`chunkwise_varlen`; ``d_o``
    ``[total_T, H, V]``, ``d_final_state`` ``[n_seqs, H, K, V]`` or None.  Returns a dict: dq, dk, dv in the q/k/v
    dtype, dbeta float32 ``[total_T, H]``, dg float32 like g (None for "delta"), dh0 float32 ``[n_seqs, H, K, V]``."""
    if variant not in _VAR:
        raise ValueError(f"unknown variant {variant!r}")
    if (g is None) != (variant == "delta"):
        raise ValueError("g must be given for 'gated' / 'kda' and omitted for 'delta'")
    cu = [int(c) for c in (cu_seqlens.tolist() if isinstance(cu_seqlens, Tensor) else cu_seqlens)]
    n = len(cu) - 1
    if n < 1 or cu[0] != 0 or cu[-1] != q.shape[0] or any(b <= a for a, b in zip(cu, cu[1:])):
        raise ValueError("cu_seqlens must rise strictly from 0 to the number of packed tokens")
    if use_qk_l2norm is None:
        use_qk_l2norm = variant != "delta"
    ops._require_cuda(q, k, v, g, beta, d_o, initial_state, d_final_state)
    total, Hq, K = q.shape
    H, V = v.shape[1], v.shape[2]
    if not ops.backward_supported(variant, K, chunk_size):
        raise NotImplementedError("the backward kernels cover chunk_size <= 64 and K <= 128 (K % 16 == 0 for 'kda')")
    for name, t in (("initial_state", initial_state), ("d_final_state", d_final_state)):
        if t is not None and tuple(t.shape) != (n, H, K, V):
            raise ValueError(f"{name} must be [n_seqs,H,K,V]={n, H, K, V}")
    if scale is None:
        scale = K ** -0.5
    dev = q.device
    native = ops._NATIVE
    common = torch.float32 if any(t.dtype not in native for t in (q, k, v)) or len({q.dtype, k.dtype, v.dtype}) > 1 else q.dtype
    qn, kn, vn, don = (t.to(common).contiguous() for t in (q, k, v, d_o))
    gn = None if g is None else ops._native(g).contiguous()
    bn = beta.to(torch.float32).contiguous()
    f32 = lambda t: None if t is None else t.to(device=dev, dtype=torch.float32).contiguous()
    h0, dhT = f32(initial_state), f32(d_final_state)
    longest = max(b - a for a, b in zip(cu, cu[1:]))
    d = ops._desc(_VAR[variant], DR_LAYOUT_BTHD, 1, H, longest, K, V, chunk_size, qn, gn, common, use_qk_l2norm, scale)
    d.qk_heads = Hq
    lib = _lib.load()
    need = int(lib.dr_workspace_bytes(ctypes.byref(d), 1))
    _lib.check(need if need < 0 else 0, "dr_workspace_bytes")
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
    dq, dk, dv = torch.empty_like(qn), torch.empty_like(kn), torch.empty_like(vn)
    dbeta = torch.empty((total, H), dtype=torch.float32, device=dev)
    dg = None if g is None else torch.empty(gn.shape, dtype=torch.float32, device=dev)
    dh0 = torch.empty((n, H, K, V), dtype=torch.float32, device=dev)
    cu_arr = (ctypes.c_int32 * (n + 1))(*cu)
    P = ops._ptr
    with torch.cuda.device(dev):
        st = lib.dr_chunk_bwd_varlen(ctypes.byref(d), P(qn), P(kn), P(vn), P(gn), P(bn), cu_arr, n, P(h0), P(don), P(dhT),
                                     P(dq), P(dk), P(dv), P(dbeta), P(dg), P(dh0), P(ws), ws.numel(),
                                     P(ops._status(dev)), ops._stream(dev))
    if st == -7:
        raise ValueError(f"chunk_size (BT={chunk_size}) must be divisible by BC=16.")
    _lib.check(st, "dr_chunk_bwd_varlen")
    return dict(dq=dq.to(q.dtype), dk=dk.to(k.dtype), dv=dv.to(v.dtype), dg=dg, dbeta=dbeta, dh0=dh0)
