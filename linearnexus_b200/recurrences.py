"""The other matrix-state scans of LinearNexus over the sm_100a C ABI: RWKV-7 DPLR, RWKV-6, Mamba-2 SSD.

Names, argument order, keyword defaults, shapes and output dtypes follow the LinearNexus functions cited per
function (paths relative to the LinearNexus tree); arrays are torch CUDA tensors.  All three run the token
recurrence with the float32 state in registers (``csrc/dr_linrec.cuh``); a chunked tensor-core form exists for the
delta-rule family only.  There is no CPU path.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import DR_LAYOUT_BHTD, DR_LAYOUT_BTHD
from .ops import _NATIVE, _is_bthd_view, _native, _ptr, _require_cuda, _status, _stream

Tensor = torch.Tensor


def _common_io(*ts) -> list:
    """Activations travel in one dtype: bf16 if all are bf16, else float32."""
    ts = [_native(t) for t in ts]
    if any(t.dtype != ts[0].dtype for t in ts):
        ts = [t.float() for t in ts]
    return ts


def _layout4(ts):
    if ts[0].shape[1] > 1 and ts[0].shape[2] > 1 and all(_is_bthd_view(t) for t in ts):
        return DR_LAYOUT_BTHD, list(ts)
    return DR_LAYOUT_BHTD, [t.contiguous() for t in ts]


def _state(x: Optional[Tensor], shape, dev) -> Optional[Tensor]:
    if x is None:
        return None
    if tuple(x.shape) != tuple(shape):
        raise ValueError(f"state must be {tuple(shape)}, got {tuple(x.shape)}")
    return x.to(device=dev, dtype=torch.float32).contiguous()


def _empty_like_layout(ref: Tensor, last: int, layout: int) -> Tensor:
    B, H, T, _ = ref.shape
    if layout == DR_LAYOUT_BTHD:
        return torch.empty(B, T, H, last, device=ref.device, dtype=ref.dtype).transpose(1, 2)
    return torch.empty(B, H, T, last, device=ref.device, dtype=ref.dtype)


# ---- RWKV-7 DPLR (modules/linear_attn/rwkv7.py) ----------------------------------------------------------------

def dplr_delta_rule_recurrent(q: Tensor, k: Tensor, v: Tensor, a: Tensor, b: Tensor, gk: Tensor, scale: float = 1.0,
                              initial_state: Optional[Tensor] = None, _out_state: Optional[Tensor] = None
                              ) -> Tuple[Tensor, Tensor]:
    """``h <- exp(gk) h + b (a^T h) + k v^T;  o = h^T (q scale)`` over the tokens (rwkv7.py:114-214).
    q, k, a, b, gk ``[B,H,T,K]``, v ``[B,H,T,V]`` -> o ``[B,H,T,V]`` in q's dtype, final state float32 ``[B,H,K,V]``."""
    _require_cuda(q, k, v, a, b, gk, initial_state)
    if q.dim() != 4 or any(t.shape != q.shape for t in (k, a, b, gk)) or v.shape[:3] != q.shape[:3]:
        raise ValueError("expected q, k, a, b, gk [B,H,T,K] and v [B,H,T,V]")
    B, H, T, K = q.shape
    V = v.shape[-1]
    od = q.dtype
    layout, (q, k, v, a, b, gk) = _layout4(_common_io(q, k, v, a, b, gk))
    h0 = _state(initial_state, (B, H, K, V), q.device)
    hT = _out_state if _out_state is not None else torch.empty(B, H, K, V, device=q.device, dtype=torch.float32)
    if T == 0:
        hT.copy_(h0) if h0 is not None else hT.zero_()
        return q.new_empty(B, H, 0, V).to(od), hT
    o = _empty_like_layout(q, V, layout)
    with torch.cuda.device(q.device):
        st = _lib.load().dr_dplr_recurrent(_ptr(q), _ptr(k), _ptr(v), _ptr(a), _ptr(b), _ptr(gk), _ptr(h0), _ptr(o), _ptr(hT),
                                           B, H, T, K, V, float(scale), _NATIVE[q.dtype], layout, _ptr(_status(q.device)), _stream(q.device))
    _lib.check(st, "dr_dplr_recurrent")
    return o.to(od), hT


def dplr_delta_rule_step(q: Tensor, k: Tensor, v: Tensor, a: Tensor, b: Tensor, gk: Tensor, state: Tensor,
                         scale: float = 1.0, inplace: bool = False) -> Tuple[Tensor, Tensor]:
    """One token (rwkv7.py:217-259): inputs ``[B,H,K]`` / ``[B,H,V]``, state ``[B,H,K,V]``.  ``inplace=True`` (an
    extension) updates a float32 contiguous state cache where it lies."""
    u = lambda t: t.unsqueeze(2)
    if inplace and not (state.dtype == torch.float32 and state.is_contiguous()):
        raise ValueError("inplace=True needs a contiguous float32 state")
    o, hT = dplr_delta_rule_recurrent(u(q), u(k), u(v), u(a), u(b), u(gk), scale, state,
                                      _out_state=state if inplace else None)
    return o.squeeze(2), hT


# ---- RWKV-6 (modules/linear_attn/rwkv6.py) ---------------------------------------------------------------------

def rwkv6_recurrent(r: Tensor, k: Tensor, v: Tensor, w: Tensor, u: Tensor, scale: float = 1.0,
                    initial_state: Optional[Tensor] = None, _out_state: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
    """``o = (h + (u k) v^T)^T (sigmoid(r) scale);  h <- exp(-exp(w)) h + k v^T`` (rwkv6.py:115-189).
    r, k, w ``[B,H,T,K]``, v ``[B,H,T,V]``, u ``[H,K]`` -> o in r's dtype, final state float32."""
    _require_cuda(r, k, v, w, u, initial_state)
    if r.dim() != 4 or k.shape != r.shape or w.shape != r.shape or v.shape[:3] != r.shape[:3]:
        raise ValueError("expected r, k, w [B,H,T,K] and v [B,H,T,V]")
    B, H, T, K = r.shape
    V = v.shape[-1]
    if tuple(u.shape) != (H, K):
        raise ValueError(f"u must be [H,K]={H, K}, got {tuple(u.shape)}")
    od = r.dtype
    layout, (r, k, v, w) = _layout4(_common_io(r, k, v, w))
    u32 = u.to(torch.float32).contiguous()
    h0 = _state(initial_state, (B, H, K, V), r.device)
    hT = _out_state if _out_state is not None else torch.empty(B, H, K, V, device=r.device, dtype=torch.float32)
    if T == 0:
        hT.copy_(h0) if h0 is not None else hT.zero_()
        return r.new_empty(B, H, 0, V).to(od), hT
    o = _empty_like_layout(r, V, layout)
    with torch.cuda.device(r.device):
        st = _lib.load().dr_rwkv6_recurrent(_ptr(r), _ptr(k), _ptr(v), _ptr(w), _ptr(u32), _ptr(h0), _ptr(o), _ptr(hT),
                                            B, H, T, K, V, float(scale), _NATIVE[r.dtype], layout, _ptr(_status(r.device)), _stream(r.device))
    _lib.check(st, "dr_rwkv6_recurrent")
    return o.to(od), hT


def rwkv6_chunkwise(r: Tensor, k: Tensor, v: Tensor, w: Tensor, u: Tensor, scale: float = 1.0,
                    initial_state: Optional[Tensor] = None, chunk_size: int = 32) -> Tuple[Tensor, Tensor]:
    """Same result as :func:`rwkv6_recurrent`.  The reference's own chunk function (rwkv6.py:192-357) cannot be
    matched: its first einsum names five axes for a four-axis operand and raises, and it reads ``w`` as a plain log
    decay where the recurrence uses ``exp(-exp(w))``.  ``RWKV6Block`` itself calls ``rwkv6_recurrent`` in "chunk"
    mode (rwkv6.py:837-850, with the note that the chunk form is wrong), so that is the function a caller of the
    block gets.  ``chunk_size`` is accepted and ignored."""
    return rwkv6_recurrent(r, k, v, w, u, scale, initial_state)


def rwkv6_step(r: Tensor, k: Tensor, v: Tensor, w: Tensor, u: Tensor, state: Tensor, scale: float = 1.0,
               inplace: bool = False) -> Tuple[Tensor, Tensor]:
    """One token (rwkv6.py:360-398): inputs ``[B,H,K]`` / ``[B,H,V]``, state ``[B,H,K,V]``; the output takes the
    promoted dtype of state and r as in the reference."""
    if inplace and not (state.dtype == torch.float32 and state.is_contiguous()):
        raise ValueError("inplace=True needs a contiguous float32 state")
    x = lambda t: t.unsqueeze(2)
    o, hT = rwkv6_recurrent(x(r), x(k), x(v), x(w), u, scale, state, _out_state=state if inplace else None)
    return o.squeeze(2).to(torch.promote_types(state.dtype, r.dtype)), hT


# ---- Mamba-2 SSD (modules/ssm/mamba2.py) -----------------------------------------------------------------------

def ssd_chunk_scan(hidden_states: Tensor, dt: Tensor, A: Tensor, B: Tensor, C: Tensor, D: Tensor, *,
                   chunk_size: int = 256, n_groups: int = 1, ssm_state: Optional[Tensor] = None,
                   dt_bias: Optional[Tensor] = None, dt_min: float = 0.001, dt_max: float = 0.1,
                   dt_limit: Tuple[float, float] = (0.0, float("inf")), _out_state: Optional[Tensor] = None
                   ) -> Tuple[Tensor, Tensor]:
    """The SSD scan (mamba2.py:161-348): ``dt' = clip(softplus(dt + dt_bias), dt_limit)``,
    ``state <- exp(A dt') state + (dt' x) B^T``, ``y = state C + D x``.  hidden_states ``[B,T,H,P]``, dt ``[B,T,H]``,
    A, D ``[H]``, B, C ``[B,T,G,N]`` -> y ``[B,T,H,P]``, state float32 ``[B,H,P,N]``.  ``chunk_size`` does not change
    the result (the reference's chunked evaluation equals this recurrence); ``dt_min`` / ``dt_max`` are unused
    there as well."""
    x = hidden_states
    _require_cuda(x, dt, A, B, C, D, ssm_state, dt_bias)
    if x.dim() != 4 or dt.shape != x.shape[:3] or B.dim() != 4 or C.shape != B.shape or B.shape[:2] != x.shape[:2]:
        raise ValueError("expected hidden_states [B,T,H,P], dt [B,T,H], B and C [B,T,G,N]")
    Bt, T, H, P = x.shape
    G, N = B.shape[2], B.shape[3]
    if G != n_groups or H % G:
        raise ValueError(f"B/C carry {G} groups; n_groups={n_groups}, heads={H}")
    od = x.dtype
    x, Bm, Cm = (t.contiguous() for t in _common_io(x, B, C))
    dtn = dt.to(torch.float32).contiguous()
    f32 = lambda t: None if t is None else t.to(torch.float32).contiguous()
    A32, D32, bias32 = f32(A), f32(D), f32(dt_bias)
    h0 = _state(ssm_state, (Bt, H, P, N), x.device)
    hT = _out_state if _out_state is not None else torch.empty(Bt, H, P, N, device=x.device, dtype=torch.float32)
    if T == 0:   # mamba2.py:218-220
        hT.copy_(h0) if h0 is not None else hT.zero_()
        return x.new_empty(Bt, 0, H, P).to(od), hT
    y = torch.empty_like(x)
    lo, hi = float(dt_limit[0]), min(float(dt_limit[1]), 3.0e38)
    with torch.cuda.device(x.device):
        st = _lib.load().dr_ssd_scan(_ptr(x), _ptr(dtn), _ptr(A32), _ptr(Bm), _ptr(Cm), _ptr(D32), _ptr(bias32), _ptr(h0),
                                     _ptr(y), _ptr(hT), Bt, T, H, P, N, G, lo, hi, _NATIVE[x.dtype], _ptr(_status(x.device)), _stream(x.device))
    _lib.check(st, "dr_ssd_scan")
    return y.to(od), hT


def ssd_recurrent_step(hidden_state: Tensor, dt: Tensor, A: Tensor, B: Tensor, C: Tensor, D: Tensor, ssm_state: Tensor, *,
                       n_groups: int = 1, dt_bias: Optional[Tensor] = None,
                       dt_limit: Tuple[float, float] = (0.0, float("inf")), inplace: bool = False) -> Tuple[Tensor, Tensor]:
    """One token (mamba2.py:351-425): hidden_state ``[B,H,P]``, dt ``[B,H]``, B, C ``[B,G,N]``, state ``[B,H,P,N]``."""
    if inplace and not (ssm_state.dtype == torch.float32 and ssm_state.is_contiguous()):
        raise ValueError("inplace=True needs a contiguous float32 state")
    y, hT = ssd_chunk_scan(hidden_state.unsqueeze(1), dt.unsqueeze(1), A, B.unsqueeze(1), C.unsqueeze(1), D,
                           n_groups=n_groups, ssm_state=ssm_state, dt_bias=dt_bias, dt_limit=dt_limit,
                           _out_state=ssm_state if inplace else None)
    return y.squeeze(1), hT
