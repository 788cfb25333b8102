"""CPU oracle for the RWKV-7 DPLR, RWKV-6 and Mamba-2 SSD scans (TEST INFRASTRUCTURE ONLY).

Restates in torch-on-CPU the pure functions of ``linearnexus/modules/linear_attn/rwkv7.py``,
``linearnexus/modules/linear_attn/rwkv6.py`` and ``linearnexus/modules/ssm/mamba2.py`` that
carry a matrix state across tokens.  It is the checker for the CUDA kernels, never the
product path; only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline /
``--impl reference`` legs may import it.

PINNED against the reference's own source: ``tests/golden/reference_vectors.npz`` holds
inputs and outputs of the reference's functions themselves, executed over a numpy stand-in
for ``jax.numpy`` (``tests/golden/make_reference_vectors.py``);
``tests/test_reference_vectors.py`` checks every function here against them.

``compute_dtype``: ``torch.float32`` follows the reference, ``torch.float64`` is the
mathematical truth for kernel checks.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

Tensor = torch.Tensor


def _state0(initial_state, shape, cd):
    return torch.zeros(*shape, dtype=cd) if initial_state is None else initial_state.to(cd).clone()


# ---- RWKV-7: diagonal-plus-low-rank transition (rwkv7.py) ----------------------------------------------------

def dplr_delta_rule_step(q, k, v, a, b, gk, state, scale: float = 1.0, compute_dtype=torch.float32):
    """One token, rwkv7.py:217-259: h <- exp(gk) * h + b (a^T h); h <- h + k v^T; o = h^T (q * scale)."""
    cd = compute_dtype
    od = q.dtype
    q, k, v, a, b, gk, h = (x.to(cd) for x in (q, k, v, a, b, gk, state))
    q = q * scale
    a_h = torch.einsum("bhk,bhkv->bhv", a, h)
    h = torch.exp(gk)[..., None] * h + b[..., None] * a_h[..., None, :]
    h = h + torch.einsum("bhk,bhv->bhkv", k, v)
    o = torch.einsum("bhkv,bhk->bhv", h, q)
    return (o.to(od) if cd == torch.float32 else o), h


def dplr_delta_rule_recurrent(q, k, v, a, b, gk, scale: float = 1.0, initial_state=None,
                              compute_dtype=torch.float32) -> Tuple[Tensor, Tensor]:
    """Scan of the step over tokens, rwkv7.py:114-214.  q, k, a, b, gk [B,H,T,K], v [B,H,T,V]."""
    cd = compute_dtype
    B, H, T, K = q.shape
    h = _state0(initial_state, (B, H, K, v.shape[-1]), cd)
    outs = []
    for t in range(T):
        o, h = dplr_delta_rule_step(q[:, :, t].to(cd), k[:, :, t], v[:, :, t], a[:, :, t], b[:, :, t], gk[:, :, t], h,
                                    scale, cd)
        outs.append(o)
    o = torch.stack(outs, dim=2) if outs else torch.zeros(B, H, 0, v.shape[-1], dtype=cd)
    return (o.to(q.dtype) if cd == torch.float32 else o), h


# ---- RWKV-6: per-channel decay with a bonus on the current token (rwkv6.py) ----------------------------------

def rwkv6_step(r, k, v, w, u, state, scale: float = 1.0, compute_dtype=torch.float32):
    """One token, rwkv6.py:360-398: o = (h + u k v^T)^T (sigmoid(r) * scale); h <- h * exp(-exp(w)) + k v^T.
    The output reads the state BEFORE this token's decay and write."""
    cd = compute_dtype
    r, k, v, w, u, h = (x.to(cd) for x in (r, k, v, w, u, state))
    r = torch.sigmoid(r) * scale
    kv = torch.einsum("bhk,bhv->bhkv", k, v)
    o = torch.einsum("bhkv,bhk->bhv", h + u[None, :, :, None] * kv, r)
    h = h * torch.exp(-torch.exp(w))[..., None] + kv
    return o, h


def rwkv6_recurrent(r, k, v, w, u, scale: float = 1.0, initial_state=None,
                    compute_dtype=torch.float32) -> Tuple[Tensor, Tensor]:
    """Scan of the step, rwkv6.py:115-189.  r, k, w [B,H,T,K], v [B,H,T,V], u [H,K]."""
    cd = compute_dtype
    B, H, T, K = r.shape
    h = _state0(initial_state, (B, H, K, v.shape[-1]), cd)
    outs = []
    for t in range(T):
        o, h = rwkv6_step(r[:, :, t], k[:, :, t], v[:, :, t], w[:, :, t], u, h, scale, cd)
        outs.append(o)
    o = torch.stack(outs, dim=2) if outs else torch.zeros(B, H, 0, v.shape[-1], dtype=cd)
    return (o.to(r.dtype) if cd == torch.float32 else o), h


# ---- Mamba-2 SSD (mamba2.py) ---------------------------------------------------------------------------------

def _dt_activation(dt, dt_bias, dt_limit):
    if dt_bias is not None:
        dt = dt + dt_bias
    dt = torch.nn.functional.softplus(dt, threshold=1e9)   # jax.nn.softplus has no linear cut-over
    return torch.clamp(dt, dt_limit[0], dt_limit[1])


def segment_sum(x: Tensor) -> Tensor:
    """mamba2.py:127-158: out[..., i, j] = sum_{j < m <= i} x[..., m] for j <= i, -inf above the diagonal."""
    L = x.shape[-1]
    e = x[..., None].expand(*x.shape, L)
    below = torch.tril(torch.ones(L, L, dtype=torch.bool), -1)
    c = torch.cumsum(torch.where(below, e, torch.zeros((), dtype=x.dtype)), dim=-2)
    lower = torch.tril(torch.ones(L, L, dtype=torch.bool), 0)
    return torch.where(lower, c, torch.full((), float("-inf"), dtype=x.dtype))


def ssd_recurrent_step(hidden_state, dt, A, B, C, D, ssm_state, *, n_groups: int = 1, dt_bias=None,
                       dt_limit=(0.0, float("inf")), compute_dtype=torch.float32):
    """One token, mamba2.py:351-425.  hidden_state [B,H,P], dt [B,H], B/C [B,G,N], state [B,H,P,N]:
    state <- exp(A dt) state + (dt x) B^T;  y = state C + D x."""
    cd = compute_dtype
    x, dt, A, Bm, Cm, D, h = (t.to(cd) for t in (hidden_state, dt, A, B, C, D, ssm_state))
    H = x.shape[1]
    dt = _dt_activation(dt, None if dt_bias is None else dt_bias.to(cd)[None, :], dt_limit)
    Bm = Bm.repeat_interleave(H // n_groups, dim=1)
    Cm = Cm.repeat_interleave(H // n_groups, dim=1)
    dA = torch.exp(A[None, :, None, None] * dt[..., None, None])
    dBx = (dt[..., None, None] * Bm[:, :, None, :]) * x[..., None]
    h = dA * h + dBx
    y = torch.einsum("bhds,bhs->bhd", h, Cm) + D[None, :, None] * x
    return y, h


def ssd_chunk_scan(hidden_states, dt, A, B, C, D, *, chunk_size: int = 256, n_groups: int = 1, ssm_state=None,
                   dt_bias=None, dt_min: float = 0.001, dt_max: float = 0.1, dt_limit=(0.0, float("inf")),
                   compute_dtype=torch.float32) -> Tuple[Tensor, Tensor]:
    """The chunked scan in the reference's five steps, mamba2.py:161-348.  hidden_states [B,T,H,P], dt [B,T,H],
    A, D [H], B/C [B,T,G,N]; returns y [B,T,H,P] and the state [B,H,P,N]."""
    cd = compute_dtype
    x, dt, A, Bm, Cm, D = (t.to(cd) for t in (hidden_states, dt, A, B, C, D))
    Bt, T, H, P = x.shape
    N = Bm.shape[-1]
    dt = _dt_activation(dt, None if dt_bias is None else dt_bias.to(cd)[None, None, :], dt_limit)
    Bm = Bm.repeat_interleave(H // n_groups, dim=2)
    Cm = Cm.repeat_interleave(H // n_groups, dim=2)
    h0 = _state0(ssm_state, (Bt, H, P, N), cd)
    if T == 0:
        return torch.zeros(Bt, 0, H, P, dtype=cd), h0
    pad = (chunk_size - T % chunk_size) % chunk_size

    def padt(t):   # zero padding along the token axis (mamba2.py:226-233)
        if pad == 0:
            return t
        return torch.cat([t, torch.zeros(t.shape[0], pad, *t.shape[2:], dtype=t.dtype)], dim=1)

    d_res = padt(x * D[None, None, :, None])
    xd = padt(x * dt[..., None])
    a_dt = padt(A[None, None, :] * dt)
    Bm, Cm = padt(Bm), padt(Cm)
    nc = (T + pad) // chunk_size
    xd = xd.reshape(Bt, nc, chunk_size, H, P)
    a_dt = a_dt.reshape(Bt, nc, chunk_size, H)
    Bc = Bm.reshape(Bt, nc, chunk_size, H, N)
    Cc = Cm.reshape(Bt, nc, chunk_size, H, N)
    d_res = d_res.reshape(Bt, nc, chunk_size, H, P)
    a_perm = a_dt.permute(0, 1, 3, 2)                       # [B, nc, H, cs]
    a_cum = torch.cumsum(a_perm, dim=-1)
    # 1. inside a chunk
    Lm = torch.exp(segment_sum(a_perm))
    G = torch.einsum("bclhn,bckhn->bchlk", Cc, Bc)
    y_diag = torch.einsum("bchlk,bchkd->bchld", G * Lm, xd.permute(0, 1, 3, 2, 4))
    # 2. what each chunk adds to the state
    decay_states = torch.exp(a_cum[..., -1:] - a_cum)
    states = torch.einsum("bnchs,bnchd->bnhds", Bc * decay_states.permute(0, 1, 3, 2)[..., None], xd)
    # 3. chunk-to-chunk recurrence
    states = torch.cat([h0[:, None], states], dim=1)
    a_end = torch.nn.functional.pad(a_cum[..., -1], (0, 0, 1, 0))     # [B, nc+1, H]
    decay_chunk = torch.exp(segment_sum(a_end.permute(0, 2, 1))).permute(0, 2, 3, 1)
    new_states = torch.einsum("bnmh,bmhds->bnhds", decay_chunk, states)
    chunk_states, final = new_states[:, :-1], new_states[:, -1]
    # 4. state -> output
    y_off = torch.einsum("bnchs,bnhds->bnchd", Cc, chunk_states) * torch.exp(a_cum).permute(0, 1, 3, 2)[..., None]
    y = y_diag.permute(0, 1, 3, 2, 4) + y_off + d_res
    return y.reshape(Bt, nc * chunk_size, H, P)[:, :T], final


def ssd_token_recurrence(hidden_states, dt, A, B, C, D, *, n_groups: int = 1, ssm_state=None, dt_bias=None,
                         dt_limit=(0.0, float("inf")), compute_dtype=torch.float64) -> Tuple[Tensor, Tensor]:
    """The step applied token by token: the function the chunked scan equals (the reference's Mamba2Block decodes
    with it after a chunked prefill, mamba2.py:351-425)."""
    Bt, T, H, P = hidden_states.shape
    h = _state0(ssm_state, (Bt, H, P, B.shape[-1]), compute_dtype)
    ys = []
    for t in range(T):
        y, h = ssd_recurrent_step(hidden_states[:, t], dt[:, t], A, B[:, t], C[:, t], D, h, n_groups=n_groups,
                                  dt_bias=dt_bias, dt_limit=dt_limit, compute_dtype=compute_dtype)
        ys.append(y)
    y = torch.stack(ys, dim=1) if ys else torch.zeros(Bt, 0, H, P, dtype=compute_dtype)
    return y, h
