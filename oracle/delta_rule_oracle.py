"""CPU oracle for the delta-rule linear-attention ops (TEST INFRASTRUCTURE ONLY).

This module restates, in torch-on-CPU, the nine pure functions of
``linearnexus/modules/linear_attn/{delta_net,gated_deltanet,kda}.py`` in the
order of operations the reference uses (where the fp32 cast sits relative to the
l2 normalisation and the scale multiply, the ``x / (||x|| + 1e-6)`` eps placement,
the ``exp(min(x, 0))`` clamps, zero padding of ragged chunks, and the output dtype
quirks).  It is the checker for the CUDA kernels; it is never the product path.
Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline /
``--impl reference`` legs may import it.

PINNED against the reference's own source: ``tests/golden/reference_vectors.npz`` holds inputs and
outputs of the reference's nine functions themselves, their source files executed over a numpy
stand-in for ``jax.numpy`` / ``lax.scan`` (``tests/golden/make_reference_vectors.py``; JAX is
not installed where this was written, and the reference ships no golden vectors).
``tests/test_reference_vectors.py`` holds every function here, in float32 and in float64, within
float32 round-off (2e-5) of those outputs, at K = V = 32/48 and at the K = V = 128, chunk 64 shapes
of the tensor-core kernels.  The gradients are the autograd of this pinned forward (the reference's
are JAX autodiff of its forward, which the stand-in cannot run).  The reference's own
self-consistency tests are re-expressed as well (chunk == recurrent, step == recurrent at T=1,
beta=0 keeps the state at zero; ``tests/test_deltanet.py:64-157,281-346``,
``tests/test_gated_deltanet.py:310-339``, ``tests/test_kda.py:219-290``).

``compute_dtype`` selects the arithmetic type: ``torch.float32`` follows the
reference (which computes everything in fp32), ``torch.float64`` gives the
mathematical truth against which both the fp32 restatement and the kernels are checked.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

Tensor = torch.Tensor


def _l2norm(x: Tensor) -> Tensor:
    # x / (||x||_2 + 1e-6), eps added to the norm (gated_deltanet.py:194-195, kda.py:244-245)
    return x / (torch.linalg.vector_norm(x, dim=-1, keepdim=True) + 1e-6)


def _state0(initial_state, b, h, kd, vd, cd):
    if initial_state is None:
        return torch.zeros(b, h, kd, vd, dtype=cd)
    return initial_state.to(cd).clone()


# ----------------------------------------------------------------------------
# DeltaNet  (delta_net.py)
# ----------------------------------------------------------------------------

def delta_rule_recurrent(q, k, v, beta, initial_state=None, scale=None, backend=None,
                         compute_dtype=torch.float32) -> Tuple[Tensor, Tensor]:
    """Token recurrence without decay; follows delta_net.py:126-213.

    No l2norm inside the op; inputs cast to fp32 first and q pre-scaled
    (delta_net.py:170-173); output uses the updated state (delta_net.py:194-198).
    """
    cd = compute_dtype
    B, H, T, K = q.shape
    V = v.shape[-1]
    od = q.dtype
    if scale is None:
        scale = K ** -0.5
    if beta.ndim == 4:
        beta = beta.squeeze(-1)
    q = q.to(cd) * torch.tensor(scale, dtype=cd)
    k = k.to(cd)
    v = v.to(cd)
    beta = beta.to(cd)
    S = _state0(initial_state, B, H, K, V, cd)
    out = torch.empty(B, H, T, V, dtype=cd)
    for t in range(T):
        k_t, v_t, q_t, b_t = k[:, :, t], v[:, :, t], q[:, :, t], beta[:, :, t]
        v_old = torch.einsum("bhkv,bhk->bhv", S, k_t)
        v_delta = b_t[..., None] * (v_t - v_old)
        S = S + torch.einsum("bhk,bhv->bhkv", k_t, v_delta)
        out[:, :, t] = torch.einsum("bhk,bhkv->bhv", q_t, S)
    return out.to(od), S.to(torch.float32 if cd == torch.float32 else cd)


def delta_rule_chunkwise(q, k, v, beta, initial_state=None, chunk_size=64, scale=None,
                         backend=None, compute_dtype=torch.float32):
    """WY chunk form; follows delta_net.py:216-354 (``backend`` is ignored there too)."""
    cd = compute_dtype
    B, H, T, K = q.shape
    V = v.shape[-1]
    od = q.dtype
    if scale is None:
        scale = K ** -0.5
    if beta.ndim == 4:
        beta = beta.squeeze(-1)
    q = q.to(cd) * torch.tensor(scale, dtype=cd)
    k = k.to(cd)
    v = v.to(cd)
    beta = beta.to(cd)
    C = chunk_size
    pad = (C - T % C) % C
    if pad:
        q = torch.nn.functional.pad(q, (0, 0, 0, pad))
        k = torch.nn.functional.pad(k, (0, 0, 0, pad))
        v = torch.nn.functional.pad(v, (0, 0, 0, pad))
        beta = torch.nn.functional.pad(beta, (0, pad))
    Tp = T + pad
    N = Tp // C
    qc = q.reshape(B, H, N, C, K)
    kc = k.reshape(B, H, N, C, K)
    vc = v.reshape(B, H, N, C, V)
    bc = beta.reshape(B, H, N, C)
    S = _state0(initial_state, B, H, K, V, cd)
    eye = torch.eye(C, dtype=cd)
    causal = torch.tril(torch.ones(C, C, dtype=cd))
    outs = []
    for n in range(N):
        q_c, k_c, v_c, b_c = qc[:, :, n], kc[:, :, n], vc[:, :, n], bc[:, :, n]
        kk = torch.einsum("bhik,bhjk->bhij", k_c, k_c)
        A = torch.tril(b_c[..., :, None] * kk, diagonal=-1)
        A_inv = torch.linalg.solve_triangular(eye + A, eye.expand_as(A).contiguous(), upper=False)
        w = A_inv @ (k_c * b_c[..., None])
        u = A_inv @ (v_c * b_c[..., None])
        v_new = u - w @ S
        o = q_c @ S + (torch.einsum("bhik,bhjk->bhij", q_c, k_c) * causal) @ v_new
        S = S + k_c.transpose(-1, -2) @ v_new
        outs.append(o)
    out = torch.stack(outs, dim=2).reshape(B, H, Tp, V)[:, :, :T]
    return out.to(od), S


def delta_rule_step(q, k, v, beta, state, scale=None, compute_dtype=torch.float32):
    """One token; follows delta_net.py:357-397."""
    cd = compute_dtype
    if beta.ndim == 3:
        beta = beta.squeeze(-1)
    K = q.shape[-1]
    if scale is None:
        scale = K ** -0.5
    od = q.dtype
    q = q.to(cd) * torch.tensor(scale, dtype=cd)
    k = k.to(cd)
    v = v.to(cd)
    beta = beta.to(cd)
    S = state.to(cd)
    v_old = torch.einsum("bhkv,bhk->bhv", S, k)
    v_delta = beta[..., None] * (v - v_old)
    S_new = S + torch.einsum("bhk,bhv->bhkv", k, v_delta)
    o = torch.einsum("bhk,bhkv->bhv", q, S_new)
    return o.to(od), S_new


def delta_rule_recurrent_pallas(q, k, v, beta, initial_state=None, scale=None,
                                compute_dtype=torch.float32):
    """Same maths as delta_rule_recurrent (kernels/pallas/delta_rule.py:47-128), including
    its shape guards: key_dim % 32 and value_dim % 64 raise RuntimeError (:108-115)."""
    K, V = q.shape[-1], v.shape[-1]
    if K % 32 != 0:
        raise RuntimeError("key_dim must be a multiple of 32")
    if V % 64 != 0:
        raise RuntimeError("value_dim must be a multiple of 64")
    return delta_rule_recurrent(q, k, v, beta, initial_state, scale, compute_dtype=compute_dtype)


# ----------------------------------------------------------------------------
# Gated DeltaNet  (gated_deltanet.py)
# ----------------------------------------------------------------------------

def gated_delta_rule_recurrent(q, k, v, g, beta, scale=None, initial_state=None,
                               use_qk_l2norm=True, compute_dtype=torch.float32):
    """Scalar-decay token recurrence; follows gated_deltanet.py:136-229.

    Cast to fp32 first (:173-177), per-step l2norm (:193-195), then scale (:197);
    decay before retrieve (:200-204)."""
    cd = compute_dtype
    B, H, T, K = q.shape
    V = v.shape[-1]
    od = q.dtype
    if scale is None:
        scale = K ** -0.5
    q, k, v, g, beta = (x.to(cd) for x in (q, k, v, g, beta))
    S = _state0(initial_state, B, H, K, V, cd)
    out = torch.empty(B, H, T, V, dtype=cd)
    sc = torch.tensor(scale, dtype=cd)
    for t in range(T):
        q_t, k_t, v_t = q[:, :, t], k[:, :, t], v[:, :, t]
        if use_qk_l2norm:
            q_t = _l2norm(q_t)
            k_t = _l2norm(k_t)
        q_t = q_t * sc
        S = S * torch.exp(g[:, :, t])[..., None, None]
        v_old = torch.einsum("bhkv,bhk->bhv", S, k_t)
        v_delta = beta[:, :, t][..., None] * (v_t - v_old)
        S = S + torch.einsum("bhk,bhv->bhkv", k_t, v_delta)
        out[:, :, t] = torch.einsum("bhk,bhkv->bhv", q_t, S)
    return out.to(od), S


def _unit_lower_solve(L: Tensor, Bm: Tensor) -> Tensor:
    """Forward substitution, one row per step (gated_deltanet.py:450-475, kda.py:575-598)."""
    C = L.shape[-1]
    X = torch.zeros_like(Bm)
    for t in range(C):
        contrib = torch.einsum("...j,...jd->...d", L[..., t, :], X)
        X[..., t, :] = Bm[..., t, :] - contrib
    return X


def _build_m_and_aqk(q, k, G, beta, BC, per_channel):
    """M = I + A_kk (unit lower) and A_qk with the reference's 16x16 tiling:
    diagonal tiles by masked pairwise exponentials, off-diagonal tiles factorised
    around the row tile's first cumulative gate with both factors exp(min(.,0))
    (gated_deltanet.py:333-439, kda.py:458-564).  q,k: [...,C,K]; G: [...,C] or [...,C,K]."""
    C = q.shape[-2]
    NC = C // BC
    cd = q.dtype
    lead = q.shape[:-2]
    M = torch.zeros(*lead, C, C, dtype=cd)
    Aqk = torch.zeros(*lead, C, C, dtype=cd)
    tri_s = torch.tril(torch.ones(BC, BC, dtype=torch.bool), diagonal=-1)
    tri_i = torch.tril(torch.ones(BC, BC, dtype=torch.bool), diagonal=0)
    ninf = torch.tensor(float("-inf"), dtype=cd)
    zero = torch.tensor(0.0, dtype=cd)
    eye = torch.eye(BC, dtype=cd)
    for i in range(NC):
        r = slice(i * BC, (i + 1) * BC)
        g_r, q_r, k_r, b_r = G[..., r, :] if per_channel else G[..., r], q[..., r, :], k[..., r, :], beta[..., r]
        if per_channel:
            d = g_r[..., :, None, :] - g_r[..., None, :, :]                      # [...,BC,BC,K]
            e_s = torch.exp(torch.where(tri_s[..., None], d, ninf))
            e_i = torch.exp(torch.where(tri_i[..., None], d, ninf))
            kk = k_r[..., :, None, :] * k_r[..., None, :, :]
            qk = q_r[..., :, None, :] * k_r[..., None, :, :]
            A0 = (kk * e_s).sum(-1)
            Aq = (qk * e_i).sum(-1)
        else:
            d = g_r[..., :, None] - g_r[..., None, :]
            e_s = torch.exp(torch.where(tri_s, d, ninf))
            e_i = torch.exp(torch.where(tri_i, d, ninf))
            kk = k_r[..., :, None, :] * k_r[..., None, :, :]
            qk = q_r[..., :, None, :] * k_r[..., None, :, :]
            A0 = (kk * e_s[..., None]).sum(-1)
            Aq = (qk * e_i[..., None]).sum(-1)
        M[..., r, r] = eye + A0 * b_r[..., :, None]
        Aqk[..., r, r] = Aq
        g_ref = g_r[..., 0, :] if per_channel else g_r[..., 0]
        for j in range(i):
            c = slice(j * BC, (j + 1) * BC)
            if per_channel:
                g_c = G[..., c, :]
                rs = torch.exp(torch.minimum(g_r - g_ref[..., None, :], zero))
                cs = torch.exp(torch.minimum(g_ref[..., None, :] - g_c, zero))
            else:
                g_c = G[..., c]
                rs = torch.exp(torch.minimum(g_r - g_ref[..., None], zero))[..., None]
                cs = torch.exp(torch.minimum(g_ref[..., None] - g_c, zero))[..., None]
            k_rs, q_rs = k_r * rs, q_r * rs
            k_cs = k[..., c, :] * cs
            M[..., r, c] = (k_rs @ k_cs.transpose(-1, -2)) * b_r[..., :, None]
            Aqk[..., r, c] = q_rs @ k_cs.transpose(-1, -2)
    return M, Aqk


def _gated_chunk_core(q, k, v, g, beta, initial_state, C, per_channel, cd):
    """Shared tail of gated_delta_rule_chunkwise / kda_chunkwise after normalisation,
    scaling and the fp32 cast: pad, chunk, cumsum, build M/A_qk, solve, chunk scan.
    (gated_deltanet.py:288-532, kda.py:387-653)."""
    B, H, T, K = q.shape
    V = v.shape[-1]
    pad = (C - T % C) % C
    if pad:
        P = torch.nn.functional.pad
        q, k, v = P(q, (0, 0, 0, pad)), P(k, (0, 0, 0, pad)), P(v, (0, 0, 0, pad))
        g = P(g, (0, 0, 0, pad)) if per_channel else P(g, (0, pad))
        beta = P(beta, (0, pad))
    Tp = T + pad
    N = Tp // C
    BC = 16
    if C % BC != 0:
        raise ValueError(f"chunk_size (BT={C}) must be divisible by BC={BC}.")
    q = q.reshape(B, H, N, C, K)
    k = k.reshape(B, H, N, C, K)
    v = v.reshape(B, H, N, C, V)
    g = g.reshape(B, H, N, C, K) if per_channel else g.reshape(B, H, N, C)
    beta = beta.reshape(B, H, N, C)
    G = torch.cumsum(g, dim=3)
    eG = torch.exp(G)
    M, Aqk = _build_m_and_aqk(q, k, G, beta, BC, per_channel)
    eGk = eG if per_channel else eG[..., None]
    rhs = torch.cat([beta[..., None] * (k * eGk), beta[..., None] * v], dim=-1)
    solved = _unit_lower_solve(M, rhs)
    w, u = solved[..., :K], solved[..., K:]
    S = _state0(initial_state, B, H, K, V, cd)
    zero = torch.tensor(0.0, dtype=cd)
    outs = []
    for n in range(N):
        q_i, k_i, u_i, w_i, A_i = q[:, :, n], k[:, :, n], u[:, :, n], w[:, :, n], Aqk[:, :, n]
        G_i, eG_i = G[:, :, n], eGk[:, :, n]
        v_i = u_i - w_i @ S
        o = (q_i * eG_i) @ S + A_i @ v_i
        if per_channel:
            S_new = S * eG[:, :, n, -1, :][..., None]
            ratio = torch.exp(torch.minimum(G_i[:, :, -1:, :] - G_i, zero))
        else:
            S_new = S * eG[:, :, n, -1][..., None, None]
            ratio = torch.exp(torch.minimum(G_i[:, :, -1:] - G_i, zero))[..., None]
        S = S_new + (ratio * k_i).transpose(-1, -2) @ v_i
        outs.append(o)
    out = torch.stack(outs, dim=2).reshape(B, H, Tp, V)[:, :, :T]
    return out, S


def gated_delta_rule_chunkwise(q, k, v, g, beta, scale=None, initial_state=None, chunk_size=64,
                               use_qk_l2norm=True, compute_dtype=torch.float32):
    """Chunk form with scalar decay; follows gated_deltanet.py:232-534.

    l2norm runs in the INPUT dtype (:273-275); the scale multiply by an fp32 scalar
    promotes to fp32 (:278); then everything is cast to fp32 (:281-285)."""
    cd = compute_dtype
    K = q.shape[-1]
    od = q.dtype
    if scale is None:
        scale = K ** -0.5
    if compute_dtype == torch.float64:
        q, k = q.to(cd), k.to(cd)
    if use_qk_l2norm:
        q = _l2norm(q)
        k = _l2norm(k)
    q = q.to(torch.promote_types(q.dtype, torch.float32)) * torch.tensor(
        scale, dtype=torch.promote_types(q.dtype, torch.float32))
    q, k, v, g, beta = (x.to(cd) for x in (q, k, v, g, beta))
    out, S = _gated_chunk_core(q, k, v, g, beta, initial_state, chunk_size, False, cd)
    return out.to(od), S


def gated_delta_rule_step(q, k, v, g, beta, state, scale=None, use_qk_l2norm=True,
                          compute_dtype=torch.float32):
    """One token with scalar decay; follows gated_deltanet.py:539-597."""
    cd = compute_dtype
    od = q.dtype
    K = q.shape[-1]
    if scale is None:
        scale = K ** -0.5
    q, k, v, g, beta, S = (x.to(cd) for x in (q, k, v, g, beta, state))
    if use_qk_l2norm:
        q = _l2norm(q)
        k = _l2norm(k)
    q = q * torch.tensor(scale, dtype=cd)
    S = S * torch.exp(g)[..., None, None]
    v_old = torch.einsum("bhkv,bhk->bhv", S, k)
    v_delta = beta[..., None] * (v - v_old)
    S_new = S + torch.einsum("bhk,bhv->bhkv", k, v_delta)
    o = torch.einsum("bhk,bhkv->bhv", q, S_new)
    return o.to(od), S_new


# ----------------------------------------------------------------------------
# KDA  (kda.py)
# ----------------------------------------------------------------------------

def kda_recurrent(q, k, v, g, beta, scale=None, initial_state=None, use_qk_l2norm=True,
                  compute_dtype=torch.float32):
    """Per-channel-decay token recurrence; follows kda.py:179-283 (beta on the key, :264)."""
    cd = compute_dtype
    B, H, T, K = q.shape
    V = v.shape[-1]
    od = q.dtype
    if scale is None:
        scale = K ** -0.5
    S = _state0(initial_state, B, H, K, V, cd)
    out = torch.empty(B, H, T, V, dtype=cd)
    for t in range(T):
        k_t, v_t, q_t = k[:, :, t].to(cd), v[:, :, t].to(cd), q[:, :, t].to(cd)
        g_t, b_t = g[:, :, t].to(cd), beta[:, :, t].to(cd)
        if use_qk_l2norm:
            q_t = _l2norm(q_t)
            k_t = _l2norm(k_t)
        q_t = q_t * scale
        S = S * torch.exp(g_t)[..., None]
        v_old = torch.einsum("bhk,bhkv->bhv", k_t, S)
        v_delta = v_t - v_old
        S = S + torch.einsum("bhk,bhv->bhkv", b_t[..., None] * k_t, v_delta)
        out[:, :, t] = torch.einsum("bhk,bhkv->bhv", q_t, S)
    return out.to(od), S


def kda_step(q, k, v, g, beta, state, scale=None, use_qk_l2norm=True, compute_dtype=torch.float32):
    """One token; follows kda.py:286-347.  Output takes the STATE's dtype (:347)."""
    cd = compute_dtype
    K = q.shape[-1]
    if scale is None:
        scale = K ** -0.5
    sd = state.dtype
    q, k, v, g, beta, S = (x.to(cd) for x in (q, k, v, g, beta, state))
    if use_qk_l2norm:
        q = _l2norm(q)
        k = _l2norm(k)
    q = q * scale
    S = S * torch.exp(g)[..., None]
    v_old = torch.einsum("bhk,bhkv->bhv", k, S)
    v_delta = v - v_old
    S_new = S + torch.einsum("bhk,bhv->bhkv", beta[..., None] * k, v_delta)
    o = torch.einsum("bhk,bhkv->bhv", q, S_new)
    return o.to(sd), S_new


def kda_chunkwise(q, k, v, g, beta, scale=None, initial_state=None, chunk_size=64,
                  use_qk_l2norm=True, compute_dtype=torch.float32):
    """Chunk form with per-channel decay; follows kda.py:350-655.

    l2norm AND the scale multiply (a Python float: no promotion) run in the input
    dtype (:379-384); the fp32 cast comes after padding (:414-418); the output is
    returned in float32 whatever the input dtype (:416,655)."""
    cd = compute_dtype
    K = q.shape[-1]
    if scale is None:
        scale = K ** -0.5
    if compute_dtype == torch.float64:
        q, k = q.to(cd), k.to(cd)
    if use_qk_l2norm:
        q = _l2norm(q)
        k = _l2norm(k)
    q = q * scale
    q, k, v, g, beta = (x.to(cd) for x in (q, k, v, g, beta))
    out, S = _gated_chunk_core(q, k, v, g, beta, initial_state, chunk_size, True, cd)
    return out.to(cd), S


# ----------------------------------------------------------------------------
# Backward: the reference has no backward function; gradients there are jax.grad
# through the chunk functions above.  The oracle differentiates the float64 token
# recurrence with torch.autograd (same function, so same gradients).
# ----------------------------------------------------------------------------

def _recurrent_autograd(variant, q, k, v, g, beta, h0, scale, use_qk_l2norm, cd):
    B, H, T, K = q.shape
    V = v.shape[-1]
    S = h0
    outs = []
    for t in range(T):
        q_t, k_t, v_t = q[:, :, t], k[:, :, t], v[:, :, t]
        if use_qk_l2norm:
            q_t = _l2norm(q_t)
            k_t = _l2norm(k_t)
        q_t = q_t * scale
        if variant == "gated":
            S = S * torch.exp(g[:, :, t])[..., None, None]
        elif variant == "kda":
            S = S * torch.exp(g[:, :, t])[..., None]
        v_old = torch.einsum("bhkv,bhk->bhv", S, k_t)
        v_delta = beta[:, :, t][..., None] * (v_t - v_old)
        S = S + torch.einsum("bhk,bhv->bhkv", k_t, v_delta)
        outs.append(torch.einsum("bhk,bhkv->bhv", q_t, S))
    return torch.stack(outs, dim=2), S


def delta_rule_grads(variant, q, k, v, g, beta, h0, do, dhT=None, scale=None, use_qk_l2norm=True,
                     compute_dtype=torch.float64):
    """Gradients (dq, dk, dv, dg, dbeta, dh0) of sum(o*do) + sum(hT*dhT) for ``variant`` in
    {"delta", "gated", "kda"}; what jax.grad of the reference op would return.
    DeltaNet ops never normalise (delta_net.py:170-173): pass use_qk_l2norm=False for "delta"."""
    cd = compute_dtype
    B, H, T, K = q.shape
    V = v.shape[-1]
    if scale is None:
        scale = K ** -0.5
    leaf = lambda x: None if x is None else x.detach().to(cd).clone().requires_grad_(True)
    q_, k_, v_, b_ = leaf(q), leaf(k), leaf(v), leaf(beta)
    g_ = leaf(g) if variant != "delta" else None
    h_ = leaf(h0 if h0 is not None else torch.zeros(B, H, K, V))
    o, hT = _recurrent_autograd(variant, q_, k_, v_, g_, b_, h_, scale, use_qk_l2norm, cd)
    loss = (o * do.to(cd)).sum()
    if dhT is not None:
        loss = loss + (hT * dhT.to(cd)).sum()
    loss.backward()
    return dict(dq=q_.grad, dk=k_.grad, dv=v_.grad, dg=None if g_ is None else g_.grad,
                dbeta=b_.grad, dh0=h_.grad, o=o.detach(), hT=hT.detach())


# ----------------------------------------------------------------------------
# Input generator shared by tests and the benchmark (seeded numpy, no JAX PRNG).
# ----------------------------------------------------------------------------

def make_inputs(variant, B, H, T, K, V, seed, io_dtype=torch.float32, h0_std=None, g_dtype=torch.float32):
    """q,k ~ N(0,1) l2-normalised in fp32; v ~ N(0,1); beta = sigmoid(N(0,1));
    g = logsigmoid(N(0,1)+4) (scalar per token for "gated", per channel for "kda")."""
    import numpy as np
    rng = np.random.default_rng(seed)
    f = lambda *s: torch.from_numpy(rng.standard_normal(s, dtype=np.float32))
    q, k, v = f(B, H, T, K), f(B, H, T, K), f(B, H, T, V)
    q, k = _l2norm(q), _l2norm(k)
    beta = torch.sigmoid(f(B, H, T))
    g = None
    if variant == "gated":
        g = torch.nn.functional.logsigmoid(f(B, H, T) + 4.0).to(g_dtype)
    elif variant == "kda":
        g = torch.nn.functional.logsigmoid(f(B, H, T, K) + 4.0).to(g_dtype)
    h0 = None if h0_std is None else f(B, H, K, V) * h0_std
    return dict(q=q.to(io_dtype), k=k.to(io_dtype), v=v.to(io_dtype), g=g, beta=beta, h0=h0)
