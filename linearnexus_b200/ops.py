"""Host-side mirror of the LinearNexus delta-rule op signatures over the sm_100a C ABI.

Each function keeps the name, argument order, keyword defaults, accepted shapes, output
dtypes and error behaviour of the LinearNexus function it replaces (cited per function,
paths relative to the LinearNexus tree); the arrays are torch CUDA tensors and the work is
done by ``libdeltarule_sm100.so``.  There is no CPU path: CPU tensors raise.

Layout: ``[B, H, T, D]`` as in the reference.  A tensor that is a transposed view of a
contiguous ``[B, T, H, D]`` array (the blocks' pre-transpose layout,
modules/linear_attn/gated_deltanet.py:785-795) is consumed in place without a copy when all
sequence inputs share that layout.
"""

from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import (DR_BF16, DR_DELTA, DR_F32, DR_GATED, DR_KDA, DR_LAYOUT_BHTD, DR_LAYOUT_BTHD,
                   DR_PATH_AUTO, DR_PATH_FP32, DR_PATH_TCGEN05, DR_PATH_SPLIT, DrDesc)

Tensor = torch.Tensor
_NATIVE = {torch.float32: DR_F32, torch.bfloat16: DR_BF16}
_PATHS = {None: DR_PATH_AUTO, "auto": DR_PATH_AUTO, "fp32": DR_PATH_FP32, "tcgen05": DR_PATH_TCGEN05,
          "split": DR_PATH_SPLIT}

# Kernel family used by the chunk entry point when a call does not say; tests set it to
# force one family ("fp32" / "tcgen05").
default_chunk_path: Optional[str] = None


def _ptr(t: Optional[Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(dev) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


# One status word per device, handed to every kernel launch; kernels OR problems into it (a bounded wait
# that ran out) and never trap.  Nothing here synchronises to look at it: `check_device_status` does, and is
# meant to be called where the host synchronises anyway.
_status_words: dict = {}


def _status(dev) -> Tensor:
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _status_words.get(idx)
    if t is None:
        t = _status_words[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return t


def check_device_status(device=None) -> None:
    """Synchronise the current stream of ``device`` and raise :class:`DeltaRuleError` (DR_ERR_DEVICE) if any
    kernel launched by this package since the last check reported a problem through the device status word;
    the word is cleared, so the next check starts clean.  The reference has nothing to mirror here: its GPU
    kernel falls back silently (delta_net.py:150-156)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        st = _lib.load().dr_check_status(_ptr(_status(dev)), _stream(dev))
    _lib.check(st, "dr_check_status")


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("linearnexus_b200 ops run on CUDA tensors only (there is no CPU fallback)")


def _native(t: Tensor) -> Tensor:
    """q/k/v/g travel as fp32 or bf16; other float types are widened to fp32."""
    return t if t.dtype in _NATIVE else t.to(torch.float32)


def _is_bthd_view(t: Tensor) -> bool:
    return t.dim() >= 3 and not t.is_contiguous() and t.transpose(1, 2).is_contiguous()


def _layout(seq_tensors) -> Tuple[int, list]:
    """Pick [B,H,T,D] (copying if needed) or the zero-copy [B,T,H,D] view layout."""
    ts = [t for t in seq_tensors if t is not None]
    if ts[0].shape[1] > 1 and ts[0].shape[2] > 1 and all(_is_bthd_view(t) for t in ts):
        return DR_LAYOUT_BTHD, list(seq_tensors)
    return DR_LAYOUT_BHTD, [None if t is None else t.contiguous() for t in seq_tensors]


def _state(initial_state, B, H, K, V, dev) -> Optional[Tensor]:
    if initial_state is None:
        return None
    if tuple(initial_state.shape) != (B, H, K, V):
        raise ValueError(f"initial_state must be [B,H,K,V]={B, H, K, V}, got {tuple(initial_state.shape)}")
    return initial_state.to(device=dev, dtype=torch.float32).contiguous()


def _desc(variant, layout, B, H, T, K, V, chunk, qkv, g, out_dtype, l2norm, scale, path=None) -> DrDesc:
    d = DrDesc()
    d.variant, d.layout = variant, layout
    d.B, d.H, d.T, d.K, d.V, d.chunk = B, H, T, K, V, chunk
    d.qkv_dtype = _NATIVE[qkv.dtype]
    d.g_dtype = _NATIVE[g.dtype] if g is not None else DR_F32
    d.out_dtype = _NATIVE[out_dtype]
    d.use_qk_l2norm = int(bool(l2norm))
    d.scale = float(scale)
    if path not in _PATHS:
        raise ValueError(f"unknown chunk path {path!r}")
    d.path = _PATHS[path]
    return d


def _seq_forward(kind, variant, q, k, v, g, beta, initial_state, scale, chunk_size, l2norm,
                 out_dtype, path=None):
    _require_cuda(q, k, v, g, beta, initial_state)
    if (q.dim() != 4 or k.shape != q.shape or v.dim() != 4 or v.shape[0] != q.shape[0] or v.shape[2] != q.shape[2]
            or v.shape[1] % q.shape[1]):
        raise ValueError("expected q,k [B,Hq,T,K] and v [B,H,T,V] with H a multiple of Hq; got "
                         f"{tuple(q.shape)}, {tuple(k.shape)}, {tuple(v.shape)}")
    B, Hq, T, K = q.shape
    H, V = v.shape[1], v.shape[-1]   # Hq < H: grouped value attention, q/k head h // (H // Hq) serves head h
    if scale is None:
        scale = K ** -0.5
    if beta.dim() == 4:
        beta = beta.squeeze(-1)
    if tuple(beta.shape) != (B, H, T):
        raise ValueError(f"beta must be [B,H,T], got {tuple(beta.shape)}")
    if variant == DR_GATED and tuple(g.shape) != (B, H, T):
        raise ValueError(f"g must be [B,H,T], got {tuple(g.shape)}")
    if variant == DR_KDA and tuple(g.shape) != (B, H, T, K):
        raise ValueError(f"g must be [B,H,T,K], got {tuple(g.shape)}")
    dev = q.device
    common = torch.float32 if any(t.dtype not in _NATIVE for t in (q, k, v)) or len({q.dtype, k.dtype, v.dtype}) > 1 else q.dtype
    qn, kn, vn = (t.to(common) for t in (q, k, v))
    gn = None if g is None else _native(g)
    bn = beta.to(torch.float32)
    layout, (qn, kn, vn, gn, bn) = _layout([qn, kn, vn, gn, bn])
    h0 = _state(initial_state, B, H, K, V, dev)
    native_out = out_dtype if out_dtype in _NATIVE else torch.float32
    if layout == DR_LAYOUT_BTHD:
        o = torch.empty((B, T, H, V), dtype=native_out, device=dev).transpose(1, 2)
    else:
        o = torch.empty((B, H, T, V), dtype=native_out, device=dev)
    hT = torch.empty((B, H, K, V), dtype=torch.float32, device=dev)
    d = _desc(variant, layout, B, H, T, K, V, chunk_size, qn, gn, native_out, l2norm, scale,
              path if path is not None else default_chunk_path)
    d.qk_heads = Hq
    lib = _lib.load()
    with torch.cuda.device(dev):
        if kind == "chunk":
            need = int(lib.dr_workspace_bytes(ctypes.byref(d), 0))
            ws = torch.empty(need, dtype=torch.uint8, device=dev) if need > 0 else None
            st = lib.dr_chunk_fwd(ctypes.byref(d), _ptr(qn), _ptr(kn), _ptr(vn), _ptr(gn), _ptr(bn),
                                  _ptr(h0), _ptr(o), _ptr(hT), _ptr(ws), max(need, 0), _ptr(_status(dev)),
                                  _stream(dev))
        else:
            st = lib.dr_recurrent_fwd(ctypes.byref(d), _ptr(qn), _ptr(kn), _ptr(vn), _ptr(gn), _ptr(bn),
                                      _ptr(h0), _ptr(o), _ptr(hT), _ptr(_status(dev)), _stream(dev))
    if st == -7:
        raise ValueError(f"chunk_size (BT={chunk_size}) must be divisible by BC=16.")
    _lib.check(st, f"dr_{kind}_fwd")
    return (o if o.dtype == out_dtype else o.to(out_dtype)), hT


def _step(variant, q, k, v, g, beta, state, scale, l2norm, out_dtype, inplace=False):
    _require_cuda(q, k, v, g, beta, state)
    if q.dim() != 3 or k.shape != q.shape or v.dim() != 3 or v.shape[0] != q.shape[0] or v.shape[1] % q.shape[1]:
        raise ValueError("expected q,k [B,Hq,K] and v [B,H,V] with H a multiple of Hq")
    B, Hq, K = q.shape
    H, V = v.shape[1], v.shape[-1]
    if scale is None:
        scale = K ** -0.5
    if tuple(state.shape) != (B, H, K, V):
        raise ValueError(f"state must be [B,H,K,V]={B, H, K, V}, got {tuple(state.shape)}")
    dev = q.device
    common = torch.float32 if any(t.dtype not in _NATIVE for t in (q, k, v)) or len({q.dtype, k.dtype, v.dtype}) > 1 else q.dtype
    qn, kn, vn = (t.to(common).contiguous() for t in (q, k, v))
    gn = None if g is None else _native(g).contiguous()
    bn = beta.to(torch.float32).contiguous()
    if inplace:
        if state.dtype != torch.float32 or not state.is_contiguous():
            raise ValueError("in-place decode needs a contiguous float32 state cache")
        s_in = s_out = state
    else:
        s_in = state.to(torch.float32).contiguous()
        s_out = torch.empty_like(s_in)
    native_out = out_dtype if out_dtype in _NATIVE else torch.float32
    o = torch.empty((B, H, V), dtype=native_out, device=dev)
    d = _desc(variant, DR_LAYOUT_BHTD, B, H, 1, K, V, 0, qn, gn, native_out, l2norm, scale)
    d.qk_heads = Hq
    with torch.cuda.device(dev):
        st = _lib.load().dr_step(ctypes.byref(d), _ptr(qn), _ptr(kn), _ptr(vn), _ptr(gn), _ptr(bn),
                                 _ptr(s_in), _ptr(s_out), _ptr(o), _ptr(_status(dev)), _stream(dev))
    _lib.check(st, "dr_step")
    return (o if o.dtype == out_dtype else o.to(out_dtype)), s_out


# ------------------------------------------------------------------------------------------
# DeltaNet  (modules/linear_attn/delta_net.py)
# ------------------------------------------------------------------------------------------

def delta_rule_recurrent(q, k, v, beta, initial_state=None, scale=None, backend=None) -> Tuple[Tensor, Tensor]:
    """Token recurrence, no decay, no l2norm inside (delta_net.py:126-213).

    ``backend`` is accepted for signature compatibility; every value runs the CUDA kernel
    (the reference's silent fallback to its JAX path, delta_net.py:150-156, has no counterpart).
    Returns ``(o.astype(q.dtype) [B,H,T,V], final_state float32 [B,H,K,V])``."""
    return _seq_forward("recurrent", DR_DELTA, q, k, v, None, beta, initial_state, scale, 0, False, q.dtype)


def delta_rule_chunkwise(q, k, v, beta, initial_state=None, chunk_size=64, scale=None, backend=None,
                         path=None) -> Tuple[Tensor, Tensor]:
    """WY chunk form (delta_net.py:216-354).  Any ``chunk_size`` >= 1; ``backend`` ignored as in the reference.
    Differentiable (``loss.backward()``) for ``chunk_size <= 64`` and ``K <= 128``; other shapes run forward only."""
    return _seq_forward("chunk", DR_DELTA, q, k, v, None, beta, initial_state, scale, chunk_size, False, q.dtype, path)


def delta_rule_step(q, k, v, beta, state, scale=None) -> Tuple[Tensor, Tensor]:
    """One decode token (delta_net.py:357-397); beta may be [B,H] or [B,H,1]."""
    if beta.dim() == 3:
        beta = beta.squeeze(-1)
    return _step(DR_DELTA, q, k, v, None, beta, state, scale, False, q.dtype)


def delta_rule_recurrent_pallas(q, k, v, beta, initial_state=None, scale=None) -> Tuple[Tensor, Tensor]:
    """Drop-in for the Pallas kernel entry point (kernels/pallas/delta_rule.py:47-281): same
    maths as :func:`delta_rule_recurrent` and the same RuntimeError guards on key_dim % 32 and
    value_dim % 64 (kernels/pallas/delta_rule.py:108-115)."""
    if not q.is_cuda:
        raise RuntimeError("the sm_100a delta-rule kernel is not usable on this machine: tensors are not on a CUDA device")
    if q.shape[-1] % 32 != 0:
        raise RuntimeError("delta-rule kernel entry requires key_dim to be a multiple of 32")
    if v.shape[-1] % 64 != 0:
        raise RuntimeError("delta-rule kernel entry requires value_dim to be a multiple of 64")
    return delta_rule_recurrent(q, k, v, beta, initial_state, scale)


# ------------------------------------------------------------------------------------------
# Gated DeltaNet  (modules/linear_attn/gated_deltanet.py)
# ------------------------------------------------------------------------------------------

def gated_delta_rule_recurrent(q, k, v, g, beta, scale=None, initial_state=None, use_qk_l2norm=True):
    """Scalar-decay token recurrence (gated_deltanet.py:136-229)."""
    return _seq_forward("recurrent", DR_GATED, q, k, v, g, beta, initial_state, scale, 0, use_qk_l2norm, q.dtype)


def gated_delta_rule_chunkwise(q, k, v, g, beta, scale=None, initial_state=None, chunk_size=64,
                               use_qk_l2norm=True, path=None):
    """Chunk form with scalar decay (gated_deltanet.py:232-534).  ``chunk_size % 16 != 0`` raises
    ValueError as the reference does (:318-321).  The kernel normalises q,k in fp32 (the
    reference does it in the input dtype, :273-275 -- strictly less accurate for bf16)."""
    return _seq_forward("chunk", DR_GATED, q, k, v, g, beta, initial_state, scale, chunk_size, use_qk_l2norm, q.dtype, path)


def gated_delta_rule_step(q, k, v, g, beta, state, scale=None, use_qk_l2norm=True, inplace=False):
    """One decode token (gated_deltanet.py:539-597).  ``inplace=True`` (an extension) updates the
    float32 ``state`` cache in place and returns it, which is what a serving loop wants; the
    default returns a new state like the functional reference."""
    return _step(DR_GATED, q, k, v, g, beta, state, scale, use_qk_l2norm, q.dtype, inplace)


# ------------------------------------------------------------------------------------------
# KDA  (modules/linear_attn/kda.py)
# ------------------------------------------------------------------------------------------

def kda_recurrent(q, k, v, g, beta, scale=None, initial_state=None, use_qk_l2norm=True):
    """Per-channel-decay token recurrence (kda.py:179-283)."""
    return _seq_forward("recurrent", DR_KDA, q, k, v, g, beta, initial_state, scale, 0, use_qk_l2norm, q.dtype)


def kda_step(q, k, v, g, beta, state, scale=None, use_qk_l2norm=True, inplace=False):
    """One decode token (kda.py:286-347).  The output takes the STATE's dtype, as in the
    reference (kda.py:347)."""
    return _step(DR_KDA, q, k, v, g, beta, state, scale, use_qk_l2norm, state.dtype, inplace)


def kda_chunkwise(q, k, v, g, beta, scale=None, initial_state=None, chunk_size=64, use_qk_l2norm=True,
                  path=None, out_dtype=None):
    """Chunk form with per-channel decay (kda.py:350-655).  The output is float32 whatever the
    input dtype, as in the reference (kda.py:416,655); ``out_dtype`` (an extension) overrides it."""
    return _seq_forward("chunk", DR_KDA, q, k, v, g, beta, initial_state, scale, chunk_size, use_qk_l2norm,
                        torch.float32 if out_dtype is None else out_dtype, path)


# ------------------------------------------------------------------------------------------
# Backward.  The reference has no backward function: its gradients are jax.grad through the
# chunk functions above.  `chunk_backward` is the explicit adjoint; the three `*_chunkwise`
# ops route through torch.autograd Functions built on it whenever an input requires grad, so
# `loss.backward()` works as `jax.grad` does on the reference.
# ------------------------------------------------------------------------------------------

_VARIANTS = {"delta": DR_DELTA, "gated": DR_GATED, "kda": DR_KDA}


def _train_prep(variant, q, k, v, g, beta, initial_state, scale, chunk_size, use_qk_l2norm, out_dtype=None):
    """Common argument handling of the backward-related entry points ([B,H,T,D] contiguous copies)."""
    var = _VARIANTS[variant]
    B, Hq, T, K = q.shape
    H, V = v.shape[1], v.shape[-1]   # Hq < H: grouped value attention (dq, dk come back summed over each group)
    if k.shape != q.shape or H % Hq:
        raise ValueError("expected q,k [B,Hq,T,K] and v [B,H,T,V] with H a multiple of Hq; got "
                         f"{tuple(q.shape)}, {tuple(k.shape)}, {tuple(v.shape)}")
    if scale is None:
        scale = K ** -0.5
    if beta.dim() == 4:
        beta = beta.squeeze(-1)
    dev = q.device
    common = torch.float32 if any(t.dtype not in _NATIVE for t in (q, k, v)) or len({q.dtype, k.dtype, v.dtype}) > 1 else q.dtype
    qn, kn, vn = (t.to(common).contiguous() for t in (q, k, v))
    gn = None if g is None else _native(g).contiguous()
    bn = beta.to(torch.float32).contiguous()
    h0 = _state(initial_state, B, H, K, V, dev)
    d = _desc(var, DR_LAYOUT_BHTD, B, H, T, K, V, chunk_size, qn, gn, common if out_dtype is None else out_dtype,
              use_qk_l2norm, scale)
    d.qk_heads = Hq
    lib = _lib.load()
    need = lib.dr_workspace_bytes(ctypes.byref(d), 1)
    if need == -7:
        raise ValueError(f"chunk_size (BT={chunk_size}) must be divisible by BC=16.")
    _lib.check(int(need) if need < 0 else 0, "dr_workspace_bytes")
    return d, lib, int(need), (qn, kn, vn, gn, bn, h0), (B, H, T, K, V, dev, common)


def chunk_forward_saving(variant, q, k, v, g, beta, initial_state=None, scale=None, chunk_size=64,
                         use_qk_l2norm=True, out_dtype=None):
    """The chunkwise forward of a training step: returns ``(o, final_state, saved)`` where ``saved`` is the
    backward workspace holding the state at the start of every chunk; pass it to ``chunk_backward(..., saved=)``
    so that the backward does not recompute the forward."""
    _require_cuda(q, k, v, g, beta, initial_state)
    if out_dtype is None:
        out_dtype = torch.float32 if variant == "kda" else q.dtype
    native_out = out_dtype if out_dtype in _NATIVE else torch.float32
    d, lib, need, (qn, kn, vn, gn, bn, h0), (B, H, T, K, V, dev, common) = _train_prep(
        variant, q, k, v, g, beta, initial_state, scale, chunk_size, use_qk_l2norm, native_out)
    ws = torch.empty(need, dtype=torch.uint8, device=dev)
    o = torch.empty((B, H, T, V), dtype=native_out, device=dev)
    hT = torch.empty((B, H, K, V), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        st = lib.dr_chunk_fwd_saving(ctypes.byref(d), _ptr(qn), _ptr(kn), _ptr(vn), _ptr(gn), _ptr(bn), _ptr(h0),
                                     _ptr(o), _ptr(hT), _ptr(ws), ws.numel(), _ptr(_status(dev)), _stream(dev))
    _lib.check(st, "dr_chunk_fwd_saving")
    return (o if o.dtype == out_dtype else o.to(out_dtype)), hT, ws


def chunk_backward(variant, q, k, v, g, beta, d_o, initial_state=None, d_final_state=None, scale=None,
                   chunk_size=64, use_qk_l2norm=True, saved=None):
    """Gradients of sum(o * d_o) + sum(final_state * d_final_state) for ``variant`` in
    {"delta", "gated", "kda"}.  Returns a dict: dq, dk [like q: with grouped q/k heads, summed over each
    group's value heads], dv [like v] in the q/k/v dtype;
    dbeta float32 [B,H,T]; dg float32 [like g] (None for "delta"); dh0 float32 [B,H,K,V].
    ``saved``: the third result of ``chunk_forward_saving`` on the same inputs (skips the forward recomputation;
    the buffer is consumed)."""
    _require_cuda(q, k, v, g, beta, d_o, initial_state, d_final_state)
    d, lib, need, (qn, kn, vn, gn, bn, h0), (B, H, T, K, V, dev, common) = _train_prep(
        variant, q, k, v, g, beta, initial_state, scale, chunk_size, use_qk_l2norm)
    don = d_o.to(common).contiguous()
    dhT = _state(d_final_state, B, H, K, V, dev)
    if saved is not None and (saved.numel() < need or saved.device != dev or saved.dtype != torch.uint8):
        raise ValueError("saved must be the workspace returned by chunk_forward_saving for the same shapes")
    ws = torch.empty(need, dtype=torch.uint8, device=dev) if saved is None else saved
    dq, dk, dv = torch.empty_like(qn), torch.empty_like(kn), torch.empty_like(vn)
    dbeta = torch.empty((B, H, T), dtype=torch.float32, device=dev)
    dg = None if g is None else torch.empty(gn.shape, dtype=torch.float32, device=dev)
    dh0 = torch.empty((B, H, K, V), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        if saved is None:
            st = lib.dr_chunk_bwd(ctypes.byref(d), _ptr(qn), _ptr(kn), _ptr(vn), _ptr(gn), _ptr(bn), _ptr(h0), _ptr(don),
                                  _ptr(dhT), _ptr(dq), _ptr(dk), _ptr(dv), _ptr(dbeta), _ptr(dg), _ptr(dh0), _ptr(ws),
                                  ws.numel(), _ptr(_status(dev)), _stream(dev))
        else:
            st = lib.dr_chunk_bwd_saved(ctypes.byref(d), _ptr(qn), _ptr(kn), _ptr(vn), _ptr(gn), _ptr(bn), _ptr(don),
                                        _ptr(dhT), _ptr(dq), _ptr(dk), _ptr(dv), _ptr(dbeta), _ptr(dg), _ptr(dh0),
                                        _ptr(ws), ws.numel(), _ptr(_status(dev)), _stream(dev))
    _lib.check(st, "dr_chunk_bwd")
    return dict(dq=dq.to(q.dtype), dk=dk.to(k.dtype), dv=dv.to(v.dtype), dg=dg, dbeta=dbeta, dh0=dh0)


def backward_supported(variant: str, K: int, chunk_size: int) -> bool:
    """Shapes the backward kernels cover: chunk_size <= 64 and K <= 128 (and K % 16 == 0 for "kda").  The forward
    entry points accept more (longer chunks and K up to 256 run on the token-recurrent kernel); the reference
    differentiates any shape through jax.grad."""
    return chunk_size <= 64 and K <= 128 and (variant != "kda" or K % 16 == 0)


class _ChunkFn(torch.autograd.Function):
    """Forward that keeps the per-chunk states for its backward (one forward per training step).  Inputs the
    saving forward does not take (grouped q/k heads, an explicit kernel path) fall back to forward + recomputation."""

    @staticmethod
    def forward(ctx, variant, q, k, v, g, beta, initial_state, scale, chunk_size, l2norm, out_dtype, path):
        saved = None
        with torch.no_grad():
            if path is None and backward_supported(variant, q.shape[-1], chunk_size):
                o, hT, saved = chunk_forward_saving(variant, q, k, v, g, beta, initial_state, scale, chunk_size,
                                                    l2norm, out_dtype)
            else:   # an explicit kernel path, or a shape only the forward covers (backward() then says so)
                o, hT = _seq_forward("chunk", _VARIANTS[variant], q, k, v, g, beta, initial_state, scale, chunk_size,
                                     l2norm, out_dtype, path)
        ctx.save_for_backward(q, k, v, g if g is not None else q.new_empty(0), beta,
                              initial_state if initial_state is not None else q.new_empty(0))
        ctx.saved_ws = saved
        ctx.meta = (variant, scale, chunk_size, l2norm, g is not None, initial_state is not None)
        return o, hT

    @staticmethod
    def backward(ctx, d_o, d_hT):
        q, k, v, g, beta, h0 = ctx.saved_tensors
        variant, scale, chunk_size, l2norm, has_g, has_h0 = ctx.meta
        if not backward_supported(variant, q.shape[-1], chunk_size):
            raise NotImplementedError(
                f"the backward kernels cover chunk_size <= 64 and K <= 128 (K % 16 == 0 for 'kda'); got chunk_size="
                f"{chunk_size}, K={q.shape[-1]}.  The forward of this shape is available (this call ran it).")
        saved, ctx.saved_ws = ctx.saved_ws, None   # consumed: a second backward recomputes
        gr = chunk_backward(variant, q, k, v, g if has_g else None, beta, d_o, h0 if has_h0 else None, d_hT,
                            scale=scale, chunk_size=chunk_size, use_qk_l2norm=l2norm, saved=saved)
        dg = gr["dg"].to(g.dtype) if has_g else None
        return (None, gr["dq"], gr["dk"], gr["dv"], dg, gr["dbeta"].reshape(beta.shape).to(beta.dtype),
                gr["dh0"].to(h0.dtype) if has_h0 else None, None, None, None, None, None)


def _wants_grad(*ts):
    return torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in ts)


_delta_chunk_nograd, _gated_chunk_nograd, _kda_chunk_nograd = delta_rule_chunkwise, gated_delta_rule_chunkwise, kda_chunkwise


def delta_rule_chunkwise(q, k, v, beta, initial_state=None, chunk_size=64, scale=None, backend=None, path=None):  # noqa: F811
    if _wants_grad(q, k, v, beta, initial_state):
        return _ChunkFn.apply("delta", q, k, v, None, beta, initial_state, scale, chunk_size, False, q.dtype, path)
    return _delta_chunk_nograd(q, k, v, beta, initial_state, chunk_size, scale, backend, path)


def gated_delta_rule_chunkwise(q, k, v, g, beta, scale=None, initial_state=None, chunk_size=64,  # noqa: F811
                               use_qk_l2norm=True, path=None):
    if _wants_grad(q, k, v, g, beta, initial_state):
        return _ChunkFn.apply("gated", q, k, v, g, beta, initial_state, scale, chunk_size, use_qk_l2norm, q.dtype, path)
    return _gated_chunk_nograd(q, k, v, g, beta, scale, initial_state, chunk_size, use_qk_l2norm, path)


def kda_chunkwise(q, k, v, g, beta, scale=None, initial_state=None, chunk_size=64, use_qk_l2norm=True,  # noqa: F811
                  path=None, out_dtype=None):
    if _wants_grad(q, k, v, g, beta, initial_state):
        return _ChunkFn.apply("kda", q, k, v, g, beta, initial_state, scale, chunk_size, use_qk_l2norm,
                              torch.float32 if out_dtype is None else out_dtype, path)
    return _kda_chunk_nograd(q, k, v, g, beta, scale, initial_state, chunk_size, use_qk_l2norm, path, out_dtype)


delta_rule_chunkwise.__doc__ = _delta_chunk_nograd.__doc__
gated_delta_rule_chunkwise.__doc__ = _gated_chunk_nograd.__doc__
kda_chunkwise.__doc__ = _kda_chunk_nograd.__doc__
