"""The element-wise steps a block runs right before and right after the delta-rule op, as single HBM passes.

Same names and argument meaning as the reference helpers they replace:

* ``depthwise_conv1d_causal(inputs, weight, bias, cache=None)`` -- ``linearnexus/core/conv.py:13-68``; with
  ``activation="silu"`` the ``jax.nn.silu`` that follows it in the blocks (``gated_deltanet.py:764-783``) is
  applied in the same pass.
* ``gated_deltanet_gates(a, b, A_log, dt_bias)`` -- ``gated_deltanet.py:804-815``; ``kda_gate`` -- ``kda.py:120-172``.
* ``rmsnorm_gated(o, weight, gate)`` -- ``RMSNorm`` (``modules/common.py:42-53``) times ``sigmoid(gate)``
  (``gated_deltanet.py:853-865``, ``FusedRMSNormGated`` ``kda.py:664-700``), reading the op's ``[B,H,T,V]`` output and
  writing the ``[B,T,H,V]`` tensor the output projection takes.

Everything stays token-major (``[B,T,H,D]``): the ops take ``x.transpose(1, 2)`` views of such arrays without
copying and answer in the same layout, so a block built from these pieces has no transposes.  CUDA tensors only; there is no CPU path.
"""
import ctypes
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import DR_BF16, DR_F32, DR_LAYOUT_BHTD, DR_LAYOUT_BTHD

Tensor = torch.Tensor
_NATIVE = {torch.float32: DR_F32, torch.bfloat16: DR_BF16}


def _ptr(t: Optional[Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(dev):
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise ValueError("linearnexus_b200.block_ops takes CUDA tensors only (there is no CPU path)")


def _act(t: Tensor) -> Tensor:
    """Activations in a dtype the kernels read (fp32 / bf16), contiguous."""
    return (t if t.dtype in _NATIVE else t.float()).contiguous()


def depthwise_conv1d_causal(inputs: Tensor, weight: Tensor, bias: Optional[Tensor] = None, *,
                            cache: Optional[Tensor] = None, activation: Optional[str] = None,
                            cache_out: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
    """``inputs`` [B,T,C], ``weight`` [kernel,C], ``bias`` [C] or None, ``cache`` [B,kernel-1,C] or None.
    Returns ``(conv_output, new_cache)`` as the reference; ``activation="silu"`` fuses the SiLU.  ``cache_out``
    may name the tensor that receives the new cache (``cache`` itself for a decode step)."""
    _cuda(inputs, weight, bias, cache, cache_out)
    if inputs.dim() != 3:
        raise ValueError("inputs must be [batch, seq, channels]")
    if activation not in (None, "silu"):
        raise ValueError("activation must be None or 'silu'")
    B, T, C = inputs.shape
    W = weight.shape[0]
    if W < 1:
        raise ValueError("kernel_size must be >= 1")
    if weight.shape != (W, C):
        raise ValueError("weight must be [kernel, channels]")
    if cache is not None and cache.shape != (B, W - 1, C):
        raise ValueError(f"cache shape must be (batch, kernel-1, channels); got {tuple(cache.shape)} for kernel_size={W}")
    x = _act(inputs)
    dev = x.device
    y = torch.empty_like(x)
    cin = None if cache is None or W == 1 else cache.to(x.dtype).contiguous()
    if W == 1:
        new_cache = torch.zeros((B, 0, C), dtype=inputs.dtype, device=dev)
    elif cache_out is not None:
        if cache_out.shape != (B, W - 1, C) or cache_out.dtype != x.dtype or not cache_out.is_contiguous():
            raise ValueError("cache_out must be a contiguous [batch, kernel-1, channels] tensor of the input dtype")
        new_cache = cache_out
    else:
        new_cache = torch.empty((B, W - 1, C), dtype=x.dtype, device=dev)
    lib = _lib.load()
    # the fp32 copies of the parameters stay bound to names until the call has been enqueued: a temporary would
    # be released (and its block handed to the next cast) before the kernel reads it
    w32 = weight.float().contiguous()
    b32 = None if bias is None else bias.float().contiguous()
    with torch.cuda.device(dev):
        st = lib.dr_short_conv_silu(_ptr(x), _ptr(w32), _ptr(b32), _ptr(cin), _ptr(y),
                                    _ptr(new_cache if W > 1 else None), B, T, C, W, _NATIVE[x.dtype],
                                    int(activation == "silu"), _stream(dev))
    _lib.check(st, "dr_short_conv_silu")
    return (y if y.dtype == inputs.dtype else y.to(inputs.dtype)), new_cache


def short_conv_silu(inputs, weight, bias=None, *, cache=None, cache_out=None):
    """``silu(depthwise_conv1d_causal(...))`` in one pass (the q/k/v preparation of the blocks)."""
    return depthwise_conv1d_causal(inputs, weight, bias, cache=cache, activation="silu", cache_out=cache_out)


def _gates(mode, a, b, A_log, bias, H, K, beta_scale, threshold):
    a2 = _act(a)
    b2 = None if b is None else _act(b)
    dev = a2.device
    B, T = a2.shape[0], a2.shape[1]
    g = torch.empty((B, T, H) if K == 1 and mode == 0 else (B, T, H, K), dtype=torch.float32, device=dev)
    beta = None if b is None else torch.empty((B, T, H), dtype=torch.float32, device=dev)
    lib = _lib.load()
    A32 = A_log.float().contiguous()          # kept alive until the call has been enqueued (see above)
    bias32 = None if bias is None else bias.float().contiguous()
    with torch.cuda.device(dev):
        st = lib.dr_gate_activations(mode, _ptr(a2), _ptr(b2), _ptr(A32), _ptr(bias32), _ptr(g), _ptr(beta),
                                     B, T, H, K, _NATIVE[a2.dtype], _NATIVE[b2.dtype] if b2 is not None else DR_F32,
                                     float(beta_scale), float(threshold), _stream(dev))
    _lib.check(st, "dr_gate_activations")
    return g, beta


def gated_deltanet_gates(a: Tensor, b: Tensor, A_log: Tensor, dt_bias: Tensor,
                         allow_neg_eigval: bool = False) -> Tuple[Tensor, Tensor]:
    """``a``, ``b`` [B,T,H] (the a_proj / b_proj outputs) -> ``(g, beta)`` fp32 [B,T,H]:
    ``g = -exp(A_log) * softplus(a + dt_bias)``, ``beta = sigmoid(b)`` (doubled with ``allow_neg_eigval``)."""
    _cuda(a, b, A_log, dt_bias)
    if a.dim() != 3 or a.shape != b.shape or A_log.shape != (a.shape[2],) or dt_bias.shape != (a.shape[2],):
        raise ValueError("expected a, b [B,T,H] and A_log, dt_bias [H]")
    return _gates(0, a, b, A_log, dt_bias, a.shape[2], 1, 2.0 if allow_neg_eigval else 1.0, 0.0)


def kda_gate(g: Tensor, A_log: Tensor, head_k_dim: int, g_bias: Optional[Tensor] = None,
             beta: Optional[Tensor] = None, threshold: float = 20.0):
    """``g`` [B,T,H*head_k_dim] -> ``(g_out [B,T,H,head_k_dim], sigmoid(beta) or None)``, fp32 (the reference casts
    g_out back to g's dtype; the ops take fp32 or bf16 decays, so cast if wanted)."""
    _cuda(g, A_log, g_bias, beta)
    H = A_log.shape[0]
    if g.dim() != 3 or g.shape[2] != H * head_k_dim:
        raise ValueError("expected g [B,T,H*head_k_dim] and A_log [H]")
    return _gates(1, g, beta, A_log, g_bias, H, head_k_dim, 1.0, threshold)


def rmsnorm_gated(o: Tensor, weight: Tensor, gate: Optional[Tensor] = None, eps: float = 1e-6,
                  o_layout: str = "bhtd", out_dtype: Optional[torch.dtype] = None) -> Tensor:
    """``o`` as the op returns it ([B,H,T,V], or [B,T,H,V] with ``o_layout="bthd"``), ``gate`` [B,T,H,V] or None,
    ``weight`` [V] -> ``RMSNorm(o) * sigmoid(gate)`` as [B,T,H,V]."""
    _cuda(o, weight, gate)
    if o_layout not in ("bhtd", "bthd") or o.dim() != 4:
        raise ValueError("o must be 4-d with o_layout 'bhtd' or 'bthd'")
    if o_layout == "bhtd" and o.dtype in _NATIVE and not o.is_contiguous() and o.transpose(1, 2).is_contiguous():
        # what the op returns for token-major inputs: a [B,H,T,V] view of a [B,T,H,V] array, taken as it is
        o, o_layout = o.transpose(1, 2), "bthd"
    o2 = _act(o)
    if o_layout == "bhtd":
        B, H, T, V = o2.shape
    else:
        B, T, H, V = o2.shape
    if weight.shape != (V,) or (gate is not None and gate.shape != (B, T, H, V)):
        raise ValueError("expected weight [V] and gate [B,T,H,V]")
    g2 = None if gate is None else _act(gate)
    out_dtype = o2.dtype if out_dtype is None else out_dtype
    y = torch.empty((B, T, H, V), dtype=out_dtype if out_dtype in _NATIVE else torch.float32, device=o2.device)
    lib = _lib.load()
    w32 = weight.float().contiguous()         # kept alive until the call has been enqueued
    with torch.cuda.device(o2.device):
        st = lib.dr_gated_rmsnorm(_ptr(o2), _ptr(g2), _ptr(w32), _ptr(y), B, H, T, V,
                                  DR_LAYOUT_BHTD if o_layout == "bhtd" else DR_LAYOUT_BTHD, _NATIVE[o2.dtype],
                                  _NATIVE[g2.dtype] if g2 is not None else DR_F32, _NATIVE[y.dtype], float(eps),
                                  _stream(o2.device))
    _lib.check(st, "dr_gated_rmsnorm")
    return y if y.dtype == out_dtype else y.to(out_dtype)
