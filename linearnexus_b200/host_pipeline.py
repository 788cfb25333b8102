"""Chunkwise forward for inputs that live in HOST memory: copies and kernels overlapped on three streams.

The ops in ``ops.py`` take device tensors.  A caller whose q, k, v (and g, beta) sit in pinned host memory
-- a data loader, an offloaded activation store, a benchmark that times end to end -- pays two PCIe transfers
around a kernel that is ~30x shorter than they are.  Every (batch, head) unit of the op is independent, so this
helper cuts the work into slices and runs

    copy stream   : H2D slice i+1        compute stream : op(slice i)        return stream : D2H slice i-1

at the same time: the kernel disappears behind the copies and the two copy directions run concurrently
(PCIe is full duplex).  Results land in caller-provided (or freshly pinned) host buffers.  The numbers are
those of the same op on the same rows: there is no approximation and no change of kernel.
"""
from typing import Optional, Tuple

import torch

from . import ops

Tensor = torch.Tensor

_FWD = {
    "delta": lambda q, k, v, g, beta, h0, kw: ops.delta_rule_chunkwise(q, k, v, beta, h0, **kw),
    "gated": lambda q, k, v, g, beta, h0, kw: ops.gated_delta_rule_chunkwise(q, k, v, g, beta, initial_state=h0, **kw),
    "kda": lambda q, k, v, g, beta, h0, kw: ops.kda_chunkwise(q, k, v, g, beta, initial_state=h0, **kw),
}


def _pinned(t: Optional[Tensor], name: str) -> None:
    if t is None:
        return
    if t.is_cuda:
        raise ValueError(f"{name} is already on the device: call the op in linearnexus_b200.ops directly")
    if not t.is_pinned():
        raise ValueError(f"{name} must be in pinned host memory (tensor.pin_memory()) for asynchronous copies")


class HostPipeline:
    """Reusable streams/events for ``chunkwise_from_host`` on one device."""

    def __init__(self, device=None):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        with torch.cuda.device(self.device):
            self.h2d = torch.cuda.Stream()
            self.compute = torch.cuda.Stream()
            self.d2h = torch.cuda.Stream()

    def chunkwise_from_host(self, variant: str, q: Tensor, k: Tensor, v: Tensor, g: Optional[Tensor], beta: Tensor,
                            initial_state: Optional[Tensor] = None, out: Optional[Tensor] = None,
                            final_state: Optional[Tensor] = None, slices: Optional[int] = None,
                            **op_kwargs) -> Tuple[Tensor, Tensor]:
        """``variant`` in {"delta", "gated", "kda"}; q, k, v, g, beta as for the chunkwise op but in pinned host
        memory, ``[B,H,T,D]``.  Returns ``(o, final_state)`` as pinned host tensors (``out`` / ``final_state`` when
        given).  ``slices``: number of pieces the work is cut into (default: one piece per 8 MB of input, at most 8,
        of the flattened batch x head axis -- every piece costs one kernel's latency, measured best at 4-8 for
        large calls -- or one per batch row when the tensors are not plain contiguous [B,H,T,D]).  The call returns when
        the results are in host memory."""
        if variant not in _FWD:
            raise ValueError(f"unknown variant {variant!r}")
        if (g is None) != (variant == "delta"):
            raise ValueError("g must be given for 'gated' / 'kda' and omitted for 'delta'")
        for name, t in (("q", q), ("k", k), ("v", v), ("g", g), ("beta", beta), ("initial_state", initial_state),
                        ("out", out), ("final_state", final_state)):
            _pinned(t, name)
        B, H, T, K = q.shape
        V = v.shape[-1]
        # Every (batch, head) unit is independent: slice the flattened unit axis (B*H) so that the first copy and
        # the last kernel / copy-back -- the parts of the pipeline that cannot overlap -- are short.  That needs
        # [B,H,T,D]-contiguous tensors with one q/k head per head; otherwise slice whole batch rows.
        flat = (q.shape[1] == v.shape[1] and beta.dim() == 3 and
                all(t is None or t.is_contiguous() for t in (q, k, v, g, beta, initial_state, out, final_state)))
        if flat:
            U = B * H
            q, k, v = q.view(1, U, T, K), k.view(1, U, T, K), v.view(1, U, T, V)
            g = None if g is None else g.view(1, U, *g.shape[2:])
            beta = beta.reshape(1, U, T)
            initial_state = None if initial_state is None else initial_state.view(1, U, K, V)
            if slices is None:
                # every slice costs one launch and a handful of copies: small calls (a few MB) go as one piece
                in_bytes = sum(t.numel() * t.element_size() for t in (q, k, v, g, beta) if t is not None)
                slices = max(1, min(8, in_bytes // (8 << 20)))
            n = max(1, min(U, int(slices)))
            bounds = [(U * i // n, U * (i + 1) // n) for i in range(n)]
            ax = 1
        else:
            U = B
            n = B if slices is None else max(1, min(int(slices), B))
            bounds = [(B * i // n, B * (i + 1) // n) for i in range(n)]
            ax = 0
        dev = self.device
        o_dtype = torch.float32 if variant == "kda" and "out_dtype" not in op_kwargs else op_kwargs.get("out_dtype", q.dtype)
        if out is None:
            out = torch.empty((B, H, T, V), dtype=o_dtype).pin_memory()
        if final_state is None:
            final_state = torch.empty((B, H, K, V), dtype=torch.float32).pin_memory()
        out_v = out.view(1, B * H, T, V) if flat else out
        fs_v = final_state.view(1, B * H, K, V) if flat else final_state
        cut = (lambda t, lo, hi: t[:, lo:hi]) if ax == 1 else (lambda t, lo, hi: t[lo:hi])
        caller = torch.cuda.current_stream(dev)
        start = torch.cuda.Event()
        start.record(caller)
        for st in (self.h2d, self.compute, self.d2h):
            st.wait_event(start)
        keep = []   # device tensors stay referenced until the final synchronisation
        for lo, hi in bounds:
            with torch.cuda.stream(self.h2d):
                ins = [None if t is None else cut(t, lo, hi).to(dev, non_blocking=True)
                       for t in (q, k, v, g, beta, initial_state)]
                ready = torch.cuda.Event()
                ready.record(self.h2d)
            with torch.cuda.stream(self.compute):
                self.compute.wait_event(ready)
                o_d, s_d = _FWD[variant](*ins, op_kwargs)
                done = torch.cuda.Event()
                done.record(self.compute)
            with torch.cuda.stream(self.d2h):
                self.d2h.wait_event(done)
                cut(out_v, lo, hi).copy_(o_d, non_blocking=True)
                cut(fs_v, lo, hi).copy_(s_d, non_blocking=True)
            for t in ins + [o_d, s_d]:
                if t is not None:
                    t.record_stream(self.compute)
                    t.record_stream(self.d2h)
            keep.append((ins, o_d, s_d))
        end = torch.cuda.Event()
        end.record(self.d2h)
        caller.wait_event(end)
        end.synchronize()
        return out, final_state


_default = {}


def chunkwise_from_host(variant, q, k, v, g, beta, **kwargs):
    """Module-level convenience over a per-device ``HostPipeline``."""
    dev = torch.cuda.current_device()
    if dev not in _default:
        _default[dev] = HostPipeline(torch.device("cuda", dev))
    return _default[dev].chunkwise_from_host(variant, q, k, v, g, beta, **kwargs)
