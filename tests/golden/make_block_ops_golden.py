"""Generates tests/golden/block_ops_golden.npz from the CPU oracle of the block steps (float64 arithmetic).

The reference has no golden vectors for its conv / gate / norm helpers and cannot be imported where this was
written (it needs jax), so these vectors come from oracle/block_ops_oracle.py in float64, cross-checked at
generation time against torch's own conv1d.  Run from the repository root:

    python tests/golden/make_block_ops_golden.py
"""
import sys
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import block_ops_oracle as O  # noqa: E402

F64 = torch.float64


def main():
    rng = np.random.default_rng(2024)
    t = lambda *s: torch.from_numpy(rng.standard_normal(s, dtype=np.float32))
    out = {}
    # causal short conv (window 4, the blocks' size) with bias and a warm cache, SiLU applied
    B, T, C, W = 2, 21, 16, 4
    x, w, bias, cache = t(B, T, C), t(W, C) * 0.5, t(C) * 0.1, t(B, W - 1, C)
    y, nc = O.short_conv_silu(x, w, bias, cache, apply_silu=True, compute_dtype=F64)
    pre, _ = O.short_conv_silu(x, w, bias, cache, apply_silu=False, compute_dtype=F64)
    ref = F.conv1d(torch.cat([cache, x], 1).double().transpose(1, 2), w.double().t().unsqueeze(1), bias.double(),
                   groups=C).transpose(1, 2)
    assert (pre - ref).abs().max() < 1e-12
    out.update({"conv.x": x, "conv.w": w, "conv.bias": bias, "conv.cache": cache, "conv.y": y, "conv.new_cache": nc})
    # gate activations of the Gated DeltaNet block and kda_gate (values on both sides of the softplus threshold)
    Bg, Tg, H, K = 2, 9, 3, 8
    a, b, A_log, dt_bias = t(Bg, Tg, H) * 3, t(Bg, Tg, H) * 3, t(H), t(H)
    g, beta = O.gdn_gate_activations(a, b, A_log, dt_bias, allow_neg_eigval=True, compute_dtype=F64)
    out.update({"gdn_gate.a": a, "gdn_gate.b": b, "gdn_gate.A_log": A_log, "gdn_gate.dt_bias": dt_bias,
                "gdn_gate.g": g, "gdn_gate.beta": beta})
    graw, gb, kb = t(Bg, Tg, H * K) * 12, t(H * K), t(Bg, Tg, H)
    gk, bk = O.kda_gate(graw, A_log, K, gb, kb, compute_dtype=F64)
    out.update({"kda_gate.g": graw, "kda_gate.A_log": A_log, "kda_gate.g_bias": gb, "kda_gate.beta": kb,
                "kda_gate.g_out": gk, "kda_gate.beta_out": bk})
    # per-head RMSNorm with the sigmoid gate; o in the op's [B,H,T,V] layout, result [B,T,H,V]
    Bn, Hn, Tn, V = 2, 3, 7, 32
    o, gate, wn = t(Bn, Hn, Tn, V), t(Bn, Tn, Hn, V), torch.from_numpy(rng.random(V, dtype=np.float32)) + 0.5
    yn = O.gated_rmsnorm(o.transpose(1, 2), wn, gate, eps=1e-5, compute_dtype=F64)
    out.update({"norm.o": o, "norm.gate": gate, "norm.w": wn, "norm.y": yn})
    np.savez_compressed(Path(__file__).with_name("block_ops_golden.npz"),
                        **{k: v.numpy() for k, v in out.items()})
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
