"""Generates tests/golden/delta_rule_golden.npz from the CPU oracle (float64 arithmetic).

The reference ships no golden vectors for the delta-rule ops and cannot be imported where
this was written (it needs jax/flax), so these vectors come from the oracle's float64 token
recurrences, cross-checked at generation time against the oracle's chunk forms (the
reference's own self-consistency tests, re-expressed).  Run from the repository root:

    python tests/golden/make_golden.py
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import delta_rule_oracle as O  # noqa: E402

F64 = torch.float64
CASES = {
    # name: (variant, B, H, T, K, V, chunk, seed, h0_std)
    "delta": ("delta", 1, 2, 40, 16, 32, 16, 11, 0.1),
    "gated": ("gated", 1, 2, 40, 16, 32, 32, 12, 0.1),
    "kda": ("kda", 1, 2, 40, 16, 32, 32, 13, 0.1),
}


def main():
    out = {}
    for name, (variant, B, H, T, K, V, C, seed, h0s) in CASES.items():
        inp = O.make_inputs(variant, B, H, T, K, V, seed, h0_std=h0s)
        q, k, v, g, beta, h0 = (inp[x] for x in ("q", "k", "v", "g", "beta", "h0"))
        # un-normalise so that the in-op l2norm has something to do
        q = q * 1.7
        k = k * 0.6
        d = lambda x: None if x is None else x.double()
        if variant == "delta":
            o, hT = O.delta_rule_recurrent(d(q), d(k), d(v), d(beta), d(h0), compute_dtype=F64)
            o2, hT2 = O.delta_rule_chunkwise(d(q), d(k), d(v), d(beta), d(h0), chunk_size=C, compute_dtype=F64)
            so, sS = O.delta_rule_step(d(q[:, :, 0]), d(k[:, :, 0]), d(v[:, :, 0]), d(beta[:, :, 0]), d(h0), compute_dtype=F64)
        elif variant == "gated":
            o, hT = O.gated_delta_rule_recurrent(d(q), d(k), d(v), d(g), d(beta), initial_state=d(h0), compute_dtype=F64)
            o2, hT2 = O.gated_delta_rule_chunkwise(d(q), d(k), d(v), d(g), d(beta), initial_state=d(h0), chunk_size=C, compute_dtype=F64)
            so, sS = O.gated_delta_rule_step(d(q[:, :, 0]), d(k[:, :, 0]), d(v[:, :, 0]), d(g[:, :, 0]), d(beta[:, :, 0]), d(h0), compute_dtype=F64)
        else:
            o, hT = O.kda_recurrent(d(q), d(k), d(v), d(g), d(beta), initial_state=d(h0), compute_dtype=F64)
            o2, hT2 = O.kda_chunkwise(d(q), d(k), d(v), d(g), d(beta), initial_state=d(h0), chunk_size=C, compute_dtype=F64)
            so, sS = O.kda_step(d(q[:, :, 0]), d(k[:, :, 0]), d(v[:, :, 0]), d(g[:, :, 0]), d(beta[:, :, 0]), d(h0), compute_dtype=F64)
        assert (o - o2).abs().max() < 1e-10 and (hT - hT2).abs().max() < 1e-10, name
        do = torch.from_numpy(np.random.default_rng(seed + 100).standard_normal((B, H, T, V), dtype=np.float32))
        dhT = torch.from_numpy(np.random.default_rng(seed + 200).standard_normal((B, H, K, V), dtype=np.float32)) * 0.1
        gr = O.delta_rule_grads(variant, q, k, v, g, beta, h0, do, dhT, use_qk_l2norm=(variant != "delta"))
        assert (gr["o"] - o).abs().max() < 1e-10
        for key, val in dict(q=q, k=k, v=v, g=g, beta=beta, h0=h0, do=do, dhT=dhT).items():
            if val is not None:
                out[f"{name}.{key}"] = val.numpy().astype(np.float32)
        out[f"{name}.chunk"] = np.int32(C)
        for key, val in dict(o=o, hT=hT, step_o=so, step_S=sS, dq=gr["dq"], dk=gr["dk"], dv=gr["dv"],
                             dg=gr["dg"], dbeta=gr["dbeta"], dh0=gr["dh0"]).items():
            if val is not None:
                out[f"{name}.{key}"] = val.numpy().astype(np.float64)
    np.savez_compressed(Path(__file__).with_name("delta_rule_golden.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
