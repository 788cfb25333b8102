"""Child process of tests/test_gpu_bounds_build.py: runs tiny and ragged shapes through the library that
DELTARULE_SM100_LIB names and writes every output to an .npz file (plus the device status bits seen)."""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
import linearnexus_b200 as L  # noqa: E402
from linearnexus_b200 import _lib  # noqa: E402
from linearnexus_b200.synthetic import make_rows  # noqa: E402


def main(out_path):
    lib = _lib.load()
    out = {"bounds_checked": np.int32(lib.dr_debug_bounds_checked())}
    cu = lambda d: {k: (None if v is None else v.cuda()) for k, v in d.items()}
    n = 0
    for T in (1, 63, 64, 65, 130):
        for (K, V) in ((64, 64), (128, 128), (24, 40)):
            for variant in ("delta", "gated", "kda"):
                for dt in (torch.float32, torch.bfloat16):
                    c = cu(make_rows(variant, 0, 1, 2, T, K, V, seed=T + K, io_dtype=dt, h0_std=0.1))
                    if variant == "delta":
                        a = (c["q"], c["k"], c["v"], c["beta"])
                        fns = ((L.delta_rule_recurrent, {}), (L.delta_rule_chunkwise, {"chunk_size": 64}),
                               (L.delta_rule_chunkwise, {"chunk_size": 64, "path": "fp32"}))
                    else:
                        a = (c["q"], c["k"], c["v"], c["g"], c["beta"])
                        rec, ch = ((L.gated_delta_rule_recurrent, L.gated_delta_rule_chunkwise) if variant == "gated"
                                   else (L.kda_recurrent, L.kda_chunkwise))
                        fns = ((rec, {}), (ch, {"chunk_size": 64}), (ch, {"chunk_size": 32, "path": "fp32"}))
                    for fn, kw in fns:
                        o, s = fn(*a, initial_state=c["h0"], **kw)
                        out[f"o{n}"], out[f"s{n}"] = o.float().cpu().numpy(), s.float().cpu().numpy()
                        n += 1
    # the other scans, odd sizes
    gen = torch.Generator().manual_seed(7)
    rn = lambda *s: torch.randn(*s, generator=gen).cuda()
    for T in (1, 9, 67):
        q, k, a, b = (rn(1, 3, T, 40) * 0.5 for _ in range(4))
        v, gk = rn(1, 3, T, 72), -rn(1, 3, T, 40).abs()
        o, s = L.dplr_delta_rule_recurrent(q, k, v, a, b, gk, initial_state=rn(1, 3, 40, 72) * 0.1)
        out[f"o{n}"], out[f"s{n}"] = o.cpu().numpy(), s.cpu().numpy(); n += 1
        o, s = L.rwkv6_recurrent(q, k, v, gk, rn(3, 40), initial_state=rn(1, 3, 40, 72) * 0.1)
        out[f"o{n}"], out[f"s{n}"] = o.cpu().numpy(), s.cpu().numpy(); n += 1
        y, s = L.ssd_chunk_scan(rn(2, T, 4, 24), rn(2, T, 4), -rn(4).abs(), rn(2, T, 2, 20), rn(2, T, 2, 20), rn(4), n_groups=2,
                                ssm_state=rn(2, 4, 24, 20) * 0.1, dt_bias=rn(4))
        out[f"o{n}"], out[f"s{n}"] = y.cpu().numpy(), s.cpu().numpy(); n += 1
    torch.cuda.synchronize()
    try:
        L.check_device_status()
        out["status_bits"] = np.int32(0)
    except _lib.DeltaRuleError:
        out["status_bits"] = np.int32(lib.dr_last_device_status())
    # the check routine itself, on an index outside its array (no memory is touched)
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    hit = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    rc = lib.dr_debug_bounds_probe(st.data_ptr(), 10, 10, hit.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    out["probe_rc"], out["probe_in_range"], out["probe_status"] = np.int32(rc), np.int32(hit.item()), np.int32(st.item())
    out["count"] = np.int32(n)
    np.savez(out_path, **out)


if __name__ == "__main__":
    main(sys.argv[1])
