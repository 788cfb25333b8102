"""Device timing of the element-wise block steps against the HBM roofline.

    python -m linearnexus_b200.bench_block_ops [--steps 20] [--warmup 5]

One JSON line per kernel at the block shape of the headline benchmark (B=8, T=4096, 16 heads of 128, bf16):
algorithmic bytes (every input read once, every output written once) over the CUDA-event time of one launch,
against the measured copy bandwidth in ``MEASURED_PEAKS.json`` next to the package (6650 GB/s if absent).
Inputs are larger than L2, so no flush is needed between launches.
"""
import argparse
import json
from pathlib import Path

import torch



def _time(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    args = ap.parse_args()
    peaks = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    peak, src = (float(json.loads(peaks.read_text())["hbm_gbs"]), "measured") if peaks.exists() else (6650.0, "fallback")
    B, T, H, D, W = 8, 4096, 16, 128, 4
    C = H * D
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(B, T, C, device="cuda", generator=g).bfloat16()
    w = torch.randn(W, C, device="cuda", generator=g)
    o = torch.randn(B, H, T, D, device="cuda", generator=g).bfloat16()
    gate = torch.randn(B, T, H, D, device="cuda", generator=g).bfloat16()
    wn = torch.rand(D, device="cuda", generator=g) + 0.5
    a, b = torch.randn(B, T, H, device="cuda", generator=g), torch.randn(B, T, H, device="cuda", generator=g)
    A_log, dt_bias = torch.zeros(H, device="cuda"), torch.zeros(H, device="cuda")
    # the C entry points on preallocated outputs: a launch costs the host a few microseconds, so back-to-back
    # launches keep the GPU busy and the event time is kernel time
    import ctypes
    from . import _lib
    lib = _lib.load()
    ptr = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    y = torch.empty_like(x)
    cache = torch.empty(B, W - 1, C, device="cuda", dtype=torch.bfloat16)
    yn = torch.empty(B, T, H, D, device="cuda", dtype=torch.bfloat16)
    go, bo = torch.empty_like(a), torch.empty_like(b)
    BF, F32 = _lib.DR_BF16, _lib.DR_F32

    def chk(status):
        _lib.check(status, "bench_block_ops")
    cases = [
        ("short_conv_silu", lambda: chk(lib.dr_short_conv_silu(ptr(x), ptr(w), None, None, ptr(y), ptr(cache), B, T, C, W,
                                                               BF, 1, st)),
         2 * x.numel() * 2 + w.numel() * 4 + B * (W - 1) * C * 2),
        ("gated_rmsnorm", lambda: chk(lib.dr_gated_rmsnorm(ptr(o), ptr(gate), ptr(wn), ptr(yn), B, H, T, D,
                                                           _lib.DR_LAYOUT_BHTD, BF, BF, BF, 1e-6, st)), 3 * o.numel() * 2),
        ("gated_rmsnorm_token_major", lambda: chk(lib.dr_gated_rmsnorm(ptr(o), ptr(gate), ptr(wn), ptr(yn), B, H, T, D,
                                                                       _lib.DR_LAYOUT_BTHD, BF, BF, BF, 1e-6, st)),
         3 * o.numel() * 2),
        ("gate_activations", lambda: chk(lib.dr_gate_activations(0, ptr(a), ptr(b), ptr(A_log), ptr(dt_bias), ptr(go),
                                                                 ptr(bo), B, T, H, 1, F32, F32, 1.0, 0.0, st)),
         4 * a.numel() * 4),
    ]
    for name, fn, nbytes in cases:
        ms = _time(fn, args.steps, args.warmup)
        gbs = nbytes / ms / 1e6
        print(json.dumps({"kernel": name, "ms": round(ms, 4), "alg_bytes": nbytes, "achieved_gbs": round(gbs, 1),
                          "peak_gbs": peak, "peak_source": src, "frac": round(gbs / peak, 3),
                          "shape": f"B={B} T={T} H={H} D={D} bf16"}))


if __name__ == "__main__":
    main()
