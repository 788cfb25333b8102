#!/usr/bin/env python
"""Benchmark of the delta-rule hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" is one pass of the hot path over one batch of seeded synthetic input.  The default
workload is the configuration the headline metric is quoted on: Gated DeltaNet chunkwise
forward, bf16 q/k/v/o with fp32 accumulation, B=8, T=4096, H=16, d_k=d_v=128, chunk 64.
With N > 1 (launched by torch.distributed.run, one rank per GPU) every rank runs the same
per-GPU batch on its own (batch x head) units -- weak scaling, no collective on the data path;
NCCL only carries the barrier and the max-over-ranks of the device time.

Rank 0 prints ONE JSON line.  `value` is device-timed throughput with inputs resident in HBM;
`e2e` is the same metric through the public op with host (pinned) inputs and outputs, copies
inside the timed region; `roofline` is the dominant kernel against the measured peak;
`cpu_baseline` is the CPU oracle timed on a bounded sample of the same workload.
`--impl reference` times that CPU path alone (the reference itself needs JAX, which is not
installed on these machines; the oracle restates its maths in torch).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402
import torch  # noqa: E402

WORKLOADS = {
    # name: variant, B, T, H, K, V, chunk, io dtype, kind
    "gdn_fwd": dict(variant="gated", B=8, T=4096, H=16, K=128, V=128, chunk=64, kind="chunk_fwd", cfg_id=2),
    "kda_fwd": dict(variant="kda", B=4, T=8192, H=32, K=128, V=128, chunk=64, kind="chunk_fwd", cfg_id=3),
    # same shape with the decay and the output in bf16 (the block's activation dtype; opt-in output dtype)
    "kda_fwd_bf16": dict(variant="kda", B=4, T=8192, H=32, K=128, V=128, chunk=64, kind="chunk_fwd", cfg_id=3,
                         g_bf16=True, out_bf16=True),
    "gdn_decode": dict(variant="gated", B=256, T=1, H=32, K=128, V=128, chunk=0, kind="decode", cfg_id=4),
    # training configuration: B=16 over 8 GPUs = 2 batch rows per GPU; forward + backward
    "gdn_fwd_bwd": dict(variant="gated", B=2, T=4096, H=16, K=128, V=128, chunk=64, kind="fwd_bwd", cfg_id=5),
    "deltanet_fwd_fp32": dict(variant="delta", B=2, T=512, H=4, K=64, V=64, chunk=64, kind="chunk_fwd", cfg_id=1),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel (ncu, see profiles/*.md)
NCU_TRAFFIC = {
    "gdn_fwd:chunk_tcgen05": 504.4e6,   # profiles/chunk_sm100_kernel_gdn_fwd.md (B=4 capture scaled by sequences)
    "kda_fwd:chunk_split_tcgen05": 3.78e9,    # profiles/kda_split_kernels.md: both kernels, B=1 capture x 4 sequences-wise
    "gdn_decode:step": 1026.8e6,        # profiles/step_kernel_gdn_decode.md (full size)
    "gdn_decode:step_stream": 1023.5e6, # same file, second capture
    "gdn_fwd_bwd:bwd_saved": 2123.1e6,  # profiles/bwd_chunk_kernel_phases.md: saving forward + pre-pass + adjoint + finalize (full size)
}


def alg_flops_per_token_head(C, K, V):
    # 3 CxCxK products + 2 CxCxV products + 3 CxKxV products at 2 flop/MAC + the triangular inverse
    return 6 * C * K + 4 * C * V + 6 * K * V + C * C / 3.0


def alg_bytes_per_token_head(w, io_bytes=2):
    K, V = w["K"], w["V"]
    if w["kind"] == "decode":
        return 2 * 4 * K * V + io_bytes * (2 * K + V) + 8 + io_bytes * V
    g_bytes = (2 if w.get("g_bf16") else 4) * K if w["variant"] == "kda" else 4
    o_bytes = 4 if w["variant"] == "kda" and not w.get("out_bf16") else io_bytes
    return io_bytes * (2 * K + V) + o_bytes * V + g_bytes + 4


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", 0.0)), "source": "measured"}
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, val in zip(names, f[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def make_host_inputs(w, seed, n_sets=1):
    """Seeded inputs on the host in the op's [B,H,T,D] layout (bf16 q,k,v; fp32 g, beta)."""
    from oracle.delta_rule_oracle import make_inputs  # input generator only; nothing is computed by the oracle here
    io = torch.float32 if w["cfg_id"] == 1 else torch.bfloat16
    sets = []
    for s in range(n_sets):
        h0 = 0.02 if w["kind"] == "decode" or w["variant"] == "kda" else None
        sets.append(make_inputs(w["variant"], w["B"], w["H"], w["T"], w["K"], w["V"], seed + s, io_dtype=io, h0_std=h0,
                                g_dtype=torch.bfloat16 if w.get("g_bf16") else torch.float32))
    return sets


def run_ours(args, w, rank, world, dev):
    import linearnexus_b200 as L
    from linearnexus_b200 import _lib
    lib = _lib.load()  # raises if the CUDA library is missing: there is no fallback

    host = make_host_inputs(w, 1234 + w["cfg_id"] + 1000 * rank)[0]
    pin = {k: (None if v is None else v.contiguous().pin_memory()) for k, v in host.items()}
    devt = {k: (None if v is None else v.to(dev, non_blocking=True)) for k, v in pin.items()}
    torch.cuda.synchronize(dev)
    decode = w["kind"] == "decode"
    tokens_per_step = w["B"] * w["T"]
    kda_kw = dict(out_dtype=torch.bfloat16) if w.get("out_bf16") else {}

    if decode:
        q, k, v, g, beta = (devt[x][:, :, 0].contiguous() if devt[x] is not None else None for x in ("q", "k", "v", "g", "beta"))
        state = devt["h0"].clone()

        def step():
            return L.gated_delta_rule_step(q, k, v, g, beta, state, inplace=True)
    elif w["kind"] == "fwd_bwd":
        from linearnexus_b200 import ops as _ops
        gen = torch.Generator().manual_seed(7)
        d_o = torch.randn(w["B"], w["H"], w["T"], w["V"], generator=gen).to(torch.bfloat16).to(dev)

        def step():   # one forward (which keeps the per-chunk states) + the backward that uses them
            o, hT, saved = _ops.chunk_forward_saving("gated", devt["q"], devt["k"], devt["v"], devt["g"], devt["beta"],
                                                     chunk_size=w["chunk"])
            gr = _ops.chunk_backward("gated", devt["q"], devt["k"], devt["v"], devt["g"], devt["beta"], d_o,
                                     chunk_size=w["chunk"], saved=saved)
            return o, gr["dq"]
    elif w["variant"] == "gated":
        def step():
            return L.gated_delta_rule_chunkwise(devt["q"], devt["k"], devt["v"], devt["g"], devt["beta"], chunk_size=w["chunk"])
    elif w["variant"] == "kda":
        def step():
            return L.kda_chunkwise(devt["q"], devt["k"], devt["v"], devt["g"], devt["beta"], initial_state=devt["h0"],
                                   chunk_size=w["chunk"], **kda_kw)
    else:
        def step():
            return L.delta_rule_chunkwise(devt["q"], devt["k"], devt["v"], devt["beta"], chunk_size=w["chunk"])

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(args.warmup):
        step()
    # short steps (the fused forward is 0.3 ms): keep warming for ~50 ms so that clocks and caches are in
    # their steady state when the timed region starts (untimed, on top of the W warm-up steps)
    torch.cuda.synchronize(dev)
    t_spin = time.perf_counter()
    while not args.no_steady_warmup and time.perf_counter() - t_spin < 0.05:
        step()
        torch.cuda.synchronize(dev)
    barrier()
    sampler = ClockSampler(dev.index)
    if rank == 0:
        sampler.start()
    # ---- device-timed region: inputs resident in HBM, K steps, CUDA events on the launch stream ----
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    n0 = _lib.launch_count()
    barrier()
    ev[0].record()
    for i in range(args.steps):
        step()
        ev[i + 1].record()
    barrier()
    launches = _lib.launch_count() - n0
    path = _lib.last_path()
    total_ms = ev[0].elapsed_time(ev[-1])
    per_launch_ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
    clocks = sampler.stop() if rank == 0 else None

    # ---- end-to-end region: host (pinned) inputs -> public op -> host outputs, copies timed ----
    names = ("q", "k", "v", "g", "beta") if not decode else ()
    fwd_bwd = w["kind"] == "fwd_bwd"
    pin_do = d_o.cpu().pin_memory() if fwd_bwd else None
    out_host = None
    e2e_steps = max(1, min(args.steps, 5))

    def e2e_step():
        nonlocal out_host
        if decode:
            qh, kh, vh, gh, bh = (pin[x][:, :, 0].contiguous().pin_memory() for x in ("q", "k", "v", "g", "beta"))
            ins = [t.to(dev, non_blocking=True) for t in (qh, kh, vh, gh, bh)]
            o, _ = L.gated_delta_rule_step(*ins, state, inplace=True)
            outs = [o]
        else:
            if not fwd_bwd:
                # the public host-memory entry point: batch slices, H2D / kernel / D2H overlapped on three streams
                if out_host is None:
                    o_dt = torch.float32 if w["variant"] == "kda" and not w.get("out_bf16") else pin["q"].dtype
                    out_host = [torch.empty((w["B"], w["H"], w["T"], w["V"]), dtype=o_dt).pin_memory(),
                                torch.empty((w["B"], w["H"], w["K"], w["V"]), dtype=torch.float32).pin_memory()]
                kw = dict(chunk_size=w["chunk"], **kda_kw)
                if pin.get("h0") is not None:
                    kw["initial_state"] = pin["h0"]
                L.chunkwise_from_host(w["variant"], pin["q"], pin["k"], pin["v"], pin["g"], pin["beta"],
                                      out=out_host[0], final_state=out_host[1], **kw)
                return out_host
            ins = {x: (None if pin[x] is None else pin[x].to(dev, non_blocking=True)) for x in names}
            if fwd_bwd:
                do_dev = pin_do.to(dev, non_blocking=True)
                o, hT, saved = _ops.chunk_forward_saving("gated", ins["q"], ins["k"], ins["v"], ins["g"], ins["beta"],
                                                         chunk_size=w["chunk"])
                gr = _ops.chunk_backward("gated", ins["q"], ins["k"], ins["v"], ins["g"], ins["beta"], do_dev,
                                         chunk_size=w["chunk"], saved=saved)
            elif w["variant"] == "gated":
                o, hT = L.gated_delta_rule_chunkwise(ins["q"], ins["k"], ins["v"], ins["g"], ins["beta"], chunk_size=w["chunk"])
            elif w["variant"] == "kda":
                o, hT = L.kda_chunkwise(ins["q"], ins["k"], ins["v"], ins["g"], ins["beta"], initial_state=devt["h0"], chunk_size=w["chunk"])
            else:
                o, hT = L.delta_rule_chunkwise(ins["q"], ins["k"], ins["v"], ins["beta"], chunk_size=w["chunk"])
            outs = [o, hT] + ([gr[x] for x in ("dq", "dk", "dv", "dg", "dbeta")] if fwd_bwd else [])
        if out_host is None:
            out_host = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in outs]
        for h_, t in zip(out_host, outs):
            h_.copy_(t, non_blocking=True)
        return outs

    e2e_step()
    barrier()
    t_e0 = torch.cuda.Event(enable_timing=True); t_e1 = torch.cuda.Event(enable_timing=True)
    t_e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    t_e1.record()
    barrier()
    e2e_ms = t_e0.elapsed_time(t_e1) / e2e_steps
    if decode:
        h2d = sum(pin[x][:, :, 0].numel() * pin[x].element_size() for x in ("q", "k", "v", "g", "beta"))
    else:
        h2d = sum(pin[x].numel() * pin[x].element_size() for x in names if pin[x] is not None)
        if fwd_bwd:
            h2d += pin_do.numel() * pin_do.element_size()
        elif pin.get("h0") is not None:
            h2d += pin["h0"].numel() * pin["h0"].element_size()
    d2h = sum(t.numel() * t.element_size() for t in out_host)

    times = torch.tensor([total_ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        torch.distributed.all_reduce(times, op=torch.distributed.ReduceOp.MAX)
    total_ms, e2e_ms = times.tolist()
    ms_per_step = total_ms / args.steps
    value = world * tokens_per_step / (ms_per_step * 1e-3)
    e2e_value = world * tokens_per_step / (e2e_ms * 1e-3)
    return dict(ms_per_step=ms_per_step, value=value, e2e_value=e2e_value, h2d=h2d, d2h=d2h,
                launches=launches, path=path, clocks=clocks, kernel_ms=float(np.mean(per_launch_ms)),
                inputs=host)


def cpu_oracle_sample(w, target_s=12.0, threads=None):
    """Times the CPU oracle (torch fp32 restatement of the reference op) on a bounded sample of
    the workload: a (batch x head) slice at the full sequence length, scaled linearly."""
    from oracle import delta_rule_oracle as O
    # torchrun exports OMP_NUM_THREADS=1: the CPU arm is meant to use every host core it can
    torch.set_num_threads(threads or os.cpu_count() or 1)
    cores = torch.get_num_threads()
    heads = 8 if w["kind"] != "decode" else w["H"]
    batch = 1 if w["kind"] != "decode" else 8
    inp = O.make_inputs(w["variant"], batch, heads, w["T"] if w["kind"] != "decode" else 1, w["K"], w["V"], seed=99,
                        io_dtype=torch.bfloat16 if w["cfg_id"] != 1 else torch.float32, h0_std=0.02)

    def once():
        if w["kind"] == "decode":
            return O.gated_delta_rule_step(inp["q"][:, :, 0], inp["k"][:, :, 0], inp["v"][:, :, 0], inp["g"][:, :, 0],
                                           inp["beta"][:, :, 0], inp["h0"])
        if w["variant"] == "gated":
            return O.gated_delta_rule_chunkwise(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], chunk_size=w["chunk"])
        if w["variant"] == "kda":
            return O.kda_chunkwise(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], initial_state=inp["h0"], chunk_size=w["chunk"])
        return O.delta_rule_chunkwise(inp["q"], inp["k"], inp["v"], inp["beta"], chunk_size=w["chunk"])

    once()  # warm-up
    t0 = time.perf_counter()
    reps = 0
    while True:
        once()
        reps += 1
        el = time.perf_counter() - t0
        if el >= target_s or reps >= 500:
            break
    sec = el / reps
    # the workload has B*H units; the sample has batch*heads of them
    scale = (batch * heads) / (w["B"] * w["H"])
    value = (w["B"] * w["T"]) * scale / sec
    sample = (f"{'gated_delta_rule_step' if w['kind'] == 'decode' else w['variant'] + ' chunkwise'} oracle (torch fp32, CPU) on "
              f"B={batch},H={heads},T={w['T']},K={w['K']},V={w['V']} ({reps} reps, {sec:.3f} s each), "
              f"scaled linearly in B*H to the full workload")
    return dict(value=value, cores=cores, sample=sample, sec_per_rep=sec, reps=reps)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="gdn_fwd", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="CPU seconds the cpu_baseline sample may take")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=0, help="override the per-GPU batch (profiling captures of a small case)")
    ap.add_argument("--no-steady-warmup", action="store_true",
                    help="skip the ~50 ms of extra untimed launches (profiler captures: keeps the launch count small)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    w = dict(WORKLOADS[args.workload])
    if args.batch:
        w["B"] = args.batch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    metric = ("decode_tokens_per_sec" if w["kind"] == "decode" else
              "delta_rule_fwd_bwd_tokens_per_sec" if w["kind"] == "fwd_bwd" else "delta_rule_fwd_tokens_per_sec")
    config = {"workload": f"{args.workload}: {w['variant']} {'decode step' if w['kind'] == 'decode' else 'chunkwise forward'} "
                          f"B={w['B']} T={w['T']} H={w['H']} d_k={w['K']} d_v={w['V']} chunk={w['chunk']} per GPU",
              "per_gpu_batch": w["B"], "global_batch": w["B"] * world, "seq_len": w["T"], "heads": w["H"],
              "sharding": f"batch x head units, {world} rank(s), no data-path collective",
              "l2": "inputs larger than L2 (no flush needed)" if w["cfg_id"] != 1 else "inputs fit in L2 (latency-bound case)"}

    if args.impl == "reference":
        if rank != 0:
            return
        steps = max(1, args.steps)
        per = max(2.0, min(args.cpu_seconds, 120.0 / max(1, steps + args.warmup)))
        vals, info = [], None
        for i in range(args.warmup + steps):
            info = cpu_oracle_sample(w, target_s=per)
            if i >= args.warmup:
                vals.append(info["value"])
        value = float(np.mean(vals))
        ms = w["B"] * w["T"] / value * 1e3
        line = {"impl": "reference", "metric": metric, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
                "steps": steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
                "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": info["cores"], "kind": "port",
                                 "sample": info["sample"]},
                "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "note": "the reference is pure JAX and JAX is not installed here; this is the CPU oracle that restates it"}
        print(json.dumps(line))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path for the product)")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=dev)
    res = run_ours(args, w, rank, world, dev)
    if world > 1:
        torch.distributed.barrier()
    if rank == 0:
        peaks = load_peaks()
        units = w["B"] * w["H"] * w["T"]
        C = w["chunk"] or 64
        # duration of the step's kernels together (one launch for the fused forward and the decode step;
        # intra + state pass for the two-kernel forward; forward + adjoint + finalize for fwd_bwd)
        ktime = res["ms_per_step"] * 1e-3
        if w["kind"] == "decode":
            alg_b = alg_bytes_per_token_head(w) * units
            roof = {"bound": "hbm", "achieved": alg_b / ktime / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s"}
        else:
            flops = alg_flops_per_token_head(C, w["K"], w["V"]) * units * (3 if w["kind"] == "fwd_bwd" else 1)
            alg_b = alg_bytes_per_token_head(w, 4 if w["cfg_id"] == 1 else 2) * units
            tf = flops / ktime / 1e12
            hb = alg_b / ktime / 1e9
            if w["variant"] == "kda":
                # 94 flop per algorithmic byte (fp32 g and output): left of the ridge, HBM is the binding roof
                roof = {"bound": "hbm", "achieved": hb, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "tensor_tflops": tf, "tensor_frac": tf / peaks["bf16_tflops"]}
            else:
                roof = {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                        "hbm_gbs": hb, "hbm_frac": hb / peaks["hbm_gbs"]}
        roof["frac"] = roof["achieved"] / roof["peak"]
        roof["peak_source"] = peaks["source"]
        roof["kernel"] = res["path"]
        roof["alg_bytes_per_launch"] = alg_b
        # DRAM bytes per launch from the ncu captures summarised under profiles/ (per workload and kernel)
        roof["traffic"] = NCU_TRAFFIC.get(f"{args.workload}:{res['path']}") if not args.batch else None
        cpu = None
        if not args.no_cpu_baseline:
            c = cpu_oracle_sample(w, target_s=args.cpu_seconds)
            cpu = {"value": c["value"], "unit": "tokens/s", "cores": c["cores"], "kind": "port", "sample": c["sample"]}
        line = {"metric": metric, "value": res["value"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32" if w["cfg_id"] == 1 else "bf16", "data": "synthetic", "config": config,
                "e2e": {"value": res["e2e_value"], "unit": "tokens/s", "h2d_bytes_per_step": res["h2d"],
                        "d2h_bytes_per_step": res["d2h"]},
                "gpu_launches": res["launches"], "clocks": res["clocks"], "roofline": roof, "cpu_baseline": cpu}
        print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
