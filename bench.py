#!/usr/bin/env python
"""Benchmark of the delta-rule hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" is one pass of the hot path over one batch of seeded synthetic input.  The default
workload is the configuration the headline metric is quoted on: Gated DeltaNet chunkwise
forward, bf16 q/k/v/o with fp32 accumulation, B=8, T=4096, H=16, d_k=d_v=128, chunk 64.

With N > 1 (launched by torch.distributed.run, one rank per GPU) the global batch is N x the per-GPU
batch; every rank builds exactly its rows of it (the rows carry their own seeds, so the cut equals
`linearnexus_b200.shard.shard_inputs` of the whole batch) and runs them with no collective on the data
path -- weak scaling.  NCCL carries the barrier, the max-over-ranks of the device time and the gather of
every rank's parity figures.  `strong` (N > 1, forward workloads) times the SAME global batch as N = 1
cut over the ranks.

Rank 0 prints ONE JSON line.  `value` is device-timed throughput with inputs resident in HBM;
`e2e` is the same metric through the public op with host (pinned) inputs and outputs, copies
inside the timed region; `roofline` is the dominant kernel against the measured peak; `parity` is the
largest error of sampled (batch, head) units of the timed configuration against the float64 recurrence
(computed outside the timed regions); `cpu_baseline` is the CPU oracle timed on a bounded sample of the
same workload.  `--impl reference` times that CPU path alone (the reference itself needs JAX, which is
not installed on these machines; the oracle restates its maths in torch).
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
    # name: variant, B (per GPU), T, H, K, V, chunk, kind
    "gdn_fwd": dict(variant="gated", B=8, T=4096, H=16, K=128, V=128, chunk=64, kind="chunk_fwd", cfg_id=2),
    # the same call on the blocks' native [B,T,H,D] storage (transposed views, no copies)
    "gdn_fwd_bthd": dict(variant="gated", B=8, T=4096, H=16, K=128, V=128, chunk=64, kind="chunk_fwd", cfg_id=2, bthd=True),
    "kda_fwd": dict(variant="kda", B=4, T=8192, H=32, K=128, V=128, chunk=64, kind="chunk_fwd", cfg_id=3),
    # same shape with the decay and the output in bf16 (the block's activation dtype; opt-in output dtype)
    "kda_fwd_bf16": dict(variant="kda", B=4, T=8192, H=32, K=128, V=128, chunk=64, kind="chunk_fwd", cfg_id=3,
                         g_bf16=True, out_bf16=True),
    # 1024 consecutive decode steps on fresh inputs walk a [1024, ...] buffer (step i uses entry i % 1024)
    "gdn_decode": dict(variant="gated", B=256, T=1, H=32, K=128, V=128, chunk=0, kind="decode", cfg_id=4),
    # training configuration: B=16 over 8 GPUs = 2 batch rows per GPU; forward + backward
    "gdn_fwd_bwd": dict(variant="gated", B=2, T=4096, H=16, K=128, V=128, chunk=64, kind="fwd_bwd", cfg_id=5),
    "deltanet_fwd_fp32": dict(variant="delta", B=2, T=512, H=4, K=64, V=64, chunk=64, kind="chunk_fwd", cfg_id=1),
    # the other matrix-state scans (token recurrence, state in registers); the reference quotes no configuration for
    # them, so they take the headline's batch, length and head count at those models' usual head sizes
    "dplr_fwd": dict(variant="dplr", B=8, T=4096, H=16, K=64, V=64, chunk=0, kind="scan", cfg_id=6),
    "rwkv6_fwd": dict(variant="rwkv6", B=8, T=4096, H=16, K=64, V=64, chunk=0, kind="scan", cfg_id=7),
    "ssd_fwd": dict(variant="ssd", B=8, T=4096, H=16, K=128, V=64, chunk=0, kind="scan", cfg_id=8, groups=1),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
DECODE_BUFFER = 1024


def alg_flops_per_token_head(C, K, V):
    # 3 CxCxK products + 2 CxCxV products + 3 CxKxV products at 2 flop/MAC + the triangular inverse
    return 6 * C * K + 4 * C * V + 6 * K * V + C * C / 3.0


def alg_bytes(w, io_bytes=2):
    """Algorithmic bytes of one step: every input and output once at its storage width."""
    B, H, T, K, V = w["B"], w["H"], w["T"], w["K"], w["V"]
    units = B * H
    if w["kind"] == "scan":
        state = units * 2 * 4 * K * V                       # initial state in, final state out
        if w["variant"] == "ssd":                           # x, y per head; B, C per group; dt float32 per head
            return B * T * (H * (2 * io_bytes * V + 4) + w["groups"] * 2 * io_bytes * K) + state
        n_key = 5 if w["variant"] == "dplr" else 3          # q k a b gk | r k w
        return units * T * io_bytes * (n_key * K + 2 * V) + state
    if w["kind"] == "decode":
        return units * (2 * 4 * K * V + io_bytes * (2 * K + V) + 8 + io_bytes * V)
    g_bytes = (2 if w.get("g_bf16") else 4) * K if w["variant"] == "kda" else (4 if w["variant"] == "gated" else 0)
    o_bytes = 4 if w["variant"] == "kda" and not w.get("out_bf16") else io_bytes
    per_token = io_bytes * (2 * K + V) + o_bytes * V + g_bytes + 4
    total = units * T * per_token + units * 4 * K * V            # + final state
    if w["variant"] == "kda":
        total += units * 4 * K * V                               # + initial state
    if w["kind"] == "fwd_bwd":
        # backward alone: read q,k,v,do and g,beta; write dq,dk,dv and dbeta,dg
        total += units * T * (io_bytes * (2 * K + 2 * V) + 8 + io_bytes * (2 * K + V) + 8)
    return total


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", 0.0)), "source": "measured"}
    return dict(FALLBACK_PEAKS, source="fallback")


def ncu_traffic(workload, path):
    """DRAM bytes per launch of the step's kernels from the committed profiler captures (null when none)."""
    p = ROOT / "profiles" / "ncu_traffic.json"
    if not p.exists():
        return None
    rec = json.loads(p.read_text()).get(f"{workload}:{path}")
    return None if rec is None else rec["dram_bytes_per_step"]


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


def h2d_probe(pin_tensors, dev, barrier, reps=3):
    """Host-to-device bandwidth of this rank with every rank copying at once: `reps` copies of the step's pinned
    inputs between two barriers, device-timed.  Explains the end-to-end figure: the copies of all ranks share the
    host's memory and PCIe roots."""
    ts = [t for t in pin_tensors if t is not None]
    dst = [torch.empty(t.shape, dtype=t.dtype, device=dev) for t in ts]
    for d_, t in zip(dst, ts):
        d_.copy_(t, non_blocking=True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(reps):
        for d_, t in zip(dst, ts):
            d_.copy_(t, non_blocking=True)
    e1.record()
    barrier()
    nbytes = reps * sum(t.numel() * t.element_size() for t in ts)
    return nbytes / (e0.elapsed_time(e1) * 1e-3) / 1e9


def host_rows(w, lo, hi):
    """Rows lo..hi-1 of the workload's global batch (pinned host memory, the op's [B,H,T,D] layout)."""
    from linearnexus_b200.synthetic import make_rows
    io = torch.float32 if w["cfg_id"] == 1 else torch.bfloat16
    h0 = 0.02 if w["kind"] == "decode" or w["variant"] == "kda" else None
    host = make_rows(w["variant"], lo, hi, w["H"], w["T"], w["K"], w["V"], seed=1234 + w["cfg_id"], io_dtype=io,
                     h0_std=h0, g_dtype=torch.bfloat16 if w.get("g_bf16") else torch.float32)
    return {k: (None if v is None else v.contiguous().pin_memory()) for k, v in host.items()}


def rel_err(got, ref):
    got, ref = got.double().cpu(), ref.double()
    return float((got - ref).abs().max() / ref.abs().max().clamp_min(1e-30))


def forward_parity(w, host, o, hT, n_units=4, seed=0):
    """Largest relative error (max|x - ref| / max|ref|) of o and the final state over `n_units` sampled (b, h)
    units against the float64 token recurrence of the oracle."""
    from oracle import delta_rule_oracle as O   # checker only: outside every timed region
    B, H = host["q"].shape[0], host["q"].shape[1]
    rng = np.random.default_rng(seed)
    units = sorted({(int(rng.integers(B)), int(rng.integers(H))) for _ in range(4 * n_units)})[:n_units]
    eo = es = 0.0
    for (b, h) in units:
        cut = lambda t: None if t is None else t[b:b + 1, h:h + 1].double()
        q, k, v, g, beta, h0 = (cut(host[x]) for x in ("q", "k", "v", "g", "beta", "h0"))
        if w["variant"] == "delta":
            ro, rS = O.delta_rule_recurrent(q, k, v, beta, h0, compute_dtype=torch.float64)
        elif w["variant"] == "gated":
            ro, rS = O.gated_delta_rule_recurrent(q, k, v, g, beta, initial_state=h0, compute_dtype=torch.float64)
        else:
            ro, rS = O.kda_recurrent(q, k, v, g, beta, initial_state=h0, compute_dtype=torch.float64)
        eo = max(eo, rel_err(o[b:b + 1, h:h + 1], ro))
        es = max(es, rel_err(hT[b:b + 1, h:h + 1], rS))
    return {"o_rel": eo, "state_rel": es, "units": len(units), "against": "float64 token recurrence (oracle)"}


# ---- the other scans (RWKV-7 DPLR, RWKV-6, Mamba-2 SSD) -----------------------------------------------------------

def scan_host_inputs(w, rows, seed, heads=None):
    """Seeded inputs of one scan workload, `rows` batch rows, float32 values rounded to bf16 where stored as bf16."""
    H, T, K, V = heads or w["H"], w["T"], w["K"], w["V"]
    rng = np.random.default_rng(seed)
    f = lambda *s, scale=1.0: torch.from_numpy(rng.standard_normal(s, dtype=np.float32)) * scale
    bf = lambda t: t.to(torch.bfloat16)
    if w["variant"] == "dplr":
        kk = torch.nn.functional.normalize(f(rows, H, T, K), dim=-1)
        return dict(q=bf(f(rows, H, T, K)), k=bf(f(rows, H, T, K, scale=0.5)), v=bf(f(rows, H, T, V)), a=bf(-kk),
                    b=bf(kk * torch.sigmoid(f(rows, H, T, K))), gk=bf(-torch.exp(f(rows, H, T, K) - 1.0)),
                    h0=f(rows, H, K, V, scale=0.02))
    if w["variant"] == "rwkv6":
        return dict(r=bf(f(rows, H, T, K)), k=bf(f(rows, H, T, K, scale=0.5)), v=bf(f(rows, H, T, V)),
                    w=bf(-f(rows, H, T, K).abs() - 0.5), u=f(H, K, scale=0.5), h0=f(rows, H, K, V, scale=0.02))
    G = w["groups"] if heads is None else 1
    return dict(x=bf(f(rows, T, H, V)), dt=f(rows, T, H, scale=0.5), A=-torch.exp(f(H, scale=0.5)),
                B=bf(f(rows, T, G, K, scale=0.5)), C=bf(f(rows, T, G, K, scale=0.5)), D=f(H), dt_bias=f(H, scale=0.3),
                h0=f(rows, H, V, K, scale=0.02))


def scan_call(mod, w, t, cd=None):
    """The public function of the workload on tensors `t`; `mod` is the package or (with cd) the oracle module."""
    kw = {} if cd is None else dict(compute_dtype=cd)
    if w["variant"] == "dplr":
        return mod.dplr_delta_rule_recurrent(t["q"], t["k"], t["v"], t["a"], t["b"], t["gk"], scale=w["K"] ** -0.5,
                                             initial_state=t["h0"], **kw)
    if w["variant"] == "rwkv6":
        return mod.rwkv6_recurrent(t["r"], t["k"], t["v"], t["w"], t["u"], scale=w["K"] ** -0.5, initial_state=t["h0"], **kw)
    return mod.ssd_chunk_scan(t["x"], t["dt"], t["A"], t["B"], t["C"], t["D"], chunk_size=256, n_groups=t["B"].shape[2],
                              ssm_state=t["h0"], dt_bias=t["dt_bias"], dt_limit=(0.001, 5.0), **kw)


def scan_unit(w, host, b, h):
    """Inputs of the single (batch b, head h) sequence, float64, for the oracle."""
    d = lambda x: x.double()
    if w["variant"] == "ssd":
        g = h // (host["x"].shape[2] // host["B"].shape[2])
        return dict(x=d(host["x"][b:b + 1, :, h:h + 1]), dt=d(host["dt"][b:b + 1, :, h:h + 1]), A=d(host["A"][h:h + 1]),
                    B=d(host["B"][b:b + 1, :, g:g + 1]), C=d(host["C"][b:b + 1, :, g:g + 1]), D=d(host["D"][h:h + 1]),
                    dt_bias=d(host["dt_bias"][h:h + 1]), h0=d(host["h0"][b:b + 1, h:h + 1]))
    out = {k: d(v[b:b + 1, h:h + 1]) for k, v in host.items() if k != "u"}
    if "u" in host:
        out["u"] = d(host["u"][h:h + 1])
    return out


def run_scan(args, w, rank, world, dev):
    import linearnexus_b200 as L
    from linearnexus_b200 import _lib
    from oracle import linear_recurrences_oracle as R   # checker only: outside every timed region
    _lib.load()
    B = w["B"]
    host = scan_host_inputs(w, B, seed=(1234 + w["cfg_id"]) * 4096 + rank)
    pin = {k: v.contiguous().pin_memory() for k, v in host.items()}
    devt = {k: v.to(dev, non_blocking=True) for k, v in pin.items()}
    torch.cuda.synchronize(dev)
    step = lambda: scan_call(L, w, devt)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(dev.index)
    if rank == 0:
        sampler.start()
    n0 = _lib.launch_count()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    barrier()
    ev[0].record()
    for i in range(args.steps):
        step()
        ev[i + 1].record()
    barrier()
    total_ms = ev[0].elapsed_time(ev[-1])
    launches = _lib.launch_count() - n0
    path = _lib.last_path()
    clocks = sampler.stop() if rank == 0 else None

    o, hT = step()
    torch.cuda.synchronize(dev)
    rng = np.random.default_rng(rank)
    units = sorted({(int(rng.integers(B)), int(rng.integers(w["H"]))) for _ in range(8)})[:2]
    eo = es = 0.0
    for (b, h) in units:
        ro, rs = scan_call(R, w, scan_unit(w, host, b, h), cd=torch.float64)
        got_o = o[b:b + 1, :, h:h + 1] if w["variant"] == "ssd" else o[b:b + 1, h:h + 1]
        eo, es = max(eo, rel_err(got_o, ro)), max(es, rel_err(hT[b:b + 1, h:h + 1], rs))
    parity = {"o_rel": eo, "state_rel": es, "units": len(units), "against": "float64 token recurrence (oracle)"}

    # end to end: pinned host inputs -> device -> public function -> pinned host outputs, all inside the timed region
    out_host = [torch.empty(o.shape, dtype=o.dtype).pin_memory(), torch.empty(hT.shape, dtype=hT.dtype).pin_memory()]

    def e2e_step():
        t = {k: v.to(dev, non_blocking=True) for k, v in pin.items()}
        oo, ss = scan_call(L, w, t)
        out_host[0].copy_(oo, non_blocking=True)
        out_host[1].copy_(ss, non_blocking=True)

    e2e_step()
    e2e_steps = max(1, min(args.steps, 5))
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record()
    for _ in range(e2e_steps):
        e2e_step()
    t1.record()
    barrier()
    e2e_ms = t0.elapsed_time(t1) / e2e_steps
    h2d_gbs = h2d_probe(list(pin.values()), dev, barrier)
    times = torch.tensor([total_ms, e2e_ms, eo, es, -h2d_gbs], dtype=torch.float64, device=dev)
    if world > 1:
        gathered = [torch.empty_like(times) for _ in range(world)]
        torch.distributed.all_gather(gathered, times)
        allv = torch.stack(gathered)
        parity["per_rank"] = allv[:, 2:4].tolist()
        parity["units"] *= world
        times = allv.max(dim=0).values
    total_ms, e2e_ms, parity["o_rel"], parity["state_rel"], neg_h2d = times.tolist()
    ms = total_ms / args.steps
    tokens = B * w["T"]
    return dict(ms_per_step=ms, value=world * tokens / (ms * 1e-3), e2e_value=world * tokens / (e2e_ms * 1e-3),
                h2d=sum(v.numel() * v.element_size() for v in pin.values()),
                d2h=sum(v.numel() * v.element_size() for v in out_host), launches=launches, path=path, clocks=clocks,
                kernel_ms=ms, parity=parity, strong=None, h2d_gbs=-neg_h2d)


def cpu_scan_sample(w, target_s=12.0):
    """The float32 CPU oracle of a scan workload on a few heads of one batch row at the full length, scaled linearly."""
    from oracle import linear_recurrences_oracle as R
    torch.set_num_threads(os.cpu_count() or 1)
    heads = 4
    inp = {k: (v.float() if v.dtype == torch.bfloat16 else v) for k, v in scan_host_inputs(w, 1, seed=99, heads=heads).items()}
    scan_call(R, w, inp, cd=torch.float32)
    t0, reps = time.perf_counter(), 0
    while True:
        scan_call(R, w, inp, cd=torch.float32)
        reps += 1
        el = time.perf_counter() - t0
        if el >= target_s or reps >= 200:
            break
    sec = el / reps
    value = w["B"] * w["T"] * (heads / (w["B"] * w["H"])) / sec
    sample = (f"{w['variant']} oracle (torch fp32, CPU) on B=1,H={heads},T={w['T']},K={w['K']},V={w['V']} "
              f"({reps} reps, {sec:.3f} s each), scaled linearly in B*H to the full workload")
    return dict(value=value, cores=torch.get_num_threads(), sample=sample, sec_per_rep=sec, reps=reps)


def run_ours(args, w, rank, world, dev):
    import linearnexus_b200 as L
    from linearnexus_b200 import _lib, ops
    _lib.load()  # raises if the CUDA library is missing: there is no fallback

    B = w["B"]
    pin = host_rows(w, rank * B, (rank + 1) * B)
    devt = {k: (None if v is None else v.to(dev, non_blocking=True)) for k, v in pin.items()}
    torch.cuda.synchronize(dev)
    decode = w["kind"] == "decode"
    fwd_bwd = w["kind"] == "fwd_bwd"
    tokens_per_step = B * w["T"]
    kda_kw = dict(out_dtype=torch.bfloat16) if w.get("out_bf16") else {}
    if w.get("bthd"):   # the blocks' storage: [B,T,H,D] arrays seen as [B,H,T,D] views (what a transpose-free block passes)
        for x in ("q", "k", "v", "g", "beta"):
            devt[x] = devt[x].transpose(1, 2).contiguous().transpose(1, 2)

    def forward(t, **extra):
        if w["variant"] == "gated":
            return L.gated_delta_rule_chunkwise(t["q"], t["k"], t["v"], t["g"], t["beta"], chunk_size=w["chunk"], **extra)
        if w["variant"] == "kda":
            return L.kda_chunkwise(t["q"], t["k"], t["v"], t["g"], t["beta"], initial_state=t["h0"], chunk_size=w["chunk"],
                                   **kda_kw, **extra)
        return L.delta_rule_chunkwise(t["q"], t["k"], t["v"], t["beta"], chunk_size=w["chunk"], **extra)

    dec = None
    if decode:
        # fresh q, k, v, g, beta for every one of DECODE_BUFFER consecutive steps, generated on the device
        gen = torch.Generator(device=dev).manual_seed(4321 + rank)
        H, K, V = w["H"], w["K"], w["V"]
        rn = lambda *s: torch.randn(*s, generator=gen, device=dev)
        nrm = lambda x: x / (x.norm(dim=-1, keepdim=True) + 1e-6)
        dec = dict(q=nrm(rn(DECODE_BUFFER, B, H, K)).bfloat16(), k=nrm(rn(DECODE_BUFFER, B, H, K)).bfloat16(),
                   v=rn(DECODE_BUFFER, B, H, V).bfloat16(),
                   g=torch.nn.functional.logsigmoid(rn(DECODE_BUFFER, B, H) + 4.0), beta=torch.sigmoid(rn(DECODE_BUFFER, B, H)))
        state0 = devt["h0"].clone()
        state = devt["h0"]
        counter = [0]

        def step():
            i = counter[0] % DECODE_BUFFER
            counter[0] += 1
            return L.gated_delta_rule_step(dec["q"][i], dec["k"][i], dec["v"][i], dec["g"][i], dec["beta"][i], state, inplace=True)
    elif fwd_bwd:
        gen = torch.Generator().manual_seed(7 + rank)
        d_o = torch.randn(B, w["H"], w["T"], w["V"], generator=gen).to(torch.bfloat16)
        pin_do = d_o.pin_memory()
        d_o = pin_do.to(dev)

        def step():   # one forward (which keeps the per-chunk states) + the backward that uses them
            o, hT, saved = ops.chunk_forward_saving("gated", devt["q"], devt["k"], devt["v"], devt["g"], devt["beta"],
                                                    chunk_size=w["chunk"])
            gr = ops.chunk_backward("gated", devt["q"], devt["k"], devt["v"], devt["g"], devt["beta"], d_o,
                                    chunk_size=w["chunk"], saved=saved)
            return o, hT, gr
    else:
        def step():
            return forward(devt)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize(dev)

    def timed(fn, steps):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        barrier()
        ev[0].record()
        for i in range(steps):
            fn()
            ev[i + 1].record()
        barrier()
        return ev[0].elapsed_time(ev[-1]), [ev[i].elapsed_time(ev[i + 1]) for i in range(steps)]

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
    n0 = _lib.launch_count()
    total_ms, per_launch_ms = timed(step, args.steps)
    launches = _lib.launch_count() - n0
    path = _lib.last_path()
    clocks = sampler.stop() if rank == 0 else None
    ops.check_device_status(dev)   # a bounded wait that ran out inside a kernel raises here

    # ---- parity of the timed configuration (outside the timed regions) ----
    if decode:
        from oracle import delta_rule_oracle as O
        n_par = min(max(args.steps, 8), 64)
        sub = [(int(b), int(h)) for b, h in np.random.default_rng(rank).integers(0, [B, w["H"]], size=(16, 2))]
        S = state0.clone()
        ref = torch.stack([state0[b, h] for b, h in sub]).double().cpu()[:, None]   # [16,1,K,V]
        eo = 0.0
        for i in range(n_par):
            o, _ = L.gated_delta_rule_step(dec["q"][i], dec["k"][i], dec["v"][i], dec["g"][i], dec["beta"][i], S, inplace=True)
            pick = lambda t: torch.stack([t[i][b, h] for b, h in sub]).double().cpu()[:, None]
            ro, ref = O.gated_delta_rule_step(pick(dec["q"]), pick(dec["k"]), pick(dec["v"]), pick(dec["g"]), pick(dec["beta"]),
                                              ref, compute_dtype=torch.float64)
            eo = max(eo, rel_err(torch.stack([o[b, h] for b, h in sub])[:, None], ro))
        es = float((torch.stack([S[b, h] for b, h in sub]).double().cpu()[:, None] - ref).abs().max())
        parity = {"o_rel": eo, "state_abs": es, "units": len(sub), "steps": n_par,
                  "against": "float64 gated_delta_rule_step (oracle), consecutive in-place steps"}
        del S
    else:
        out = step()
        torch.cuda.synchronize(dev)
        parity = forward_parity(w, pin, out[0], out[1], seed=rank)
    ops.check_device_status(dev)

    # ---- end-to-end region: host (pinned) inputs -> public op -> host outputs, copies timed ----
    names = ("q", "k", "v", "g", "beta")
    out_host = None
    e2e_steps = max(1, min(args.steps, 5))

    def e2e_step():
        nonlocal out_host
        if decode:
            i = counter[0] % 8
            counter[0] += 1
            ins = [e2e_in[x][i].to(dev, non_blocking=True) for x in names]
            o, _ = L.gated_delta_rule_step(*ins, state, inplace=True)
            outs = [o]
        elif not fwd_bwd and not w.get("bthd"):
            # the public host-memory entry point: batch slices, H2D / kernel / D2H overlapped on three streams
            if out_host is None:
                o_dt = torch.float32 if w["variant"] == "kda" and not w.get("out_bf16") else pin["q"].dtype
                out_host = [torch.empty((B, w["H"], w["T"], w["V"]), dtype=o_dt).pin_memory(),
                            torch.empty((B, w["H"], w["K"], w["V"]), dtype=torch.float32).pin_memory()]
            kw = dict(chunk_size=w["chunk"], **kda_kw)
            if pin.get("h0") is not None:
                kw["initial_state"] = pin["h0"]
            L.chunkwise_from_host(w["variant"], pin["q"], pin["k"], pin["v"], pin["g"], pin["beta"],
                                  out=out_host[0], final_state=out_host[1], **kw)
            return
        else:
            ins = {x: (None if pin[x] is None else pin[x].to(dev, non_blocking=True)) for x in names}
            ins["h0"] = devt["h0"]
            if w.get("bthd"):
                for x in names:
                    ins[x] = ins[x].transpose(1, 2).contiguous().transpose(1, 2)
            if fwd_bwd:
                do_dev = pin_do.to(dev, non_blocking=True)
                o, hT, saved = ops.chunk_forward_saving("gated", ins["q"], ins["k"], ins["v"], ins["g"], ins["beta"],
                                                        chunk_size=w["chunk"])
                gr = ops.chunk_backward("gated", ins["q"], ins["k"], ins["v"], ins["g"], ins["beta"], do_dev,
                                        chunk_size=w["chunk"], saved=saved)
                outs = [o, hT] + [gr[x] for x in ("dq", "dk", "dv", "dg", "dbeta")]
            else:
                outs = list(forward(ins))
        if out_host is None:
            out_host = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in outs]
        for h_, t in zip(out_host, outs):
            h_.copy_(t, non_blocking=True)

    if decode:
        e2e_in = {x: dec[x][:8].cpu().pin_memory() for x in names}   # host copies of the first buffer entries
        counter[0] = 0
        e2e_steps = min(e2e_steps, 8)
    e2e_step()
    t_e0 = torch.cuda.Event(enable_timing=True); t_e1 = torch.cuda.Event(enable_timing=True)
    barrier()
    t_e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    t_e1.record()
    barrier()
    e2e_ms = t_e0.elapsed_time(t_e1) / e2e_steps
    if decode:
        h2d = sum(e2e_in[x][0].numel() * e2e_in[x].element_size() for x in names)
    else:
        h2d = sum(pin[x].numel() * pin[x].element_size() for x in names if pin[x] is not None)
        if fwd_bwd:
            h2d += pin_do.numel() * pin_do.element_size()
        elif pin.get("h0") is not None and not w.get("bthd"):
            h2d += pin["h0"].numel() * pin["h0"].element_size()
    d2h = sum(t.numel() * t.element_size() for t in out_host)
    h2d_gbs = h2d_probe([e2e_in[x] for x in names] if decode else [pin[x] for x in names], dev, barrier)

    # ---- strong scaling of the forward: the N = 1 global batch cut over the ranks ----
    strong = None
    if world > 1 and w["kind"] == "chunk_fwd" and not args.no_strong:
        from linearnexus_b200.shard import shard_inputs
        Bg = B                                    # the same global batch as a 1-GPU run
        whole = {k: v for k, v in host_rows(w, 0, Bg).items()}
        mine, mode = shard_inputs(whole, world, rank)
        md = {k: (None if v is None else v.contiguous().to(dev)) for k, v in mine.items()}
        if w.get("bthd"):
            for x in names:
                md[x] = md[x].transpose(1, 2).contiguous().transpose(1, 2)
        for _ in range(3):
            forward(md)
        s_ms, _ = timed(lambda: forward(md), args.steps)
        so, sh = forward(md)
        torch.cuda.synchronize(dev)
        sp = forward_parity(w, mine, so, sh, n_units=2, seed=rank)
        strong = dict(ms=s_ms / args.steps, mode=mode, units=int(md["q"].shape[0] * md["q"].shape[1]), parity=sp)

    times = torch.tensor([total_ms, e2e_ms, strong["ms"] if strong else 0.0, parity["o_rel"],
                          parity.get("state_rel", parity.get("state_abs", 0.0)),
                          strong["parity"]["o_rel"] if strong else 0.0, strong["parity"]["state_rel"] if strong else 0.0,
                          -h2d_gbs],
                         dtype=torch.float64, device=dev)
    per_rank = per_rank_ms = None
    if world > 1:
        gathered = [torch.empty_like(times) for _ in range(world)]
        torch.distributed.all_gather(gathered, times)     # NCCL: every rank's times and parity figures
        allv = torch.stack(gathered)
        per_rank = allv[:, 3:5].tolist()
        per_rank_ms = (allv[:, 0] / args.steps).tolist()
        times = allv.max(dim=0).values                     # slowest rank, worst error
    total_ms, e2e_ms, strong_ms, p_o, p_s, sp_o, sp_s, neg_h2d = times.tolist()   # max over ranks; slowest copy
    parity["o_rel"] = p_o
    parity["state_rel" if "state_rel" in parity else "state_abs"] = p_s
    if per_rank is not None:
        parity["per_rank"] = per_rank
        parity["units"] = parity["units"] * world
    ms_per_step = total_ms / args.steps
    res = dict(ms_per_step=ms_per_step, value=world * tokens_per_step / (ms_per_step * 1e-3),
               e2e_value=world * tokens_per_step / (e2e_ms * 1e-3), h2d=h2d, d2h=d2h, launches=launches, path=path,
               clocks=clocks, kernel_ms=float(np.mean(per_launch_ms)), parity=parity, strong=None, h2d_gbs=-neg_h2d,
               per_rank_ms=per_rank_ms)
    if strong:
        res["strong"] = {"global_batch": B, "units_per_rank": strong["units"], "sharded_over": strong["mode"],
                         "ms_per_step": strong_ms, "value": B * w["T"] / (strong_ms * 1e-3), "unit": "tokens/s",
                         "parity": {"o_rel": sp_o, "state_rel": sp_s},
                         "note": "one CTA per (batch, head) sequence: the cut leaves units_per_rank CTAs for 148 SMs, "
                                 "so the step time stays that of one sequence"}
    return res


def cpu_oracle_sample(w, target_s=12.0, threads=None):
    """Times the CPU oracle (torch fp32 restatement of the reference op) on a bounded sample of
    the workload: a (batch x head) slice at the full sequence length, scaled linearly."""
    if w["kind"] == "scan":
        return cpu_scan_sample(w, target_s)
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
    sample = (f"{'gated_delta_rule_step' if w['kind'] == 'decode' else w['variant'] + ' chunkwise'} oracle (torch fp32, CPU, forward only) on "
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
    ap.add_argument("--no-strong", action="store_true", help="skip the strong-scaling sub-record of multi-GPU forward runs")
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
              "delta_rule_fwd_bwd_tokens_per_sec" if w["kind"] == "fwd_bwd" else
              f"{w['variant']}_scan_fwd_tokens_per_sec" if w["kind"] == "scan" else "delta_rule_fwd_tokens_per_sec")
    what = {"decode": "decode step", "fwd_bwd": "chunkwise forward + backward", "scan": "scan forward"}.get(w["kind"], "chunkwise forward")
    config = {"workload": f"{args.workload}: {w['variant']} {what} "
                          f"B={w['B']} T={w['T']} H={w['H']} d_k={w['K']} d_v={w['V']} chunk={w['chunk']} per GPU"
                          + (", inputs stored [B,T,H,D]" if w.get("bthd") else ""),
              "per_gpu_batch": w["B"], "global_batch": w["B"] * world, "seq_len": w["T"], "heads": w["H"],
              "sharding": f"rows of one seeded global batch, {world} rank(s), no data-path collective",
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
                "note": "the reference is pure JAX and JAX is not installed here; this is the CPU oracle that restates it. "
                        "One host times a bounded sample and the figure is its throughput in tokens/s, which does not "
                        "depend on how many GPUs the other arm uses: at N > 1 it is the rate at which this host's cores "
                        "would work through the N-GPU global batch"}
        print(json.dumps(line))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path for the product)")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=dev)
    res = run_scan(args, w, rank, world, dev) if w["kind"] == "scan" else run_ours(args, w, rank, world, dev)
    if world > 1:
        torch.distributed.barrier()
    if rank == 0:
        peaks = load_peaks()
        units = w["B"] * w["H"] * w["T"]
        C = w["chunk"] or 64
        # duration of the step's kernels together (one launch for the fused forward and the decode step;
        # intra + state pass for the two-kernel forward; forward + pre-pass + adjoint + finalize for fwd_bwd)
        ktime = res["ms_per_step"] * 1e-3
        alg_b = alg_bytes(w, 4 if w["cfg_id"] == 1 else 2)
        if w["kind"] in ("decode", "scan"):
            roof = {"bound": "hbm", "achieved": alg_b / ktime / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s"}
        else:
            flops = alg_flops_per_token_head(C, w["K"], w["V"]) * units * (3 if w["kind"] == "fwd_bwd" else 1)
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
        roof["traffic"] = ncu_traffic(args.workload, res["path"]) if not args.batch else None
        cpu = None
        if not args.no_cpu_baseline:
            c = cpu_oracle_sample(w, target_s=args.cpu_seconds)
            cpu = {"value": c["value"], "unit": "tokens/s", "cores": c["cores"], "kind": "port", "sample": c["sample"]}
        line = {"metric": metric, "value": res["value"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32" if w["cfg_id"] == 1 or w["kind"] == "scan" else "bf16", "data": "synthetic",
                "config": config,
                "e2e": {"value": res["e2e_value"], "unit": "tokens/s", "h2d_bytes_per_step": res["h2d"],
                        "d2h_bytes_per_step": res["d2h"],
                        # pinned host -> device GB/s of the slowest rank with all ranks copying at once (the ceiling of e2e)
                        "h2d_gbs_slowest_rank": res["h2d_gbs"]},
                "gpu_launches": res["launches"], "clocks": res["clocks"], "roofline": roof, "parity": res["parity"],
                "cpu_baseline": cpu}
        if res["strong"]:
            line["strong"] = res["strong"]
        if res.get("per_rank_ms"):
            line["ms_per_step_per_rank"] = res["per_rank_ms"]   # `ms_per_step` is their maximum
        print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
