"""Per-phase cycle counts of the chunk kernels (developer tool).

The kernels carry ``clock64()`` counters that are compiled in only with ``-DDR_PROFILE``.  This module
builds that variant of the library next to the normal one (``libdeltarule_sm100_prof.so``), runs one of
the workloads below on seeded synthetic inputs and prints the average cycles per chunk and phase as seen
by one thread of one CTA.  Numbers taken from this build are for finding the slow phase only; benchmark
figures always come from the normal build.

    python -m linearnexus_b200.profile_phases gdn      # fused tcgen05 forward, B=8 T=4096 H=16
    python -m linearnexus_b200.profile_phases kda      # intra-chunk pass of the two-kernel forward
    python -m linearnexus_b200.profile_phases bwd      # adjoint kernel, bf16 inputs
    python -m linearnexus_b200.profile_phases bwd_kda  # adjoint kernel of the per-channel-decay variant (CUDA cores)
"""
import ctypes
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PROF_LIB = os.path.join(HERE, "libdeltarule_sm100_prof.so")

GDN = {0: "P barrier (scalars visible)", 2: "P wait stage + issue next K,Q", 3: "P wait D1", 4: "P epilogue 1 (X, A_qk, rk)",
       1: "P issue next D1 / decay scan", 5: "P inverse, Tb/Tw, q norms, arrive",
       16: "C wait for the producer", 17: "C issue U^T,W^T + state pass", 22: "C wait U^T,W^T; W tile", 23: "C issue Vn (8 products, thread 0)", 18: "C output epilogue + barrier",
       19: "C wait Vn (+ issue Dq)", 20: "C Vn -> bf16", 21: "C Do, state update + wait"}
KDA = {149: "issue global loads q,k,g", 147: "first use -> smem, norms", 148: "V copy to the record", 140: "barrier", 141: "prefix sum of the decay",
       142: "A_kk, A_qk on mma.sync", 143: "exact diagonal blocks (if any) + barrier", 144: "inverse",
       145: "record tiles (Tb, A_qk, Qg, Kd)", 146: "W product + tile"}
KDA_STATE = {170: "wait record", 171: "wait state update of previous chunk", 172: "state pass", 173: "output epilogue of previous chunk",
             174: "wait Vn", 175: "Vn -> bf16"}
BWD = {150: "loop barrier", 151: "stage q,k,v,dO,S0", 152: "decay scan", 153: "X, A build", 154: "R (+ barrier)",
       155: "inverse, Vn = T R", 156: "dVn", 157: "dR = T^T dVn", 158: "dV, dbeta, dA, dM", 159: "per (row, channel) products",
       160: "dS0"}


def build():
    from . import _lib
    src = os.path.join(HERE, "csrc", "dr_api.cu")
    inc = os.path.join(os.path.dirname(HERE), "include")
    newest = max(os.path.getmtime(os.path.join(HERE, "csrc", f)) for f in os.listdir(os.path.join(HERE, "csrc")))
    if os.path.exists(PROF_LIB) and os.path.getmtime(PROF_LIB) >= newest:
        return
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
           "-Xcompiler", "-fPIC", "-DDR_PROFILE", f"-I{inc}", f"-I{os.path.join(HERE, 'csrc')}", "-o", PROF_LIB, src]
    subprocess.run(cmd, check=True)


def _inputs(torch, variant, B, H, T, seed=1):
    g = torch.Generator().manual_seed(seed)
    n = lambda *s: torch.randn(*s, generator=g)
    q, k, v = n(B, H, T, 128), n(B, H, T, 128), n(B, H, T, 128)
    beta = torch.sigmoid(n(B, H, T))
    gg = torch.nn.functional.logsigmoid(n(B, H, T, 128) + 4.0) if variant == "kda" else \
        torch.nn.functional.logsigmoid(n(B, H, T) + 4.0)
    return [x.bfloat16().cuda() for x in (q, k, v)] + [gg.cuda(), beta.cuda()]


def main(which):
    build()
    import torch
    import linearnexus_b200 as L
    from linearnexus_b200 import _lib, ops
    from pathlib import Path
    _lib.LIB_PATH = Path(PROF_LIB)   # nothing has been loaded yet: the loader opens this build instead
    lib = _lib.load()
    buf = (ctypes.c_ulonglong * 192)()
    if which == "gdn":
        B, H, T, names = 8, 16, 4096, GDN
        q, k, v, g, beta = _inputs(torch, "gated", B, H, T)
        run = lambda: L.gated_delta_rule_chunkwise(q, k, v, g, beta)
        per = T // 64
    elif which == "kda":
        B, H, T, names = 4, 32, 2048, KDA
        q, k, v, g, beta = _inputs(torch, "kda", B, H, T)
        run = lambda: L.kda_chunkwise(q, k, v, g, beta)
        per = 1          # the profiled CTA handles one chunk
    else:
        B, H, T, names = 2, 16, 1024, BWD
        variant = "kda" if which == "bwd_kda" else "gated"
        q, k, v, g, beta = _inputs(torch, variant, B, H, T)
        d_o = torch.randn(B, H, T, 128, device="cuda").bfloat16()
        run = lambda: ops.chunk_backward(variant, q, k, v, g, beta, d_o, chunk_size=64)
        per = T // 64
    for _ in range(3):   # the counters are cleared by every read: the last launch is reported
        run()
        torch.cuda.synchronize()
        lib.dr_debug_read_profile(buf)
    print(f"{which}: B={B} H={H} T={T}, cycles per chunk")
    total = 0
    for i, nm in names.items():
        print(f"  {nm:44s} {buf[i] / per:10.0f}")
        total += buf[i] / per
    print(f"  {'sum':44s} {total:10.0f}")
    if which == "kda":
        print("state kernel (workers, thread 0 of CTA 0), cycles per chunk")
        for i, nm in KDA_STATE.items():
            print(f"  {nm:44s} {buf[i] / (T // 64):10.0f}")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "gdn")
