"""Parity at the sizes the benchmark times: every BASELINE configuration is launched at its full grid and
checked against the float64 token recurrence of the oracle -- all (batch, head) units at a reduced length,
and a sample of units at the full length (the float64 recurrence of every unit at full length would take
minutes on the host).  Tolerances are the configuration's own: relative error max|x - ref| / max|ref| <= 2e-2
on outputs and final state for bf16 inputs; the same bar for the gradients of the bf16 training
step; for the decode steps the fp32 state cache within 1e-4 of the float64 steps after all 1024 updates and the
bf16 budget on the outputs."""
import numpy as np
import pytest
import torch

import linearnexus_b200 as L
from linearnexus_b200 import _lib, ops
from linearnexus_b200.synthetic import make_rows
from oracle import delta_rule_oracle as O

pytestmark = pytest.mark.gpu
BF16_TOL = 2e-2


def _rel(a, b):
    a, b = a.double().cpu(), b.double()
    return ((a - b).abs().max() / b.abs().max().clamp_min(1e-30)).item()


def _cuda(d):
    return {k: (None if v is None else v.cuda()) for k, v in d.items()}


def _truth(variant, inp, b, h):
    cut = lambda t: None if t is None else t[b:b + 1, h:h + 1].double()
    q, k, v, g, beta, h0 = (cut(inp[x]) for x in ("q", "k", "v", "g", "beta", "h0"))
    if variant == "gated":
        return O.gated_delta_rule_recurrent(q, k, v, g, beta, initial_state=h0, compute_dtype=torch.float64)
    return O.kda_recurrent(q, k, v, g, beta, initial_state=h0, compute_dtype=torch.float64)


def _sample_units(B, H, n, seed):
    rng = np.random.default_rng(seed)
    return sorted({(int(rng.integers(B)), int(rng.integers(H))) for _ in range(8 * n)})[:n]


# ---- cfg 2: Gated DeltaNet forward, bf16, B=8, H=16, K=V=128, chunk 64 ---------------------------------------

def test_cfg2_all_128_sequences_at_reduced_length():
    inp = make_rows("gated", 0, 8, 16, 512, 128, 128, seed=2, io_dtype=torch.bfloat16)
    cu = _cuda(inp)
    o, hT = L.gated_delta_rule_chunkwise(cu["q"], cu["k"], cu["v"], cu["g"], cu["beta"])
    assert _lib.last_path() == "chunk_tcgen05"
    ops.check_device_status()
    d = lambda x: inp[x].double()
    ro, rS = O.gated_delta_rule_recurrent(d("q"), d("k"), d("v"), d("g"), d("beta"), compute_dtype=torch.float64)
    # per unit, so that one bad sequence cannot hide behind the largest one
    for b in range(8):
        for h in range(16):
            assert _rel(o[b, h], ro[b, h]) <= BF16_TOL, (b, h)
            assert _rel(hT[b, h], rS[b, h]) <= BF16_TOL, (b, h)


def test_cfg2_full_length_full_grid_sampled_units():
    inp = make_rows("gated", 0, 8, 16, 4096, 128, 128, seed=2, io_dtype=torch.bfloat16)
    cu = _cuda(inp)
    o, hT = L.gated_delta_rule_chunkwise(cu["q"], cu["k"], cu["v"], cu["g"], cu["beta"])
    assert _lib.last_path() == "chunk_tcgen05"
    ops.check_device_status()
    assert torch.isfinite(o.float()).all() and torch.isfinite(hT).all()
    for (b, h) in _sample_units(8, 16, 8, seed=0):
        ro, rS = _truth("gated", inp, b, h)
        assert _rel(o[b:b + 1, h:h + 1], ro) <= BF16_TOL, (b, h)
        assert _rel(hT[b:b + 1, h:h + 1], rS) <= BF16_TOL, (b, h)
    # the same call on [B,T,H,D] storage (the TMA maps of that layout) gives the same bits
    tr = lambda x: x.transpose(1, 2).contiguous().transpose(1, 2)
    o2, hT2 = L.gated_delta_rule_chunkwise(tr(cu["q"]), tr(cu["k"]), tr(cu["v"]), tr(cu["g"]), tr(cu["beta"]))
    assert torch.equal(o2, o) and torch.equal(hT2, hT)


# ---- cfg 3: KDA forward, bf16, B=4, H=32, K=V=128, random initial state ---------------------------------------

@pytest.mark.parametrize("strong_decay", [False, True])
def test_cfg3_all_128_sequences_at_reduced_length(strong_decay):
    inp = make_rows("kda", 0, 4, 32, 512, 128, 128, seed=3, io_dtype=torch.bfloat16, h0_std=0.02)
    if strong_decay:   # the reference's own kernel benchmark draws g uniformly from [-10, 0] per channel
        gen = torch.Generator().manual_seed(5)
        inp["g"] = -10.0 * torch.rand(inp["g"].shape, generator=gen)
    cu = _cuda(inp)
    o, hT = L.kda_chunkwise(cu["q"], cu["k"], cu["v"], cu["g"], cu["beta"], initial_state=cu["h0"])
    assert _lib.last_path() == "chunk_split_tcgen05" and o.dtype == torch.float32
    ops.check_device_status()
    d = lambda x: inp[x].double()
    ro, rS = O.kda_recurrent(d("q"), d("k"), d("v"), d("g"), d("beta"), initial_state=d("h0"), compute_dtype=torch.float64)
    for b in range(4):
        for h in range(32):
            assert _rel(o[b, h], ro[b, h]) <= BF16_TOL, (b, h)
            # with g in [-10, 0] the final state is whatever the last few tokens wrote: compare against the largest
            # entry of the whole batch rather than of a unit that may have decayed to almost nothing
            assert ((hT[b, h].double().cpu() - rS[b, h]).abs().max() / rS.abs().max()).item() <= BF16_TOL, (b, h)


def test_cfg3_full_length_full_grid_sampled_units():
    inp = make_rows("kda", 0, 4, 32, 8192, 128, 128, seed=3, io_dtype=torch.bfloat16, h0_std=0.02)
    cu = _cuda(inp)
    o, hT = L.kda_chunkwise(cu["q"], cu["k"], cu["v"], cu["g"], cu["beta"], initial_state=cu["h0"])
    assert _lib.last_path() == "chunk_split_tcgen05"
    ops.check_device_status()
    assert torch.isfinite(o).all() and torch.isfinite(hT).all()
    for (b, h) in _sample_units(4, 32, 8, seed=1):
        ro, rS = _truth("kda", inp, b, h)
        assert _rel(o[b:b + 1, h:h + 1], ro) <= BF16_TOL, (b, h)
        assert _rel(hT[b:b + 1, h:h + 1], rS) <= BF16_TOL, (b, h)


# ---- cfg 4: 1024 consecutive in-place decode steps on the full B=256, H=32 cache ------------------------------

def test_cfg4_1024_consecutive_decode_steps_in_place():
    B, H, K, V, steps = 256, 32, 128, 128, 1024
    gen = torch.Generator(device="cuda").manual_seed(4)
    rn = lambda *s: torch.randn(*s, generator=gen, device="cuda")
    nrm = lambda x: x / (x.norm(dim=-1, keepdim=True) + 1e-6)
    q, k = nrm(rn(steps, B, H, K)).bfloat16(), nrm(rn(steps, B, H, K)).bfloat16()
    v = rn(steps, B, H, V).bfloat16()
    g = torch.nn.functional.logsigmoid(rn(steps, B, H) + 4.0)
    beta = torch.sigmoid(rn(steps, B, H))
    S = rn(B, H, K, V) * 0.02
    sub = _sample_units(B, H, 16, seed=4)
    ib = torch.tensor([b for b, _ in sub], device="cuda")
    ih = torch.tensor([h for _, h in sub], device="cuda")
    pick = lambda t: t[ib, ih].double().cpu()[:, None]   # the 16 followed units as a [16, 1, ...] batch
    ref = pick(S)
    worst_o = 0.0
    for i in range(steps):
        o, S2 = L.gated_delta_rule_step(q[i], k[i], v[i], g[i], beta[i], S, inplace=True)
        assert S2.data_ptr() == S.data_ptr()
        ro, ref = O.gated_delta_rule_step(pick(q[i]), pick(k[i]), pick(v[i]), pick(g[i]), pick(beta[i]), ref,
                                          compute_dtype=torch.float64)
        if i % 64 == 0 or i == steps - 1:
            worst_o = max(worst_o, _rel(pick(o), ro))
    assert _lib.last_path() == "step_stream"
    ops.check_device_status()
    assert worst_o <= BF16_TOL            # o is rounded to bf16
    # the fp32 cache itself after 1024 in-place updates: fp32 accumulation error only
    assert (pick(S) - ref).abs().max().item() <= 1e-4 * max(1.0, ref.abs().max().item())


# ---- cfg 5: Gated DeltaNet forward + backward, bf16, 2 batch rows per GPU, H=16 -------------------------------

def _grad_check(inp, d_o, got, groups, tol):
    """`groups`: list of (b, h_lo, h_hi): the float64 autograd of the recurrence runs on a few heads at a time
    (it keeps every per-token state: ~0.6 MB per token and head)."""
    for (b, lo, hi) in groups:
        cut = lambda t: None if t is None else t[b:b + 1, lo:hi]
        ref = O.delta_rule_grads("gated", cut(inp["q"]), cut(inp["k"]), cut(inp["v"]), cut(inp["g"]), cut(inp["beta"]), None,
                                 cut(d_o))
        for h in range(lo, hi):
            for name in ("dq", "dk", "dv", "dg", "dbeta", "dh0"):
                assert _rel(got[name][b, h], ref[name][0, h - lo]) <= tol, (name, b, h)
            assert _rel(got["o"][b, h], ref["o"][0, h - lo]) <= BF16_TOL, ("o", b, h)
            assert _rel(got["hT"][b, h], ref["hT"][0, h - lo]) <= BF16_TOL, ("hT", b, h)


@pytest.mark.parametrize("T,all_units", [(1024, True), (4096, False)])
def test_cfg5_training_step_gradients(T, all_units):
    B, H = 2, 16
    inp = make_rows("gated", 0, B, H, T, 128, 128, seed=5, io_dtype=torch.bfloat16)
    gen = torch.Generator().manual_seed(55)
    d_o = torch.randn(B, H, T, 128, generator=gen).bfloat16()
    cu = _cuda(inp)
    o, hT, saved = ops.chunk_forward_saving("gated", cu["q"], cu["k"], cu["v"], cu["g"], cu["beta"])
    got = ops.chunk_backward("gated", cu["q"], cu["k"], cu["v"], cu["g"], cu["beta"], d_o.cuda(), saved=saved)
    ops.check_device_status()
    got.update(o=o, hT=hT)
    if all_units:
        groups = [(b, lo, lo + 4) for b in range(B) for lo in range(0, H, 4)]
    else:
        groups = [(b, h, h + 1) for (b, h) in _sample_units(B, H, 2, seed=5)]
    _grad_check(inp, d_o, got, groups, tol=2e-2)
