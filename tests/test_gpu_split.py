"""GPU tests of the two-kernel chunk forward (chunk-parallel intra pass + tcgen05 state pass): KDA with
per-channel decay, and the scalar-decay / decay-free variants through the same kernels, each against
the float64 token recurrence of the oracle and against the exact fp32 chunk kernel."""
import pytest
import torch

import linearnexus_b200 as L
from linearnexus_b200 import _lib
from oracle import delta_rule_oracle as O

pytestmark = pytest.mark.gpu
BF16_TOL = 2e-2  # max|x - ref| / max|ref| for bf16 inputs with fp32 accumulation


def _rel(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return ((a - b).abs().max() / b.abs().max().clamp_min(1e-30)).item()


def _truth(variant, inp):
    d = lambda x: None if x is None else x.double()
    q, k, v, g, beta, h0 = (d(inp[x]) for x in ("q", "k", "v", "g", "beta", "h0"))
    if variant == "delta":
        return O.delta_rule_recurrent(q, k, v, beta, h0, compute_dtype=torch.float64)
    if variant == "gated":
        return O.gated_delta_rule_recurrent(q, k, v, g, beta, initial_state=h0, compute_dtype=torch.float64)
    return O.kda_recurrent(q, k, v, g, beta, initial_state=h0, compute_dtype=torch.float64)


def _run(variant, inp, path, **kw):
    cu = {k: (None if v is None else v.cuda()) for k, v in inp.items()}
    if variant == "delta":
        out = L.delta_rule_chunkwise(cu["q"], cu["k"], cu["v"], cu["beta"], cu["h0"], chunk_size=64, path=path)
    elif variant == "gated":
        out = L.gated_delta_rule_chunkwise(cu["q"], cu["k"], cu["v"], cu["g"], cu["beta"], initial_state=cu["h0"],
                                           chunk_size=64, path=path)
    else:
        out = L.kda_chunkwise(cu["q"], cu["k"], cu["v"], cu["g"], cu["beta"], initial_state=cu["h0"],
                              chunk_size=64, path=path, **kw)
    return out


@pytest.mark.parametrize("g_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,H,T,h0", [(1, 1, 64, None), (1, 2, 128, 0.02), (2, 3, 200, 0.02), (1, 2, 1, 0.02),
                                      (1, 2, 1024, None)])
def test_kda_split_parity(B, H, T, h0, g_dtype):
    inp = O.make_inputs("kda", B, H, T, 128, 128, seed=T + H, io_dtype=torch.bfloat16, h0_std=h0, g_dtype=g_dtype)
    o, hT = _run("kda", inp, None)           # AUTO: the split path is the default for this shape
    assert _lib.last_path() == "chunk_split_tcgen05"
    torch.cuda.synchronize()
    ro, rS = _truth("kda", inp)
    assert o.dtype == torch.float32 and hT.dtype == torch.float32   # kda_chunkwise returns float32 (kda.py:655)
    assert torch.isfinite(o).all() and torch.isfinite(hT).all()
    assert _rel(o, ro) <= BF16_TOL, f"output rel err {_rel(o, ro)}"
    assert _rel(hT, rS) <= BF16_TOL, f"state rel err {_rel(hT, rS)}"
    o2, hT2 = _run("kda", inp, "split")
    assert torch.equal(o, o2) and torch.equal(hT, hT2)
    o3, hT3 = _run("kda", inp, "fp32")
    assert _lib.last_path() == "chunk_fp32"
    assert _rel(o, o3) <= BF16_TOL and _rel(hT, hT3) <= BF16_TOL


@pytest.mark.parametrize("decay", [-2.0, -3.0, -8.0, -40.0])
def test_kda_split_strong_decay(decay):
    """Strong log decay per token and channel: e^{-G} over a chunk would overflow fp32.  Off-diagonal
    sub-blocks keep every exponent <= 0; a diagonal sub-block whose decay range passes 2^64 in some
    channel (here: -3 and below) is recomputed exactly, the others use the product form."""
    inp = O.make_inputs("kda", 1, 2, 192, 128, 128, seed=5, io_dtype=torch.bfloat16, h0_std=0.02)
    inp["g"] = torch.full_like(inp["g"], decay)
    inp["g"][:, :, ::7] = -0.01
    inp["g"][:, :, 64:96, :64] = -0.05   # one sub-block pair mild in half of the channels
    o, hT = _run("kda", inp, "split")
    torch.cuda.synchronize()
    ro, rS = _truth("kda", inp)
    assert torch.isfinite(o).all() and torch.isfinite(hT).all()
    assert _rel(o, ro) <= BF16_TOL and _rel(hT, rS) <= BF16_TOL


def test_kda_split_bf16_output_and_bthd():
    inp = O.make_inputs("kda", 2, 3, 130, 128, 128, seed=9, io_dtype=torch.bfloat16, h0_std=0.02)
    ro, rS = _truth("kda", inp)
    o, hT = _run("kda", inp, "split", out_dtype=torch.bfloat16)
    assert o.dtype == torch.bfloat16
    assert _rel(o, ro) <= BF16_TOL and _rel(hT, rS) <= BF16_TOL
    # [B,T,H,D] storage viewed as [B,H,T,D]: served without a copy
    cu = {k: (None if v is None else v.cuda()) for k, v in inp.items()}
    tr = lambda x: x.transpose(1, 2).contiguous().transpose(1, 2)
    o2, hT2 = L.kda_chunkwise(tr(cu["q"]), tr(cu["k"]), tr(cu["v"]), tr(cu["g"]), tr(cu["beta"]),
                              initial_state=cu["h0"], chunk_size=64, path="split")
    assert _lib.last_path() == "chunk_split_tcgen05"
    assert _rel(o2, ro) <= BF16_TOL and _rel(hT2, rS) <= BF16_TOL


@pytest.mark.parametrize("variant", ["gated", "delta"])
def test_split_serves_scalar_and_no_decay(variant):
    inp = O.make_inputs(variant, 1, 2, 200, 128, 128, seed=3, io_dtype=torch.bfloat16, h0_std=0.02)
    o, hT = _run(variant, inp, "split")
    assert _lib.last_path() == "chunk_split_tcgen05"
    ro, rS = _truth(variant, inp)
    assert _rel(o, ro) <= BF16_TOL and _rel(hT, rS) <= BF16_TOL
    o1, hT1 = _run(variant, inp, "tcgen05")
    assert _rel(o, o1) <= BF16_TOL and _rel(hT, hT1) <= BF16_TOL


def test_split_without_workspace_is_refused():
    """No silent downgrade: the two-kernel path without its workspace is DR_ERR_WORKSPACE, by name or by AUTO."""
    import ctypes
    from linearnexus_b200 import ops
    inp = O.make_inputs("kda", 1, 1, 64, 128, 128, seed=1, io_dtype=torch.bfloat16)
    cu = {k: (None if v is None else v.cuda()) for k, v in inp.items()}
    lib = _lib.load()
    o = torch.empty(1, 1, 64, 128, device="cuda")
    hT = torch.empty(1, 1, 128, 128, device="cuda")
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for path, want in ((None, -5), ("split", -5), ("fp32", 0)):
        d = ops._desc(_lib.DR_KDA, _lib.DR_LAYOUT_BHTD, 1, 1, 64, 128, 128, 64, cu["q"], cu["g"], torch.float32, True,
                      128 ** -0.5, path)
        st = lib.dr_chunk_fwd(ctypes.byref(d), vp(cu["q"]), vp(cu["k"]), vp(cu["v"]), vp(cu["g"]), vp(cu["beta"]),
                              None, vp(o), vp(hT), None, 0, None, stream)
        assert st == want
    assert _lib.last_path() == "chunk_fp32"
    torch.cuda.synchronize()
