"""GPU tests of the tcgen05/TMEM path: the descriptor plumbing against a plain matmul, then the
tensor-core chunk kernel against the float64 oracle and against the fp32 CUDA-core kernel."""
import ctypes

import pytest
import torch

import linearnexus_b200 as L
from linearnexus_b200 import _lib
from oracle import delta_rule_oracle as O

pytestmark = pytest.mark.gpu
BF16_TOL = 2e-2


def _rel(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return ((a - b).abs().max() / b.abs().max().clamp_min(1e-30)).item()


@pytest.mark.parametrize("a_tmem", [0, 1, 2, 5, 6, 8])
@pytest.mark.parametrize("b_mn", [0, 1])
@pytest.mark.parametrize("kd,n", [(128, 64), (128, 128), (64, 64), (64, 128)])
def test_umma_plumbing(a_tmem, b_mn, kd, n):
    g = torch.Generator(device="cpu").manual_seed(kd + n + 2 * a_tmem + b_mn)
    # a_tmem: 0 A in smem K-major, 1 A in TMEM, 2 A in smem MN-major; +4 sets the negate-A flag;
    # +8 runs M = 64 (only the first 64 rows of A and D are meaningful)
    A = torch.randn(128, kd, generator=g).bfloat16().cuda()
    B = torch.randn(n, kd, generator=g).bfloat16().cuda()
    Bsrc = B.t().contiguous() if b_mn else B
    Asrc = A.t().contiguous() if (a_tmem & 3) == 2 else A
    D = torch.full((128, n), float("nan"), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    st = _lib.load().dr_debug_umma_selftest(vp(Asrc), vp(Bsrc), vp(D), kd, n, a_tmem, b_mn, vp(status),
                                            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(st, "dr_debug_umma_selftest")
    torch.cuda.synchronize()
    assert status.item() == 0, "a bounded mbarrier wait ran out"
    ref = A.float() @ B.float().t() * (-1.0 if a_tmem & 4 else 1.0)
    rows = 64 if a_tmem & 8 else 128
    assert (D[:rows] - ref[:rows]).abs().max().item() <= 1e-3 * max(1.0, ref.abs().max().item())


def _truth(variant, inp):
    d = lambda x: None if x is None else x.double()
    q, k, v, g, beta, h0 = (d(inp[x]) for x in ("q", "k", "v", "g", "beta", "h0"))
    if variant == "delta":
        return O.delta_rule_recurrent(q, k, v, beta, h0, compute_dtype=torch.float64)
    return O.gated_delta_rule_recurrent(q, k, v, g, beta, initial_state=h0, compute_dtype=torch.float64)


def _run(variant, inp, path):
    cu = {k: (None if v is None else v.cuda()) for k, v in inp.items()}
    if variant == "delta":
        out = L.delta_rule_chunkwise(cu["q"], cu["k"], cu["v"], cu["beta"], cu["h0"], chunk_size=64, path=path)
    else:
        out = L.gated_delta_rule_chunkwise(cu["q"], cu["k"], cu["v"], cu["g"], cu["beta"], initial_state=cu["h0"],
                                           chunk_size=64, path=path)
    assert _lib.last_path() == ("chunk_tcgen05" if path == "tcgen05" else "chunk_fp32")
    return out


@pytest.mark.parametrize("variant", ["gated", "delta"])
@pytest.mark.parametrize("B,H,T,h0", [(1, 1, 64, None), (1, 2, 128, 0.02), (2, 3, 200, 0.02), (1, 2, 1, 0.02), (1, 4, 1024, None)])
def test_tcgen05_chunk_parity(variant, B, H, T, h0):
    inp = O.make_inputs(variant, B, H, T, 128, 128, seed=T + H, io_dtype=torch.bfloat16, h0_std=h0)
    inp["q"] = (inp["q"].float() * 1.5).bfloat16()
    o, hT = _run(variant, inp, "tcgen05")
    torch.cuda.synchronize()
    ro, rS = _truth(variant, inp)
    assert o.dtype == torch.bfloat16 and hT.dtype == torch.float32
    assert torch.isfinite(o.float()).all() and torch.isfinite(hT).all()
    assert _rel(o, ro) <= BF16_TOL, f"output rel err {_rel(o, ro)}"
    assert _rel(hT, rS) <= BF16_TOL, f"state rel err {_rel(hT, rS)}"
    o2, hT2 = _run(variant, inp, "tcgen05")
    assert torch.equal(o, o2) and torch.equal(hT, hT2)
    o3, hT3 = _run(variant, inp, "fp32")
    assert _rel(o, o3) <= BF16_TOL and _rel(hT, hT3) <= BF16_TOL


def test_tcgen05_is_default_for_headline_shape():
    inp = O.make_inputs("gated", 1, 1, 64, 128, 128, seed=1, io_dtype=torch.bfloat16)
    cu = {k: (None if v is None else v.cuda()) for k, v in inp.items()}
    L.gated_delta_rule_chunkwise(cu["q"], cu["k"], cu["v"], cu["g"], cu["beta"])
    assert _lib.last_path() == "chunk_tcgen05"
    L.gated_delta_rule_chunkwise(cu["q"].float(), cu["k"].float(), cu["v"].float(), cu["g"], cu["beta"])
    assert _lib.last_path() == "recurrent"   # no tensor-core kernel for fp32 storage: the token recurrence
    L.gated_delta_rule_chunkwise(cu["q"].float(), cu["k"].float(), cu["v"].float(), cu["g"], cu["beta"], path="fp32")
    assert _lib.last_path() == "chunk_fp32"


@pytest.mark.parametrize("variant", ["gated", "delta"])
@pytest.mark.parametrize("T", [100, 320])
def test_tcgen05_without_tma_inputs(variant, T):
    """Inputs the tensor maps cannot describe -- [B,T,H,D] storage (rows of a sequence not contiguous) or a
    length that is not a multiple of 8 -- take the per-thread copy path of the same kernel: same results."""
    inp = O.make_inputs(variant, 2, 3, T, 128, 128, seed=T, io_dtype=torch.bfloat16, h0_std=0.02)
    o, hT = _run(variant, inp, "tcgen05")
    ro, rS = _truth(variant, inp)
    assert _rel(o, ro) <= BF16_TOL and _rel(hT, rS) <= BF16_TOL
    cu = {k: (None if v is None else v.cuda()) for k, v in inp.items()}
    tr = lambda x: None if x is None else x.transpose(1, 2).contiguous().transpose(1, 2)
    if variant == "delta":
        o2, hT2 = L.delta_rule_chunkwise(tr(cu["q"]), tr(cu["k"]), tr(cu["v"]), tr(cu["beta"]), cu["h0"], chunk_size=64,
                                         path="tcgen05")
    else:
        o2, hT2 = L.gated_delta_rule_chunkwise(tr(cu["q"]), tr(cu["k"]), tr(cu["v"]), tr(cu["g"]), tr(cu["beta"]),
                                               initial_state=cu["h0"], chunk_size=64, path="tcgen05")
    assert _lib.last_path() == "chunk_tcgen05"
    assert o2.transpose(1, 2).is_contiguous()
    # the two load paths feed identical tiles to identical products
    if T % 8 == 0:
        assert _rel(o2, ro) <= BF16_TOL and _rel(hT2, rS) <= BF16_TOL
    else:
        assert torch.equal(o2, o) and torch.equal(hT2, hT)
