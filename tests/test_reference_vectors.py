"""The oracle against the reference's own code.

``tests/golden/reference_vectors.npz`` holds inputs and outputs of the reference's functions themselves
(its source files executed over a numpy stand-in for ``jax.numpy``; see
``tests/golden/make_reference_vectors.py``).  Both sides compute in float32, so the bound is float32
round-off of sums in a different order: max|x - ref| <= 2e-5 * max(1, max|ref|).  The float64 oracle, which
the kernel tests use as truth, has to sit within the same bound of the reference's float32 result.
"""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import block_ops_oracle as BO
from oracle import delta_rule_oracle as O
from oracle import linear_recurrences_oracle as R

VEC = np.load(Path(__file__).parent / "golden" / "reference_vectors.npz")
TOL = 2e-5


def T(case, key):
    name = f"{case}.{key}"
    return torch.from_numpy(VEC[name]) if name in VEC.files else None


def close(got, ref, tol=TOL):
    got, ref = got.double(), ref.double()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    err = (got - ref).abs().max().item()
    assert err <= tol * max(1.0, ref.abs().max().item()), err


DELTA_CASES = ["delta", "gated", "kda", "gated128", "kda128"]


def _variant(case):
    return case.replace("128", "")


def _run(case, form, cd):
    v = _variant(case)
    q, k, val, g, beta, h0 = (T(case, x) for x in ("q", "k", "v", "g", "beta", "h0"))
    C = int(VEC[f"{case}.chunk"])
    if form == "step":
        cut = lambda t: None if t is None else t[:, :, 0]
        if v == "delta":
            return O.delta_rule_step(cut(q), cut(k), cut(val), cut(beta), h0, compute_dtype=cd)
        fn = O.gated_delta_rule_step if v == "gated" else O.kda_step
        return fn(cut(q), cut(k), cut(val), cut(g), cut(beta), h0, compute_dtype=cd)
    if v == "delta":
        if form == "recurrent":
            return O.delta_rule_recurrent(q, k, val, beta, initial_state=h0, compute_dtype=cd)
        return O.delta_rule_chunkwise(q, k, val, beta, initial_state=h0, chunk_size=C, compute_dtype=cd)
    if form == "recurrent":
        fn = O.gated_delta_rule_recurrent if v == "gated" else O.kda_recurrent
        return fn(q, k, val, g, beta, initial_state=h0, compute_dtype=cd)
    fn = O.gated_delta_rule_chunkwise if v == "gated" else O.kda_chunkwise
    return fn(q, k, val, g, beta, initial_state=h0, chunk_size=C, compute_dtype=cd)


@pytest.mark.parametrize("case", DELTA_CASES)
@pytest.mark.parametrize("form", ["recurrent", "chunk", "step"])
@pytest.mark.parametrize("cd", [torch.float32, torch.float64])
def test_delta_rule_oracle_matches_reference_source(case, form, cd):
    o, s = _run(case, form, cd)
    close(o, T(case, f"o_{form}"))
    close(s, T(case, f"hT_{form}"))


def test_reference_output_dtypes_and_shapes():
    # every function of the reference returned float32 for float32 inputs, the state as [B,H,K,V]
    for case in DELTA_CASES:
        B, H, Tn, K = VEC[f"{case}.q"].shape
        V = VEC[f"{case}.v"].shape[-1]
        for form in ("recurrent", "chunk"):
            assert VEC[f"{case}.o_{form}"].shape == (B, H, Tn, V) and VEC[f"{case}.o_{form}"].dtype == np.float32
            assert VEC[f"{case}.hT_{form}"].shape == (B, H, K, V)
        assert VEC[f"{case}.o_step"].shape == (B, H, V)


@pytest.mark.parametrize("cd", [torch.float32, torch.float64])
def test_dplr_oracle_matches_reference_source(cd):
    q, k, v, a, b, gk, h0 = (T("dplr", x) for x in ("q", "k", "v", "a", "b", "gk", "h0"))
    sc = float(VEC["dplr.scale"])
    o, s = R.dplr_delta_rule_recurrent(q, k, v, a, b, gk, scale=sc, initial_state=h0, compute_dtype=cd)
    close(o, T("dplr", "o")), close(s, T("dplr", "hT"))
    c = lambda t: t[:, :, 0]
    o1, s1 = R.dplr_delta_rule_step(c(q), c(k), c(v), c(a), c(b), c(gk), h0, scale=sc, compute_dtype=cd)
    close(o1, T("dplr", "o_step")), close(s1, T("dplr", "hT_step"))


@pytest.mark.parametrize("cd", [torch.float32, torch.float64])
def test_rwkv6_oracle_matches_reference_source(cd):
    r, k, v, w, u, h0 = (T("rwkv6", x) for x in ("r", "k", "v", "w", "u", "h0"))
    sc = float(VEC["rwkv6.scale"])
    o, s = R.rwkv6_recurrent(r, k, v, w, u, scale=sc, initial_state=h0, compute_dtype=cd)
    close(o, T("rwkv6", "o")), close(s, T("rwkv6", "hT"))
    c = lambda t: t[:, :, 0]
    o1, s1 = R.rwkv6_step(c(r), c(k), c(v), c(w), u, h0, scale=sc, compute_dtype=cd)
    close(o1, T("rwkv6", "o_step")), close(s1, T("rwkv6", "hT_step"))


@pytest.mark.parametrize("cd", [torch.float32, torch.float64])
def test_ssd_oracle_matches_reference_source(cd):
    x, dt, A, Bm, Cm, D, bias, h0 = (T("ssd", n) for n in ("x", "dt", "A", "B", "C", "D", "dt_bias", "h0"))
    lim = tuple(float(t) for t in VEC["ssd.dt_limit"])
    kw = dict(n_groups=int(VEC["ssd.groups"]), dt_bias=bias, dt_limit=lim, compute_dtype=cd)
    y, s = R.ssd_chunk_scan(x, dt, A, Bm, Cm, D, chunk_size=int(VEC["ssd.chunk"]), ssm_state=h0, **kw)
    close(y, T("ssd", "y")), close(s, T("ssd", "hT"))
    # the token recurrence is the same function of the inputs as the chunked scan
    y2, s2 = R.ssd_token_recurrence(x, dt, A, Bm, Cm, D, ssm_state=h0, **kw)
    close(y2, T("ssd", "y")), close(s2, T("ssd", "hT"))
    y1, s1 = R.ssd_recurrent_step(x[:, 0], dt[:, 0], A, Bm[:, 0], Cm[:, 0], D, h0, **kw)
    close(y1, T("ssd", "y_step")), close(s1, T("ssd", "hT_step"))


def test_kda_gate_oracle_matches_reference_source():
    g, b = BO.kda_gate(T("kda_gate", "g_in"), T("kda_gate", "A_log"), 8, g_bias=T("kda_gate", "g_bias"),
                       beta=T("kda_gate", "beta_in"))
    close(g, T("kda_gate", "g_out")), close(b, T("kda_gate", "beta_out"))


def test_padding_helpers_match_reference_source():
    from linearnexus_b200 import varlen
    mask = T("padding", "mask")
    idx, cu = varlen.compute_unpadded_indices(mask)
    assert idx.tolist() == VEC["padding.indices"].tolist() and cu.tolist() == VEC["padding.cu_seqlens"].tolist()
    x = T("padding", "x")
    flat = varlen.unpad(x, idx)
    assert torch.equal(flat, T("padding", "flat"))
    assert torch.equal(varlen.pad(flat, idx, 3, 5), T("padding", "back"))


def test_conv_oracle_matches_reference_source():
    x, w, b, cache = (T("conv", n) for n in ("x", "weight", "bias", "cache"))
    y, c = BO.short_conv_silu(x, w, b, apply_silu=False)
    close(y, T("conv", "y_cold")), close(c, T("conv", "cache_cold"))
    y, c = BO.short_conv_silu(x, w, None, cache=cache, apply_silu=False)
    close(y, T("conv", "y_warm")), close(c, T("conv", "cache_warm"))


def test_norm_oracle_matches_reference_source():
    o, gate, w = T("norm", "o"), T("norm", "gate"), T("norm", "weight")
    close(BO.gated_rmsnorm(o, w, None, eps=1e-6), T("norm", "rmsnorm_eps1e-6"))
    close(BO.gated_rmsnorm(o, w, gate, eps=1e-5), T("norm", "fused_eps1e-5"))


@pytest.mark.parametrize("case", ["delta", "gated", "kda"])
def test_oracle_gradients_match_derivatives_of_reference_source(case):
    """The fixtures hold d/de L(x + e * dir) of L = sum(o * do) + sum(hT * dhT) for the reference's chunk form, by
    central differences of its own source run in float64.  <grad, dir> of the oracle's backward has to give the same
    number for every input (1e-6 relative to the size of the terms summed)."""
    names = [n for n in ("q", "k", "v", "g", "beta", "h0") if f"{case}.{n}" in VEC.files]
    gr = O.delta_rule_grads(case, T(case, "q"), T(case, "k"), T(case, "v"), T(case, "g"), T(case, "beta"), T(case, "h0"),
                            T(case, "do"), T(case, "dhT"), use_qk_l2norm=(case != "delta"))
    for n in names:
        grad = gr["d" + n].double()
        d = T(case, "dir_" + n).double()
        want = float(VEC[f"{case}.dL_{n}"])
        size = (grad * d).abs().sum().item()
        assert abs((grad * d).sum().item() - want) <= 1e-6 * max(size, 1.0), (n, (grad * d).sum().item(), want)


# ---- the CUDA kernels against the same vectors ------------------------------------------------------------------

def _cuda(t):
    return None if t is None else t.cuda()


@pytest.mark.gpu
@pytest.mark.parametrize("case", DELTA_CASES)
def test_cuda_chunk_and_recurrent_match_reference_source(case):
    """float32 storage through the fp32 kernels: 1e-4 (tf32-free, fp32 accumulation in a different order)."""
    import linearnexus_b200 as L
    v = _variant(case)
    q, k, val, g, beta, h0 = (_cuda(T(case, x)) for x in ("q", "k", "v", "g", "beta", "h0"))
    C = int(VEC[f"{case}.chunk"])
    if v == "delta":
        o, s = L.delta_rule_chunkwise(q, k, val, beta, initial_state=h0, chunk_size=C)
        o2, s2 = L.delta_rule_recurrent(q, k, val, beta, initial_state=h0)
        o1, s1 = L.delta_rule_step(q[:, :, 0], k[:, :, 0], val[:, :, 0], beta[:, :, 0], h0)
    elif v == "gated":
        o, s = L.gated_delta_rule_chunkwise(q, k, val, g, beta, initial_state=h0, chunk_size=C)
        o2, s2 = L.gated_delta_rule_recurrent(q, k, val, g, beta, initial_state=h0)
        o1, s1 = L.gated_delta_rule_step(q[:, :, 0], k[:, :, 0], val[:, :, 0], g[:, :, 0], beta[:, :, 0], h0)
    else:
        o, s = L.kda_chunkwise(q, k, val, g, beta, initial_state=h0, chunk_size=C)
        o2, s2 = L.kda_recurrent(q, k, val, g, beta, initial_state=h0)
        o1, s1 = L.kda_step(q[:, :, 0], k[:, :, 0], val[:, :, 0], g[:, :, 0], beta[:, :, 0], h0)
    tol = 1e-4
    close(o.cpu(), T(case, "o_chunk"), tol), close(s.cpu(), T(case, "hT_chunk"), tol)
    close(o2.cpu(), T(case, "o_recurrent"), tol), close(s2.cpu(), T(case, "hT_recurrent"), tol)
    close(o1.cpu(), T(case, "o_step"), tol), close(s1.cpu(), T(case, "hT_step"), tol)


@pytest.mark.gpu
@pytest.mark.parametrize("case", ["gated128", "kda128"])
def test_cuda_tensor_core_kernels_match_reference_source(case):
    """The inputs of these cases are exactly representable in bf16, so the bf16 tensors the tcgen05 kernels read
    hold the very numbers the reference's code saw; the bound is the bf16 budget of the configuration
    (max|x - ref| <= 2e-2 max|ref|) on outputs and final state."""
    import linearnexus_b200 as L
    from linearnexus_b200 import _lib, ops
    v = _variant(case)
    q, k, val = (_cuda(T(case, x)).bfloat16() for x in ("q", "k", "v"))
    assert torch.equal(q.float().cpu(), T(case, "q"))
    g, beta, h0 = (_cuda(T(case, x)) for x in ("g", "beta", "h0"))
    if v == "gated":
        o, s = L.gated_delta_rule_chunkwise(q, k, val, g, beta, initial_state=h0, chunk_size=64)
        assert _lib.last_path() == "chunk_tcgen05"
    else:
        o, s = L.kda_chunkwise(q, k, val, g, beta, initial_state=h0, chunk_size=64)
        assert _lib.last_path() == "chunk_split_tcgen05"
    ops.check_device_status()
    ro, rs = T(case, "o_chunk").double(), T(case, "hT_chunk").double()
    assert ((o.double().cpu() - ro).abs().max() / ro.abs().max()).item() <= 2e-2
    assert ((s.double().cpu() - rs).abs().max() / rs.abs().max()).item() <= 2e-2


@pytest.mark.gpu
@pytest.mark.parametrize("case", ["delta", "gated", "kda"])
def test_cuda_backward_matches_derivatives_of_reference_source(case):
    """loss.backward() through the CUDA chunk forward + backward, float32 storage: <grad, dir> against the central
    differences of the reference's own source (1e-3 of the size of the terms summed: the backward kernels use tf32
    tensor-core products)."""
    import linearnexus_b200 as L
    names = [n for n in ("q", "k", "v", "g", "beta", "h0") if f"{case}.{n}" in VEC.files]
    x = {n: T(case, n).cuda().requires_grad_(True) for n in names}
    C = int(VEC[f"{case}.chunk"])
    if case == "delta":
        o, s = L.delta_rule_chunkwise(x["q"], x["k"], x["v"], x["beta"], initial_state=x["h0"], chunk_size=C)
    elif case == "gated":
        o, s = L.gated_delta_rule_chunkwise(x["q"], x["k"], x["v"], x["g"], x["beta"], initial_state=x["h0"], chunk_size=C)
    else:
        o, s = L.kda_chunkwise(x["q"], x["k"], x["v"], x["g"], x["beta"], initial_state=x["h0"], chunk_size=C)
    ((o.float() * T(case, "do").cuda()).sum() + (s * T(case, "dhT").cuda()).sum()).backward()
    for n in names:
        grad, d = x[n].grad.double().cpu(), T(case, "dir_" + n).double()
        want = float(VEC[f"{case}.dL_{n}"])
        size = (grad * d).abs().sum().item()
        assert abs((grad * d).sum().item() - want) <= 1e-3 * max(size, 1.0), (n, (grad * d).sum().item(), want)
