"""GPU parity of the backward (dq, dk, dv, dbeta, dg, dh0) against autograd of the float64 oracle,
which is what jax.grad of the reference functions computes."""
import pytest
import torch

import linearnexus_b200 as L
from linearnexus_b200 import ops
from oracle import delta_rule_oracle as O

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return ((a - b).abs().max() / b.abs().max().clamp_min(1e-30)).item()


def _check(variant, B, H, T, K, V, C, io=torch.float32, tol=2e-4, h0_std=0.1, with_dhT=True):
    inp = O.make_inputs(variant, B, H, T, K, V, seed=T + K + C, io_dtype=io, h0_std=h0_std)
    if io == torch.float32:
        inp["q"] = inp["q"] * 1.3
        inp["k"] = inp["k"] * 0.7
    gen = torch.Generator().manual_seed(5)
    do = torch.randn(B, H, T, V, generator=gen).to(io)
    dhT = torch.randn(B, H, K, V, generator=gen) * 0.1 if with_dhT else None
    l2 = variant != "delta"
    f = lambda x: None if x is None else x.float() if x.dtype == torch.bfloat16 else x
    ref = O.delta_rule_grads(variant, f(inp["q"]), f(inp["k"]), f(inp["v"]), inp["g"], inp["beta"], inp["h0"], f(do), dhT,
                             use_qk_l2norm=l2)
    cu = lambda x: None if x is None else x.cuda()
    got = ops.chunk_backward(variant, cu(inp["q"]), cu(inp["k"]), cu(inp["v"]), cu(inp["g"]), cu(inp["beta"]), cu(do),
                             initial_state=cu(inp["h0"]), d_final_state=cu(dhT), chunk_size=C, use_qk_l2norm=l2)
    torch.cuda.synchronize()
    for name in ("dq", "dk", "dv", "dbeta", "dg", "dh0"):
        if ref[name] is None:
            assert got[name] is None
            continue
        assert got[name].shape == ref[name].shape, name
        err = _rel(got[name], ref[name])
        assert err <= tol, f"{variant} {name}: rel err {err}"
    return got


@pytest.mark.parametrize("variant", ["delta", "gated", "kda"])
@pytest.mark.parametrize("shape", [(1, 2, 64, 32, 32, 64), (2, 2, 100, 16, 48, 32), (1, 1, 130, 64, 64, 64), (1, 2, 40, 128, 128, 16)])
def test_backward_fp32(variant, shape):
    _check(variant, *shape)


def test_backward_golden_fixture(golden):
    for name in ("delta", "gated", "kda"):
        G = lambda key: torch.from_numpy(golden[f"{name}.{key}"]).cuda() if f"{name}.{key}" in golden.files else None
        got = ops.chunk_backward(name, G("q"), G("k"), G("v"), G("g"), G("beta"), G("do"), initial_state=G("h0"),
                                 d_final_state=G("dhT"), chunk_size=int(golden[f"{name}.chunk"]), use_qk_l2norm=(name != "delta"))
        for key in ("dq", "dk", "dv", "dg", "dbeta", "dh0"):
            if G(key) is not None:
                assert _rel(got[key], G(key)) <= 2e-4, (name, key)


def test_backward_bf16_headline_head_size():
    """bf16 q,k,v,do with fp32 accumulation at d_k = d_v = 128, chunk 64 (the training configuration's head)."""
    got = _check("gated", 1, 2, 256, 128, 128, 64, io=torch.bfloat16, tol=2e-2, h0_std=0.02)
    assert got["dq"].dtype == torch.bfloat16 and got["dg"].dtype == torch.float32


def test_autograd_through_the_op():
    inp = O.make_inputs("gated", 1, 2, 96, 32, 32, seed=9, h0_std=0.1)
    leaf = {k_: (None if v_ is None else v_.cuda().requires_grad_(True)) for k_, v_ in inp.items()}
    o, hT = L.gated_delta_rule_chunkwise(leaf["q"], leaf["k"], leaf["v"], leaf["g"], leaf["beta"], initial_state=leaf["h0"],
                                         chunk_size=32)
    gen = torch.Generator().manual_seed(1)
    do = torch.randn(o.shape, generator=gen)
    dhT = torch.randn(hT.shape, generator=gen) * 0.1
    ((o * do.cuda()).sum() + (hT * dhT.cuda()).sum()).backward()
    ref = O.delta_rule_grads("gated", inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["h0"], do, dhT)
    for name, key in (("q", "dq"), ("k", "dk"), ("v", "dv"), ("g", "dg"), ("beta", "dbeta"), ("h0", "dh0")):
        assert _rel(leaf[name].grad, ref[key]) <= 2e-4, key


@pytest.mark.parametrize("variant,io,K,tol", [("gated", torch.bfloat16, 128, 2e-2), ("delta", torch.bfloat16, 128, 2e-2),
                                              ("kda", torch.bfloat16, 128, 2e-2), ("gated", torch.float32, 32, 2e-4),
                                              ("kda", torch.float32, 16, 2e-4)])
def test_saving_forward_then_saved_backward(variant, io, K, tol):
    """One forward per training step: chunk_forward_saving returns the forward's results plus the per-chunk states;
    chunk_backward(saved=...) must give the gradients of the recomputing backward (and of the float64 oracle)."""
    from linearnexus_b200 import _lib
    B, H, T, C = 1, 2, 200, 64 if K == 128 else 32
    inp = O.make_inputs(variant, B, H, T, K, K, seed=21, io_dtype=io, h0_std=0.02)
    gen = torch.Generator().manual_seed(6)
    do = torch.randn(B, H, T, K, generator=gen).to(io)
    l2 = variant != "delta"
    cu = {k_: (None if v_ is None else v_.cuda()) for k_, v_ in inp.items()}
    o, hT, saved = ops.chunk_forward_saving(variant, cu["q"], cu["k"], cu["v"], cu["g"], cu["beta"], cu["h0"],
                                            chunk_size=C, use_qk_l2norm=l2)
    assert _lib.last_path() == "fwd_saving"
    # same forward results as the plain op (same kernels for gated/delta; KDA's default op is the same two-kernel path)
    if variant == "delta":
        o2, hT2 = L.delta_rule_chunkwise(cu["q"], cu["k"], cu["v"], cu["beta"], cu["h0"], chunk_size=C)
    elif variant == "gated":
        o2, hT2 = L.gated_delta_rule_chunkwise(cu["q"], cu["k"], cu["v"], cu["g"], cu["beta"], initial_state=cu["h0"], chunk_size=C)
    else:
        o2, hT2 = L.kda_chunkwise(cu["q"], cu["k"], cu["v"], cu["g"], cu["beta"], initial_state=cu["h0"], chunk_size=C)
    assert o.dtype == o2.dtype and torch.equal(o, o2) and torch.equal(hT, hT2)
    got = ops.chunk_backward(variant, cu["q"], cu["k"], cu["v"], cu["g"], cu["beta"], do.cuda(), initial_state=cu["h0"],
                             chunk_size=C, use_qk_l2norm=l2, saved=saved)
    assert _lib.last_path() == "bwd_saved"
    again = ops.chunk_backward(variant, cu["q"], cu["k"], cu["v"], cu["g"], cu["beta"], do.cuda(), initial_state=cu["h0"],
                               chunk_size=C, use_qk_l2norm=l2)
    f = lambda x: None if x is None else x.float() if x.dtype == torch.bfloat16 else x
    ref = O.delta_rule_grads(variant, f(inp["q"]), f(inp["k"]), f(inp["v"]), inp["g"], inp["beta"], inp["h0"], f(do), None,
                             use_qk_l2norm=l2)
    for name in ("dq", "dk", "dv", "dbeta", "dg", "dh0"):
        if ref[name] is None:
            continue
        # same checkpoints, same adjoint (dbeta and dg are summed with atomics: equal up to summation order)
        if name in ("dbeta", "dg"):
            assert _rel(got[name], again[name]) <= 1e-5, name
        else:
            assert torch.equal(got[name], again[name]), name
        assert _rel(got[name], ref[name]) <= tol, (variant, name, _rel(got[name], ref[name]))


def test_autograd_uses_the_saved_states():
    from linearnexus_b200 import _lib
    inp = O.make_inputs("gated", 1, 2, 128, 128, 128, seed=4, io_dtype=torch.bfloat16)
    leaf = {k_: (None if v_ is None else v_.cuda().requires_grad_(v_.is_floating_point())) for k_, v_ in inp.items()}
    nf = _lib.launch_count()
    o, hT = L.gated_delta_rule_chunkwise(leaf["q"], leaf["k"], leaf["v"], leaf["g"], leaf["beta"])
    assert _lib.last_path() == "fwd_saving"
    # the forward that keeps the per-chunk states, with the adjoint's chunk-parallel pre-pass beside it
    assert _lib.launch_count() - nf == 2
    n0 = _lib.launch_count()
    (o.float().square().sum() + hT.sum()).backward()
    torch.cuda.synchronize()
    # adjoint + finalize only: no forward recomputation, no pre-pass (the path name is per host thread; autograd
    # runs elsewhere, so the launch counter is the witness)
    assert _lib.launch_count() - n0 == 2
    assert leaf["q"].grad is not None and torch.isfinite(leaf["q"].grad.float()).all()


@pytest.mark.parametrize("variant", ["gated", "delta"])
@pytest.mark.parametrize("K,V,T,Hq,H", [(16, 8, 70, 2, 2), (32, 40, 130, 1, 3), (48, 64, 64, 2, 4), (80, 24, 100, 1, 2),
                                        (96, 96, 65, 3, 3), (112, 16, 129, 1, 1), (128, 72, 257, 2, 4), (128, 128, 1, 1, 2)])
def test_tensor_core_backward_odd_shapes(variant, K, V, T, Hq, H):
    """bf16 inputs (tf32 tensor-core adjoint, 16 warps) against the exact fp32 path on the same values: channel
    counts that leave warps idle, value slices with a ragged last slice, ragged chunks, grouped q/k heads."""
    from linearnexus_b200 import ops
    gen = torch.Generator(device="cuda").manual_seed(K * 1000 + V)
    r = lambda *s: torch.randn(*s, device="cuda", generator=gen)
    B = 2
    q, k, v = r(B, Hq, T, K).bfloat16(), r(B, Hq, T, K).bfloat16(), r(B, H, T, V).bfloat16()
    beta = torch.sigmoid(r(B, H, T))
    g = torch.nn.functional.logsigmoid(r(B, H, T) + 3) if variant == "gated" else None
    d_o, d_hT, h0 = (r(B, H, T, V) * 0.1).bfloat16(), r(B, H, K, V) * 0.1, r(B, H, K, V) * 0.05
    a = ops.chunk_backward(variant, q, k, v, g, beta, d_o, h0, d_hT)
    b = ops.chunk_backward(variant, q.float(), k.float(), v.float(), g, beta, d_o.float(), h0, d_hT)
    for name in ("dq", "dk", "dv", "dbeta", "dg", "dh0"):
        if a[name] is None:
            continue
        x, y = a[name].float(), b[name].float()
        assert torch.isfinite(x).all(), name
        err = (x - y).abs().max() / y.abs().max().clamp_min(1e-20)
        assert err <= 2e-2, (name, float(err))   # the bf16 bar: max|x - ref| / max|ref|


def test_forward_of_grad_inputs_runs_for_shapes_the_backward_does_not_cover():
    """chunk_size 128 has a forward (token-recurrent kernel) but no backward: a call on requires_grad inputs still
    returns the forward result, and only .backward() reports the limit."""
    inp = O.make_inputs("gated", 1, 2, 256, 64, 64, seed=4)
    cu = {k: (None if v is None else v.cuda()) for k, v in inp.items()}
    q = cu["q"].clone().requires_grad_(True)
    o, hT = L.gated_delta_rule_chunkwise(q, cu["k"], cu["v"], cu["g"], cu["beta"], chunk_size=128)
    with torch.no_grad():
        o2, hT2 = L.gated_delta_rule_chunkwise(cu["q"], cu["k"], cu["v"], cu["g"], cu["beta"], chunk_size=128)
    assert torch.equal(o, o2) and torch.equal(hT, hT2)
    with pytest.raises(NotImplementedError, match="chunk_size <= 64"):
        o.sum().backward()
