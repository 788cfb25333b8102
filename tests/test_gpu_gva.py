"""Grouped value attention: q and k with fewer heads than v.  The kernels index q/k head h // (H // Hq) instead of
reading copies made by a repeat (gated_deltanet.py:798-801, kda.py:917-922): results must equal the op on the
repeated tensors bit for bit, on every forward path."""
import pytest
import torch

import linearnexus_b200 as L
from linearnexus_b200 import _lib
from oracle import delta_rule_oracle as O

pytestmark = pytest.mark.gpu


def _inputs(variant, B, Hq, H, T, K, V, dtype, seed=5):
    inp = O.make_inputs(variant, B, H, T, K, V, seed=seed, io_dtype=dtype, h0_std=0.02)
    cu = {k: (None if v is None else v.cuda()) for k, v in inp.items()}
    q, k = cu["q"][:, :Hq].contiguous(), cu["k"][:, :Hq].contiguous()
    rep = H // Hq
    return cu, q, k, q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)


@pytest.mark.parametrize("variant,path,dtype,K", [
    ("gated", "tcgen05", torch.bfloat16, 128), ("delta", "tcgen05", torch.bfloat16, 128),
    ("gated", "split", torch.bfloat16, 128), ("kda", None, torch.bfloat16, 128),
    ("gated", "fp32", torch.float32, 64), ("kda", "fp32", torch.float32, 32), ("delta", "fp32", torch.float32, 64)])
def test_chunk_forward_grouped_heads(variant, path, dtype, K):
    B, Hq, H, T = 2, 2, 6, 200
    cu, q, k, qr, kr = _inputs(variant, B, Hq, H, T, K, K, dtype)
    def run(qq, kk):
        if variant == "delta":
            return L.delta_rule_chunkwise(qq, kk, cu["v"], cu["beta"], cu["h0"], chunk_size=64, path=path)
        if variant == "gated":
            return L.gated_delta_rule_chunkwise(qq, kk, cu["v"], cu["g"], cu["beta"], initial_state=cu["h0"], path=path)
        return L.kda_chunkwise(qq, kk, cu["v"], cu["g"], cu["beta"], initial_state=cu["h0"], path=path)
    o, hT = run(q, k)
    used = _lib.last_path()
    o2, hT2 = run(qr, kr)
    assert _lib.last_path() == used
    assert o.shape == (B, H, T, K) and hT.shape == (B, H, K, K)
    assert torch.equal(o, o2) and torch.equal(hT, hT2)


@pytest.mark.parametrize("variant", ["delta", "gated", "kda"])
def test_recurrent_and_step_grouped_heads(variant):
    B, Hq, H, T, K, V = 2, 2, 4, 12, 64, 64
    cu, q, k, qr, kr = _inputs(variant, B, Hq, H, T, K, V, torch.float32)
    if variant == "delta":
        a = L.delta_rule_recurrent(q, k, cu["v"], cu["beta"], cu["h0"])
        b = L.delta_rule_recurrent(qr, kr, cu["v"], cu["beta"], cu["h0"])
    elif variant == "gated":
        a = L.gated_delta_rule_recurrent(q, k, cu["v"], cu["g"], cu["beta"], initial_state=cu["h0"])
        b = L.gated_delta_rule_recurrent(qr, kr, cu["v"], cu["g"], cu["beta"], initial_state=cu["h0"])
    else:
        a = L.kda_recurrent(q, k, cu["v"], cu["g"], cu["beta"], initial_state=cu["h0"])
        b = L.kda_recurrent(qr, kr, cu["v"], cu["g"], cu["beta"], initial_state=cu["h0"])
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    sl = lambda x: None if x is None else x[:, :, 0]
    if variant == "delta":
        a = L.delta_rule_step(sl(q), sl(k), sl(cu["v"]), sl(cu["beta"]), cu["h0"])
        b = L.delta_rule_step(sl(qr), sl(kr), sl(cu["v"]), sl(cu["beta"]), cu["h0"])
    elif variant == "gated":
        a = L.gated_delta_rule_step(sl(q), sl(k), sl(cu["v"]), sl(cu["g"]), sl(cu["beta"]), cu["h0"])
        b = L.gated_delta_rule_step(sl(qr), sl(kr), sl(cu["v"]), sl(cu["g"]), sl(cu["beta"]), cu["h0"])
    else:
        a = L.kda_step(sl(q), sl(k), sl(cu["v"]), sl(cu["g"]), sl(cu["beta"]), cu["h0"])
        b = L.kda_step(sl(qr), sl(kr), sl(cu["v"]), sl(cu["g"]), sl(cu["beta"]), cu["h0"])
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def test_streamed_decode_grouped_heads():
    B, Hq, H, K, V = 40, 2, 8, 128, 128
    cu, q, k, qr, kr = _inputs("gated", B, Hq, H, 1, K, V, torch.bfloat16)
    sl = lambda x: x[:, :, 0]
    a = L.gated_delta_rule_step(sl(q), sl(k), sl(cu["v"]), sl(cu["g"]), sl(cu["beta"]), cu["h0"])
    assert _lib.last_path() == "step_stream"
    b = L.gated_delta_rule_step(sl(qr), sl(kr), sl(cu["v"]), sl(cu["g"]), sl(cu["beta"]), cu["h0"])
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def test_grouped_heads_rejected_where_unsupported():
    cu, q, k, qr, kr = _inputs("gated", 1, 1, 2, 64, 128, 128, torch.bfloat16)
    with pytest.raises(ValueError):
        L.gated_delta_rule_chunkwise(torch.cat([q, q, q], 1), torch.cat([k, k, k], 1), cu["v"], cu["g"], cu["beta"])  # 2 % 3


@pytest.mark.parametrize("variant,dtype,K", [
    ("gated", torch.bfloat16, 128), ("delta", torch.bfloat16, 128), ("kda", torch.bfloat16, 128),
    ("gated", torch.float32, 64), ("kda", torch.float32, 32), ("delta", torch.float32, 64)])
@pytest.mark.parametrize("saving", [False, True])
def test_chunk_backward_grouped_heads(variant, dtype, K, saving):
    """dq, dk of a shared q/k head are the sums over its group of the gradients the op gives on repeated
    tensors; dv, dbeta, dg, dh0 (per value head) are those gradients themselves."""
    B, Hq, H, T = 2, 2, 6, 200
    rep = H // Hq
    cu, q, k, qr, kr = _inputs(variant, B, Hq, H, T, K, K, dtype)
    gen = torch.Generator().manual_seed(11)
    d_o = (torch.randn(B, H, T, K, generator=gen) * 0.1).to(dtype).cuda()
    d_hT = (torch.randn(B, H, K, K, generator=gen) * 0.1).cuda()
    g = cu["g"]

    def run(qq, kk):
        saved = None
        if saving:
            *_, saved = L.ops.chunk_forward_saving(variant, qq, kk, cu["v"], g, cu["beta"], cu["h0"])
        return L.ops.chunk_backward(variant, qq, kk, cu["v"], g, cu["beta"], d_o, cu["h0"], d_hT, saved=saved)
    a, b = run(q, k), run(qr, kr)
    assert a["dq"].shape == q.shape and a["dk"].shape == k.shape
    # bf16 results are rounded per head before the reference sum and after it in the grouped call
    tol = 1e-5 if dtype == torch.float32 else 1.5e-2
    for name in ("dq", "dk"):
        ref = b[name].float().view(B, Hq, rep, T, K).sum(2)
        err = (a[name].float() - ref).abs().max() / ref.abs().max()
        assert err <= tol, (name, float(err))
    for name in ("dv", "dbeta", "dg", "dh0"):
        if a[name] is None:
            assert b[name] is None
            continue
        ref = b[name].float()
        err = (a[name].float() - ref).abs().max() / ref.abs().max().clamp_min(1e-30)
        assert err <= 1e-5, (name, float(err))


def test_autograd_grouped_heads():
    """loss.backward() through the op with Hq < H: one saving forward, gradients of the shape of q and k."""
    B, Hq, H, T, K = 1, 2, 4, 192, 128
    cu, q, k, qr, kr = _inputs("gated", B, Hq, H, T, K, K, torch.bfloat16)
    q.requires_grad_(True); k.requires_grad_(True)
    v = cu["v"].clone().requires_grad_(True)
    o, hT = L.gated_delta_rule_chunkwise(q, k, v, cu["g"], cu["beta"], initial_state=cu["h0"])
    (o.float().square().mean() + hT.square().mean()).backward()
    assert q.grad.shape == q.shape and k.grad.shape == k.shape and v.grad.shape == v.shape
    assert torch.isfinite(q.grad.float()).all() and q.grad.float().abs().max() > 0
