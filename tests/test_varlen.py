"""Packed (variable-length) batches: the padding helpers against the behaviour of the reference's
core/padding.py (CPU), and the packed chunkwise op against the oracle run on each sequence alone (GPU)."""
import numpy as np
import pytest
import torch

import linearnexus_b200 as L
from linearnexus_b200 import _lib
from oracle import delta_rule_oracle as O


def test_padding_helpers_round_trip():
    mask = torch.tensor([[1, 1, 1, 0, 0], [1, 0, 0, 0, 0], [1, 1, 1, 1, 1]])
    idx, cu = L.compute_unpadded_indices(mask)
    assert idx.dtype == torch.int32 and cu.dtype == torch.int32
    assert idx.tolist() == [0, 1, 2, 5, 10, 11, 12, 13, 14] and cu.tolist() == [0, 3, 4, 9]
    x = torch.arange(3 * 5 * 2, dtype=torch.float32).reshape(3, 5, 2)
    packed = L.unpad(x, idx)
    assert packed.shape == (9, 2) and torch.equal(packed[3], x[1, 0])
    back = L.pad(packed, idx, 3, 5)
    assert torch.equal(back, x * mask[..., None])          # padded positions come back as zeros
    with pytest.raises(ValueError):
        L.compute_unpadded_indices(torch.ones(2, 3, 4))
    with pytest.raises(ValueError):
        L.pad(packed[:-1], idx, 3, 5)


def _packed(variant, lens, H, K, V, io, seed):
    seqs = [O.make_inputs(variant, 1, H, T, K, V, seed=seed + i, io_dtype=io, h0_std=0.05) for i, T in enumerate(lens)]
    cat = lambda name: None if seqs[0][name] is None else torch.cat([s[name][0].transpose(0, 1) for s in seqs], dim=0)
    packed = {name: cat(name) for name in ("q", "k", "v", "g", "beta")}     # [total_T, H, ...]
    packed["h0"] = torch.cat([s["h0"] for s in seqs], dim=0)                # [n, H, K, V]
    cu = np.concatenate([[0], np.cumsum(lens)]).tolist()
    return seqs, packed, cu


def _truth(variant, s):
    d = lambda x: None if s[x] is None else s[x].double()
    if variant == "delta":
        return O.delta_rule_recurrent(d("q"), d("k"), d("v"), d("beta"), d("h0"), compute_dtype=torch.float64)
    if variant == "gated":
        return O.gated_delta_rule_recurrent(d("q"), d("k"), d("v"), d("g"), d("beta"), initial_state=d("h0"), compute_dtype=torch.float64)
    return O.kda_recurrent(d("q"), d("k"), d("v"), d("g"), d("beta"), initial_state=d("h0"), compute_dtype=torch.float64)


@pytest.mark.gpu
@pytest.mark.parametrize("variant,io,K,tol", [("gated", torch.bfloat16, 128, 2e-2), ("kda", torch.bfloat16, 128, 2e-2),
                                              ("delta", torch.float32, 64, 1e-4), ("gated", torch.float32, 32, 1e-4)])
def test_packed_forward_equals_each_sequence_alone(variant, io, K, tol):
    lens = [200, 64, 1, 333, 72]     # ragged tails, a single token, multiples of 8 and not
    seqs, packed, cu = _packed(variant, lens, 2, K, K, io, seed=40)
    cu_t = {k: (None if v is None else v.cuda()) for k, v in packed.items()}
    o, hT = L.chunkwise_varlen(variant, cu_t["q"], cu_t["k"], cu_t["v"], cu_t["g"], cu_t["beta"], cu,
                               initial_state=cu_t["h0"])
    L.check_device_status()
    assert o.shape == (sum(lens), 2, K) and hT.shape == (len(lens), 2, K, K)
    for i, s in enumerate(seqs):
        ro, rS = _truth(variant, s)
        got = o[cu[i]:cu[i + 1]].transpose(0, 1)[None].double().cpu()
        if io == torch.float32:
            assert (got - ro).abs().max().item() <= tol and (hT[i:i + 1].double().cpu() - rS).abs().max().item() <= tol
        else:
            assert ((got - ro).abs().max() / ro.abs().max()).item() <= tol, i
            assert ((hT[i:i + 1].double().cpu() - rS).abs().max() / rS.abs().max()).item() <= tol, i


@pytest.mark.gpu
def test_packed_batch_is_differentiable():
    lens = [96, 40]
    seqs, packed, cu = _packed("gated", lens, 2, 64, 64, torch.float32, seed=50)
    t = {k: (None if v is None else v.cuda()) for k, v in packed.items()}
    q = t["q"].clone().requires_grad_(True)
    o, hT = L.chunkwise_varlen("gated", q, t["k"], t["v"], t["g"], t["beta"], cu, initial_state=t["h0"])
    gen = torch.Generator().manual_seed(1)
    d_o = torch.randn(o.shape, generator=gen)
    (o * d_o.cuda()).sum().backward()
    for i, s in enumerate(seqs):
        do_i = d_o[cu[i]:cu[i + 1]].transpose(0, 1)[None]
        ref = O.delta_rule_grads("gated", s["q"], s["k"], s["v"], s["g"], s["beta"], s["h0"], do_i)
        got = q.grad[cu[i]:cu[i + 1]].transpose(0, 1)[None].double().cpu()
        assert ((got - ref["dq"]).abs().max() / ref["dq"].abs().max()).item() <= 2e-4


def test_packed_entry_point_validates_offsets():
    lib = _lib.load()
    import ctypes
    d = _lib.DrDesc()
    d.variant, d.layout, d.B, d.H, d.T, d.K, d.V, d.chunk = 1, 1, 1, 1, 64, 64, 64, 64
    bad = (ctypes.c_int32 * 3)(0, 10, 10)      # an empty sequence
    assert lib.dr_chunk_fwd_varlen(ctypes.byref(d), 16, 16, 16, 16, 16, bad, 2, None, 16, None, None, 0, None, None) == -2
    d.layout = 0                               # packed batches are token-major
    ok = (ctypes.c_int32 * 2)(0, 10)
    assert lib.dr_chunk_fwd_varlen(ctypes.byref(d), 16, 16, 16, 16, 16, ok, 1, None, 16, None, None, 0, None, None) == -2


@pytest.mark.gpu
@pytest.mark.parametrize("variant,io,K,tol", [("gated", torch.bfloat16, 128, 2e-2), ("kda", torch.float32, 32, 2e-4),
                                              ("delta", torch.float32, 64, 2e-4)])
def test_packed_backward_equals_each_sequence_alone(variant, io, K, tol):
    """dr_chunk_bwd_varlen against the float64 oracle's gradients of every sequence taken alone."""
    lens = [130, 64, 1, 77]
    H = 2
    seqs, packed, cu = _packed(variant, lens, H, K, K, io, seed=60)
    t = {k: (None if v is None else v.cuda()) for k, v in packed.items()}
    gen = torch.Generator().manual_seed(2)
    d_o = torch.randn(sum(lens), H, K, generator=gen).to(io)
    d_hT = torch.randn(len(lens), H, K, K, generator=gen) * 0.1
    got = L.chunk_backward_varlen(variant, t["q"], t["k"], t["v"], t["g"], t["beta"], d_o.cuda(), cu,
                                  initial_state=t["h0"], d_final_state=d_hT.cuda())
    L.check_device_status()
    assert got["dq"].shape == t["q"].shape and got["dbeta"].shape == (sum(lens), H) and got["dh0"].shape == (len(lens), H, K, K)
    f = lambda x: None if x is None else (x.float() if x.dtype == torch.bfloat16 else x)
    rel = lambda a, b: ((a.double().cpu() - b.double()).abs().max() / b.double().abs().max().clamp_min(1e-30)).item()
    for i, s in enumerate(seqs):
        do_i = f(d_o[cu[i]:cu[i + 1]]).transpose(0, 1)[None]
        ref = O.delta_rule_grads(variant, f(s["q"]), f(s["k"]), f(s["v"]), s["g"], s["beta"], s["h0"], do_i, d_hT[i:i + 1],
                                 use_qk_l2norm=(variant != "delta"))
        sl = slice(cu[i], cu[i + 1])
        tok = lambda x: x[sl].transpose(0, 1)[None]       # packed [T_i, H, ...] -> [1, H, T_i, ...]
        if lens[i] > 1:   # a one-token sequence has gradients near zero in places: compared through the others' scale
            for name in ("dq", "dk", "dv"):
                assert rel(tok(got[name]), ref[name]) <= tol, (i, name)
            assert rel(tok(got["dbeta"]), ref["dbeta"]) <= tol, (i, "dbeta")
            if ref["dg"] is not None:
                assert rel(tok(got["dg"]), ref["dg"]) <= tol, (i, "dg")
        assert rel(got["dh0"][i:i + 1], ref["dh0"]) <= tol, (i, "dh0")
