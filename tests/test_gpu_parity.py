"""GPU parity: every op of the drop-in surface through the C ABI against the CPU oracle.

Tolerances (stated by the task): fp32 inputs -> max-abs error <= 1e-4; bf16 inputs with fp32
accumulation -> max|x - ref| / max|ref| <= 2e-2 on outputs and final state.
"""
import numpy as np
import pytest
import torch

import linearnexus_b200 as L
from linearnexus_b200 import _lib
from oracle import delta_rule_oracle as O

pytestmark = pytest.mark.gpu
F64 = torch.float64
FP32_TOL = 1e-4
BF16_TOL = 2e-2


def _cuda(x):
    return None if x is None else x.cuda()


def _rel(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return ((a - b).abs().max() / b.abs().max().clamp_min(1e-30)).item()


def _abs(a, b):
    return (a.double().cpu() - b.double().cpu()).abs().max().item()


def _run(variant, kind, inp, chunk=64, path=None, **kw):
    q, k, v, g, beta, h0 = (_cuda(inp[x]) for x in ("q", "k", "v", "g", "beta", "h0"))
    if variant == "delta":
        if kind == "chunk":
            return L.delta_rule_chunkwise(q, k, v, beta, h0, chunk_size=chunk, path=path, **kw)
        return L.delta_rule_recurrent(q, k, v, beta, h0, **kw)
    if variant == "gated":
        if kind == "chunk":
            return L.gated_delta_rule_chunkwise(q, k, v, g, beta, initial_state=h0, chunk_size=chunk, path=path, **kw)
        return L.gated_delta_rule_recurrent(q, k, v, g, beta, initial_state=h0, **kw)
    if kind == "chunk":
        return L.kda_chunkwise(q, k, v, g, beta, initial_state=h0, chunk_size=chunk, path=path, **kw)
    return L.kda_recurrent(q, k, v, g, beta, initial_state=h0, **kw)


def _truth(variant, inp, **kw):
    d = lambda x: None if x is None else x.double()
    q, k, v, g, beta, h0 = (d(inp[x]) for x in ("q", "k", "v", "g", "beta", "h0"))
    if variant == "delta":
        return O.delta_rule_recurrent(q, k, v, beta, h0, compute_dtype=F64, **kw)
    if variant == "gated":
        return O.gated_delta_rule_recurrent(q, k, v, g, beta, initial_state=h0, compute_dtype=F64, **kw)
    return O.kda_recurrent(q, k, v, g, beta, initial_state=h0, compute_dtype=F64, **kw)


@pytest.mark.parametrize("name", ["delta", "gated", "kda"])
@pytest.mark.parametrize("kind", ["recurrent", "chunk"])
def test_golden_fixture(golden, name, kind):
    G = lambda key: torch.from_numpy(golden[f"{name}.{key}"]) if f"{name}.{key}" in golden.files else None
    inp = dict(q=G("q"), k=G("k"), v=G("v"), g=G("g"), beta=G("beta"), h0=G("h0"))
    o, hT = _run(name, kind, inp, chunk=int(golden[f"{name}.chunk"]), path="fp32")
    assert _abs(o, G("o")) <= FP32_TOL
    assert _abs(hT, G("hT")) <= FP32_TOL
    assert hT.dtype == torch.float32
    q, k, v, g, beta, h0 = (_cuda(inp[x]) for x in ("q", "k", "v", "g", "beta", "h0"))
    if name == "delta":
        so, sS = L.delta_rule_step(q[:, :, 0], k[:, :, 0], v[:, :, 0], beta[:, :, 0], h0)
    elif name == "gated":
        so, sS = L.gated_delta_rule_step(q[:, :, 0], k[:, :, 0], v[:, :, 0], g[:, :, 0], beta[:, :, 0], h0)
    else:
        so, sS = L.kda_step(q[:, :, 0], k[:, :, 0], v[:, :, 0], g[:, :, 0], beta[:, :, 0], h0)
    assert _abs(so, G("step_o")) <= FP32_TOL
    assert _abs(sS, G("step_S")) <= FP32_TOL


SHAPES = [
    # B, H, T, K, V, chunk
    (2, 4, 32, 16, 32, 16),     # reference test shape (tests/test_deltanet.py:64-90)
    (2, 2, 64, 8, 8, 64),       # reference KDA test shape (tests/test_kda.py:252-290)
    (1, 2, 1, 32, 64, 16),      # single token
    (1, 2, 63, 64, 64, 64),     # one short chunk
    (1, 2, 65, 64, 64, 64),     # one token into the second chunk
    (1, 3, 130, 128, 128, 64),  # ragged tail, headline head size
    (1, 2, 50, 32, 48, 32),     # reference padding case T=50, chunk=32 (tests/test_gated_deltanet.py:229-247); V not a multiple of 32
    (1, 1, 96, 100, 36, 32),    # K, V not powers of two
]


@pytest.mark.parametrize("variant", ["delta", "gated", "kda"])
@pytest.mark.parametrize("kind", ["recurrent", "chunk"])
@pytest.mark.parametrize("shape", SHAPES)
def test_fp32_parity(variant, kind, shape):
    B, H, T, K, V, C = shape
    inp = O.make_inputs(variant, B, H, T, K, V, seed=sum(shape) + 7 * len(variant), h0_std=0.1)
    inp["q"] = inp["q"] * 1.3
    kw = {} if variant == "delta" else {"use_qk_l2norm": True}
    o, hT = _run(variant, kind, inp, chunk=C, path="fp32", **kw)
    ro, rS = _truth(variant, inp, **kw)
    assert o.shape == (B, H, T, V) and hT.shape == (B, H, K, V)
    assert _abs(o, ro) <= FP32_TOL, _lib.last_path()
    assert _abs(hT, rS) <= FP32_TOL
    # determinism: a second run is bit-identical (catches races)
    o2, hT2 = _run(variant, kind, inp, chunk=C, path="fp32", **kw)
    assert torch.equal(o, o2) and torch.equal(hT, hT2)


def test_config1_deltanet_fp32():
    """DeltaNet forward fp32, B=2,T=512,H=4,d=64, chunk 64, zero state: the reference's own
    CPU-runnable configuration."""
    inp = O.make_inputs("delta", 2, 4, 512, 64, 64, seed=1235)
    o, hT = _run("delta", "chunk", inp, chunk=64)
    ro, rS = O.delta_rule_recurrent(inp["q"].double(), inp["k"].double(), inp["v"].double(), inp["beta"].double(), compute_dtype=F64)
    co, cS = O.delta_rule_chunkwise(inp["q"], inp["k"], inp["v"], inp["beta"], chunk_size=64)
    assert _abs(o, ro) <= FP32_TOL and _abs(hT, rS) <= FP32_TOL
    assert _abs(o, co) <= FP32_TOL and _abs(hT, cS) <= FP32_TOL


@pytest.mark.parametrize("variant", ["delta", "gated", "kda"])
@pytest.mark.parametrize("kind", ["recurrent", "chunk"])
def test_bf16_io_parity(variant, kind):
    B, H, T, K, V = 1, 2, 200, 128, 128
    inp = O.make_inputs(variant, B, H, T, K, V, seed=77, io_dtype=torch.bfloat16, h0_std=0.02)
    o, hT = _run(variant, kind, inp, chunk=64, path="fp32")
    ro, rS = _truth(variant, {k_: (v_.float() if v_ is not None and v_.dtype == torch.bfloat16 else v_) for k_, v_ in inp.items()})
    assert o.dtype == (torch.float32 if (variant == "kda" and kind == "chunk") else torch.bfloat16)
    assert _rel(o, ro) <= BF16_TOL and _rel(hT, rS) <= BF16_TOL


def test_beta_zero_keeps_state_zero_and_beta_rank4():
    inp = O.make_inputs("delta", 1, 2, 40, 16, 32, seed=3)
    q, k, v = (_cuda(inp[x]) for x in "qkv")
    _, s = L.delta_rule_chunkwise(q, k, v, torch.zeros(1, 2, 40, 1, device="cuda"), chunk_size=8)
    assert s.abs().max().item() == 0
    o1, s1 = L.delta_rule_recurrent(q, k, v, _cuda(inp["beta"])[..., None])
    o2, s2 = L.delta_rule_recurrent(q, k, v, _cuda(inp["beta"]))
    assert torch.equal(o1, o2) and s1.abs().max().item() > 0


def test_gated_chunk_size_not_multiple_of_16_raises():
    inp = O.make_inputs("gated", 1, 1, 20, 16, 16, seed=3)
    with pytest.raises(ValueError, match="divisible"):
        _run("gated", "chunk", inp, chunk=24)
    _run("delta", "chunk", O.make_inputs("delta", 1, 1, 20, 16, 16, seed=3), chunk=24)  # DeltaNet has no such rule


def test_pallas_entry_guards_and_result():
    inp = O.make_inputs("delta", 1, 2, 33, 32, 64, seed=4)
    q, k, v, beta = (_cuda(inp[x]) for x in ("q", "k", "v", "beta"))
    o, s = L.delta_rule_recurrent_pallas(q, k, v, beta)
    ro, rS = _truth("delta", inp)
    assert _abs(o, ro) <= FP32_TOL and _abs(s, rS) <= FP32_TOL
    with pytest.raises(RuntimeError):
        L.delta_rule_recurrent_pallas(q[..., :16], k[..., :16], v, beta)
    with pytest.raises(RuntimeError):
        L.delta_rule_recurrent_pallas(q, k, v[..., :32], beta)


def test_bthd_view_is_consumed_without_copy():
    """Inputs that are transposed views of [B,T,H,D] arrays (the blocks' native layout)."""
    inp = O.make_inputs("gated", 2, 3, 70, 32, 64, seed=8)
    cu = {k_: _cuda(v_) for k_, v_ in inp.items()}
    as_view = lambda t: t.transpose(1, 2).contiguous().transpose(1, 2)
    o1, s1 = L.gated_delta_rule_chunkwise(cu["q"], cu["k"], cu["v"], cu["g"], cu["beta"], chunk_size=32, path="fp32")
    o2, s2 = L.gated_delta_rule_chunkwise(as_view(cu["q"]), as_view(cu["k"]), as_view(cu["v"]), as_view(cu["g"]),
                                          as_view(cu["beta"]), chunk_size=32, path="fp32")
    assert o2.transpose(1, 2).is_contiguous()
    assert torch.equal(o1, o2) and torch.equal(s1, s2)
    o3, s3 = L.gated_delta_rule_recurrent(as_view(cu["q"]), as_view(cu["k"]), as_view(cu["v"]), as_view(cu["g"]), as_view(cu["beta"]))
    ro, rS = _truth("gated", inp)
    assert _abs(o3, ro) <= FP32_TOL and _abs(s3, rS) <= FP32_TOL


@pytest.mark.parametrize("variant", ["delta", "gated", "kda"])
@pytest.mark.parametrize("shape", [(2, 4, 16, 32), (3, 2, 128, 128), (1, 2, 100, 36), (1, 1, 256, 256), (2, 2, 8, 8)])
def test_step_parity_and_inplace(variant, shape):
    B, H, K, V = shape
    inp = O.make_inputs(variant, B, H, 6, K, V, seed=K + V, h0_std=0.02)
    S_ref = inp["h0"].double()
    S_gpu = inp["h0"].cuda().clone()
    for t in range(6):
        sl = lambda x: None if x is None else x[:, :, t]
        q, k, v, g, beta = (sl(inp[x]) for x in ("q", "k", "v", "g", "beta"))
        if variant == "delta":
            ro, S_ref = O.delta_rule_step(q.double(), k.double(), v.double(), beta.double(), S_ref, compute_dtype=F64)
            o, S_new = L.delta_rule_step(_cuda(q), _cuda(k), _cuda(v), _cuda(beta), S_gpu)
            S_gpu = S_new
        elif variant == "gated":
            ro, S_ref = O.gated_delta_rule_step(q.double(), k.double(), v.double(), g.double(), beta.double(), S_ref, compute_dtype=F64)
            o, S_new = L.gated_delta_rule_step(_cuda(q), _cuda(k), _cuda(v), _cuda(g), _cuda(beta), S_gpu, inplace=True)
            assert S_new.data_ptr() == S_gpu.data_ptr()
        else:
            ro, S_ref = O.kda_step(q.double(), k.double(), v.double(), g.double(), beta.double(), S_ref, compute_dtype=F64)
            o, S_new = L.kda_step(_cuda(q), _cuda(k), _cuda(v), _cuda(g), _cuda(beta), S_gpu, inplace=True)
            assert o.dtype == S_gpu.dtype
        assert _abs(o, ro) <= FP32_TOL
        assert _abs(S_gpu, S_ref) <= FP32_TOL


def test_step_bf16_io_decode_config_shape():
    """Decode configuration head shape (d_k=d_v=128, bf16 q,k,v, fp32 cache) on a batch subset."""
    B, H, K, V = 4, 32, 128, 128
    inp = O.make_inputs("gated", B, H, 8, K, V, seed=1238, io_dtype=torch.bfloat16, h0_std=0.02)
    S_ref = inp["h0"].double()
    S_gpu = inp["h0"].cuda().clone()
    for t in range(8):
        q, k, v, g, beta = (inp[x][:, :, t] for x in ("q", "k", "v", "g", "beta"))
        ro, S_ref = O.gated_delta_rule_step(q.double(), k.double(), v.double(), g.double(), beta.double(), S_ref, compute_dtype=F64)
        o, _ = L.gated_delta_rule_step(_cuda(q), _cuda(k), _cuda(v), _cuda(g), _cuda(beta), S_gpu, inplace=True)
        assert o.dtype == torch.bfloat16
        assert _rel(o, ro) <= BF16_TOL
    assert _rel(S_gpu, S_ref) <= 1e-4


@pytest.mark.parametrize("variant", ["delta", "gated", "kda"])
def test_step_streamed_kernel_many_units(variant):
    """More than two (batch, head) units per SM at d_k = d_v = 128: the persistent, TMA-pipelined decode kernel.
    Three steps, in place and out of place, against the float64 step."""
    from linearnexus_b200 import _lib
    B, H, K, V = 41, 8, 128, 128
    inp = O.make_inputs(variant, B, H, 3, K, V, seed=77, io_dtype=torch.bfloat16, h0_std=0.02)
    S_ref = inp["h0"].double()
    S_gpu = inp["h0"].cuda().clone()
    for t in range(3):
        sl = lambda x: None if x is None else x[:, :, t]
        q, k, v, g, beta = (sl(inp[x]) for x in ("q", "k", "v", "g", "beta"))
        if variant == "delta":
            ro, S_ref = O.delta_rule_step(q.double(), k.double(), v.double(), beta.double(), S_ref, compute_dtype=F64)
            o, S_gpu = L.delta_rule_step(_cuda(q), _cuda(k), _cuda(v), _cuda(beta), S_gpu)
        elif variant == "gated":
            ro, S_ref = O.gated_delta_rule_step(q.double(), k.double(), v.double(), g.double(), beta.double(), S_ref, compute_dtype=F64)
            o, _ = L.gated_delta_rule_step(_cuda(q), _cuda(k), _cuda(v), _cuda(g), _cuda(beta), S_gpu, inplace=True)
        else:
            ro, S_ref = O.kda_step(q.double(), k.double(), v.double(), g.double(), beta.double(), S_ref, compute_dtype=F64)
            o, _ = L.kda_step(_cuda(q), _cuda(k), _cuda(v), _cuda(g), _cuda(beta), S_gpu, inplace=True)
        assert _lib.last_path() == "step_stream"
        assert _rel(o, ro) <= BF16_TOL
        assert _rel(S_gpu, S_ref) <= 1e-4
