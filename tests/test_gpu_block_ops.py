"""The element-wise steps around the op (short conv + SiLU, gate activations, gated RMSNorm) against the CPU
restatement of the reference helpers (oracle/block_ops_oracle.py).  fp32: max-abs 1e-5 relative to the largest
reference value; bf16: one bf16 rounding of the result (2^-8 relative) plus the same."""
import pytest
import torch

import linearnexus_b200 as L
from linearnexus_b200 import block_ops as BO
from oracle import block_ops_oracle as O

pytestmark = pytest.mark.gpu


def _close(got, ref, dtype):
    tol = 1e-5 if dtype == torch.float32 else 2.0 ** -7
    ref = ref.double()
    err = (got.double().cpu() - ref).abs().max() / ref.abs().max().clamp_min(1e-30)
    assert err <= tol, float(err)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,T,C,W,bias,cache,silu", [
    (2, 100, 256, 4, False, False, True),      # the blocks' configuration
    (2, 100, 256, 4, True, True, True),
    (1, 1, 512, 4, False, True, True),         # decode step with a cache
    (3, 33, 64, 2, True, True, False),
    (2, 70, 128, 7, False, True, True),        # wide window, two tiles
    (2, 2, 64, 4, False, True, True),          # T shorter than the history
    (2, 40, 128, 1, True, False, True),        # kernel_size 1: the input (+ bias), weight unused
    (1, 4096, 2048, 4, False, False, True)])
def test_short_conv_silu(dtype, B, T, C, W, bias, cache, silu):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(B, T, C, generator=g).to(dtype)
    w = torch.randn(W, C, generator=g) * 0.5
    bs = torch.randn(C, generator=g) if bias else None
    ch = torch.randn(B, W - 1, C, generator=g).to(dtype) if cache and W > 1 else None
    y_ref, c_ref = O.short_conv_silu(x, w, bs, ch, apply_silu=silu)
    y, c = BO.depthwise_conv1d_causal(x.cuda(), w.cuda(), None if bs is None else bs.cuda(),
                                      cache=None if ch is None else ch.cuda(), activation="silu" if silu else None)
    assert y.shape == x.shape and y.dtype == dtype and c.shape == c_ref.shape
    _close(y, y_ref, dtype)
    assert torch.equal(c.cpu(), c_ref)   # the cache is a copy of input rows


def test_short_conv_decode_updates_cache_in_place_and_matches_prefill():
    """T steps one at a time through the cache give the rows of the full-sequence call."""
    g = torch.Generator().manual_seed(4)
    B, T, C, W = 2, 9, 128, 4
    x = torch.randn(B, T, C, generator=g).cuda()
    w = torch.randn(W, C, generator=g).cuda()
    y_all, c_all = BO.short_conv_silu(x, w)
    cache = torch.zeros(B, W - 1, C, device="cuda")
    rows = []
    for t in range(T):
        y, c = BO.short_conv_silu(x[:, t:t + 1].contiguous(), w, cache=cache, cache_out=cache)
        assert c.data_ptr() == cache.data_ptr()
        rows.append(y)
    assert torch.allclose(torch.cat(rows, 1), y_all, atol=1e-6, rtol=1e-6)
    assert torch.equal(cache, c_all)


def test_short_conv_feeds_the_op_without_transposes():
    """conv + SiLU output [B,T,H*D] viewed as [B,T,H,D] is read by the op in place (transposed views)."""
    g = torch.Generator().manual_seed(5)
    B, T, H, D = 1, 128, 2, 64
    mk = lambda: torch.randn(B, T, H * D, generator=g).cuda()
    w = (torch.randn(4, H * D, generator=g) * 0.5).cuda()
    q, k, v = (BO.short_conv_silu(mk(), w)[0].view(B, T, H, D) for _ in range(3))
    a, b = torch.randn(B, T, H, generator=g).cuda(), torch.randn(B, T, H, generator=g).cuda()
    gg, beta = BO.gated_deltanet_gates(a, b, torch.zeros(H).cuda(), torch.zeros(H).cuda())
    view = lambda t: t.transpose(1, 2)                 # [B,H,T,..] views of the token-major arrays: no copies
    o1, s1 = L.gated_delta_rule_chunkwise(view(q), view(k), view(v), view(gg), view(beta))
    assert o1.transpose(1, 2).is_contiguous()          # the op answered in the same layout
    tr = lambda t: t.transpose(1, 2).contiguous()
    o2, s2 = L.gated_delta_rule_chunkwise(tr(q), tr(k), tr(v), tr(gg), tr(beta))
    assert torch.equal(o1, o2) and torch.equal(s1, s2)
    wn = torch.rand(D, generator=g).cuda() + 0.5
    gate = torch.randn(B, T, H, D, generator=g).cuda()
    y1, y2 = BO.rmsnorm_gated(o1, wn, gate), BO.rmsnorm_gated(o2, wn, gate)
    assert y1.shape == (B, T, H, D) and torch.equal(y1, y2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("neg", [False, True])
def test_gated_deltanet_gates(dtype, neg):
    g = torch.Generator().manual_seed(6)
    B, T, H = 2, 77, 6
    a = (torch.randn(B, T, H, generator=g) * 4).to(dtype)
    b = (torch.randn(B, T, H, generator=g) * 4).to(dtype)
    A_log, dt_bias = torch.randn(H, generator=g), torch.randn(H, generator=g)
    g_ref, b_ref = O.gdn_gate_activations(a, b, A_log, dt_bias, neg)
    gg, beta = BO.gated_deltanet_gates(a.cuda(), b.cuda(), A_log.cuda(), dt_bias.cuda(), neg)
    assert gg.dtype == torch.float32 and gg.shape == (B, T, H) and beta.shape == (B, T, H)
    _close(gg, g_ref, torch.float32)
    _close(beta, b_ref, torch.float32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("with_bias,with_beta", [(True, True), (False, False)])
def test_kda_gate(dtype, with_bias, with_beta):
    g = torch.Generator().manual_seed(7)
    B, T, H, K = 2, 50, 3, 32
    x = (torch.randn(B, T, H * K, generator=g) * 12).to(dtype)   # crosses the softplus threshold of 20
    A_log = torch.randn(H, generator=g)
    bias = torch.randn(H * K, generator=g) if with_bias else None
    beta = torch.randn(B, T, H, generator=g) if with_beta else None
    g_ref, b_ref = O.kda_gate(x.float() if with_bias else x, A_log, K, bias, beta)
    gg, bb = BO.kda_gate(x.cuda(), A_log.cuda(), K, None if bias is None else bias.cuda(),
                         None if beta is None else beta.cuda())
    assert gg.shape == (B, T, H, K)
    _close(gg, g_ref, torch.float32)
    if with_beta:
        _close(bb, b_ref, torch.float32)
    else:
        assert bb is None


@pytest.mark.parametrize("odt,gdt,ydt", [(torch.bfloat16, torch.bfloat16, torch.bfloat16),
                                         (torch.float32, torch.float32, torch.float32),
                                         (torch.float32, torch.bfloat16, torch.bfloat16),
                                         (torch.bfloat16, None, torch.float32)])
@pytest.mark.parametrize("layout", ["bhtd", "bthd"])
@pytest.mark.parametrize("V", [128, 64, 256, 20])
def test_rmsnorm_gated(odt, gdt, ydt, layout, V):
    g = torch.Generator().manual_seed(8)
    B, H, T = 2, 3, 37
    o = torch.randn(B, H, T, V, generator=g).to(odt)
    gate = None if gdt is None else torch.randn(B, T, H, V, generator=g).to(gdt)
    w = torch.rand(V, generator=g) + 0.5
    ref = O.gated_rmsnorm(o.transpose(1, 2), w, gate, eps=1e-5)
    oin = o if layout == "bhtd" else o.transpose(1, 2).contiguous()
    y = BO.rmsnorm_gated(oin.cuda(), w.cuda(), None if gate is None else gate.cuda(), eps=1e-5, o_layout=layout,
                         out_dtype=ydt)
    assert y.shape == (B, T, H, V) and y.dtype == ydt
    _close(y, ref, ydt)


def test_block_ops_full_size_properties():
    """At the benchmark's size: the conv of a constant sequence is constant after the history, the norm of a
    scaled input is unchanged, and outputs are finite."""
    B, T, H, D = 8, 4096, 16, 128
    x = torch.ones(B, T, H * D, device="cuda", dtype=torch.bfloat16)
    w = torch.full((4, H * D), 0.25, device="cuda")
    y, c = BO.short_conv_silu(x, w)
    assert torch.all(y[:, 3:] == y[:, 3:4]) and torch.equal(c, x[:, -3:])
    o = torch.randn(B, H, T, D, device="cuda", dtype=torch.bfloat16)
    wn = torch.ones(D, device="cuda")
    y1 = BO.rmsnorm_gated(o, wn, eps=0.0)
    y2 = BO.rmsnorm_gated(o * 4, wn, eps=0.0)
    assert torch.isfinite(y1.float()).all() and torch.equal(y1, y2)


def test_block_ops_against_golden_vectors():
    """The kernels on the committed fixtures (float64 oracle outputs, tests/golden/make_block_ops_golden.py)."""
    import numpy as np
    from pathlib import Path
    G = np.load(Path(__file__).parent / "golden" / "block_ops_golden.npz")
    c = lambda k: torch.from_numpy(G[k]).cuda()
    y, nc = BO.short_conv_silu(c("conv.x"), c("conv.w"), c("conv.bias"), cache=c("conv.cache"))
    _close(y, torch.from_numpy(G["conv.y"]), torch.float32)
    assert torch.equal(nc.cpu(), torch.from_numpy(G["conv.new_cache"]))
    g, beta = BO.gated_deltanet_gates(c("gdn_gate.a"), c("gdn_gate.b"), c("gdn_gate.A_log"), c("gdn_gate.dt_bias"), True)
    _close(g, torch.from_numpy(G["gdn_gate.g"]), torch.float32)
    _close(beta, torch.from_numpy(G["gdn_gate.beta"]), torch.float32)
    gk, bk = BO.kda_gate(c("kda_gate.g"), c("kda_gate.A_log"), 8, c("kda_gate.g_bias"), c("kda_gate.beta"))
    _close(gk, torch.from_numpy(G["kda_gate.g_out"]), torch.float32)
    _close(bk, torch.from_numpy(G["kda_gate.beta_out"]), torch.float32)
    yn = BO.rmsnorm_gated(c("norm.o"), c("norm.w"), c("norm.gate"), eps=1e-5)
    _close(yn, torch.from_numpy(G["norm.y"]), torch.float32)


def test_parameters_of_a_bf16_model_and_strided_parameters():
    """Parameters that are not fp32-contiguous (a bf16 model; a strided slice of a fused parameter) are converted
    inside the wrappers; the converted copies must stay alive until the kernel has been enqueued.  A_log and dt_bias
    (and weight / bias rows) have the same size, which is exactly the case where a released temporary would be
    handed to the next conversion."""
    g = torch.Generator().manual_seed(12)
    B, T, H = 2, 64, 8
    a = (torch.randn(B, T, H, generator=g) * 3).bfloat16()
    b = (torch.randn(B, T, H, generator=g) * 3).bfloat16()
    A_log = torch.randn(H, generator=g).bfloat16()
    dt_bias = torch.randn(H, generator=g).bfloat16()
    g_ref, b_ref = O.gdn_gate_activations(a, b, A_log.float(), dt_bias.float(), False)
    gg, beta = BO.gated_deltanet_gates(a.cuda(), b.cuda(), A_log.cuda(), dt_bias.cuda())
    _close(gg, g_ref, torch.float32)
    _close(beta, b_ref, torch.float32)
    # strided fp32 parameters: every second entry of a wider tensor
    wide = torch.randn(2 * H, generator=g)
    A2, d2 = wide[::2], torch.randn(2 * H, generator=g)[1::2]
    g_ref, b_ref = O.gdn_gate_activations(a, b, A2, d2, True)
    gg, beta = BO.gated_deltanet_gates(a.cuda(), b.cuda(), wide.cuda()[::2], d2.cuda(), True)
    _close(gg, g_ref, torch.float32)
    _close(beta, b_ref, torch.float32)
    # conv taps and bias in bf16, both [.., C] with W == 1 row of bias-sized data next to them
    C, W = 128, 4
    x = torch.randn(B, T, C, generator=g).bfloat16()
    w = (torch.randn(W, C, generator=g) * 0.5).bfloat16()
    bs = torch.randn(C, generator=g).bfloat16()
    y_ref, _ = O.short_conv_silu(x, w.float(), bs.float(), None, apply_silu=True)
    y, _ = BO.short_conv_silu(x.cuda(), w.cuda(), bs.cuda())
    _close(y, y_ref, torch.bfloat16)
    # norm weight in bf16 and as a strided view
    V = 128
    o = torch.randn(B, H, T, V, generator=g).bfloat16()
    gate = torch.randn(B, T, H, V, generator=g).bfloat16()
    nw = (torch.rand(2 * V, generator=g) + 0.5)
    ref = O.gated_rmsnorm(o.transpose(1, 2), nw[::2], gate, eps=1e-5)
    y = BO.rmsnorm_gated(o.cuda(), nw.cuda()[::2], gate.cuda(), eps=1e-5)
    _close(y, ref, torch.bfloat16)
    ref = O.gated_rmsnorm(o.transpose(1, 2), nw[:V].bfloat16().float(), gate, eps=1e-5)
    y = BO.rmsnorm_gated(o.cuda(), nw[:V].bfloat16().cuda(), gate.cuda(), eps=1e-5)
    _close(y, ref, torch.bfloat16)
