"""CPU tests of the oracle: the reference's own self-consistency tests re-expressed, plus the
committed golden vectors (float64 token recurrence)."""
import numpy as np
import pytest
import torch

from oracle import delta_rule_oracle as O

F64 = torch.float64


def _t(a):
    return torch.from_numpy(np.asarray(a))


def _rand(shape, seed):
    return torch.from_numpy(np.random.default_rng(seed).standard_normal(shape, dtype=np.float32))


def test_deltanet_recurrent_vs_chunkwise_parity():
    # tests/test_deltanet.py:64-90 -- B=2,H=4,T=32,dk=16,dv=32, chunk 8, rtol=atol=1e-3
    q, k, v = _rand((2, 4, 32, 16), 0), _rand((2, 4, 32, 16), 1), _rand((2, 4, 32, 32), 2)
    beta = torch.sigmoid(_rand((2, 4, 32), 3))
    q, k = O._l2norm(q), O._l2norm(k)
    o1, s1 = O.delta_rule_recurrent(q, k, v, beta)
    o2, s2 = O.delta_rule_chunkwise(q, k, v, beta, chunk_size=8)
    assert torch.allclose(o1, o2, rtol=1e-3, atol=1e-3)
    assert torch.allclose(s1, s2, rtol=1e-3, atol=1e-3)


def test_deltanet_step_matches_recurrent():
    # tests/test_deltanet.py:134-157
    q, k, v = _rand((2, 4, 1, 16), 0), _rand((2, 4, 1, 16), 1), _rand((2, 4, 1, 32), 2)
    beta = torch.sigmoid(_rand((2, 4, 1), 3))
    q, k = O._l2norm(q), O._l2norm(k)
    o1, s1 = O.delta_rule_recurrent(q, k, v, beta)
    o2, s2 = O.delta_rule_step(q[:, :, 0], k[:, :, 0], v[:, :, 0], beta[:, :, 0], torch.zeros(2, 4, 16, 32))
    assert torch.allclose(o1[:, :, 0], o2, rtol=1e-5)
    assert torch.allclose(s1, s2, rtol=1e-5)


def test_deltanet_initial_state_changes_output():
    # tests/test_deltanet.py:92-113
    q, k, v = O._l2norm(_rand((2, 4, 16, 16), 0)), O._l2norm(_rand((2, 4, 16, 16), 1)), _rand((2, 4, 16, 32), 2)
    beta = torch.sigmoid(_rand((2, 4, 16), 3))
    h0 = _rand((2, 4, 16, 32), 4) * 0.1
    o0, _ = O.delta_rule_recurrent(q, k, v, beta)
    o1, _ = O.delta_rule_recurrent(q, k, v, beta, initial_state=h0)
    assert not torch.allclose(o0, o1)


def test_beta_zero_keeps_state_zero():
    # tests/test_deltanet.py:281-297
    q, k, v = _rand((1, 2, 8, 16), 0), _rand((1, 2, 8, 16), 1), _rand((1, 2, 8, 32), 2)
    _, s = O.delta_rule_recurrent(q, k, v, torch.zeros(1, 2, 8))
    assert s.abs().max() == 0
    _, s = O.delta_rule_recurrent(q, k, v, torch.ones(1, 2, 8))
    assert s.abs().max() > 0


def test_gated_step_matches_recurrent():
    # tests/test_gated_deltanet.py:310-339
    q, k, v = _rand((2, 4, 16), 0), _rand((2, 4, 16), 1), _rand((2, 4, 32), 2)
    g = -torch.rand(2, 4, generator=torch.Generator().manual_seed(3))
    beta = torch.rand(2, 4, generator=torch.Generator().manual_seed(4))
    o1, s1 = O.gated_delta_rule_step(q, k, v, g, beta, torch.zeros(2, 4, 16, 32))
    o2, s2 = O.gated_delta_rule_recurrent(q[:, :, None], k[:, :, None], v[:, :, None], g[:, :, None], beta[:, :, None])
    assert torch.allclose(o1, o2[:, :, 0], rtol=1e-4, atol=1e-4)
    assert torch.allclose(s1, s2, rtol=1e-4, atol=1e-4)


def test_gated_chunk_matches_recurrent_multi_chunk():
    # the reference only checks finiteness here (tests/test_gated_deltanet.py:249-284); the
    # oracle is held to closeness.
    inp = O.make_inputs("gated", 1, 2, 100, 16, 32, seed=5)
    o1, s1 = O.gated_delta_rule_recurrent(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], scale=1.0)
    o2, s2 = O.gated_delta_rule_chunkwise(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], scale=1.0, chunk_size=32)
    assert torch.allclose(o1, o2, rtol=1e-4, atol=1e-5)
    assert torch.allclose(s1, s2, rtol=1e-4, atol=1e-5)


def test_gated_chunk_size_must_divide_16():
    inp = O.make_inputs("gated", 1, 1, 20, 8, 8, seed=5)
    with pytest.raises(ValueError):
        O.gated_delta_rule_chunkwise(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], chunk_size=24)


def test_kda_chunk_matches_recurrent():
    # tests/test_kda.py:252-290 -- B=2,H=2,T=64,dk=dv=8, one chunk, g in [-0.5,0], 2e-3
    q, k, v = _rand((2, 2, 64, 8), 0), _rand((2, 2, 64, 8), 1), _rand((2, 2, 64, 8), 2)
    g = -0.5 * torch.rand(2, 2, 64, 8, generator=torch.Generator().manual_seed(3))
    beta = torch.rand(2, 2, 64, generator=torch.Generator().manual_seed(4))
    o1, s1 = O.kda_recurrent(q, k, v, g, beta)
    o2, s2 = O.kda_chunkwise(q, k, v, g, beta, chunk_size=64)
    assert torch.allclose(o1, o2, rtol=2e-3, atol=2e-3)
    assert torch.allclose(s1, s2, rtol=2e-3, atol=2e-3)


def test_kda_step_matches_recurrent_and_dtype_quirks():
    # tests/test_kda.py:219-250; output dtype quirks kda.py:347 (state dtype) and :655 (float32)
    q, k, v = _rand((2, 2, 8), 0), _rand((2, 2, 8), 1), _rand((2, 2, 8), 2)
    g = -torch.rand(2, 2, 8, generator=torch.Generator().manual_seed(3))
    beta = torch.rand(2, 2, generator=torch.Generator().manual_seed(4))
    o1, s1 = O.kda_step(q.bfloat16(), k.bfloat16(), v.bfloat16(), g, beta, torch.zeros(2, 2, 8, 8))
    assert o1.dtype == torch.float32
    o2, s2 = O.kda_recurrent(q.bfloat16()[:, :, None], k.bfloat16()[:, :, None], v.bfloat16()[:, :, None], g[:, :, None], beta[:, :, None])
    assert o2.dtype == torch.bfloat16
    assert torch.allclose(o1, o2[:, :, 0].float(), rtol=1e-2, atol=1e-2)
    assert torch.allclose(s1, s2, rtol=1e-4, atol=1e-4)
    o3, _ = O.kda_chunkwise(q.bfloat16()[:, :, None].expand(2, 2, 16, 8), k.bfloat16()[:, :, None].expand(2, 2, 16, 8),
                            v.bfloat16()[:, :, None].expand(2, 2, 16, 8), g[:, :, None].expand(2, 2, 16, 8),
                            beta[:, :, None].expand(2, 2, 16), chunk_size=16)
    assert o3.dtype == torch.float32


def test_stronger_decay_shrinks_state():
    # tests/test_kda.py:743-766
    inp = O.make_inputs("kda", 1, 2, 32, 8, 8, seed=9)
    _, s_weak = O.kda_recurrent(inp["q"], inp["k"], inp["v"], torch.full_like(inp["g"], -0.01), inp["beta"])
    _, s_strong = O.kda_recurrent(inp["q"], inp["k"], inp["v"], torch.full_like(inp["g"], -1.0), inp["beta"])
    assert s_strong.norm() < s_weak.norm()


@pytest.mark.parametrize("name", ["delta", "gated", "kda"])
def test_oracle_fp32_against_golden(golden, name):
    """fp32 restatements (recurrent, chunk, step) against the committed float64 vectors."""
    G = lambda key: _t(golden[f"{name}.{key}"]) if f"{name}.{key}" in golden.files else None
    q, k, v, g, beta, h0 = G("q"), G("k"), G("v"), G("g"), G("beta"), G("h0")
    C = int(golden[f"{name}.chunk"])
    if name == "delta":
        o1, s1 = O.delta_rule_recurrent(q, k, v, beta, h0)
        o2, s2 = O.delta_rule_chunkwise(q, k, v, beta, h0, chunk_size=C)
        so, sS = O.delta_rule_step(q[:, :, 0], k[:, :, 0], v[:, :, 0], beta[:, :, 0], h0)
    elif name == "gated":
        o1, s1 = O.gated_delta_rule_recurrent(q, k, v, g, beta, initial_state=h0)
        o2, s2 = O.gated_delta_rule_chunkwise(q, k, v, g, beta, initial_state=h0, chunk_size=C)
        so, sS = O.gated_delta_rule_step(q[:, :, 0], k[:, :, 0], v[:, :, 0], g[:, :, 0], beta[:, :, 0], h0)
    else:
        o1, s1 = O.kda_recurrent(q, k, v, g, beta, initial_state=h0)
        o2, s2 = O.kda_chunkwise(q, k, v, g, beta, initial_state=h0, chunk_size=C)
        so, sS = O.kda_step(q[:, :, 0], k[:, :, 0], v[:, :, 0], g[:, :, 0], beta[:, :, 0], h0)
    for got, key in ((o1, "o"), (o2, "o"), (s1, "hT"), (s2, "hT"), (so, "step_o"), (sS, "step_S")):
        assert (got.double() - G(key)).abs().max() < 1e-5, key


@pytest.mark.parametrize("name", ["delta", "gated", "kda"])
def test_oracle_grads_against_golden(golden, name):
    G = lambda key: _t(golden[f"{name}.{key}"]) if f"{name}.{key}" in golden.files else None
    gr = O.delta_rule_grads(name, G("q"), G("k"), G("v"), G("g"), G("beta"), G("h0"), G("do"), G("dhT"),
                            use_qk_l2norm=(name != "delta"))
    for key in ("dq", "dk", "dv", "dg", "dbeta", "dh0"):
        if G(key) is not None:
            assert (gr[key] - G(key)).abs().max() < 1e-9, key


def test_block_ops_oracle_against_torch_primitives():
    """The restated conv / norm against torch's own conv1d and a direct formula; kernel_size 1 returns the input."""
    import torch.nn.functional as F
    from oracle import block_ops_oracle as BO
    g = torch.Generator().manual_seed(0)
    B, T, C, W = 2, 19, 8, 4
    x, w = torch.randn(B, T, C, generator=g), torch.randn(W, C, generator=g)
    cache, bias = torch.randn(B, W - 1, C, generator=g), torch.randn(C, generator=g)
    y, nc = BO.short_conv_silu(x, w, bias, cache, apply_silu=False)
    xx = torch.cat([cache, x], 1).transpose(1, 2)                       # [B,C,W-1+T]
    ref = F.conv1d(xx, w.t().unsqueeze(1), bias, groups=C).transpose(1, 2)
    assert torch.allclose(y, ref, atol=1e-5) and torch.equal(nc, torch.cat([cache, x], 1)[:, -(W - 1):])
    y1, nc1 = BO.short_conv_silu(x, torch.randn(1, C, generator=g), None, None, apply_silu=False)
    assert torch.equal(y1, x) and nc1.shape == (B, 0, C)
    # prefill == step-by-step decode through the cache
    c = torch.zeros(B, W - 1, C)
    rows = []
    for t in range(T):
        r, c = BO.short_conv_silu(x[:, t:t + 1], w, None, c)
        rows.append(r)
    assert torch.allclose(torch.cat(rows, 1), BO.short_conv_silu(x, w)[0], atol=1e-6)
    o, wt, gate = torch.randn(3, 5, 16, generator=g), torch.rand(16, generator=g), torch.randn(3, 5, 16, generator=g)
    yn = BO.gated_rmsnorm(o, wt, gate, eps=1e-5)
    assert torch.allclose(yn, o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + 1e-5) * wt * torch.sigmoid(gate), atol=1e-6)
    gk, bk = BO.kda_gate(torch.full((1, 1, 4), 30.0), torch.zeros(2), 2, None, torch.zeros(1, 1, 2))
    assert torch.allclose(gk, torch.full((1, 1, 2, 2), -30.0)) and torch.allclose(bk, torch.full((1, 1, 2), 0.5))


def test_block_ops_oracle_fp32_against_golden():
    """The fp32 restatement of the block steps against the committed float64 vectors."""
    import numpy as np
    from pathlib import Path
    from oracle import block_ops_oracle as BO
    G = np.load(Path(__file__).parent / "golden" / "block_ops_golden.npz")
    T_ = lambda k: torch.from_numpy(G[k])
    y, nc = BO.short_conv_silu(T_("conv.x"), T_("conv.w"), T_("conv.bias"), T_("conv.cache"))
    assert (y.double() - T_("conv.y")).abs().max() < 1e-5 and torch.equal(nc, T_("conv.new_cache"))
    g, beta = BO.gdn_gate_activations(T_("gdn_gate.a"), T_("gdn_gate.b"), T_("gdn_gate.A_log"), T_("gdn_gate.dt_bias"), True)
    assert (g.double() - T_("gdn_gate.g")).abs().max() < 1e-5 and (beta.double() - T_("gdn_gate.beta")).abs().max() < 1e-6
    gk, bk = BO.kda_gate(T_("kda_gate.g"), T_("kda_gate.A_log"), 8, T_("kda_gate.g_bias"), T_("kda_gate.beta"))
    assert (gk.double() - T_("kda_gate.g_out")).abs().max() < 1e-4 and (bk.double() - T_("kda_gate.beta_out")).abs().max() < 1e-6
    yn = BO.gated_rmsnorm(T_("norm.o").transpose(1, 2), T_("norm.w"), T_("norm.gate"), eps=1e-5)
    assert (yn.double() - T_("norm.y")).abs().max() < 1e-5
