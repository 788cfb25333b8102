"""RWKV-7 DPLR, RWKV-6 and Mamba-2 SSD scans on the GPU: against the reference's own outputs (fixtures made by running
its source, tests/golden/make_reference_vectors.py) and against the float64 oracle on seeded inputs at larger sizes.
float32 storage: max|x - ref| <= 1e-4 max(1, max|ref|) (float32 sums in another order).  bf16 storage: the inputs are
rounded to bf16 first and the float64 oracle runs on the rounded values, so only the bf16 rounding of the OUTPUT and
float32 accumulation remain: 1e-2 relative to max|ref| on outputs, 1e-4 on the float32 state."""
from pathlib import Path

import numpy as np
import pytest
import torch

import linearnexus_b200 as L
from linearnexus_b200 import _lib
from oracle import linear_recurrences_oracle as R

pytestmark = pytest.mark.gpu
VEC = np.load(Path(__file__).parent / "golden" / "reference_vectors.npz")
G = lambda case, key: torch.from_numpy(VEC[f"{case}.{key}"]).cuda()


def close(got, ref, tol=1e-4):
    got, ref = got.double().cpu(), ref.double().cpu()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    err = (got - ref).abs().max().item()
    assert err <= tol * max(1.0, ref.abs().max().item()), err


def rel(got, ref):
    got, ref = got.double().cpu(), ref.double().cpu()
    return ((got - ref).abs().max() / ref.abs().max().clamp_min(1e-30)).item()


# ---- the reference's own outputs -------------------------------------------------------------------------------

def test_dplr_matches_reference_source():
    q, k, v, a, b, gk, h0 = (G("dplr", x) for x in ("q", "k", "v", "a", "b", "gk", "h0"))
    sc = float(VEC["dplr.scale"])
    o, s = L.dplr_delta_rule_recurrent(q, k, v, a, b, gk, scale=sc, initial_state=h0)
    assert _lib.last_path() == "dplr_recurrent"
    close(o, G("dplr", "o")), close(s, G("dplr", "hT"))
    c = lambda t: t[:, :, 0]
    o1, s1 = L.dplr_delta_rule_step(c(q), c(k), c(v), c(a), c(b), c(gk), h0, scale=sc)
    close(o1, G("dplr", "o_step")), close(s1, G("dplr", "hT_step"))
    # token-major storage (transposed views of [B,T,H,D] arrays) is read in place and gives the same bits
    tr = lambda x: x.transpose(1, 2).contiguous().transpose(1, 2)
    o2, s2 = L.dplr_delta_rule_recurrent(tr(q), tr(k), tr(v), tr(a), tr(b), tr(gk), scale=sc, initial_state=h0)
    assert torch.equal(o2, o) and torch.equal(s2, s)


def test_rwkv6_matches_reference_source():
    r, k, v, w, u, h0 = (G("rwkv6", x) for x in ("r", "k", "v", "w", "u", "h0"))
    sc = float(VEC["rwkv6.scale"])
    o, s = L.rwkv6_recurrent(r, k, v, w, u, scale=sc, initial_state=h0)
    assert _lib.last_path() == "rwkv6_recurrent"
    close(o, G("rwkv6", "o")), close(s, G("rwkv6", "hT"))
    o2, s2 = L.rwkv6_chunkwise(r, k, v, w, u, scale=sc, initial_state=h0, chunk_size=16)
    assert torch.equal(o2, o) and torch.equal(s2, s)
    c = lambda t: t[:, :, 0]
    o1, s1 = L.rwkv6_step(c(r), c(k), c(v), c(w), u, h0, scale=sc)
    close(o1, G("rwkv6", "o_step")), close(s1, G("rwkv6", "hT_step"))


def test_ssd_matches_reference_source():
    x, dt, A, Bm, Cm, D, bias, h0 = (G("ssd", n) for n in ("x", "dt", "A", "B", "C", "D", "dt_bias", "h0"))
    lim = tuple(float(t) for t in VEC["ssd.dt_limit"])
    kw = dict(n_groups=int(VEC["ssd.groups"]), dt_bias=bias, dt_limit=lim)
    y, s = L.ssd_chunk_scan(x, dt, A, Bm, Cm, D, chunk_size=int(VEC["ssd.chunk"]), ssm_state=h0, **kw)
    assert _lib.last_path() == "ssd_scan"
    close(y, G("ssd", "y")), close(s, G("ssd", "hT"))
    y1, s1 = L.ssd_recurrent_step(x[:, 0], dt[:, 0], A, Bm[:, 0], Cm[:, 0], D, h0, **kw)
    close(y1, G("ssd", "y_step")), close(s1, G("ssd", "hT_step"))


# ---- what the reference's tests assert (tests/test_rwkv6.py, tests/test_rwkv7.py, tests/test_mamba2.py) -----------

def _randn(gen, *s, scale=1.0):
    return torch.randn(*s, generator=gen) * scale


def test_rwkv6_reference_test_properties():
    gen = torch.Generator().manual_seed(0)
    B, H, T, K = 2, 2, 8, 16
    r, k, v = (_randn(gen, B, H, T, K).cuda() for _ in range(3))
    w = -_randn(gen, B, H, T, K).abs().cuda()
    u = _randn(gen, H, K).cuda()
    o, s = L.rwkv6_recurrent(r, k, v, w, u)
    assert o.shape == (B, H, T, K) and s.shape == (B, H, K, K) and torch.isfinite(o).all() and torch.isfinite(s).all()
    o_init, _ = L.rwkv6_recurrent(r, k, v, w, u, initial_state=_randn(gen, B, H, K, K).cuda())
    assert not torch.allclose(o, o_init, rtol=1e-4)
    # one step == the recurrence at T = 1 (tests/test_rwkv6.py: test_step_matches_first_recurrent_step)
    z = torch.zeros(B, H, K, K, device="cuda")
    o1, s1 = L.rwkv6_step(r[:, :, 0], k[:, :, 0], v[:, :, 0], w[:, :, 0], u, z)
    oT, sT = L.rwkv6_recurrent(r[:, :, :1], k[:, :, :1], v[:, :, :1], w[:, :, :1], u)
    assert torch.allclose(o1, oT[:, :, 0], rtol=1e-4) and torch.allclose(s1, sT, rtol=1e-4)
    # decay = exp(-exp(w)): w = -10 forgets less than w = -0.1 (test_decay_behavior)
    _, weak = L.rwkv6_recurrent(r, k, v, torch.full_like(w, -10.0), u)
    _, strong = L.rwkv6_recurrent(r, k, v, torch.full_like(w, -0.1), u)
    assert weak.norm() > strong.norm()


def test_dplr_step_chain_equals_recurrence_and_inplace():
    gen = torch.Generator().manual_seed(1)
    B, H, T, K, V = 2, 3, 6, 16, 24
    q, k, a, b = (_randn(gen, B, H, T, K, scale=0.5).cuda() for _ in range(4))
    v = _randn(gen, B, H, T, V).cuda()
    gk = -_randn(gen, B, H, T, K).abs().cuda()
    h0 = _randn(gen, B, H, K, V, scale=0.1).cuda()
    o, s = L.dplr_delta_rule_recurrent(q, k, v, a, b, gk, initial_state=h0)
    S = h0.clone()
    for t in range(T):
        ot, S2 = L.dplr_delta_rule_step(q[:, :, t], k[:, :, t], v[:, :, t], a[:, :, t], b[:, :, t], gk[:, :, t], S, inplace=True)
        assert S2.data_ptr() == S.data_ptr()
        close(ot, o[:, :, t], 1e-5)
    close(S, s, 1e-5)


def test_ssd_reference_test_properties():
    # tests/test_mamba2.py: constant inputs, chunk 8, shapes; an initial state changes the final state
    Bt, T, H, P, N = 2, 16, 4, 32, 64
    dev = "cuda"
    x, dt = torch.ones(Bt, T, H, P, device=dev), torch.full((Bt, T, H), 0.1, device=dev)
    A, D = -torch.ones(H, device=dev), torch.ones(H, device=dev)
    Bm = Cm = torch.ones(Bt, T, 1, N, device=dev)
    y, s = L.ssd_chunk_scan(x, dt, A, Bm, Cm, D, chunk_size=8, n_groups=1)
    assert y.shape == (Bt, T, H, P) and s.shape == (Bt, H, P, N)
    ry, rs = R.ssd_chunk_scan(x.cpu(), dt.cpu(), A.cpu(), Bm.cpu(), Cm.cpu(), D.cpu(), chunk_size=8, compute_dtype=torch.float64)
    close(y, ry), close(s, rs)
    init = torch.full((Bt, H, P, N), 0.5, device=dev)
    _, s2 = L.ssd_chunk_scan(x[:, :8], dt[:, :8], A, Bm[:, :8], Cm[:, :8], D, chunk_size=8, ssm_state=init)
    assert not torch.allclose(s2, init)
    y0, s0 = L.ssd_chunk_scan(x[:, :0], dt[:, :0], A, Bm[:, :0], Cm[:, :0], D, ssm_state=init)   # empty sequence
    assert y0.shape == (Bt, 0, H, P) and torch.equal(s0, init)


# ---- larger seeded cases against the float64 oracle --------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("K,V", [(64, 64), (128, 128), (40, 72)])
def test_dplr_against_float64_oracle(dtype, K, V):
    gen = torch.Generator().manual_seed(K + V)
    B, H, T = 2, 3, 200
    rd = lambda t: t.to(dtype)
    q, k = rd(_randn(gen, B, H, T, K)), rd(_randn(gen, B, H, T, K, scale=0.5))
    kk = torch.nn.functional.normalize(_randn(gen, B, H, T, K), dim=-1)
    a, b = rd(-kk), rd(kk * torch.sigmoid(_randn(gen, B, H, T, K)))
    v, gk = rd(_randn(gen, B, H, T, V)), rd(-torch.exp(_randn(gen, B, H, T, K) - 1.0))
    h0 = _randn(gen, B, H, K, V, scale=0.1)
    sc = K ** -0.5
    o, s = L.dplr_delta_rule_recurrent(*(t.cuda() for t in (q, k, v, a, b, gk)), scale=sc, initial_state=h0.cuda())
    assert o.dtype == dtype and s.dtype == torch.float32
    ro, rs = R.dplr_delta_rule_recurrent(*(t.double() for t in (q, k, v, a, b, gk)), scale=sc, initial_state=h0,
                                         compute_dtype=torch.float64)
    assert rel(o, ro) <= (1e-4 if dtype == torch.float32 else 1e-2)
    assert rel(s, rs) <= 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("K,V", [(64, 64), (128, 128), (24, 100)])
def test_rwkv6_against_float64_oracle(dtype, K, V):
    gen = torch.Generator().manual_seed(K + V + 1)
    B, H, T = 2, 3, 200
    rd = lambda t: t.to(dtype)
    r, k, v = rd(_randn(gen, B, H, T, K)), rd(_randn(gen, B, H, T, K, scale=0.5)), rd(_randn(gen, B, H, T, V))
    w = rd(-_randn(gen, B, H, T, K).abs() - 0.5)
    u, h0 = _randn(gen, H, K, scale=0.5), _randn(gen, B, H, K, V, scale=0.1)
    o, s = L.rwkv6_recurrent(r.cuda(), k.cuda(), v.cuda(), w.cuda(), u.cuda(), scale=K ** -0.5, initial_state=h0.cuda())
    assert o.dtype == dtype and s.dtype == torch.float32
    ro, rs = R.rwkv6_recurrent(r.double(), k.double(), v.double(), w.double(), u.double(), scale=K ** -0.5,
                               initial_state=h0, compute_dtype=torch.float64)
    assert rel(o, ro) <= (1e-4 if dtype == torch.float32 else 1e-2)
    assert rel(s, rs) <= 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,P,N,G", [(8, 64, 128, 1), (6, 32, 64, 3), (4, 40, 20, 4)])
def test_ssd_against_float64_oracle(dtype, H, P, N, G):
    gen = torch.Generator().manual_seed(H + P + N)
    Bt, T = 2, 300
    rd = lambda t: t.to(dtype)
    x, Bm, Cm = rd(_randn(gen, Bt, T, H, P)), rd(_randn(gen, Bt, T, G, N, scale=0.5)), rd(_randn(gen, Bt, T, G, N, scale=0.5))
    dt = _randn(gen, Bt, T, H, scale=0.5)
    A, D, bias = -torch.exp(_randn(gen, H, scale=0.5)), _randn(gen, H), _randn(gen, H, scale=0.3)
    h0 = _randn(gen, Bt, H, P, N, scale=0.1)
    kw = dict(n_groups=G, dt_bias=bias, dt_limit=(0.001, 5.0))
    y, s = L.ssd_chunk_scan(x.cuda(), dt.cuda(), A.cuda(), Bm.cuda(), Cm.cuda(), D.cuda(), chunk_size=64,
                            ssm_state=h0.cuda(), n_groups=G, dt_bias=bias.cuda(), dt_limit=(0.001, 5.0))
    assert y.dtype == dtype and s.dtype == torch.float32 and s.shape == (Bt, H, P, N)
    ry, rs = R.ssd_chunk_scan(x.double(), dt.double(), A.double(), Bm.double(), Cm.double(), D.double(), chunk_size=64,
                              ssm_state=h0, compute_dtype=torch.float64, **kw)
    assert rel(y, ry) <= (1e-4 if dtype == torch.float32 else 1e-2)
    assert rel(s, rs) <= 1e-4


def test_bad_arguments_raise():
    z = torch.zeros(1, 2, 4, 8, device="cuda")
    with pytest.raises(ValueError):
        L.rwkv6_recurrent(z, z, z, z, torch.zeros(3, 8, device="cuda"))
    with pytest.raises(ValueError):
        L.dplr_delta_rule_recurrent(z, z, z, z, z[:, :, :2], z)
    with pytest.raises(RuntimeError):
        L.rwkv6_recurrent(z.cpu(), z.cpu(), z.cpu(), z.cpu(), torch.zeros(2, 8))
    with pytest.raises(ValueError):
        L.ssd_chunk_scan(torch.zeros(1, 4, 3, 8, device="cuda"), torch.zeros(1, 4, 3, device="cuda"), torch.zeros(3, device="cuda"),
                         torch.zeros(1, 4, 2, 8, device="cuda"), torch.zeros(1, 4, 2, 8, device="cuda"), torch.zeros(3, device="cuda"),
                         n_groups=2)


def test_rwkv6_token_major_views_give_the_same_bits():
    r, k, v, w, u, h0 = (G("rwkv6", x) for x in ("r", "k", "v", "w", "u", "h0"))
    tr = lambda x: x.transpose(1, 2).contiguous().transpose(1, 2)
    o, s = L.rwkv6_recurrent(r, k, v, w, u, scale=0.5, initial_state=h0)
    o2, s2 = L.rwkv6_recurrent(tr(r), tr(k), tr(v), tr(w), u, scale=0.5, initial_state=h0)
    assert torch.equal(o2, o) and torch.equal(s2, s)
    assert not o2.is_contiguous() and o2.transpose(1, 2).is_contiguous()   # the output keeps the inputs' storage order
