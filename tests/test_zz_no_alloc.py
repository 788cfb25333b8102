"""dr_chunk_bwd_static: the backward for callers that cannot allocate a workspace.

Some hosts of this library have no allocator to offer at call time -- a compiled runtime that
planned all of its buffers ahead and owns the rest of the GPU, or a plug-in that must leave its
framework's memory pool alone.  For them the library carries a fixed 32 MiB scratch array of its
own.  This test drives that entry point straight through the C ABI, twice in a row (the array is
shared between calls and still holds the first call's data when the second starts), and requires
the same gradients as the regular entry point with a caller-provided workspace.  It also checks
that a request larger than the built-in array is refused instead of overrunning it.  The file is
named so that pytest collects it after every other test.
"""
import ctypes

import pytest
import torch

from linearnexus_b200 import _lib
from oracle import delta_rule_oracle as O

pytestmark = pytest.mark.gpu
STATIC_BYTES = 32 << 20


def _vp(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _desc(B, H, T, K, V, C):
    d = _lib.DrDesc()
    d.variant, d.layout = _lib.DR_GATED, _lib.DR_LAYOUT_BHTD
    d.B, d.H, d.T, d.K, d.V, d.chunk = B, H, T, K, V, C
    d.qkv_dtype = d.g_dtype = d.out_dtype = _lib.DR_F32
    d.use_qk_l2norm, d.scale = 1, K ** -0.5
    return d


def _inputs(B, H, T, K, V, seed):
    inp = O.make_inputs("gated", B, H, T, K, V, seed=seed, h0_std=0.1)
    gen = torch.Generator().manual_seed(seed)
    inp["do"] = torch.randn(B, H, T, V, generator=gen)
    inp["dhT"] = torch.randn(B, H, K, V, generator=gen) * 0.1
    return {k: v.cuda().contiguous() for k, v in inp.items()}


def _outputs(B, H, T, K, V):
    mk = lambda *s: torch.full(s, float("nan"), device="cuda")
    return dict(dq=mk(B, H, T, K), dk=mk(B, H, T, K), dv=mk(B, H, T, V), dbeta=mk(B, H, T), dg=mk(B, H, T), dh0=mk(B, H, K, V))


def _run(lib, d, x, static):
    B, H, T, K, V = d.B, d.H, d.T, d.K, d.V
    out = _outputs(B, H, T, K, V)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    head = [ctypes.byref(d), _vp(x["q"]), _vp(x["k"]), _vp(x["v"]), _vp(x["g"]), _vp(x["beta"]), _vp(x["h0"]),
            _vp(x["do"]), _vp(x["dhT"]), _vp(out["dq"]), _vp(out["dk"]), _vp(out["dv"]), _vp(out["dbeta"]),
            _vp(out["dg"]), _vp(out["dh0"])]
    if static:
        st = lib.dr_chunk_bwd_static(*head, None, stream)
    else:
        need = lib.dr_workspace_bytes(ctypes.byref(d), 1)
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        st = lib.dr_chunk_bwd(*head, _vp(ws), need, None, stream)
    torch.cuda.synchronize()
    return st, out


def test_static_scratch_backward_matches_workspace_backward_twice():
    lib = _lib.load()
    # two different problems back to back: the second call finds the first call's leftovers in the array
    for (B, H, T, K, V, C, seed) in [(2, 2, 200, 64, 64, 64, 1), (1, 3, 96, 32, 48, 32, 2)]:
        d = _desc(B, H, T, K, V, C)
        assert 0 < lib.dr_workspace_bytes(ctypes.byref(d), 1) <= STATIC_BYTES
        x = _inputs(B, H, T, K, V, seed)
        st_ref, ref = _run(lib, d, x, static=False)
        st_new, got = _run(lib, d, x, static=True)
        assert st_ref == 0 and st_new == 0, (st_ref, st_new, lib.dr_strerror(st_new))
        assert _lib.last_path() == "bwd_static"
        for name in ref:
            assert torch.isfinite(got[name]).all(), name
            denom = ref[name].abs().max().clamp_min(1e-30)
            # same kernels on the same inputs; the only run-to-run difference is the order of fp32 atomic adds
            assert ((got[name] - ref[name]).abs().max() / denom).item() <= 2e-4, name


def test_static_scratch_backward_bf16_tensor_core_shape_against_the_oracle():
    """K = V = 128, bf16: the saving forward on tcgen05, the pre-pass and the tensor-core adjoint all work out of
    the built-in array.  Checked against the float64 autograd of the recurrence (2e-2 relative, the bf16 bar),
    not only against the workspace entry point."""
    lib = _lib.load()
    B, H, T, K, V = 1, 2, 256, 128, 128
    d = _desc(B, H, T, K, V, 64)
    d.qkv_dtype = d.out_dtype = _lib.DR_BF16
    assert 0 < lib.dr_workspace_bytes(ctypes.byref(d), 1) <= STATIC_BYTES
    inp = O.make_inputs("gated", B, H, T, K, V, seed=9, io_dtype=torch.bfloat16, h0_std=0.02)
    gen = torch.Generator().manual_seed(9)
    inp["do"] = torch.randn(B, H, T, V, generator=gen).bfloat16()
    inp["dhT"] = torch.randn(B, H, K, V, generator=gen) * 0.1
    x = {k: v.cuda().contiguous() for k, v in inp.items()}
    ref = O.delta_rule_grads("gated", inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], inp["h0"], inp["do"], inp["dhT"])
    for _ in range(2):   # twice in a row: the second call finds the first call's leftovers in the array
        mk = lambda *s, dt=torch.float32: torch.full(s, float("nan"), device="cuda", dtype=dt)
        out = dict(dq=mk(B, H, T, K, dt=torch.bfloat16), dk=mk(B, H, T, K, dt=torch.bfloat16), dv=mk(B, H, T, V, dt=torch.bfloat16),
                   dbeta=mk(B, H, T), dg=mk(B, H, T), dh0=mk(B, H, K, V))
        st = lib.dr_chunk_bwd_static(ctypes.byref(d), _vp(x["q"]), _vp(x["k"]), _vp(x["v"]), _vp(x["g"]), _vp(x["beta"]),
                                     _vp(x["h0"]), _vp(x["do"]), _vp(x["dhT"]), _vp(out["dq"]), _vp(out["dk"]), _vp(out["dv"]),
                                     _vp(out["dbeta"]), _vp(out["dg"]), _vp(out["dh0"]), None,
                                     ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        assert st == 0, lib.dr_strerror(st)
        for name in out:
            got, want = out[name].double().cpu(), ref[name].double()
            assert torch.isfinite(got).all(), name
            assert ((got - want).abs().max() / want.abs().max()).item() <= 2e-2, name


def test_static_scratch_limit_is_enforced():
    lib = _lib.load()
    d = _desc(8, 16, 4096, 128, 128, 64)  # needs hundreds of MiB of scratch
    assert lib.dr_workspace_bytes(ctypes.byref(d), 1) > STATIC_BYTES
    one = torch.zeros(64, device="cuda")
    p = _vp(one)
    st = lib.dr_chunk_bwd_static(ctypes.byref(d), p, p, p, p, p, None, p, None, p, p, p, p, p, None, None, None)
    assert st == -11
    assert b"static" in lib.dr_strerror(st)
