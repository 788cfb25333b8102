"""The device status word: a bounded wait that runs out is reported to the host instead of trapping or hanging.

The failing wait is made in the allowed form only: a kernel waits, with the library's own bounded wait
limited to a few attempts, on an mbarrier that nothing ever arrives on.  It gives up, sets DR_DEV_TIMEOUT
and returns; the context stays usable and the next launch on the same GPU is correct."""
import ctypes

import pytest
import torch

import linearnexus_b200 as L
from linearnexus_b200 import _lib, ops
from oracle import delta_rule_oracle as O

pytestmark = pytest.mark.gpu


def test_wait_that_runs_out_sets_status_and_host_raises():
    lib = _lib.load()
    dev = torch.device("cuda", torch.cuda.current_device())
    ops.check_device_status()                       # clean to start with
    word = ops._status(dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    st = lib.dr_debug_wait_timeout(ctypes.c_void_p(word.data_ptr()), 32, stream)
    assert st == 0
    with pytest.raises(_lib.DeltaRuleError) as ei:
        ops.check_device_status()
    assert ei.value.status == -10 and "bounded wait" in str(ei.value)
    assert lib.dr_last_device_status() == 1         # DR_DEV_TIMEOUT
    assert word.item() == 0                         # reported once, then cleared
    ops.check_device_status()
    # the context is intact: the next launches are correct and leave the word clean
    inp = O.make_inputs("gated", 1, 2, 192, 128, 128, seed=5, io_dtype=torch.bfloat16, h0_std=0.02)
    cu = {k: (None if v is None else v.cuda()) for k, v in inp.items()}
    o, hT = L.gated_delta_rule_chunkwise(cu["q"], cu["k"], cu["v"], cu["g"], cu["beta"], initial_state=cu["h0"])
    ops.check_device_status()
    ro, rS = O.gated_delta_rule_recurrent(*(inp[x].double() for x in ("q", "k", "v", "g", "beta")),
                                          initial_state=inp["h0"].double(), compute_dtype=torch.float64)
    assert ((o.double().cpu() - ro).abs().max() / ro.abs().max()).item() <= 2e-2
    assert ((hT.double().cpu() - rS).abs().max() / rS.abs().max()).item() <= 2e-2


def test_the_status_word_names_the_wait_that_gave_up():
    """The wait routine of the tcgen05 kernels, run to the end of its bound (about a second) on an mbarrier that
    nothing arrives on: DR_DEV_TIMEOUT plus the barrier number and warp group of that wait in bits 8..15; a second
    wait of the same CTA returns at once and leaves the record alone; the context stays usable."""
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    ops.check_device_status()
    word = ops._status(dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.dr_debug_wait_site(ctypes.c_void_p(word.data_ptr()), 23, 2, stream) == 0
    with pytest.raises(_lib.DeltaRuleError) as ei:
        ops.check_device_status()
    bits = lib.dr_last_device_status()
    assert bits & 1 and _lib.device_status_site(bits) == (23, 2)
    assert "barrier 23 of warp group 2" in str(ei.value)
    ops.check_device_status()                       # cleared
    x = torch.arange(8, device=dev).sum().item()    # the context is intact
    assert x == 28


def test_every_op_family_passes_the_status_word_and_leaves_it_clean():
    """Forward (fused, two-kernel, fp32), decode (streamed and per-unit kernel) and training pair all run with a
    live status word; none of them reports anything on healthy inputs."""
    inp = O.make_inputs("kda", 1, 2, 128, 128, 128, seed=6, io_dtype=torch.bfloat16, h0_std=0.02)
    cu = {k: (None if v is None else v.cuda()) for k, v in inp.items()}
    L.kda_chunkwise(cu["q"], cu["k"], cu["v"], cu["g"], cu["beta"], initial_state=cu["h0"])
    L.kda_recurrent(cu["q"], cu["k"], cu["v"], cu["g"], cu["beta"], initial_state=cu["h0"])
    B, H = 16, 32   # enough units for the streamed decode kernel
    S = torch.randn(B, H, 128, 128, device="cuda") * 0.02
    q = torch.randn(B, H, 128, device="cuda", dtype=torch.bfloat16)
    g = -torch.rand(B, H, device="cuda")
    beta = torch.rand(B, H, device="cuda")
    L.gated_delta_rule_step(q, q, q, g, beta, S, inplace=True)
    assert _lib.last_path() == "step_stream"
    L.gated_delta_rule_step(q[:1, :2], q[:1, :2], q[:1, :2], g[:1, :2], beta[:1, :2], S[:1, :2].contiguous())
    assert _lib.last_path() == "step"
    gi = O.make_inputs("gated", 1, 2, 128, 128, 128, seed=7, io_dtype=torch.bfloat16)
    gc = {k: (None if v is None else v.cuda()) for k, v in gi.items()}
    o, hT, saved = ops.chunk_forward_saving("gated", gc["q"], gc["k"], gc["v"], gc["g"], gc["beta"])
    ops.chunk_backward("gated", gc["q"], gc["k"], gc["v"], gc["g"], gc["beta"], torch.ones_like(o), saved=saved)
    ops.check_device_status()
