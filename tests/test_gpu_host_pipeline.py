"""GPU tests of the host-memory entry point (batch slices, copies and kernels overlapped on three streams):
its results are those of the plain op on the same rows."""
import pytest
import torch

import linearnexus_b200 as L
from oracle import delta_rule_oracle as O

pytestmark = pytest.mark.gpu


def _pin(inp):
    return {k: (None if v is None else v.contiguous().pin_memory()) for k, v in inp.items()}


@pytest.mark.parametrize("variant,slices", [("gated", None), ("gated", 2), ("kda", 3), ("delta", 1)])
def test_from_host_equals_device_op(variant, slices):
    inp = O.make_inputs(variant, 3, 2, 200, 128, 128, seed=11, io_dtype=torch.bfloat16, h0_std=0.02)
    pin = _pin(inp)
    o, hT = L.chunkwise_from_host(variant, pin["q"], pin["k"], pin["v"], pin["g"], pin["beta"],
                                  initial_state=pin["h0"], slices=slices, chunk_size=64)
    assert not o.is_cuda and o.is_pinned() and hT.is_pinned()
    cu = {k: (None if v is None else v.cuda()) for k, v in inp.items()}
    if variant == "gated":
        ro, rS = L.gated_delta_rule_chunkwise(cu["q"], cu["k"], cu["v"], cu["g"], cu["beta"], initial_state=cu["h0"])
    elif variant == "kda":
        ro, rS = L.kda_chunkwise(cu["q"], cu["k"], cu["v"], cu["g"], cu["beta"], initial_state=cu["h0"])
    else:
        ro, rS = L.delta_rule_chunkwise(cu["q"], cu["k"], cu["v"], cu["beta"], cu["h0"])
    assert o.dtype == ro.dtype
    assert torch.equal(o, ro.cpu()) and torch.equal(hT, rS.cpu())


def test_from_host_reuses_caller_buffers_and_checks_arguments():
    inp = O.make_inputs("gated", 2, 2, 64, 128, 128, seed=3, io_dtype=torch.bfloat16)
    pin = _pin(inp)
    out = torch.empty(2, 2, 64, 128, dtype=torch.bfloat16).pin_memory()
    st = torch.empty(2, 2, 128, 128).pin_memory()
    o, hT = L.chunkwise_from_host("gated", pin["q"], pin["k"], pin["v"], pin["g"], pin["beta"], out=out, final_state=st)
    assert o.data_ptr() == out.data_ptr() and hT.data_ptr() == st.data_ptr()
    with pytest.raises(ValueError):
        L.chunkwise_from_host("gated", inp["q"], pin["k"], pin["v"], pin["g"], pin["beta"])   # q not pinned
    with pytest.raises(ValueError):
        L.chunkwise_from_host("gated", pin["q"].cuda(), pin["k"], pin["v"], pin["g"], pin["beta"])
    with pytest.raises(ValueError):
        L.chunkwise_from_host("delta", pin["q"], pin["k"], pin["v"], pin["g"], pin["beta"])   # g given for delta
