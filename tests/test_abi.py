"""CPU tests of the drop-in boundary: the library loads, exports every symbol the header
declares, and host-side validation returns the documented status codes (no kernel runs)."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

import linearnexus_b200 as L
from linearnexus_b200 import _lib

ROOT = Path(__file__).resolve().parents[1]


def _header_functions():
    text = "".join(p.read_text() for p in sorted((ROOT / "include").glob("*.h")))
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dr_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = _header_functions()
    assert set(_lib.EXPORTS) <= set(names)
    for n in names:
        assert hasattr(lib, n), n
    assert b"sm_100a" in lib.dr_version()


def test_desc_struct_matches_header():
    assert ctypes.sizeof(_lib.DrDesc) == 16 * 4


def _desc(**kw):
    d = _lib.DrDesc()
    d.variant, d.layout, d.B, d.H, d.T, d.K, d.V, d.chunk = 1, 0, 1, 1, 64, 128, 128, 64
    d.qkv_dtype = d.g_dtype = d.out_dtype = 0
    d.scale = 1.0
    for k, v in kw.items():
        setattr(d, k, v)
    return d


def test_validation_status_codes():
    lib = _lib.load()
    call = lambda d, g=8: lib.dr_chunk_fwd(ctypes.byref(d), 16, 16, 16, g, 16, None, 16, None, None, 0, None, None)
    assert lib.dr_chunk_fwd(ctypes.byref(_desc()), None, 16, 16, 16, 16, None, 16, None, None, 0, None, None) == -1
    assert call(_desc(K=130)) == -2
    assert call(_desc(V=1024)) == -2
    assert call(_desc(qkv_dtype=7)) == -3
    assert call(_desc(), g=16 + 2) == -4          # misaligned g (a scalar fp32 decay needs 4-byte alignment)
    assert call(_desc(variant=2), g=16 + 4) == -4  # per-channel decay rows are read 16 bytes at a time
    assert call(_desc(variant=0), g=16) == -6     # DeltaNet must not get g
    assert call(_desc(variant=1), g=None) == -6   # Gated DeltaNet needs g
    assert call(_desc(chunk=24), g=16) == -7      # reference: ValueError when chunk % 16 != 0
    assert call(_desc(variant=5), g=16) == -6
    assert lib.dr_step(ctypes.byref(_desc(T=2)), 16, 16, 16, 16, 16, 16, 16, 16, None, None) == -2
    assert lib.dr_workspace_bytes(ctypes.byref(_desc()), 0) == 0
    for s in range(-11, 1):
        assert lib.dr_strerror(s)
    assert lib.dr_check_status(None, None) == -1            # the status word is required
    assert lib.dr_debug_wait_timeout(None, 16, None) == -1
    assert lib.dr_debug_wait_timeout(16, 0, None) == -2     # attempts out of range, refused before any launch
    assert lib.dr_debug_wait_site(None, 1, 1, None) == -1
    assert lib.dr_debug_wait_site(16, 64, 0, None) == -2 and lib.dr_debug_wait_site(16, 0, 4, None) == -2


def test_device_status_maps_to_an_exception():
    """Host side of the status word: DR_ERR_DEVICE becomes a DeltaRuleError that names the DR_DEV_* bits."""
    with pytest.raises(_lib.DeltaRuleError) as ei:
        _lib.check(-10, "dr_check_status")
    assert ei.value.status == -10 and "device-side" in str(ei.value)


def test_status_word_names_where_a_wait_gave_up():
    """Bits 8..15 of the status word: barrier number (6 bits) and warp group (2 bits) of the first wait that ran out."""
    assert _lib.device_status_site(0) is None
    assert _lib.device_status_site(2) is None                      # an index check alone carries no site
    assert _lib.device_status_site(0x9701) == (23, 2)              # barrier 23 of the control block, third group
    assert _lib.device_status_site(0x0001 | (63 << 8) | (3 << 14)) == (63, 3)


def test_two_kernel_forward_without_workspace_is_an_error_not_a_downgrade():
    """KDA at the tensor-core shape resolves to the two-kernel path; a call that brings no workspace gets
    DR_ERR_WORKSPACE whether the path was chosen by AUTO or by name (validation only: nothing is launched)."""
    import torch
    from linearnexus_b200 import ops
    lib = _lib.load()
    q = torch.empty(0, dtype=torch.bfloat16)
    g = torch.empty(0, dtype=torch.float32)
    for path in (None, "split"):
        d = ops._desc(_lib.DR_KDA, _lib.DR_LAYOUT_BHTD, 1, 1, 64, 128, 128, 64, q, g, torch.float32, True, 0.1, path)
        assert lib.dr_chunk_fwd(ctypes.byref(d), 16, 16, 16, 16, 16, None, 16, None, None, 0, None, None) == -5
    d = ops._desc(_lib.DR_KDA, _lib.DR_LAYOUT_BHTD, 1, 1, 64, 128, 128, 64, q, g, torch.float32, True, 0.1, "split")
    assert lib.dr_chunk_fwd(ctypes.byref(d), 16, 16, 16, 16, 16, None, 16, None, 24, 1 << 30, None, None) == -4


def test_ops_refuse_cpu_tensors():
    q = torch.randn(1, 1, 16, 16)
    with pytest.raises(RuntimeError, match="CUDA"):
        L.gated_delta_rule_chunkwise(q, q, q, torch.zeros(1, 1, 16), torch.ones(1, 1, 16))
    with pytest.raises(RuntimeError):
        L.delta_rule_recurrent_pallas(q, q, q, torch.ones(1, 1, 16))


def test_backend_selection_is_single_backend():
    assert L.select_kernel_backend(None) == L.KernelBackend.SM100
    assert L.select_kernel_backend("pallas") == L.KernelBackend.SM100
    assert L.select_kernel_backend("reference") == L.KernelBackend.SM100
    with pytest.raises(ValueError):
        L.select_kernel_backend("tpu")


def test_state_factories_cpu():
    s = L.GatedDeltaNetState.zeros(2, 4, 16, 32, key_dim_total=64, value_dim=128, device="cpu")
    assert s.S.shape == (2, 4, 16, 32) and s.S.dtype == torch.float32
    assert s.conv_state_q.shape == (2, 3, 64) and s.conv_state_v.shape == (2, 3, 128)
    s = L.KDAState.zeros(2, 4, 16, 32, device="cpu")
    assert s.conv_state_q is None
    s = L.DeltaNetState.zeros(2, 4, 16, 32, conv_channels=64, device="cpu")
    assert s.conv_state.shape == (2, 3, 64)


def test_forward_workspace_sizes_need_no_gpu():
    """dr_workspace_bytes(desc, 0): one 82 432-byte record per (sequence, 64-token chunk) for the two-kernel
    forward (KDA by default, any variant when asked for), nothing for the kernels that need no scratch."""
    import ctypes
    import torch
    from linearnexus_b200 import ops
    lib = _lib.load()
    q = torch.empty(0, dtype=torch.bfloat16)
    g = torch.empty(0, dtype=torch.float32)
    def need(variant, path, B=2, H=3, T=130, K=128, V=128, qkv=q):
        d = ops._desc(variant, _lib.DR_LAYOUT_BHTD, B, H, T, K, V, 64, qkv, g, torch.float32, True, 0.1, path)
        return int(lib.dr_workspace_bytes(ctypes.byref(d), 0))
    assert need(_lib.DR_KDA, None) == 2 * 3 * 3 * 82432
    assert need(_lib.DR_KDA, "fp32") == 0
    assert need(_lib.DR_GATED, None) == 0
    assert need(_lib.DR_GATED, "split") == 2 * 3 * 3 * 82432
    assert need(_lib.DR_KDA, None, K=64) == 0                      # not the tensor-core shape: fp32 kernel
    assert need(_lib.DR_KDA, None, qkv=torch.empty(0)) == 0        # fp32 inputs stay on the exact kernel


def test_grouped_head_count_is_validated_on_the_host():
    """DrDesc.qk_heads: 0 or a divisor of H; anything else is a shape error before any launch."""
    import ctypes
    import torch
    from linearnexus_b200 import ops
    lib = _lib.load()
    q = torch.empty(0, dtype=torch.bfloat16)
    g = torch.empty(0, dtype=torch.float32)
    def status(qk_heads):
        d = ops._desc(_lib.DR_GATED, _lib.DR_LAYOUT_BHTD, 2, 6, 64, 128, 128, 64, q, g, torch.bfloat16, True, 0.1, None)
        d.qk_heads = qk_heads
        return int(lib.dr_workspace_bytes(ctypes.byref(d), 0))
    assert status(0) == 0 and status(6) == 0 and status(2) == 0 and status(1) == 0
    assert status(4) == -2 and status(12) == -2 and status(-1) == -2


def test_host_pipeline_argument_checks_need_no_gpu():
    import pytest
    import torch
    from linearnexus_b200 import host_pipeline
    host_pipeline._pinned(None, "g")
    with pytest.raises(ValueError):
        host_pipeline._pinned(torch.zeros(4), "q")          # pageable host memory


def test_block_op_entry_points_validate_on_the_host():
    """Bad arguments of the conv / gate / norm entry points are refused before any CUDA call."""
    lib = _lib.load()
    buf = ctypes.create_string_buffer(256)
    p = ctypes.cast(buf, ctypes.c_void_p)
    al = ctypes.c_void_p((p.value + 15) & ~15)
    assert lib.dr_short_conv_silu(None, al, None, None, al, None, 1, 1, 8, 4, 1, 1, None) == -1
    assert lib.dr_short_conv_silu(al, al, None, None, ctypes.c_void_p(al.value + 16), None, 1, 1, 12, 4, 1, 1, None) == -2
    assert lib.dr_short_conv_silu(al, al, None, None, ctypes.c_void_p(al.value + 16), None, 1, 1, 8, 9, 1, 1, None) == -2
    assert lib.dr_short_conv_silu(al, al, None, None, al, None, 1, 1, 8, 4, 1, 1, None) == -9      # in place
    assert lib.dr_short_conv_silu(al, al, None, None, ctypes.c_void_p(al.value + 8), None, 1, 1, 8, 4, 1, 1, None) == -4
    y = ctypes.c_void_p(al.value + 64)
    w4 = ctypes.c_void_p(al.value + 4)        # the taps and the bias are read as float4: 4-byte alignment is not enough
    assert lib.dr_short_conv_silu(al, w4, None, None, y, None, 1, 1, 8, 4, 1, 1, None) == -4
    assert lib.dr_short_conv_silu(al, al, w4, None, y, None, 1, 1, 8, 4, 1, 1, None) == -4
    assert lib.dr_short_conv_silu(al, w4, None, None, y, None, 1, 1, 8, 1, 1, 1, None) != -4     # W == 1: weight unused
    assert lib.dr_gate_activations(2, al, None, al, None, al, None, 1, 1, 1, 1, 0, 0, 1.0, 20.0, None) == -6
    assert lib.dr_gate_activations(0, al, None, al, None, al, None, 1, 1, 1, 4, 0, 0, 1.0, 20.0, None) == -2
    assert lib.dr_gate_activations(0, al, al, al, None, al, None, 1, 1, 1, 1, 0, 0, 1.0, 20.0, None) == -1
    assert lib.dr_gated_rmsnorm(al, None, al, al, 1, 1, 1, 6, 0, 0, 0, 0, 1e-6, None) == -2
    assert lib.dr_gated_rmsnorm(al, None, al, al, 1, 1, 1, 8, 0, 7, 0, 0, 1e-6, None) == -3
    assert lib.dr_gated_rmsnorm(al, None, al, al, 1, 1, 1, 8, 0, 0, 0, 0, 1e-6, None) == -9        # in place, transposing
