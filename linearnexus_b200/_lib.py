"""Loader and ctypes bindings for ``libdeltarule_sm100.so`` (the C ABI in include/deltarule_sm100.h).

The library is built in-tree by :func:`build_library` (``nvcc`` for sm_100a) and loaded from
the package directory.  There is no fallback: if the shared object is missing or a call
fails, an exception is raised.
"""

from __future__ import annotations

import ctypes
import os
import subprocess
import threading
from pathlib import Path

_PKG = Path(__file__).resolve().parent
_ROOT = _PKG.parent
# DELTARULE_SM100_LIB points the loader at another build of the same library (profiling builds).
LIB_PATH = Path(os.environ.get("DELTARULE_SM100_LIB", _PKG / "libdeltarule_sm100.so"))
# the same sources with the index checks compiled in (-DDR_BOUNDS_CHECK); tests load it through DELTARULE_SM100_LIB
BOUNDS_LIB_PATH = _PKG / "libdeltarule_sm100_bounds.so"
_SOURCES = ["dr_api.cu", "dr_scans.cu"]   # translation units, compiled side by side
_HEADERS = sorted(f.name for f in list((_PKG / "csrc").glob("*.cuh")) + list((_PKG / "csrc").glob("*.h")))

# DrVariant / DrDtype / DrLayout / DrChunkPath (include/deltarule_sm100.h)
DR_DELTA, DR_GATED, DR_KDA = 0, 1, 2
DR_F32, DR_BF16 = 0, 1
DR_LAYOUT_BHTD, DR_LAYOUT_BTHD = 0, 1
DR_PATH_AUTO, DR_PATH_FP32, DR_PATH_TCGEN05, DR_PATH_SPLIT = 0, 1, 2, 3

# bits of the device status word (DR_DEV_* in include/deltarule_sm100.h)
DEVICE_STATUS_BITS = {1: "a bounded wait on an mbarrier ran out", 2: "an index check failed"}


def device_status_site(word: int):
    """(barrier number, warp group) of the first wait that gave up in a tcgen05 kernel, from bits 8..15 of the device
    status word (DR_DEV_SITE in include/deltarule_sm100.h); None when the word carries no timeout."""
    if not word & 1:
        return None
    site = (word >> 8) & 0xFF
    return site & 0x3F, site >> 6

EXPORTS = ["dr_version", "dr_strerror", "dr_last_cuda_error", "dr_launch_count", "dr_last_path",
           "dr_workspace_bytes", "dr_chunk_fwd", "dr_recurrent_fwd", "dr_step", "dr_chunk_bwd",
           "dr_debug_umma_selftest", "dr_chunk_bwd_static", "dr_chunk_fwd_saving", "dr_chunk_bwd_saved",
           "dr_short_conv_silu", "dr_gate_activations", "dr_gated_rmsnorm", "dr_check_status",
           "dr_last_device_status", "dr_debug_wait_timeout", "dr_chunk_fwd_varlen", "dr_dplr_recurrent",
           "dr_rwkv6_recurrent", "dr_ssd_scan", "dr_debug_bounds_checked", "dr_debug_bounds_probe", "dr_chunk_bwd_varlen", "dr_debug_wait_site"]


class DrDesc(ctypes.Structure):
    _fields_ = [
        ("variant", ctypes.c_int32), ("layout", ctypes.c_int32),
        ("B", ctypes.c_int32), ("H", ctypes.c_int32), ("T", ctypes.c_int32),
        ("K", ctypes.c_int32), ("V", ctypes.c_int32), ("chunk", ctypes.c_int32),
        ("qkv_dtype", ctypes.c_int32), ("g_dtype", ctypes.c_int32), ("out_dtype", ctypes.c_int32),
        ("use_qk_l2norm", ctypes.c_int32), ("scale", ctypes.c_float), ("path", ctypes.c_int32),
        ("qk_heads", ctypes.c_int32), ("reserved", ctypes.c_int32),
    ]


class DeltaRuleError(RuntimeError):
    """A C-ABI call returned a negative DrStatus."""

    def __init__(self, status: int, text: str, where: str):
        super().__init__(f"{where}: {text} (DrStatus {status})")
        self.status = status


def nvcc_flags() -> list[str]:
    return ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
            f"-I{_ROOT / 'include'}", f"-I{_PKG / 'csrc'}"]


def nvcc_command(out: Path | None = None, extra: list[str] | None = None) -> list[str]:
    """One nvcc invocation that compiles and links every unit (profiling builds; `build_library` compiles the units in
    parallel instead)."""
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc] + nvcc_flags() + ["-shared"] + (extra or [])
    cmd += ["-o", str(out or LIB_PATH)] + [str(_PKG / "csrc" / s) for s in _SOURCES]
    return cmd


def library_is_stale(path: Path | None = None) -> bool:
    path = path or LIB_PATH
    if not path.exists():
        return True
    t = path.stat().st_mtime
    deps = [_PKG / "csrc" / f for f in _SOURCES + _HEADERS] + list((_ROOT / "include").glob("*.h"))
    return any(d.exists() and d.stat().st_mtime > t for d in deps)


def build_library(force: bool = False, verbose: bool = False, bounds: bool = False) -> Path:
    """Compile the CUDA sources for sm_100a into the package directory (cross-compiles without a GPU): one object
    per translation unit, the units in parallel, then one link.  ``bounds=True`` builds the debug library with the
    index checks (BOUNDS_LIB_PATH) instead."""
    target = BOUNDS_LIB_PATH if bounds else LIB_PATH
    extra = ["-DDR_BOUNDS_CHECK"] if bounds else []
    if force or library_is_stale(target):
        import tempfile
        nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
        with tempfile.TemporaryDirectory(prefix="deltarule_sm100_") as tmp:
            objs, procs = [], []
            for src in _SOURCES:
                obj = Path(tmp) / (Path(src).stem + ".o")
                cmd = [nvcc] + nvcc_flags() + extra + ["-c", "-o", str(obj), str(_PKG / "csrc" / src)]
                objs.append(obj)
                procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)))
            link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(target)] + [str(o) for o in objs]
            failed = ""
            for cmd, pr in procs:
                out, err = pr.communicate()
                if verbose or pr.returncode:
                    print(" ".join(cmd))
                    print(out, err)
                if pr.returncode:
                    failed += err
            if failed:
                raise RuntimeError("nvcc failed building libdeltarule_sm100.so:\n" + failed)
            res = subprocess.run(link, capture_output=True, text=True)
            if verbose or res.returncode:
                print(" ".join(link))
                print(res.stdout, res.stderr)
            if res.returncode:
                raise RuntimeError("nvcc failed linking libdeltarule_sm100.so:\n" + res.stderr)
    return target


_lib = None
_lock = threading.Lock()


def load() -> ctypes.CDLL:
    """Load the shared library (once) and declare the argument types of every export."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                "(there is no CPU or PyTorch fallback for these ops)")
        lib = ctypes.CDLL(str(LIB_PATH))
        vp, fp, ip = ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p
        dp = ctypes.POINTER(DrDesc)
        lib.dr_version.restype = ctypes.c_char_p
        lib.dr_strerror.restype = ctypes.c_char_p
        lib.dr_strerror.argtypes = [ctypes.c_int]
        lib.dr_last_cuda_error.restype = ctypes.c_int
        lib.dr_launch_count.restype = ctypes.c_uint64
        lib.dr_last_path.restype = ctypes.c_char_p
        lib.dr_workspace_bytes.restype = ctypes.c_int64
        lib.dr_workspace_bytes.argtypes = [dp, ctypes.c_int]
        lib.dr_chunk_fwd.restype = ctypes.c_int
        lib.dr_chunk_fwd.argtypes = [dp, vp, vp, vp, vp, fp, fp, vp, fp, vp, ctypes.c_size_t, ip, vp]
        lib.dr_chunk_fwd_varlen.restype = ctypes.c_int
        lib.dr_chunk_fwd_varlen.argtypes = [dp, vp, vp, vp, vp, fp, ctypes.POINTER(ctypes.c_int32), ctypes.c_int32, fp, vp, fp,
                                            vp, ctypes.c_size_t, ip, vp]
        lib.dr_recurrent_fwd.restype = ctypes.c_int
        lib.dr_recurrent_fwd.argtypes = [dp, vp, vp, vp, vp, fp, fp, vp, fp, ip, vp]
        lib.dr_step.restype = ctypes.c_int
        lib.dr_step.argtypes = [dp, vp, vp, vp, vp, fp, fp, fp, vp, ip, vp]
        lib.dr_check_status.restype = ctypes.c_int
        lib.dr_check_status.argtypes = [ip, vp]
        lib.dr_last_device_status.restype = ctypes.c_int
        lib.dr_debug_wait_timeout.restype = ctypes.c_int
        lib.dr_debug_wait_timeout.argtypes = [ip, ctypes.c_uint32, vp]
        lib.dr_debug_wait_site.restype = ctypes.c_int
        lib.dr_debug_wait_site.argtypes = [ip, ctypes.c_uint32, ctypes.c_uint32, vp]
        lib.dr_chunk_bwd.restype = ctypes.c_int
        lib.dr_chunk_bwd.argtypes = [dp, vp, vp, vp, vp, fp, fp, vp, fp, vp, vp, vp, fp, fp, fp, vp,
                                     ctypes.c_size_t, ip, vp]
        lib.dr_chunk_bwd_varlen.restype = ctypes.c_int
        lib.dr_chunk_bwd_varlen.argtypes = [dp, vp, vp, vp, vp, fp, ctypes.POINTER(ctypes.c_int32), ctypes.c_int32, fp, vp, fp,
                                            vp, vp, vp, fp, fp, fp, vp, ctypes.c_size_t, ip, vp]
        lib.dr_chunk_bwd_static.restype = ctypes.c_int
        lib.dr_chunk_bwd_static.argtypes = [dp, vp, vp, vp, vp, fp, fp, vp, fp, vp, vp, vp, fp, fp, fp, ip, vp]
        lib.dr_chunk_fwd_saving.restype = ctypes.c_int
        lib.dr_chunk_fwd_saving.argtypes = [dp, vp, vp, vp, vp, fp, fp, vp, fp, vp, ctypes.c_size_t, ip, vp]
        lib.dr_chunk_bwd_saved.restype = ctypes.c_int
        lib.dr_chunk_bwd_saved.argtypes = [dp, vp, vp, vp, vp, fp, vp, fp, vp, vp, vp, fp, fp, fp, vp,
                                           ctypes.c_size_t, ip, vp]
        ci, cf = ctypes.c_int, ctypes.c_float
        lib.dr_short_conv_silu.restype = ctypes.c_int
        lib.dr_short_conv_silu.argtypes = [vp, fp, fp, vp, vp, vp, ci, ci, ci, ci, ci, ci, vp]
        lib.dr_gate_activations.restype = ctypes.c_int
        lib.dr_gate_activations.argtypes = [ci, vp, vp, fp, fp, fp, fp, ci, ci, ci, ci, ci, ci, cf, cf, vp]
        lib.dr_gated_rmsnorm.restype = ctypes.c_int
        lib.dr_gated_rmsnorm.argtypes = [vp, vp, fp, vp, ci, ci, ci, ci, ci, ci, ci, ci, cf, vp]
        lib.dr_dplr_recurrent.restype = ctypes.c_int
        lib.dr_dplr_recurrent.argtypes = [vp, vp, vp, vp, vp, vp, fp, vp, fp, ci, ci, ci, ci, ci, cf, ci, ci, ip, vp]
        lib.dr_rwkv6_recurrent.restype = ctypes.c_int
        lib.dr_rwkv6_recurrent.argtypes = [vp, vp, vp, vp, fp, fp, vp, fp, ci, ci, ci, ci, ci, cf, ci, ci, ip, vp]
        lib.dr_ssd_scan.restype = ctypes.c_int
        lib.dr_ssd_scan.argtypes = [vp, vp, fp, vp, vp, fp, fp, fp, vp, fp, ci, ci, ci, ci, ci, ci, cf, cf, ci, ip, vp]
        lib.dr_debug_bounds_checked.restype = ctypes.c_int
        lib.dr_debug_bounds_probe.restype = ctypes.c_int
        lib.dr_debug_bounds_probe.argtypes = [ip, ctypes.c_int64, ctypes.c_int64, ip, vp]
        lib.dr_debug_umma_selftest.restype = ctypes.c_int
        lib.dr_debug_umma_selftest.argtypes = [vp, vp, fp, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ip, vp]
        _lib = lib
    return _lib


def check(status: int, where: str) -> None:
    if status < 0:
        lib = load()
        text = lib.dr_strerror(status).decode()
        if status == -8:
            text += f" (cudaError {lib.dr_last_cuda_error()})"
        if status == -10:
            bits = lib.dr_last_device_status()
            text += " (" + ", ".join(n for b, n in DEVICE_STATUS_BITS.items() if bits & b) + f"; status word 0x{bits & 0xffffffff:x}"
            site = device_status_site(bits)
            text += f", first at barrier {site[0]} of warp group {site[1]})" if site else ")"
        raise DeltaRuleError(status, text, where)


def launch_count() -> int:
    return int(load().dr_launch_count())


def last_path() -> str:
    return load().dr_last_path().decode()
