"""The debug build with index checks (-DDR_BOUNDS_CHECK) on tiny, ragged and odd shapes: T in {1, 63, 64, 65, 130},
d in {64, 128} and a size that is a multiple of nothing, every variant, fp32 and bf16, through the recurrence, the AUTO
chunk path and the fp32 chunk kernel, plus the RWKV / SSD scans.  No index may leave its array (status word clean),
and the outputs must equal the release build's bit for bit: the checks change nothing but what they skip.  The release
run is repeated as well: the same launch twice has to give the same bits (a race would not)."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from linearnexus_b200 import _lib

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def _run(lib_path, out):
    env = dict(os.environ, DELTARULE_SM100_LIB=str(lib_path))
    res = subprocess.run([sys.executable, str(ROOT / "tests" / "bounds_build_child.py"), str(out)], env=env,
                         capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    return np.load(out)


def test_debug_build_finds_no_index_outside_its_array_and_changes_no_bits(tmp_path):
    if not _lib.BOUNDS_LIB_PATH.exists():
        _lib.build_library(bounds=True)
    rel = _run(_lib.LIB_PATH, tmp_path / "release.npz")
    rel2 = _run(_lib.LIB_PATH, tmp_path / "release2.npz")
    dbg = _run(_lib.BOUNDS_LIB_PATH, tmp_path / "debug.npz")
    assert int(rel["bounds_checked"]) == 0 and int(dbg["bounds_checked"]) == 1
    assert int(dbg["status_bits"]) == 0 and int(rel["status_bits"]) == 0
    n = int(rel["count"])
    assert n == int(dbg["count"]) and n > 250
    for i in range(n):
        for key in (f"o{i}", f"s{i}"):
            assert np.array_equal(rel[key], rel2[key]), f"release run differs from itself in {key}"
            assert np.array_equal(rel[key], dbg[key]), f"debug build differs in {key}"
    # the check routine: index 10 of an array of 10 is outside; only the debug build raises the status bit
    assert int(dbg["probe_rc"]) == 0 and int(dbg["probe_in_range"]) == 0 and int(dbg["probe_status"]) == 2
    assert int(rel["probe_in_range"]) == 1 and int(rel["probe_status"]) == 0
