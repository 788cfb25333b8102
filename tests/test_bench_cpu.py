"""bench.py on the CPU: the algorithmic byte and flop counts behind the roofline figures, and the reference arm's line."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
import bench  # noqa: E402


def test_algorithmic_bytes_of_the_benchmarked_configurations():
    W = bench.WORKLOADS
    # Gated DeltaNet forward, bf16, B=8 T=4096 H=16 d=128: 1032 B per token and head + the final state
    assert bench.alg_bytes(W["gdn_fwd"]) == 524288 * 1032 + 128 * 4 * 128 * 128 == 549453824
    # KDA forward, fp32 g and fp32 output: q, k, v bf16 + g, o fp32 + beta, and both states
    assert bench.alg_bytes(W["kda_fwd"]) == 1048576 * (3 * 256 + 2 * 512 + 4) + 2 * 128 * 4 * 128 * 128
    # decode: 132 104 B per (batch, head) and step
    assert bench.alg_bytes(W["gdn_decode"]) == 8192 * 132104
    # training step per GPU: 1032 + 1808 B per token and head (+ the final state of the forward)
    assert bench.alg_bytes(W["gdn_fwd_bwd"]) == 131072 * 2840 + 32 * 4 * 128 * 128
    # scans: every vector once at its storage width, both states
    assert bench.alg_bytes(W["dplr_fwd"]) == 524288 * 2 * (5 * 64 + 2 * 64) + 128 * 2 * 4 * 64 * 64
    assert bench.alg_bytes(W["ssd_fwd"]) == 8 * 4096 * (16 * (2 * 2 * 64 + 4) + 1 * 2 * 2 * 128) + 128 * 2 * 4 * 128 * 64


def test_algorithmic_flops_per_token_and_head():
    assert round(bench.alg_flops_per_token_head(64, 128, 128)) == 181589
    assert round(bench.alg_flops_per_token_head(64, 64, 64)) == 66901


def test_reference_arm_prints_one_contract_line():
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "deltanet_fwd_fp32",
                          "--steps", "1", "--warmup", "0", "--cpu-seconds", "2"], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-1000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "tokens/s" and line["higher_is_better"] is True
    assert line["value"] > 0 and line["e2e"]["value"] == line["value"]
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert "workload" in line["config"]
