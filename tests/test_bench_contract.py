"""CPU: bench.py's reference arm runs without a GPU and prints one JSON line with the agreed keys."""
import json
import os
import subprocess
import sys

from conftest import ROOT


def test_reference_arm_prints_one_json_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "c1",
                        "--steps", "1", "--warmup", "1"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "TOPS" and d["value"] > 0
    for key in ("metric", "n_gpus", "steps", "warmup", "higher_is_better", "scaling", "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert d["config"]["workload"].startswith("c1")
    assert d["scaling"] == "strong" and d["metric"].endswith("M=1024 N=1024 K=1024")
    assert set(d["config"]) == {"workload", "shard", "l2", "variant"}


def test_both_arms_describe_the_same_work():
    """The reference arm and this library's arm build `metric` and `config` with the same two
    functions, from the problem that is actually computed at that number of GPUs."""
    sys.path.insert(0, ROOT)
    import bench
    assert bench.metric_name("m8", 8, "strong") == "INT4 GEMM TOPS at M=8192 N=8192 K=8192"
    assert bench.metric_name("m8", 8, "weak") == "INT4 GEMM TOPS at M=8192 N=65536 K=8192"
    c = bench.describe_config("m8", 8, "strong")
    assert c["workload"] == "m8: M=8192 N=8192 K=8192" and c["shard"].startswith("8 x (M=8192, N=1024, K=8192)")
    assert bench.describe_config("c5", 8, "strong")["shard"].startswith("8 x (M=8192, N=3584, K=8192)")
    assert bench.metric_name("c4", 1, "strong").startswith("INT4 GEMM achieved HBM GB/s")
