"""Command-line contract of bench.py that can be checked without a GPU: the reference arm answers with one JSON line
and exit code 0, the argument parser knows the documented flags and defaults to one GPU."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1",
                        "--steps", "2", "--warmup", "3"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and isinstance(rec.get("unavailable"), str) and rec["unavailable"]


def test_reference_arm_prints_only_on_rank_zero():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                       capture_output=True, text=True, timeout=120, env=env)
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_flags_and_defaults():
    sys.path.insert(0, ROOT)
    try:
        import bench
    finally:
        sys.path.pop(0)
    argv = sys.argv
    try:
        sys.argv = ["bench.py"]
        a = bench.parse()
        assert a.gpus == 1 and a.impl == "ours" and a.steps > 0 and a.warmup >= 3
        sys.argv = ["bench.py", "--gpus", "8", "--steps", "5", "--warmup", "4", "--no-graph", "--no-shard-master",
                    "--no-e2e"]
        a = bench.parse()
        assert (a.gpus, a.steps, a.warmup) == (8, 5, 4) and a.no_graph and a.no_shard_master and a.no_e2e
        assert not a.no_baseline and a.dataset_batches >= 2 and a.loader_workers >= 1
    finally:
        sys.argv = argv


def test_reference_cpu_arm_of_the_secondary_benchmarks():
    """``bench_configs.py --impl cpu_ref`` needs no GPU: it times the restated reference loops (reduced size for the
    wide MLP) and prints one JSON line per configuration."""
    for cfg in ("wide_mlp", "mnist"):
        r = subprocess.run([sys.executable, os.path.join(ROOT, "bench_configs.py"), "--impl", "cpu_ref", "--config",
                            cfg, "--steps", "1"], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr[-2000:]
        rec = json.loads(r.stdout.strip().splitlines()[-1])
        assert rec["impl"] == "cpu_ref" and rec["samples_per_s"] > 0 and rec["gflops"] > 0
        assert rec["reduced_size"] == (cfg == "wide_mlp")
