"""The benchmark script's reference arm and its command line, checked without a GPU: the arm times the reference's CPU
forward (or the oracle port where the reference was not built) and must print one JSON line of the agreed shape; ranks
other than 0 leave without work; both arms describe the workload with the same string."""
import json
import os
import subprocess
import sys
import types

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BENCH = os.path.join(ROOT, "bench.py")


def _run(extra, env_extra=None):
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "LOCAL_RANK", "WORLD_SIZE")}
    env.update(env_extra or {})
    return subprocess.run([sys.executable, BENCH, *extra], capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)


def test_reference_arm_prints_the_agreed_line():
    r = _run(["--impl", "reference", "--steps", "1", "--warmup", "1"])
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "mlp_forward_samples_per_sec" and line["unit"] == "samples/s"
    assert line["higher_is_better"] is True and line["n_gpus"] == 1 and line["steps"] == 1 and line["warmup"] == 1
    assert line["value"] > 0 and line["ms_per_step"] > 0 and line["vs_baseline"] is None and line["gpu_launches"] == 0
    # throughput and step time describe the same run: 65536 rows per step
    assert abs(line["value"] * line["ms_per_step"] * 1e-3 / 65536 - 1.0) < 1e-6
    cb = line["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["value"] == line["value"] and "65536 rows" in cb["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    # the workload string is the one the GPU arm prints for its default configuration
    sys.path.insert(0, ROOT)
    import bench
    args = types.SimpleNamespace(workload="mlp", topo=bench.WORKLOADS["mlp"][0], dtype="int8", batch=65536)
    assert line["config"]["workload"] == bench.workload_name(args)


def test_reference_arm_runs_on_rank_zero_only():
    r = _run(["--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "1"], {"RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2"})
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_defaults_follow_the_workload():
    sys.path.insert(0, ROOT)
    import bench
    old = sys.argv
    try:
        sys.argv = ["bench.py"]
        a = bench.parse()
        assert (a.gpus, a.workload, a.dtype, a.batch, a.math) == (1, "mlp", "int8", 65536, "auto") and a.steps >= 1 and a.warmup >= 3
        sys.argv = ["bench.py", "--workload", "large"]
        a = bench.parse()
        assert (a.dtype, a.batch, a.topo[0], a.topo[-1]) == ("int4", 1, 8192, 1000)
        sys.argv = ["bench.py", "--workload", "wide", "--batch", "256"]
        a = bench.parse()
        assert (a.dtype, a.batch) == ("bf16", 256)
    finally:
        sys.argv = old
    # algorithmic work of the default configuration: 923408 multiply-adds per row, weights once in the stored precision
    assert bench.flops_per_sample(bench.TOPO) == 2 * 923408 == bench.FLOP_PER_SAMPLE
    nbytes = bench.algorithmic_bytes([8192, 16384, 16384, 8192, 1000], "int4", 1)
    weights = (8192 * 16384 + 16384 * 16384 + 16384 * 8192 + 8192 * 1000) // 2
    assert weights < nbytes < weights + 100_000
