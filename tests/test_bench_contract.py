"""The benchmark entry point's contract that can be checked without a GPU."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_reports_unavailable_and_exits_zero():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2",
                        "--warmup", "1"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr[-1000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and len(line["unavailable"]) > 10


def test_bench_configs_name_the_baseline_models():
    sys.path.insert(0, ROOT)
    import bench

    deep = bench.CONFIGS["deep"]
    assert deep["hidden"] == [(8192, "gelu")] * 8 and deep["classes"] == 1000 and deep["batch"] == 512 and deep["tile"] == "bf16"
    assert deep["opt"][0] == "momentum" and deep["opt"][2] == 0.9 and deep["strategy"] == "ps4"
    wide = bench.CONFIGS["wide"]
    assert wide["hidden"] == [(4096, "relu")] * 3 and wide["x"] == 784 and wide["batch"] == 1024 and wide["tile"] == "tf32"
    cnn = bench.CONFIGS["cnn"]
    assert cnn["conv"] == [(32, 3, 1, 1), (64, 3, 2, 1), (64, 3, 2, 1)] and cnn["hidden"] == [(128, "relu")]
    assert bench.SWITCH == {"metric": "grad_norm", "window": 50, "threshold": 1e-2}
