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


def test_suite_history_turns_into_svg_charts_and_an_index(tmp_path):
    import json
    import subprocess
    import sys
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    hist = tmp_path / "history.jsonl"
    recs = [dict(suite="strategies", model="lenet5", suite_label=lab, samples_per_sec=v, epochs_per_sec=v / 4096, final_loss=0.01, accuracy=0.9, repeat=rep)
            for lab, v in (("ar-3w", 9000.0), ("ps-3w-2s", 8000.0)) for rep in range(2)]
    recs[1]["samples_per_sec"] = 9500.0
    hist.write_text("\n".join(json.dumps(r) for r in recs) + "\n")
    r = subprocess.run([sys.executable, os.path.join(root, "bench", "plots.py"), "--history", str(hist)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    assert json.loads(r.stdout.strip().splitlines()[-1])["plots"] == 4
    svg = (tmp_path / "strategies_lenet5_samples_per_sec.svg").read_text()
    assert svg.startswith("<svg") and "ar-3w" in svg and "9.2k" in svg and svg.count("<rect") == 3      # background + two bars
    assert "strategies_lenet5_accuracy.svg" in (tmp_path / "plots.md").read_text()


def test_cluster_tooling_generates_compose_and_hosts_block(tmp_path):
    import subprocess
    import sys
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "docker-compose.yml"
    r = subprocess.run([sys.executable, os.path.join(root, "docker", "compose_up.py"), "--nodes", "3", "--rate", "10mbit", "--dry-run",
                        "--file", str(out)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    text = out.read_text()
    assert text.count("dockerfile: docker/Dockerfile") == 3 and '"40002:40002"' in text and "rate --rate 10mbit node-0 node-1 node-2" in text
    hosts = tmp_path / "hosts"
    hosts.write_text("127.0.0.1 localhost\n")
    for n in (2, 3):     # the second call replaces the block instead of appending another one
        r = subprocess.run([sys.executable, os.path.join(root, "docker", "fill_hosts.py"), "--nodes", str(n), "--write", str(hosts)],
                           capture_output=True, text=True, timeout=60)
        assert r.returncode == 0, r.stderr
    h = hosts.read_text()
    assert h.startswith("127.0.0.1 localhost\n") and h.count("ono nodes") == 2 and h.count("node-") == 3
