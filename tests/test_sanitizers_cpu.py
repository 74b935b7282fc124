"""The C++ runtime under AddressSanitizer + UBSan and under ThreadSanitizer: instrumented ``ono-orchestrator`` and
``ono-node`` run whole sessions (in-process rank threads on the dynamic barrier, and a remote native rank over the
control channel) and must finish without a single report. The reference runs no sanitizer
(.github/workflows/test.yml:29-30) and its one ``unsafe impl Sync`` store is the one that hangs
(parameter_server/src/storage/wild/shard.rs:10-17)."""
import json
import os
import socket
import subprocess
import time

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bins(kind):
    from oxidized_neural_orchestra_b200 import build

    if build.sanitizer_cxx(kind) is None:
        pytest.skip(f"no compiler here links the {kind} sanitizer runtime")
    return {p.name: str(p) for p in build.build_bins(sanitize=kind, only=("ono-node", "ono-orchestrator"))}


@pytest.fixture(scope="module")
def _both_built():
    """Build the address and the thread variants side by side (they are independent compiler runs)."""
    import concurrent.futures as cf

    from oxidized_neural_orchestra_b200 import build

    kinds = [k for k in ("address", "thread") if build.sanitizer_cxx(k) is not None]
    with cf.ThreadPoolExecutor(max_workers=2) as ex:
        list(ex.map(lambda k: build.build_bins(sanitize=k, only=("ono-node", "ono-orchestrator")), kinds))
    return kinds


@pytest.fixture(scope="module", params=["address", "thread"])
def san(request, _both_built):
    env = dict(os.environ, ONO_LOG="warn", ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1",
               TSAN_OPTIONS="halt_on_error=0:second_deadlock_stack=1")
    return request.param, _bins(request.param), env


def _write(tmp_path, addrs, algorithm, extra=None):
    rng = np.random.default_rng(1)
    xs = rng.random((36, 5)).astype(np.float32)
    ys = np.eye(3, dtype=np.float32)[rng.integers(0, 3, 36)]
    model = {"layers": [{"dense": {"output_size": 6, "init": "xavier_uniform", "act_fn": {"tanh": {"amp": 1.0}}}},
                        {"dense": {"output_size": 3, "init": "xavier_uniform", "act_fn": "softmax"}}]}
    tr = {"addrs": addrs, "algorithm": algorithm,
          "dataset": {"src": {"inline": {"samples": xs.reshape(-1).tolist(), "labels": ys.reshape(-1).tolist()}}, "x_size": 5, "y_size": 3},
          "optimizer": {"adam": {"lr": 0.05, "b1": 0.9, "b2": 0.999, "eps": 1e-8}}, "loss_fn": "cross_entropy",
          "batch_size": 6, "max_epochs": 4, "offline_epochs": 0, "seed": 5}
    tr.update(extra or {})
    mp, tp = tmp_path / "model.json", tmp_path / "training.json"
    mp.write_text(json.dumps(model))
    tp.write_text(json.dumps(tr))
    return str(mp), str(tp)


def _clean(kind, r):
    assert r.returncode == 0, r.stderr[-3000:]
    assert "Sanitizer" not in r.stderr and "runtime error:" not in r.stderr, r.stderr[-3000:]
    return json.loads(r.stdout.strip().splitlines()[-1])


def test_in_process_rank_threads_are_clean(san, tmp_path):
    kind, bins, env = san
    for algorithm in ("all_reduce", {"parameter_server": {"nservers": 1, "synchronizer": "barrier", "store": "blocking"}},
                      {"parameter_server": {"nservers": 1, "synchronizer": "non_blocking", "store": "wild"}}):
        mp, tp = _write(tmp_path, ["cpu:0", "cpu:1", "cpu:2"], algorithm)
        r = subprocess.run([bins["ono-orchestrator"], mp, tp, "--quiet"], capture_output=True, text=True, timeout=600, env=env)
        res = _clean(kind, r)
        assert res["stop_reason"] == "max_epochs" and len(res["loss_history"]) == 4


def test_remote_native_rank_over_the_control_channel_is_clean(san, tmp_path):
    kind, bins, env = san
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    node = subprocess.Popen([bins["ono-node"], "--port", str(port), "--device", "cpu"], env=env, stderr=subprocess.PIPE, text=True)
    try:
        for _ in range(200):
            try:
                socket.create_connection(("127.0.0.1", port), timeout=0.2).close()
                break
            except OSError:
                time.sleep(0.05)
        mp, tp = _write(tmp_path, [f"127.0.0.1:{port}"], "all_reduce")
        r = subprocess.run([bins["ono-orchestrator"], mp, tp, "--quiet"], capture_output=True, text=True, timeout=600, env=env)
        res = _clean(kind, r)
        assert res["loss_history"][-1] < res["loss_history"][0]
    finally:
        node.terminate()
        try:
            _, err = node.communicate(timeout=60)
        except subprocess.TimeoutExpired:
            node.kill()
            _, err = node.communicate()
    assert "Sanitizer" not in err and "runtime error:" not in err, err[-3000:]


def test_native_mesh_between_node_processes_is_clean(san, tmp_path):
    """Three instrumented node processes exchanging among themselves: the barrier exchange, the sparse serializer, the
    non-blocking exchange (receiver + transmitter + worker thread per rank, pushes applied under the shard lock), the
    strategy switch (re-partition, dataset hand-over, new roles) in place and the sparse ring."""
    kind, bins, env = san
    ports = []
    for _ in range(3):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            ports.append(s.getsockname()[1])
    nodes = [subprocess.Popen([bins["ono-node"], "--port", str(p), "--device", "cpu"], env=env, stderr=subprocess.PIPE, text=True)
             for p in ports]
    errs = []
    try:
        for p in ports:
            for _ in range(200):
                try:
                    socket.create_connection(("127.0.0.1", p), timeout=0.2).close()
                    break
                except OSError:
                    time.sleep(0.05)
        addrs = [f"127.0.0.1:{p}" for p in ports]
        for algorithm, extra in (({"parameter_server": {"nservers": 1, "synchronizer": "barrier", "store": "blocking"}},
                                  {"serializer": {"sparse_capable": {"r": 0.2}}}),
                                 ({"parameter_server": {"nservers": 1, "synchronizer": "non_blocking", "store": "blocking"}}, {}),
                                 ({"parameter_server": {"nservers": 1, "synchronizer": "non_blocking", "store": "wild"}},
                                  {"b200": {"wire_dtype": "f16"}}),
                                 ({"strategy_switch": {"nservers": 1, "synchronizer": "non_blocking", "store": "blocking"}},
                                  {"b200": {"switch_window": 2, "switch_threshold": 10.0}}),
                                 ("all_reduce", {"serializer": {"sparse_capable": {"r": 0.2}}})):
            mp, tp = _write(tmp_path, addrs, algorithm, extra)
            r = subprocess.run([bins["ono-orchestrator"], mp, tp, "--quiet"], capture_output=True, text=True, timeout=600, env=env)
            res = _clean(kind, r)
            assert res["stop_reason"] == "max_epochs" and len(res["loss_history"]) == 4
            assert res.get("metrics", {}).get("data_plane") == "native tcp mesh"
    finally:
        for n in nodes:
            n.terminate()
        for n in nodes:
            try:
                _, err = n.communicate(timeout=60)
            except subprocess.TimeoutExpired:
                n.kill()
                _, err = n.communicate()
            errs.append(err)
    for err in errs:
        assert "Sanitizer" not in err and "runtime error:" not in err, err[-3000:]
