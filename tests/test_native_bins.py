"""The native executables: ``ono-orchestrator`` (headless run from model.json + training.json) and
``ono-node`` (role-agnostic listener; node/src/main.rs:27-54, router.rs:79-220, stat_service.rs:69-152)."""
import json
import os
import shutil
import socket
import subprocess
import sys
import time

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.skipif(shutil.which("g++") is None, reason="needs a C++ compiler")


@pytest.fixture(scope="module")
def bins():
    from oxidized_neural_orchestra_b200 import build

    built = {p.name: str(p) for p in build.build_bins()}
    assert {"ono-node", "ono-orchestrator"} <= set(built)
    return built


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _configs(tmp_path, addrs, algorithm="all_reduce", epochs=6):
    rng = np.random.default_rng(0)
    xs = rng.random((40, 6)).astype(np.float32)
    ys = np.eye(3, dtype=np.float32)[rng.integers(0, 3, 40)]
    model = {"layers": [{"dense": {"output_size": 5, "init": "xavier_uniform", "act_fn": {"tanh": {"amp": 1.0}}}},
                        {"dense": {"output_size": 3, "init": "xavier_uniform", "act_fn": "softmax"}}]}
    tr = {"addrs": addrs, "algorithm": algorithm,
          "dataset": {"src": {"inline": {"samples": xs.reshape(-1).tolist(), "labels": ys.reshape(-1).tolist()}}, "x_size": 6, "y_size": 3},
          "optimizer": {"adam": {"lr": 0.05, "b1": 0.9, "b2": 0.999, "eps": 1e-8}}, "loss_fn": "cross_entropy",
          "batch_size": 5, "max_epochs": epochs, "offline_epochs": 0, "seed": 3}
    mp, tp = tmp_path / "model.json", tmp_path / f"training_{len(addrs)}_{addrs[0].split(':')[0]}.json"
    mp.write_text(json.dumps(model))
    tp.write_text(json.dumps(tr))
    return str(mp), str(tp), model, tr, xs, ys


def _run_orchestrator(bins, mp, tp, *extra, timeout=300):
    r = subprocess.run([bins["ono-orchestrator"], mp, tp, "--quiet", *extra], capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, r.stderr[-2000:]
    return json.loads(r.stdout.strip().splitlines()[-1])


def _python_reference(model, tr, xs, ys):
    import orchestra
    from orchestra import Sequential, orchestrate
    from orchestra.activations import Softmax, Tanh
    from orchestra.arch import Dense
    from orchestra.datasets import InlineDataset
    from orchestra.initialization import XavierUniform
    from orchestra.loss_fns import CrossEntropy
    from orchestra.optimizers import Adam

    m = Sequential([Dense(5, XavierUniform(), Tanh()), Dense(3, XavierUniform(), Softmax())])
    cfg = orchestra.all_reduce([f"cpu:{i}" for i in range(len(tr["addrs"]))], InlineDataset(xs, ys, 6, 3), Adam(0.05),
                               CrossEntropy(), tr["max_epochs"], 5, seed=3)
    return orchestrate(m, cfg).wait(quiet=True)


def test_orchestrator_trains_in_process_and_writes_the_reference_checkpoint_layout(bins, tmp_path):
    mp, tp, model, tr, xs, ys = _configs(tmp_path, ["cpu:0", "cpu:1", "cpu:2"])
    out = tmp_path / "m.safetensors"
    res = _run_orchestrator(bins, mp, tp, "--save", str(out))
    ref = _python_reference(model, tr, xs, ys)
    assert res["stop_reason"] == "max_epochs" and res["n_params"] == 53
    assert np.allclose(res["loss_history"], ref.loss_history(), rtol=1e-6)
    from orchestra import _orchestra as core

    tensors = {t[0]: (t[1], np.asarray(t[2])) for t in core.load_safetensors(str(out))}
    order = ["layer_0.weight", "layer_0.bias", "layer_1.weight", "layer_1.bias"]
    assert sorted(tensors) == sorted(order)
    assert list(tensors["layer_0.weight"][0]) == [6, 5] and list(tensors["layer_1.bias"][0]) == [3]
    flat = np.concatenate([tensors[k][1].reshape(-1) for k in order])
    assert np.allclose(flat, ref.weights_array(), atol=1e-6)


def test_orchestrator_rejects_an_invalid_config(bins, tmp_path):
    mp, tp, *_ = _configs(tmp_path, ["cpu:0"])
    bad = json.loads(open(tp).read())
    bad["batch_size"] = 10_000
    open(tp, "w").write(json.dumps(bad))
    r = subprocess.run([bins["ono-orchestrator"], mp, tp], capture_output=True, text=True, timeout=60)
    assert r.returncode == 1 and "batch_size" in r.stderr


@pytest.fixture()
def cxx_nodes(bins):
    ports = [_free_port() for _ in range(3)]
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), ONO_LOG="warn")
    procs = [subprocess.Popen([bins["ono-node"], "--port", str(p), "--device", "cpu"], env=env) for p in ports]
    for p in ports:                      # wait until each listens (a refused probe is not a session)
        for _ in range(100):
            try:
                socket.create_connection(("127.0.0.1", p), timeout=0.2).close()
                break
            except OSError:
                time.sleep(0.05)
    yield [f"127.0.0.1:{p}" for p in ports]
    for p in procs:
        p.kill()
    for p in procs:
        p.wait(timeout=30)


def test_nodes_serve_a_single_rank_natively_and_many_ranks_through_rank_processes(bins, cxx_nodes, tmp_path):
    mp, tp, model, tr, xs, ys = _configs(tmp_path, cxx_nodes[:1])
    one = _run_orchestrator(bins, mp, tp)
    assert one["stop_reason"] == "max_epochs" and one["loss_history"][-1] < one["loss_history"][0]
    mp, tp, model, tr, xs, ys = _configs(tmp_path, cxx_nodes)
    three = _run_orchestrator(bins, mp, tp)
    ref = _python_reference(model, tr, xs, ys)
    assert np.allclose(three["loss_history"], ref.loss_history(), rtol=1e-6)
    # the nodes went back to listening: a second session on the same processes, this time planned from a latency probe
    cfg = json.loads(open(tp).read())
    cfg["b200"] = {"probe": True}
    open(tp, "w").write(json.dumps(cfg))
    again = _run_orchestrator(bins, mp, tp)
    assert np.allclose(again["loss_history"], three["loss_history"], rtol=1e-9)


def test_node_latency_probe_answers_with_min_max_mean_per_peer(cxx_nodes):
    from oxidized_neural_orchestra_b200.runtime import wire

    chs = []
    for a in cxx_nodes[:2]:
        host, port = a.rsplit(":", 1)
        ch = wire.connect(host, int(port))
        ch.connect_as("Orchestrator")
        assert ch.peer_entity == "Node"
        chs.append(ch)
    # node 0 only accepts, node 1 pings node 0 (orchestrator/src/configs/stat_requester.rs:52-72)
    chs[0].send_command({"stats_request": {"ping": {"addrs": [], "rounds": 5, "incoming": 1}}})
    chs[1].send_command({"stats_request": {"ping": {"addrs": [cxx_nodes[0]], "rounds": 5, "incoming": 0}}})
    _, r1 = chs[1].recv(timeout=30)
    _, r0 = chs[0].recv(timeout=30)
    rtts = r1["stats_response"]["stats"]["ping"]["rtts"]
    assert list(rtts) == [cxx_nodes[0]]
    st = rtts[cxx_nodes[0]]
    assert 0 < st["min"] <= st["mean"] <= st["max"] < 1e9
    assert r0["stats_response"]["stats"]["ping"]["rtts"] == {}
    for ch in chs:
        ch.send_command("disconnect")
        ch.close()


def test_orchestui_renders_the_dashboard_and_autosaves_into_the_model_repository(bins, tmp_path):
    mp, tp, model, tr, xs, ys = _configs(tmp_path, ["cpu:0", "cpu:1", "cpu:2"],
                                         algorithm={"parameter_server": {"nservers": 1, "synchronizer": "barrier", "store": "blocking"}})
    r = subprocess.run([bins["orchestui"], "--render-once", mp, tp, "--size", "120x34"], capture_output=True, text=True,
                       timeout=120, cwd=tmp_path)
    assert r.returncode == 0, r.stderr[-2000:]
    frame = r.stdout
    for panel in ("average loss", "workers", "log", "parameters", "topology"):
        assert panel in frame
    assert "finished: max_epochs" in frame and "parameter server" in frame and "progress 6/6" in frame
    saved = list((tmp_path / "safetensors").glob("*_*.safetensors"))     # <adjective>_<term>.safetensors
    assert len(saved) == 1
    from orchestra import _orchestra as core

    assert sum(np.asarray(t[2]).size for t in core.load_safetensors(str(saved[0]))) == 53


def test_orchestui_interactive_screens_driven_by_a_key_script(bins, tmp_path):
    """The interactive path without a terminal: menu -> configuration (examples carousel, typed paths) -> dashboard with
    the animated topology -> stop / save pop-ups -> repository screen listing the saved models."""
    mp, tp, model, tr, xs, ys = _configs(tmp_path, ["cpu:0", "cpu:1", "cpu:2"], algorithm="all_reduce")
    script = ("<dump>"                                   # the menu
              "<enter><right><dump>"                     # configuration screen, second example
              f"{os.path.basename(mp)}<tab>{os.path.basename(tp)}<dump><enter>"
              "<wait><dump>"                             # dashboard after the run has finished (auto-saved)
              "w<bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs>"
              "<bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs><bs>safetensors/mine.safetensors<dump><enter>"
              "m<down><enter><dump><esc>"                # back to the menu, repository screen
              "<down><enter>")                           # quit
    r = subprocess.run([bins["orchestui"], "--script", script, "--size", "120x34"], capture_output=True, text=True, timeout=120,
                       cwd=tmp_path)
    assert r.returncode == 0, r.stderr[-2000:]
    frames = r.stdout.split("=== frame ===\n")[1:]
    assert len(frames) == 6
    menu, config, typed, dash, saveas, repo = frames
    assert "Start training" in menu and "Repository" in menu
    assert "example 2/3" in config and "parameter_server" in config
    assert os.path.basename(mp) in typed and os.path.basename(tp) in typed
    assert "finished: max_epochs" in dash and "ring all-reduce" in dash and "w0" in dash and "w2" in dash and "→" in dash
    assert "save model" in saveas and "mine.safetensors" in saveas
    assert "trained-model repository" in repo and "mine.safetensors" in repo and "layer_0.weight [6, 5]" in repo
    assert (tmp_path / "safetensors" / "mine.safetensors").exists() and len(list((tmp_path / "safetensors").glob("*.safetensors"))) == 2


def test_several_cpu_ranks_run_natively_over_a_tcp_mesh_between_the_nodes(bins, cxx_nodes, tmp_path):
    """Three ono-node processes, each one CPU rank on the C++ engine, exchanging gradients over TCP among themselves
    (no rank process, no gloo): parameter server with two co-located... servers and the reference's f16 gradient wire,
    checked against the in-process cluster running the same plan."""
    import orchestra
    from orchestra import Sequential, orchestrate
    from orchestra.activations import Softmax, Tanh
    from orchestra.arch import Dense
    from orchestra.datasets import InlineDataset
    from orchestra.initialization import XavierUniform
    from orchestra.loss_fns import CrossEntropy
    from orchestra.optimizers import Adam
    from orchestra.store import BlockingStore
    from orchestra.sync import BarrierSync

    for b200 in ({}, {"wire_dtype": "f16"}):
        mp, tp, model, tr, xs, ys = _configs(tmp_path, cxx_nodes, algorithm={"parameter_server": {
            "nservers": 1, "synchronizer": "barrier", "store": "blocking"}})
        cfg = json.loads(open(tp).read())
        cfg["b200"] = b200
        cfg["early_stopping"] = None
        open(tp, "w").write(json.dumps(cfg))
        got = _run_orchestrator(bins, mp, tp)
        m = Sequential([Dense(5, XavierUniform(), Tanh()), Dense(3, XavierUniform(), Softmax())])
        ref = orchestrate(m, orchestra.parameter_server([f"cpu:{i}" for i in range(3)], 1, InlineDataset(xs, ys, 6, 3), Adam(0.05),
                                                        CrossEntropy(), BarrierSync(), BlockingStore(), tr["max_epochs"], 5, seed=3,
                                                        b200=b200 or None)).wait(quiet=True)
        assert got["stop_reason"] == "max_epochs"
        assert np.allclose(got["loss_history"], ref.loss_history(), rtol=1e-5)
        assert got.get("metrics", {}).get("data_plane") == "native tcp mesh"
    # the sparse serializer on the same mesh: thresholded (offset, f16 run) messages per worker and server shard, unsent
    # entries stay in the workers' residuals; same thresholds (same seeds) as the in-process cluster
    from orchestra.serializer import SparseSerializer

    mp, tp, model, tr, xs, ys = _configs(tmp_path, cxx_nodes, algorithm={"parameter_server": {
        "nservers": 1, "synchronizer": "barrier", "store": "blocking"}})
    cfg = json.loads(open(tp).read())
    cfg["serializer"] = {"sparse_capable": {"r": 0.3}}
    cfg["early_stopping"] = None
    open(tp, "w").write(json.dumps(cfg))
    got = _run_orchestrator(bins, mp, tp)
    m = Sequential([Dense(5, XavierUniform(), Tanh()), Dense(3, XavierUniform(), Softmax())])
    ref = orchestrate(m, orchestra.parameter_server([f"cpu:{i}" for i in range(3)], 1, InlineDataset(xs, ys, 6, 3), Adam(0.05),
                                                    CrossEntropy(), BarrierSync(), BlockingStore(), tr["max_epochs"], 5, seed=3,
                                                    serializer=SparseSerializer(0.3))).wait(quiet=True)
    dense = orchestrate(m, orchestra.parameter_server([f"cpu:{i}" for i in range(3)], 1, InlineDataset(xs, ys, 6, 3), Adam(0.05),
                                                      CrossEntropy(), BarrierSync(), BlockingStore(), tr["max_epochs"], 5, seed=3)).wait(quiet=True)
    assert got.get("metrics", {}).get("data_plane") == "native tcp mesh"
    assert np.allclose(got["loss_history"], ref.loss_history(), rtol=1e-5)
    assert not np.array_equal(ref.loss_history(), dense.loss_history())      # the serializer does change the run


def test_published_rows_run_on_native_node_processes(bins, tmp_path):
    """`bench/suites.py --nodes tcp`: one ono-node process per node on loopback ports, the orchestrator's session over
    them, a throughput table against the reference's published figures."""
    out = tmp_path / "pub"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench", "suites.py"), "--suite", "published", "--nodes", "tcp", "--model", "lenet5",
                        "--rows", "192", "--epochs", "2", "--only", "AR 3w offline 0 b64,PS blocking 3w+2s", "--out", str(out)],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    table = (out / "published_tcp.md").read_text()
    rows = [l for l in table.splitlines() if l.startswith("| lenet5 |")]
    assert len(rows) == 2 and "| 9675 |" in rows[0] and "| 9970 |" in rows[1]
    recs = [json.loads(l) for l in (out / "history.jsonl").read_text().splitlines()]
    assert all(rec["epochs"] == 2 and rec["samples_per_sec"] > 0 and np.isfinite(rec["final_loss"]) for rec in recs)
    assert [rec["nodes"] for rec in recs] == [3, 5]


def test_sparse_serializer_runs_natively_between_node_processes(bins, cxx_nodes, tmp_path):
    """A model large enough for the thresholded (offset, f16 run) encoding to beat the dense one: the node processes ship
    those records over the TCP mesh, servers lift them, workers keep what they did not send; the run equals the in-process
    cluster's (same thresholds from the same seeds) and differs from a run without the serializer."""
    import orchestra
    from orchestra import Sequential, orchestrate
    from orchestra.activations import Softmax, Tanh
    from orchestra.arch import Dense
    from orchestra.datasets import InlineDataset
    from orchestra.initialization import XavierUniform
    from orchestra.loss_fns import CrossEntropy
    from orchestra.optimizers import GradientDescent
    from orchestra.serializer import SparseSerializer
    from orchestra.store import BlockingStore
    from orchestra.sync import BarrierSync

    rng = np.random.default_rng(1)
    xs = rng.random((60, 6)).astype(np.float32)
    ys = np.eye(3, dtype=np.float32)[rng.integers(0, 3, 60)]
    model = Sequential([Dense(64, XavierUniform(), Tanh()), Dense(3, XavierUniform(), Softmax())])

    def run(addrs, ser):
        tr = orchestra.parameter_server(addrs, 1, InlineDataset(xs, ys, 6, 3), GradientDescent(0.5), CrossEntropy(), BarrierSync(),
                                        BlockingStore(), 6, 10, seed=3, serializer=ser)
        return orchestrate(model, tr).wait(quiet=True)

    native = run(cxx_nodes, SparseSerializer(0.05))
    inproc = run([f"cpu:{i}" for i in range(3)], SparseSerializer(0.05))
    dense = run([f"cpu:{i}" for i in range(3)], None)
    assert (native.metrics() or {}).get("data_plane") == "native tcp mesh"
    assert np.allclose(native.loss_history(), inproc.loss_history(), rtol=1e-5)
    assert np.abs(native.weights_array() - inproc.weights_array()).max() < 1e-5
    # with 5 % of the entries per message the run is visibly not the dense one
    assert np.abs(np.asarray(inproc.loss_history()) - np.asarray(dense.loss_history())).max() > 1e-4


@pytest.mark.parametrize("store", ["blocking", "wild"])
def test_non_blocking_parameter_server_runs_natively_between_node_processes(bins, cxx_nodes, tmp_path, store):
    """Non-blocking synchroniser on node processes: every push is applied on arrival, alone, and answered with the owner's
    shard as it stands then (blocking store: divided by the number of workers; wild store: applied as it is). The order of
    arrival is not fixed, so the check is that the run ends, learns, and stayed on the native data plane."""
    import orchestra
    from orchestra import Sequential, orchestrate
    from orchestra.activations import Softmax, Tanh
    from orchestra.arch import Dense
    from orchestra.datasets import InlineDataset
    from orchestra.initialization import XavierUniform
    from orchestra.loss_fns import CrossEntropy
    from orchestra.optimizers import GradientDescent
    from orchestra.serializer import SparseSerializer
    from orchestra.store import BlockingStore, WildStore
    from orchestra.sync import NonBlockingSync

    rng = np.random.default_rng(2)
    labels = rng.integers(0, 3, 90)
    xs = (np.eye(3, dtype=np.float32)[labels] @ rng.random((3, 6)).astype(np.float32) + 0.1 * rng.random((90, 6)).astype(np.float32))
    ys = np.eye(3, dtype=np.float32)[labels]
    model = Sequential([Dense(32, XavierUniform(), Tanh()), Dense(3, XavierUniform(), Softmax())])
    for ser, b200 in ((None, None), (None, {"wire_dtype": "f16"}), (SparseSerializer(0.1), None)):
        tr = orchestra.parameter_server(cxx_nodes, 1, InlineDataset(xs, ys, 6, 3), GradientDescent(0.2 if store == "wild" else 0.6),
                                        CrossEntropy(), NonBlockingSync(), WildStore() if store == "wild" else BlockingStore(), 12, 15,
                                        seed=3, serializer=ser, b200=b200)
        m = orchestrate(model, tr).wait(quiet=True)
        hist = m.loss_history()
        assert (m.metrics() or {}).get("data_plane") == "native tcp mesh"
        assert len(hist) == 12 and np.isfinite(hist).all() and hist[-1] < 0.8 * hist[0], hist


@pytest.mark.parametrize("sync", ["barrier", "non_blocking"])
def test_strategy_switch_runs_natively_between_node_processes(bins, cxx_nodes, tmp_path, sync):
    """All-reduce, then the switch: the promoted node keeps its ranges, stops training and hands its samples to the two
    remaining workers, which carry on against it as a parameter server; all of it inside the node processes. With the
    barrier synchroniser the run equals the in-process cluster's."""
    import orchestra
    from orchestra import Sequential, orchestrate
    from orchestra.activations import Softmax, Tanh
    from orchestra.arch import Dense
    from orchestra.datasets import InlineDataset
    from orchestra.initialization import XavierUniform
    from orchestra.loss_fns import CrossEntropy
    from orchestra.optimizers import GradientDescentWithMomentum
    from orchestra.store import BlockingStore
    from orchestra.sync import BarrierSync, NonBlockingSync

    rng = np.random.default_rng(4)
    labels = rng.integers(0, 3, 96)
    xs = (np.eye(3, dtype=np.float32)[labels] @ rng.random((3, 6)).astype(np.float32) + 0.1 * rng.random((96, 6)).astype(np.float32))
    ys = np.eye(3, dtype=np.float32)[labels]
    model = Sequential([Dense(16, XavierUniform(), Tanh()), Dense(3, XavierUniform(), Softmax())])

    def run(addrs):
        tr = orchestra.strategy_switch(addrs, 1, InlineDataset(xs, ys, 6, 3), GradientDescentWithMomentum(0.3, 0.9), CrossEntropy(),
                                       BarrierSync() if sync == "barrier" else NonBlockingSync(), BlockingStore(), 10, 8, seed=3,
                                       b200={"switch_window": 2, "switch_threshold": 10.0})
        return orchestrate(model, tr).wait(quiet=True)

    native = run(cxx_nodes)
    met = native.metrics() or {}
    assert met.get("data_plane") == "native tcp mesh" and met.get("switched") is True
    hist = native.loss_history()
    assert len(hist) == 10 and np.isfinite(hist).all() and hist[-1] < hist[0]
    if sync == "barrier":
        inproc = run([f"cpu:{i}" for i in range(3)])
        assert (inproc.metrics() or {}).get("switched") is True
        assert np.allclose(hist, inproc.loss_history(), rtol=1e-5)
        assert np.abs(native.weights_array() - inproc.weights_array()).max() < 1e-5


def test_sparse_ring_all_reduce_runs_natively_between_node_processes(bins, cxx_nodes, tmp_path):
    """The reference's ring with its sparse serializer on node processes: every hop's chunk thresholded and encoded anew,
    residuals kept at the senders; the run equals the in-process cluster's ring hop for hop (same seeds), also through a
    strategy switch whose second phase carries the serializer on."""
    import orchestra
    from orchestra import Sequential, orchestrate
    from orchestra.activations import Softmax, Tanh
    from orchestra.arch import Dense
    from orchestra.datasets import InlineDataset
    from orchestra.initialization import XavierUniform
    from orchestra.loss_fns import CrossEntropy
    from orchestra.optimizers import GradientDescentWithMomentum
    from orchestra.serializer import SparseSerializer
    from orchestra.store import BlockingStore
    from orchestra.sync import BarrierSync

    rng = np.random.default_rng(6)
    labels = rng.integers(0, 3, 96)
    xs = (np.eye(3, dtype=np.float32)[labels] @ rng.random((3, 6)).astype(np.float32) + 0.1 * rng.random((96, 6)).astype(np.float32))
    ys = np.eye(3, dtype=np.float32)[labels]
    model = Sequential([Dense(64, XavierUniform(), Tanh()), Dense(3, XavierUniform(), Softmax())])
    opt = lambda: GradientDescentWithMomentum(0.3, 0.9)

    def ar(addrs, ser):
        return orchestrate(model, orchestra.all_reduce(addrs, InlineDataset(xs, ys, 6, 3), opt(), CrossEntropy(), 8, 8, seed=3,
                                                       serializer=ser)).wait(quiet=True)

    def ss(addrs):
        tr = orchestra.strategy_switch(addrs, 1, InlineDataset(xs, ys, 6, 3), opt(), CrossEntropy(), BarrierSync(), BlockingStore(), 8, 8,
                                       seed=3, serializer=SparseSerializer(0.05), b200={"switch_window": 2, "switch_threshold": 10.0})
        return orchestrate(model, tr).wait(quiet=True)

    cpu = [f"cpu:{i}" for i in range(3)]
    native, inproc, dense = ar(cxx_nodes, SparseSerializer(0.05)), ar(cpu, SparseSerializer(0.05)), ar(cpu, None)
    assert (native.metrics() or {}).get("data_plane") == "native tcp mesh"
    assert np.allclose(native.loss_history(), inproc.loss_history(), rtol=1e-5)
    assert np.abs(native.weights_array() - inproc.weights_array()).max() < 1e-5
    assert np.abs(np.asarray(inproc.loss_history()) - np.asarray(dense.loss_history())).max() > 1e-4
    native, inproc = ss(cxx_nodes), ss(cpu)
    assert (native.metrics() or {}).get("data_plane") == "native tcp mesh" and (native.metrics() or {}).get("switched") is True
    assert np.allclose(native.loss_history(), inproc.loss_history(), rtol=1e-5)


def test_orchestrator_binary_resumes_with_optimizer_state(bins, tmp_path):
    """`ono-orchestrator` on in-process CPU ranks: `b200.state_path` writes the optimizer-state sidecar (the file the Python
    runtime writes), and a second run from `--save`d weights + that sidecar continues the first: 3 + 3 epochs give the
    losses of 6."""
    from oxidized_neural_orchestra_b200.utils.state import load_state

    mp, tp, model, tr, xs, ys = _configs(tmp_path, ["cpu:0", "cpu:1"], epochs=6)
    whole = _run_orchestrator(bins, mp, tp)

    def write(epochs, b200):
        cfg = json.loads(open(tp).read())
        cfg["max_epochs"], cfg["b200"], cfg["early_stopping"] = epochs, b200, None
        path = tmp_path / f"t_{epochs}_{len(b200)}.json"
        path.write_text(json.dumps(cfg))
        return str(path)

    w, st = str(tmp_path / "half.safetensors"), str(tmp_path / "half.state.safetensors")
    half = _run_orchestrator(bins, mp, write(3, {"state_path": st}), "--save", w)
    side = load_state(st, 53)
    assert side["meta"]["epochs"] == "3" and side["meta"]["optimizer"] == "adam" and np.abs(side["m"]).max() > 0 and side["v"].max() > 0
    rest = _run_orchestrator(bins, mp, write(3, {"init_from": w, "init_state_from": st}))
    assert np.allclose(half["loss_history"] + rest["loss_history"], whole["loss_history"], rtol=1e-5)
    cold = _run_orchestrator(bins, mp, write(3, {"init_from": w, "start_epoch": 3}))
    assert not np.allclose(cold["loss_history"], whole["loss_history"][3:], rtol=1e-5)
