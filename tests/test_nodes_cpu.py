"""Role-agnostic node processes over the TCP control channel, with gloo ranks on CPU.

Three real node processes await specs (node/README.md:3-7); the orchestrator hands out roles, ships
the dataset partitions, relays events and collects the final parameters. Results must equal the
in-process CPU cluster's, which runs the same C++ trainer on the same partitions.
"""
import numpy as np
import pytest

import orchestra
from orchestra import Sequential, orchestrate
from orchestra.activations import Softmax, Tanh
from orchestra.arch import Dense
from orchestra.datasets import InlineDataset
from orchestra.initialization import XavierUniform
from orchestra.loss_fns import CrossEntropy
from orchestra.optimizers import Adam, GradientDescent
from orchestra.store import BlockingStore
from orchestra.sync import BarrierSync
from oxidized_neural_orchestra_b200.runtime import wire
from oxidized_neural_orchestra_b200.runtime.launch import spawn_nodes


@pytest.fixture(scope="module")
def nodes():
    procs, addrs = spawn_nodes(3, "cpu", once=False)
    yield addrs
    for p in procs:
        p.kill()
    for p in procs:
        p.wait(timeout=30)


def _setup():
    rng = np.random.default_rng(0)
    xs = rng.random((40, 6), dtype=np.float32)
    ys = np.eye(3, dtype=np.float32)[rng.integers(0, 3, 40)]
    return Sequential([Dense(5, XavierUniform(), Tanh()), Dense(3, XavierUniform(), Softmax())]), xs, ys


def test_nodes_match_in_process_cluster(nodes):
    model, xs, ys = _setup()
    for make in (
        lambda a: orchestra.all_reduce(a, InlineDataset(xs, ys, 6, 3), Adam(0.05), CrossEntropy(), 6, 5, seed=3),
        lambda a: orchestra.parameter_server(a, 1, InlineDataset(xs, ys, 6, 3), GradientDescent(0.3), CrossEntropy(),
                                             BarrierSync(), BlockingStore(), 6, 5, seed=3, offline_epochs=1),
    ):
        got = orchestrate(model, make(nodes)).wait(quiet=True)
        ref = orchestrate(model, make([f"cpu:{i}" for i in range(3)])).wait(quiet=True)
        assert got.stop_reason == "max_epochs"
        assert np.allclose(got.loss_history(), ref.loss_history(), rtol=1e-6)
        assert np.abs(got.weights_array() - ref.weights_array()).max() < 1e-6


def test_nodes_strategy_switch_and_stop(nodes):
    model, xs, ys = _setup()
    tr = orchestra.strategy_switch(nodes, 1, InlineDataset(xs, ys, 6, 3), Adam(0.01), CrossEntropy(), BarrierSync(),
                                   BlockingStore(), 12, 5, seed=3, b200={"switch_window": 2, "switch_threshold": 10.0})
    s = orchestrate(model, tr)
    kinds = [ev["kind"] for ev in s.events()]
    assert "switch" in kinds and "upgraded" in kinds and kinds[-1] == "complete"
    m = s.wait(quiet=True)
    assert m.metrics()["switched"] is True and len(m.weights()) == 6 * 5 + 5 + 5 * 3 + 3
    tr = orchestra.all_reduce(nodes, InlineDataset(xs, ys, 6, 3), GradientDescent(0.01), CrossEntropy(), 100000, 5, seed=3)
    s = orchestrate(model, tr)
    s.stop()
    m = s.wait(quiet=True)
    assert m.stop_reason == "stopped" and len(m.loss_history()) < 100000


def test_runs_without_a_seed_start_every_rank_from_the_same_parameters(nodes):
    """No seed in the configuration (the public API's default): rank 0 draws one and every rank uses it. With a zero
    learning rate nothing moves, so what comes back is the initial vector. Parameter-server ranks own disjoint slices
    and the final gather takes each slice from its owner: the result equals the all-reduce run's (rank 0's replica)
    only if all ranks generated the same vector... which also needs the same seed in both runs, so each run is instead
    checked against its own loss: identical replicas give every worker the loss of the same model on its partition,
    and two epochs at zero learning rate give the same losses twice."""
    model, xs, ys = _setup()
    tr = orchestra.parameter_server(nodes, 2, InlineDataset(xs, ys, 6, 3), GradientDescent(1e-30), CrossEntropy(), BarrierSync(),
                                    BlockingStore(), 2, 40, b200={"colocate": True, "sharding": "even"})
    s = orchestrate(model, tr)
    per_worker = {}
    for ev in s.events():
        if ev["kind"] == "losses":
            per_worker.setdefault(ev["worker"], []).extend(ev["losses"])
    m = s.wait(quiet=True)
    w = m.weights_array()
    assert len(per_worker) == 3 and np.isfinite(w).all() and np.abs(w).max() > 0
    # the gathered vector is a patchwork of the three owners' slices; evaluate it on each worker's partition with the
    # CPU engine: a worker whose replica differed from the patchwork would have reported a different loss
    from orchestra import _orchestra as core
    import json

    plan = json.loads(core.adapt_configs(json.dumps(model.to_config()), tr.to_json()))
    for wk in plan["workers"]:
        b, e = wk["partition"]
        spec = dict(wk["spec"]["trainer"])
        t = core.RoundTrainer(json.dumps(spec), xs[b:e].reshape(-1), ys[b:e].reshape(-1), True)
        _, _, losses, _ = t.train(w.copy(), np.zeros_like(w))
        got = per_worker[plan["workers"].index(wk)]
        assert abs(losses[0] - got[0]) < 1e-6 and abs(got[0] - got[1]) < 1e-6


def test_gradient_norm_switch_on_cpu_ranks(nodes):
    """switch_metric "grad_norm": the norm of the averaged gradient drives the switch instead of the losses."""
    model, xs, ys = _setup()
    tr = orchestra.strategy_switch(nodes, 1, InlineDataset(xs, ys, 6, 3), Adam(0.01), CrossEntropy(), BarrierSync(),
                                   BlockingStore(), 12, 5, seed=3,
                                   b200={"switch_metric": "grad_norm", "switch_window": 3, "switch_threshold": 10.0})
    s = orchestrate(model, tr)
    evs = list(s.events())
    kinds = [ev["kind"] for ev in evs]
    m = s.wait(quiet=True)
    assert "switch" in kinds and "upgraded" in kinds
    per = {}
    for ev in evs:
        if ev["kind"] == "losses":
            per.setdefault(ev["worker"], []).extend(ev["losses"])
    longest = max(per.values(), key=len)      # a worker that was not promoted reports for all twelve epochs
    assert m.metrics()["switched"] is True and len(longest) == 12 and longest[-1] < longest[0]
    assert min(len(v) for v in per.values()) < 12                          # the promoted one stopped training at the switch


def test_latency_probe_feeds_the_planner(nodes):
    """All-pairs ping between the node processes, then a session planned from the measured round-trip times."""
    from oxidized_neural_orchestra_b200.runtime.node import obtain_stats

    stats = obtain_stats(nodes, rounds=4)
    assert set(stats) == set(nodes)
    for a in nodes:
        assert set(stats[a]) == set(nodes) - {a} and all(0 < v < 10**9 for v in stats[a].values())
        assert all(stats[a][b] == stats[b][a] for b in stats[a])
    model, xs, ys = _setup()
    tr = orchestra.parameter_server(nodes, 1, InlineDataset(xs, ys, 6, 3), GradientDescent(0.3), CrossEntropy(), BarrierSync(),
                                    BlockingStore(), 4, 5, seed=3, b200={"probe": True})
    m = orchestrate(model, tr).wait(quiet=True)
    assert m.stop_reason == "max_epochs" and len(m.loss_history()) == 4


def test_wire_framing_and_handshake_round_trip():
    import socket
    import struct
    import threading

    lsock = wire.listen("127.0.0.1", 0)
    port = lsock.getsockname()[1]
    got = {}

    def server():
        c, _ = lsock.accept()
        ch = wire.Channel(c)
        ch.accept_as("Node", "11111111-1111-1111-1111-111111111111")
        got["entity"] = ch.peer_entity
        got["xs"], got["ys"] = ch.recv_dataset()
        got["cmd"] = ch.recv()
        raw = c.recv(12)  # the next frame's header, byte for byte
        got["raw"] = raw
        ch.close()

    t = threading.Thread(target=server)
    t.start()
    ch = wire.connect("127.0.0.1", port)
    ch.connect_as("Orchestrator")
    assert ch.peer_entity == "Node"
    xs, ys = np.arange(10, dtype=np.float32), np.arange(4, dtype=np.float32)
    ch.send_dataset(xs, ys, chunk_bytes=16)  # 4-float chunks (share_dataset/tests.rs uses chunk_size 4)
    ch.send_command({"report_loss": {"losses": [0.5, float("nan")]}})
    ch.send_floats(wire.KIND_PARAMS, np.zeros(2, dtype=np.float32))
    t.join()
    assert got["entity"] == "Orchestrator"
    assert np.array_equal(got["xs"], xs) and np.array_equal(got["ys"], ys)
    kind, cmd = got["cmd"]
    assert kind == "control" and cmd["report_loss"]["losses"][0] == 0.5 and cmd["report_loss"]["losses"][1] is None
    assert got["raw"] == struct.pack(">QI", 12, 5)  # u64 BE length (kind + payload), u32 BE kind
    ch.close()
    lsock.close()
