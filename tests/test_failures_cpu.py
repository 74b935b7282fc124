"""Failure detection with the failure made on the host: a node process that dies, a barrier member that
leaves, a peer that stops answering on the control channel. Nothing here touches a GPU.

Reference behaviour being matched: a worker io error ends the session with an error event
(orchestrator/src/sessions/worker_listener.rs:99-104, event_listener.rs:128-132); a departing barrier
member never deadlocks the others (parameter_server/src/synchronization/barrier.rs:30-38).
"""
import os
import threading
import time

import numpy as np
import pytest

import orchestra
from orchestra import Sequential, orchestrate
from orchestra import _orchestra as core
from orchestra.activations import Softmax, Tanh
from orchestra.arch import Dense
from orchestra.datasets import InlineDataset
from orchestra.initialization import XavierUniform
from orchestra.loss_fns import CrossEntropy
from orchestra.optimizers import GradientDescent
from oxidized_neural_orchestra_b200.runtime import wire
from oxidized_neural_orchestra_b200.runtime.launch import spawn_nodes

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_dyn_barrier_survivors_pass_when_a_member_leaves():
    b = core.DynBarrier(3)
    leaders, passed = [], []

    def member(i, rounds):
        for _ in range(rounds):
            leaders.append(bool(b.wait()))
            passed.append(i)
        if rounds < 3:
            b.leave()

    ts = [threading.Thread(target=member, args=(i, 3 if i < 2 else 1)) for i in range(3)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(timeout=20)
    assert not any(t.is_alive() for t in ts), "a survivor is stuck behind the member that left"
    assert b.size() == 2
    assert sum(leaders) == 3 and len(passed) == 7       # one leader per generation, 3 + 3 + 1 passages


def test_a_node_that_dies_mid_run_ends_the_session_with_an_error():
    procs, addrs = spawn_nodes(3, "cpu", once=True)
    try:
        rng = np.random.default_rng(0)
        xs = rng.random((60, 6), dtype=np.float32)
        ys = np.eye(3, dtype=np.float32)[rng.integers(0, 3, 60)]
        model = Sequential([Dense(5, XavierUniform(), Tanh()), Dense(3, XavierUniform(), Softmax())])
        tr = orchestra.all_reduce(addrs, InlineDataset(xs, ys, 6, 3), GradientDescent(0.01), CrossEntropy(), 1_000_000, 5,
                                  seed=1, b200={"comm_timeout_s": 5.0})
        s = orchestrate(model, tr)
        box = {}

        def waiter():
            try:
                box["model"] = s.wait(quiet=True)
            except RuntimeError as e:
                box["error"] = str(e)

        t = threading.Thread(target=waiter, daemon=True)
        t.start()
        time.sleep(2.0)                 # let a few rounds go through
        procs[2].kill()                 # the exact child this test started
        t.join(timeout=90)
        assert not t.is_alive(), "the session hung after a node died"
        assert "error" in box and ("lost" in box["error"] or "Error" in box["error"] or "error" in box["error"])
    finally:
        for p in procs:
            p.kill()
        for p in procs:
            p.wait(timeout=30)


def test_a_node_that_stops_answering_is_dropped_after_the_heartbeat_timeout():
    """The process stays alive and its connection open, it just stops running (SIGSTOP): only the missing
    heartbeats tell the orchestrator."""
    import signal

    procs, addrs = spawn_nodes(2, "cpu", once=True)
    try:
        rng = np.random.default_rng(0)
        xs = rng.random((60, 6), dtype=np.float32)
        ys = np.eye(3, dtype=np.float32)[rng.integers(0, 3, 60)]
        model = Sequential([Dense(5, XavierUniform(), Tanh()), Dense(3, XavierUniform(), Softmax())])
        tr = orchestra.all_reduce(addrs, InlineDataset(xs, ys, 6, 3), GradientDescent(0.01), CrossEntropy(), 1_000_000, 5,
                                  seed=1, b200={"comm_timeout_s": 4.0, "heartbeat_s": 0.25, "heartbeat_timeout_s": 2.0})
        s = orchestrate(model, tr)
        box = {}

        def waiter():
            try:
                box["model"] = s.wait(quiet=True)
            except RuntimeError as e:
                box["error"] = str(e)

        t = threading.Thread(target=waiter, daemon=True)
        t.start()
        time.sleep(1.5)
        procs[1].send_signal(signal.SIGSTOP)       # exactly the child started above
        t.join(timeout=60)
        assert not t.is_alive(), "the session hung behind a silent node"
        assert "silent" in box.get("error", "") or "lost" in box.get("error", "") or "rror" in box.get("error", "")
    finally:
        for p in procs:
            try:
                p.send_signal(signal.SIGCONT)
            except OSError:
                pass
            p.kill()
        for p in procs:
            p.wait(timeout=30)


def test_control_channel_reports_a_silent_peer_instead_of_blocking():
    lsock = wire.listen("127.0.0.1", 0)
    port = lsock.getsockname()[1]
    ch = wire.connect("127.0.0.1", port)
    conn, _ = lsock.accept()            # accepted, but the peer never answers the handshake
    t0 = time.perf_counter()
    with pytest.raises((TimeoutError, ConnectionError, OSError)):
        ch.recv(timeout=0.3)
    assert time.perf_counter() - t0 < 5.0
    conn.close()
    ch.close()
    lsock.close()


@pytest.mark.parametrize("sync", ["barrier", "non_blocking"])
def test_a_native_node_that_dies_mid_run_ends_the_session_with_an_error(sync):
    """Native node processes exchanging over their TCP mesh: one of them is killed mid-run; the others' receiver /
    transmitter threads see the closed socket (or run into the communication time limit), the session reports an
    error and nothing hangs."""
    import socket
    import subprocess

    from orchestra.store import BlockingStore
    from orchestra.sync import BarrierSync, NonBlockingSync

    exe = os.path.join(ROOT, "bin", "ono-node")
    if not os.path.exists(exe):
        pytest.skip("bin/ono-node is not built")
    ports = []
    for _ in range(3):
        with socket.socket() as sk:
            sk.bind(("127.0.0.1", 0))
            ports.append(sk.getsockname()[1])
    procs = [subprocess.Popen([exe, "--port", str(p), "--device", "cpu"], env=dict(os.environ, ONO_LOG="error")) for p in ports]
    try:
        for p in ports:
            for _ in range(200):
                try:
                    socket.create_connection(("127.0.0.1", p), timeout=0.2).close()
                    break
                except OSError:
                    time.sleep(0.05)
        rng = np.random.default_rng(0)
        xs = rng.random((60, 6), dtype=np.float32)
        ys = np.eye(3, dtype=np.float32)[rng.integers(0, 3, 60)]
        model = Sequential([Dense(5, XavierUniform(), Tanh()), Dense(3, XavierUniform(), Softmax())])
        tr = orchestra.parameter_server([f"127.0.0.1:{p}" for p in ports], 1, InlineDataset(xs, ys, 6, 3), GradientDescent(0.01), CrossEntropy(),
                                        BarrierSync() if sync == "barrier" else NonBlockingSync(), BlockingStore(), 1_000_000, 5, seed=1,
                                        b200={"comm_timeout_s": 5.0})
        s = orchestrate(model, tr)
        box = {}

        def waiter():
            try:
                box["model"] = s.wait(quiet=True)
            except RuntimeError as e:
                box["error"] = str(e)

        t = threading.Thread(target=waiter, daemon=True)
        t.start()
        time.sleep(1.5)                 # let some rounds go through
        procs[2].kill()                 # the exact child this test started
        t.join(timeout=90)
        assert not t.is_alive(), "the session hung after a node died"
        assert "error" in box, box
    finally:
        for p in procs:
            p.kill()
        for p in procs:
            p.wait(timeout=30)
