"""Launcher convenience: start one node process per local device and run a session on them.

The reference brings its nodes up by hand or with docker compose (docker/compose_up.py, Makefile:57-68);
on one box the equivalent is to fork ``runtime.node`` once per GPU (or per CPU rank), each listening on
a free loopback port, and to hand those addresses to the ordinary ``host:port`` session.
"""
from __future__ import annotations

import os
import socket
import subprocess
import sys
import time

from . import wire


def spawn_nodes(n: int, device: str, gpus: list[int] | None = None, once: bool = True) -> tuple[list[subprocess.Popen], list[str]]:
    procs, addrs = [], []
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    env = dict(os.environ)
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    for i in range(n):
        port = wire.free_port()
        cmd = [sys.executable, "-m", "oxidized_neural_orchestra_b200.runtime.node", "--host", "127.0.0.1", "--port",
               str(port), "--device", device] + (["--once"] if once else [])
        if device == "gpu":
            cmd += ["--gpu", str(gpus[i] if gpus else i)]
        procs.append(subprocess.Popen(cmd, env=env))
        addrs.append(f"127.0.0.1:{port}")
    deadline = time.time() + 120
    for a, p in zip(addrs, procs):
        host, port = a.rsplit(":", 1)
        while True:
            if p.poll() is not None:
                raise RuntimeError(f"node process for {a} exited with code {p.returncode}")
            try:
                socket.create_connection((host, int(port)), timeout=1).close()
                break
            except OSError:
                if time.time() > deadline:
                    raise RuntimeError(f"node {a} did not start listening")
                time.sleep(0.2)
    return procs, addrs


class SpawnedHandle:
    """A RemoteHandle that also owns (and reaps) the node processes it started."""

    def __init__(self, inner, procs):
        self._inner, self._procs = inner, procs
        self.n_workers = inner.n_workers

    def stop(self):
        self._inner.stop()

    def events(self):
        return self._inner.events()

    def result(self):
        try:
            return self._inner.result()
        finally:
            for p in self._procs:
                try:
                    p.wait(timeout=60)
                except subprocess.TimeoutExpired:
                    p.kill()


def start_spawned_session(plan, model_cfg, training_cfg, dataset, device: str = "gpu"):
    """``gpu:<i>`` (or ``cpuproc:<i>``) addresses from a plain process: fork the nodes, then connect."""
    import json

    from orchestra import _orchestra as core

    from .node import RemoteHandle
    from .session import load_dataset_arrays

    addrs = training_cfg["addrs"]
    gpus = [int(a.split(":", 1)[1]) for a in addrs] if device == "gpu" else None
    procs, node_addrs = spawn_nodes(len(addrs), device, gpus)
    # Ranks are positions in `addrs`; the plan is recomputed by every node from the same documents,
    # so the node addresses replace the symbolic ones consistently everywhere.
    cfg = dict(training_cfg)
    cfg["addrs"] = node_addrs
    plan2 = json.loads(core.adapt_configs(json.dumps(model_cfg), json.dumps(cfg)))
    xs, ys = load_dataset_arrays(dataset)
    try:
        inner = RemoteHandle(plan2, model_cfg, cfg, xs, ys, dataset.x_size, dataset.y_size)
    except BaseException:
        for p in procs:
            p.kill()
        raise
    return SpawnedHandle(inner, procs)


def main(argv=None) -> None:
    """``python -m oxidized_neural_orchestra_b200.runtime.launch --nodes N [--base-port P] [--device cpu|gpu] [--native]``:
    bring up N listening nodes on this machine and keep them running until interrupted (the local stand-in for
    the reference's ``make cluster-up``: docker/gen_compose.py:44-151 starts node-i on port 40000+i)."""
    import argparse
    import signal

    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("--nodes", type=int, default=3)
    ap.add_argument("--base-port", type=int, default=40000)
    ap.add_argument("--device", choices=("cpu", "gpu"), default=None)
    ap.add_argument("--native", action="store_true", help="start the C++ ono-node executable instead of the Python node")
    ap.add_argument("--pid-file", default=None, help="write this launcher's pid here (SIGTERM to it stops the nodes it started)")
    a = ap.parse_args(argv)
    if a.pid_file:
        with open(a.pid_file, "w") as f:
            f.write(str(os.getpid()))
    device = a.device
    if device is None:
        import torch

        device = "gpu" if torch.cuda.is_available() else "cpu"
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    env = dict(os.environ)
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    procs = []
    for i in range(a.nodes):
        port = a.base_port + i
        if a.native:
            cmd = [os.path.join(root, "bin", "ono-node"), "--port", str(port)] + (["--gpu", str(i)] if device == "gpu" else ["--device", "cpu"])
        else:
            cmd = [sys.executable, "-m", "oxidized_neural_orchestra_b200.runtime.node", "--host", "127.0.0.1", "--port", str(port),
                   "--device", device] + (["--gpu", str(i)] if device == "gpu" else [])
        procs.append(subprocess.Popen(cmd, env=env))
        print(f"node-{i}: 127.0.0.1:{port} ({device})", file=sys.stderr)
    signal.signal(signal.SIGTERM, lambda *_: sys.exit(0))
    try:
        for p in procs:
            p.wait()
    except (KeyboardInterrupt, SystemExit):
        pass
    finally:
        for p in procs:      # exactly the children started above
            if p.poll() is None:
                p.terminate()
        if a.pid_file and os.path.exists(a.pid_file):
            os.remove(a.pid_file)
        for p in procs:
            try:
                p.wait(timeout=10)
            except subprocess.TimeoutExpired:
                p.kill()


if __name__ == "__main__":
    main()
