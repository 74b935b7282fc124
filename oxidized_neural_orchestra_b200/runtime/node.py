"""The role-agnostic node process and the orchestrator's view of it.

Like the reference's ``node`` binary (node/src/main.rs:27-54, node/src/router.rs:79-220) a node
listens on ``HOST:PORT``, waits for an orchestrator, and only learns what it is (worker, parameter
server, both) from the spec it is handed. One session at a time; after ``disconnect`` it goes back to
listening.

    PORT=40000 python -m oxidized_neural_orchestra_b200.runtime.node [--device gpu --gpu 0 | --device cpu]

Session protocol on the control channel (wire.py): ``connect/accept`` handshake, ``create_node{spec}``
followed by the node's dataset partition (``share_dataset_size`` / data chunks / ``eof`` twice), then
the node streams ``event`` messages (rank 0 relays every worker's losses), honours ``stop_after_epoch``,
finishes with ``done`` and serves ``request_params`` until ``disconnect``.
"""
from __future__ import annotations

import argparse
import json
import os
import queue
import sys
import threading
import time
import uuid

import numpy as np

from . import wire


def run_rank(job: dict, xs: np.ndarray, ys: np.ndarray, emit, stop_event, device_kind: str, gpu: int | None = None) -> dict:
    """Join the process group described by ``job`` and run this node's rank to completion."""
    import torch
    import torch.distributed as dist

    from orchestra import _orchestra as core

    rank, world = job["rank"], job["world"]
    plan = job.get("plan") or json.loads(core.adapt_configs(json.dumps(job["model"]), json.dumps(job["training"]),
                                                          json.dumps(job.get("stats") or {}) if job.get("stats") else ""))
    own_group = False
    if world > 1 and not dist.is_initialized():
        import datetime

        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = job["master_addr"], str(job["master_port"])
        # a collective whose peer died ends with an error after this long instead of waiting forever
        limit = datetime.timedelta(seconds=float(plan["b200"].get("comm_timeout_s", 300.0)))
        if device_kind == "gpu":
            torch.cuda.set_device(gpu or 0)
            dist.init_process_group("nccl", rank=rank, world_size=world, timeout=limit,
                                    device_id=torch.device("cuda", gpu or 0))
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world, timeout=limit)
        own_group = True
    try:
        if device_kind == "gpu":
            from .gpu_run import run
            from .gpu_worker import GpuRank

            dev = torch.device("cuda", gpu or 0)
            torch.cuda.set_device(dev)
            return run(GpuRank(plan, rank, world, dev, xs, ys, emit, stop_event))
        from .cpu_rank import CpuRank

        return CpuRank(plan, rank, world, xs, ys, emit, stop_event).run()
    finally:
        if own_group:
            dist.destroy_process_group()


def serve(host: str, port: int, device_kind: str, gpu: int | None, once: bool = False, ready: threading.Event | None = None) -> None:
    """Accept loop of a node (router.rs:79-113)."""
    node_id = str(uuid.uuid4())
    lsock = wire.listen(host, port)
    if ready is not None:
        ready.set()
    while True:
        conn, _ = lsock.accept()
        ch = wire.Channel(conn)
        try:
            ch.accept_as("Node", node_id)
        except (ConnectionError, OSError, ValueError):
            ch.close()  # a port probe or a stranger: not a session
            continue
        if ch.peer_entity == "Node":      # a peer measuring latency: answer its pings (stat_service.rs:107-152)
            _answer_pings(ch)
            ch.close()
            continue
        try:
            _session(ch, device_kind, gpu, lsock, node_id)
        except (ConnectionError, OSError) as e:
            print(f"[ono-node {host}:{port}] session ended: {e}", file=sys.stderr)
        finally:
            ch.close()
        if once:
            lsock.close()
            return


def _answer_pings(ch: wire.Channel) -> None:
    try:
        while True:
            kind, msg = ch.recv(timeout=30)
            if kind == "control" and msg == "ping":
                ch.send_command("pong")
            else:
                return
    except (ConnectionError, OSError, TimeoutError):
        return


def _serve_ping_stats(lsock, node_id: str, req: dict) -> dict:
    """All-pairs latency probe (node/src/stat_service.rs:69-152): connect to ``addrs`` and time ``rounds`` ping/pong
    round trips with each, while answering the pings of ``incoming`` peers that connect to this node."""
    rounds, incoming = int(req["rounds"]), int(req["incoming"])
    threads = []

    def responder():
        try:
            conn, _ = lsock.accept()
        except OSError:
            return
        c = wire.Channel(conn)
        try:
            c.accept_as("Node", node_id)
            _answer_pings(c)
        except (ConnectionError, OSError, ValueError):
            pass
        c.close()

    lsock.settimeout(30)
    for _ in range(incoming):
        t = threading.Thread(target=responder, daemon=True)
        t.start()
        threads.append(t)
    rtts = {}
    for addr in req["addrs"]:
        host, port = addr.rsplit(":", 1)
        try:
            c = wire.connect(host, int(port), timeout=10)
            c.connect_as("Node", node_id)
            samples = []
            for _ in range(rounds):
                t0 = time.perf_counter_ns()
                c.send_command("ping")
                kind, msg = c.recv(timeout=10)
                if msg != "pong":
                    raise ConnectionError("expected pong")
                samples.append(time.perf_counter_ns() - t0)
            c.send_command("disconnect")
            c.close()
            rtts[addr] = {"min": float(min(samples)), "max": float(max(samples)), "mean": float(sum(samples) / len(samples))}
        except (ConnectionError, OSError, TimeoutError) as e:
            print(f"[ono-node] ping {addr}: {e}", file=sys.stderr)
    for t in threads:
        t.join()
    lsock.settimeout(None)
    return {"stats_response": {"stats": {"ping": {"rtts": rtts}}}}


def obtain_stats(addrs: list[str], rounds: int = 10) -> dict:
    """Orchestrator side of the probe (orchestrator/src/configs/stat_requester.rs:32-72): node i pings nodes 0..i-1 and
    accepts the n-i-1 later ones. Returns ``{addr: {peer: max_rtt_ns}}`` (symmetric), the planner's input."""
    chs = []
    for a in addrs:
        host, port = a.rsplit(":", 1)
        ch = wire.connect(host, int(port))
        ch.connect_as("Orchestrator")
        chs.append(ch)
    n = len(addrs)
    for i, ch in enumerate(chs):
        ch.send_command({"stats_request": {"ping": {"addrs": addrs[:i], "rounds": rounds, "incoming": n - i - 1}}})
    stats: dict = {a: {} for a in addrs}
    for i, ch in enumerate(chs):
        _, msg = ch.recv(timeout=120)
        body = msg.get("stats_response", {}).get("stats") if isinstance(msg, dict) else None
        rtts = body.get("ping", {}).get("rtts", {}) if isinstance(body, dict) else {}
        for peer, st in rtts.items():
            stats[addrs[i]][peer] = int(st["max"])
            stats[peer][addrs[i]] = int(st["max"])
        ch.send_command("disconnect")
        ch.close()
    return stats


def _session(ch: wire.Channel, device_kind: str, gpu: int | None, lsock=None, node_id: str = "") -> None:
    while True:
        kind, msg = ch.recv(timeout=None)
        if kind != "control":
            continue
        if msg == "disconnect":
            return
        if isinstance(msg, dict) and "stats_request" in msg:
            req = msg["stats_request"].get("ping") if isinstance(msg["stats_request"], dict) else None
            if req is not None and lsock is not None:
                ch.send_command(_serve_ping_stats(lsock, node_id, req))
            else:
                ch.send_command({"stats_response": {"stats": []}})
            continue
        if msg == "ping":
            ch.send_command("pong")
            continue
        if isinstance(msg, dict) and "create_node" in msg:
            job = msg["create_node"]["spec"]
            xs, ys = ch.recv_dataset()
            stop_event = threading.Event()
            send_lock = threading.Lock()
            result: dict = {}

            def emit(ev):
                if job["rank"] == 0 or ev["kind"] in ("complete", "error"):
                    with send_lock:
                        ch.send_command({"event": ev})

            def body():
                try:
                    result.update(run_rank(job, xs, ys, emit, stop_event, device_kind, gpu))
                except BaseException as e:
                    emit({"kind": "error", "worker": 0, "losses": [], "text": f"{type(e).__name__}: {e}"})
                    emit({"kind": "complete", "worker": 0, "losses": [], "text": "error"})
                with send_lock:
                    ch.send_command("done")

            t = threading.Thread(target=body, daemon=True)
            t.start()
            # liveness: a counter the orchestrator watches; a node whose process is alive but whose rank is stuck
            # keeps beating, so the beat also carries whether the training thread is still running
            hb_every = float(job["training"].get("b200", {}).get("heartbeat_s", 2.0) or 0.0)
            hb_stop = threading.Event()

            def beat():
                k = 0
                while not hb_stop.wait(hb_every):
                    k += 1
                    try:
                        with send_lock:
                            ch.send_command({"event": {"kind": "heartbeat", "worker": job["rank"], "losses": [],
                                                       "text": json.dumps({"beat": k, "training": t.is_alive()})}})
                    except OSError:
                        return

            if hb_every > 0:
                threading.Thread(target=beat, daemon=True).start()
            # serve the orchestrator while training runs and afterwards (all_reduce.rs:137-152)
            while True:
                kind, m = ch.recv(timeout=None)
                if kind != "control":
                    continue
                if m == "stop_after_epoch":
                    stop_event.set()
                elif m == "abort":
                    # another node was lost: stop at the next boundary; a collective that is already waiting
                    # for the dead peer ends by its own time limit and reports through body()
                    stop_event.set()
                elif m == "request_params":
                    t.join()
                    p = result.get("params")
                    with send_lock:
                        ch.send_floats(wire.KIND_PARAMS, p if p is not None else np.zeros(0, dtype=np.float32))
                        ch.send_command({"event": {"kind": "metrics", "worker": 0, "losses": [],
                                                   "text": json.dumps(_jsonable(result.get("metrics", {})))}})
                elif m == "disconnect":
                    stop_event.set()
                    hb_stop.set()
                    t.join()
                    return


def _jsonable(d: dict) -> dict:
    out = {}
    for k, v in d.items():
        if isinstance(v, (np.floating, np.integer)):
            v = v.item()
        out[k] = v
    return out


class RemoteHandle:
    """Orchestrator side of a run on listening nodes (orchestrator/src/sessions/session.rs:57-167)."""

    def __init__(self, plan: dict, model_cfg: dict, training_cfg: dict, xs: np.ndarray, ys: np.ndarray, x_size: int, y_size: int,
                 stats: dict | None = None):
        addrs = training_cfg["addrs"]
        self.n_workers = len(plan["workers"])
        self._q: queue.Queue = queue.Queue()
        self._chs: list[wire.Channel] = []
        self._done_nodes = 0
        self._params = None
        self._metrics: dict = {}
        self._closed = False
        self._events_finished = False
        self._failed = False
        b200 = training_cfg.get("b200") or {}
        self._hb_timeout = float(b200.get("heartbeat_timeout_s", 0.0) or 0.0)   # 0 = do not judge liveness by beats
        self._last_seen = [time.monotonic()] * len(addrs)
        self._node_done = [False] * len(addrs)
        master_port = wire.free_port()
        master_addr = addrs[0].rsplit(":", 1)[0]
        part = {w["rank"]: w["partition"] for w in plan["workers"]}
        my_id = str(uuid.uuid4())
        for rank, addr in enumerate(addrs):
            host, port = addr.rsplit(":", 1)
            ch = wire.connect(host, int(port))
            ch.connect_as("Orchestrator", my_id)
            if ch.peer_entity != "Node":
                raise ConnectionError(f"{addr} answered as {ch.peer_entity}, expected a node")
            self._chs.append(ch)
        for rank, ch in enumerate(self._chs):
            job = {"model": model_cfg, "training": training_cfg, "rank": rank, "world": len(addrs), "stats": stats, "plan": plan,
                   "master_addr": "127.0.0.1" if master_addr in ("localhost", "127.0.0.1") else master_addr,
                   "master_port": master_port}
            ch.send_command({"create_node": {"spec": job}})
            b, e = part.get(rank, (0, 0))
            ch.send_dataset(xs[b * x_size:e * x_size], ys[b * y_size:e * y_size])
        self._threads = [threading.Thread(target=self._reader, args=(r, ch), daemon=True) for r, ch in enumerate(self._chs)]
        for t in self._threads:
            t.start()
        if self._hb_timeout > 0:
            threading.Thread(target=self._watchdog, daemon=True).start()

    def _watchdog(self):
        """Declare a node dead after `heartbeat_timeout_s` of silence (its process may hang without closing the
        connection) and end the session the way a lost connection does."""
        while not self._closed and not self._events_finished:
            time.sleep(min(1.0, self._hb_timeout / 4))
            now = time.monotonic()
            for r, seen in enumerate(self._last_seen):
                if not self._node_done[r] and not self._failed and now - seen > self._hb_timeout:
                    self._node_done[r] = True
                    self._q.put(("event", r, {"kind": "error", "worker": r, "losses": [],
                                               "text": f"node {r} lost: silent for {now - seen:.1f} s"}))
                    self._q.put(("done", r, None))
                    self._abort(r)
                    self._chs[r].close()

    def _reader(self, rank: int, ch: wire.Channel):
        try:
            while True:
                kind, msg = ch.recv(timeout=None)
                if kind == "params":
                    if rank == 0:
                        self._params = np.array(msg, dtype=np.float32)
                    continue
                if msg == "done":
                    self._node_done[rank] = True
                    self._q.put(("done", rank, None))
                    if rank != 0:
                        return
                    continue
                self._last_seen[rank] = time.monotonic()
                if isinstance(msg, dict) and "event" in msg:
                    ev = msg["event"]
                    if ev["kind"] == "heartbeat":
                        continue
                    if ev["kind"] == "metrics":
                        self._metrics = json.loads(ev["text"])
                        self._q.put(("metrics", rank, None))
                        return
                    self._q.put(("event", rank, ev))
        except (ConnectionError, OSError) as e:
            self._q.put(("event", rank, {"kind": "error", "worker": rank, "losses": [], "text": f"node {rank} lost: {e}"}))
            self._q.put(("done", rank, None))
            self._abort(rank)

    def _abort(self, lost_rank: int):
        """Tell the surviving nodes that a member is gone (the reference ends the whole session on a worker
        io error: orchestrator/src/sessions/event_listener.rs:128-132)."""
        self._failed = True
        for r, ch in enumerate(self._chs):
            if r != lost_rank:
                try:
                    ch.send_command("abort")
                except OSError:
                    pass

    def close(self):
        """Drop every control connection (nodes go back to listening)."""
        for ch in self._chs:
            try:
                ch.send_command("disconnect")
            except OSError:
                pass
            ch.close()
        self._closed = True

    def stop(self):
        for ch in self._chs:
            try:
                ch.send_command("stop_after_epoch")
            except OSError:
                pass

    def events(self):
        if self._events_finished:
            return
        done, complete_ev = 0, None
        while done < len(self._chs):
            what, rank, ev = self._q.get()
            if what == "done":
                done += 1
            elif what == "event":
                if ev["kind"] == "complete":
                    if rank == 0:
                        complete_ev = ev
                    continue
                yield ev
        self._events_finished = True
        if self._failed:
            complete_ev = {"kind": "complete", "worker": 0, "losses": [], "text": "error"}
        yield complete_ev or {"kind": "complete", "worker": 0, "losses": [], "text": "error"}

    def result(self):
        if not self._closed:
            self._chs[0].send_command("request_params")
            while True:
                what, rank, ev = self._q.get()
                if what == "metrics":
                    break
            for ch in self._chs:
                try:
                    ch.send_command("disconnect")
                except OSError:
                    pass
                ch.close()
            self._closed = True
        return (self._params if self._params is not None else np.zeros(0, dtype=np.float32)), self._metrics


def start_remote_session(plan, model_cfg, training_cfg, dataset):
    from .session import load_dataset_arrays

    xs, ys = load_dataset_arrays(dataset)
    stats = None
    if (training_cfg.get("b200") or {}).get("probe"):
        # measure the nodes' pairwise latency first and let the planner place servers / order the ring by it
        from orchestra import _orchestra as core

        stats = obtain_stats(training_cfg["addrs"])
        plan = json.loads(core.adapt_configs(json.dumps(model_cfg), json.dumps(training_cfg), json.dumps(stats)))
    return RemoteHandle(plan, model_cfg, training_cfg, xs, ys, dataset.x_size, dataset.y_size, stats)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description="role-agnostic training node (awaits a spec from an orchestrator)")
    ap.add_argument("--host", default=os.environ.get("HOST", "127.0.0.1"))
    ap.add_argument("--port", type=int, default=int(os.environ["PORT"]) if "PORT" in os.environ else None)
    ap.add_argument("--device", choices=("cpu", "gpu"), default=None)
    ap.add_argument("--gpu", type=int, default=None)
    ap.add_argument("--once", action="store_true", help="serve one session, then exit")
    a = ap.parse_args(argv)
    if a.port is None:
        ap.error("a port is required (--port or the PORT environment variable)")
    kind = a.device
    if kind is None:
        import torch

        kind = "gpu" if torch.cuda.is_available() else "cpu"
    print(f"[ono-node] listening on {a.host}:{a.port} ({kind})", file=sys.stderr)
    serve(a.host, a.port, kind, a.gpu, once=a.once)


if __name__ == "__main__":
    main()
