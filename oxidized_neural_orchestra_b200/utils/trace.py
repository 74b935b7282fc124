"""Run tracing and metrics records.

The reference's observability is the training-event stream plus stderr logs
(orchestrator/src/sessions/mod.rs:47-70, node/README.md:56-70); its benchmark harness derives
``samples_per_sec`` and friends from wall clocks (benchmarks/issue/metrics.py:11-32). Here every rank can
additionally write

* a Chrome-trace JSON (``chrome://tracing`` / Perfetto): host spans taken with ``perf_counter`` and device
  spans taken with CUDA events on the training stream, one process row per rank;
* a JSONL metrics file with one record per epoch: loss, samples/s (device-timed), mean/max step time,
  strategy in force, bytes copied per step.

Both are off unless a path is configured (``b200.trace_path`` / ``b200.metrics_path``; ``{rank}`` in the path
is replaced by the rank number, otherwise ``.rank<N>`` is appended for ranks above 0).
"""
from __future__ import annotations

import json
import time
from contextlib import contextmanager


def _path_for(path: str, rank: int) -> str:
    if "{rank}" in path:
        return path.replace("{rank}", str(rank))
    return path if rank == 0 else f"{path}.rank{rank}"


class Tracer:
    def __init__(self, path: str | None, rank: int = 0):
        self.path = _path_for(path, rank) if path else None
        self.rank = rank
        self.t0 = time.perf_counter()
        self.events: list[dict] = []
        self._device: list[tuple[str, object, object, dict]] = []
        self._anchor = None

    @property
    def on(self) -> bool:
        return self.path is not None

    def _us(self, t: float) -> float:
        return (t - self.t0) * 1e6

    @contextmanager
    def span(self, name: str, **args):
        """Host span (wall clock)."""
        if not self.on:
            yield
            return
        t = time.perf_counter()
        try:
            yield
        finally:
            self.events.append({"name": name, "ph": "X", "pid": self.rank, "tid": 0, "ts": self._us(t),
                                "dur": (time.perf_counter() - t) * 1e6, "args": args})

    def instant(self, name: str, **args):
        if self.on:
            self.events.append({"name": name, "ph": "i", "s": "p", "pid": self.rank, "tid": 0,
                                "ts": self._us(time.perf_counter()), "args": args})

    def device_anchor(self, stream) -> None:
        """Record the event device spans are measured from, and the host time it corresponds to."""
        if not self.on or self._anchor is not None:
            return
        import torch

        ev = torch.cuda.Event(enable_timing=True)
        ev.record(stream)
        ev.synchronize()
        self._anchor = (ev, time.perf_counter())

    def device_span(self, name: str, start_event, end_event, **args) -> None:
        """Device span between two already recorded CUDA events; resolved when the trace is written."""
        if self.on:
            self._device.append((name, start_event, end_event, args))

    def write(self) -> str | None:
        if not self.on:
            return None
        evs = list(self.events)
        if self._anchor is not None:
            a_ev, a_t = self._anchor
            for name, s, e, args in self._device:
                try:
                    ts = self._us(a_t) + a_ev.elapsed_time(s) * 1e3
                    dur = s.elapsed_time(e) * 1e3
                except RuntimeError:
                    continue
                evs.append({"name": name, "ph": "X", "pid": self.rank, "tid": 1, "ts": ts, "dur": dur, "args": args})
        meta = [{"name": "process_name", "ph": "M", "pid": self.rank, "args": {"name": f"rank {self.rank}"}},
                {"name": "thread_name", "ph": "M", "pid": self.rank, "tid": 0, "args": {"name": "host"}},
                {"name": "thread_name", "ph": "M", "pid": self.rank, "tid": 1, "args": {"name": "training stream"}}]
        with open(self.path, "w") as f:
            json.dump({"traceEvents": meta + evs, "displayTimeUnit": "ms"}, f)
        return self.path


class MetricsSink:
    """Append-only JSONL; field names follow the reference harness where it has them
    (benchmarks/issue/results.py:16-25: ``samples_per_sec``, ``epochs_per_sec``, ``final_loss``)."""

    def __init__(self, path: str | None, rank: int = 0):
        self.path = _path_for(path, rank) if path else None
        self.rank = rank
        if self.path:
            open(self.path, "w").close()

    @property
    def on(self) -> bool:
        return self.path is not None

    def write(self, **record) -> None:
        if not self.on:
            return
        record.setdefault("rank", self.rank)
        record.setdefault("time", time.time())
        with open(self.path, "a") as f:
            f.write(json.dumps(record) + "\n")
