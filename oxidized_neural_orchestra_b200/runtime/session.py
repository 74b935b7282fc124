"""Orchestrator-side session: validates, plans, starts the ranks and relays their events.

Counterpart of orchestrator/src/lib.rs:52-89 (``train``) and orchestrator/src/sessions/session.rs.
Addresses select the backend of a run:

* ``cpu:<i>``     – in-process CPU ranks (threads) running the C++ oracle engine and strategies;
* ``gpu:<i>``     – one process per local GPU, started by this session unless the caller already runs
                    inside such a process group (``torchrun``), in which case the ranks are reused;
* ``host:port``   – a node process that is already listening there (``python -m
                    oxidized_neural_orchestra_b200.runtime.node``), as in the reference.
"""
from __future__ import annotations

import json
import queue
import threading

import numpy as np

from orchestra import _orchestra as core


def load_dataset_arrays(dataset) -> tuple[np.ndarray, np.ndarray]:
    """Samples and labels of an InlineDataset / LocalDataset as flat float32 arrays."""
    if hasattr(dataset, "samples"):
        return dataset.samples, dataset.labels
    sp = core.ensure_binary_dataset(dataset.samples_path)  # csv/tsv -> .bin (dataset_format.rs:58-86)
    lp = core.ensure_binary_dataset(dataset.labels_path)
    return np.fromfile(sp, dtype="<f4"), np.fromfile(lp, dtype="<f4")


class CpuHandle:
    """Run handle over the in-process CPU cluster."""

    def __init__(self, plan: dict, training_cfg: dict, xs, ys, x_size, y_size):
        b = plan["b200"]
        ser = training_cfg.get("serializer", "base")
        sparse = isinstance(ser, dict)
        self.n_workers = len(plan["workers"])
        self._cluster = core.LocalCluster(json.dumps(plan), xs, ys, x_size, y_size,
                                          wire="f16" if b.get("wire_dtype") == "f16" else "f32",
                                          sparse=sparse, sparse_r=ser["sparse_capable"]["r"] if sparse else 0.0,
                                          leaky_relu_exact=b.get("leaky_relu_exact", True),
                                          switch_resets_progress=b.get("switch_resets_progress", False))
        self._cluster.start()
        self._done = False

    def stop(self):
        self._cluster.request_stop()

    def events(self):
        while not self._done:
            ev = self._cluster.next_event(200)
            if ev is None:
                continue
            if ev["kind"] == "complete":
                self._done = True
            yield ev

    def result(self):
        self._cluster.join()
        return self._cluster.final_params(), {"switched": self._cluster.switched()}


def start_session(model_cfg: dict, training_cfg: dict, dataset):
    """Validate + plan (C++ core), then start the ranks. Returns a run handle."""
    addrs = training_cfg["addrs"]
    model_js, training_js = json.dumps(model_cfg), json.dumps(training_cfg)
    kinds = {a.split(":", 1)[0] if a.split(":", 1)[0] in ("cpu", "gpu") else "tcp" for a in addrs}
    if len(kinds) > 1:
        raise ValueError("addrs must all be cpu:<i>, all gpu:<i>, or all host:port")
    kind = kinds.pop() if kinds else "tcp"
    if kind == "cpu":
        plan = json.loads(core.adapt_configs(model_js, training_js))
        xs, ys = load_dataset_arrays(dataset)
        return CpuHandle(plan, training_cfg, xs, ys, dataset.x_size, dataset.y_size)
    from .gpu_session import start_gpu_session

    return start_gpu_session(model_cfg, training_cfg, dataset, kind)
