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
        # Resume (additive to the reference, which exports weights only): the weights come through the plan
        # (`b200.init_from` becomes inline parameter generators), the optimizer state and the position in the shuffle
        # sequence from the sidecar a previous run wrote (`b200.state_path`, CPU or GPU ranks: same file).
        state, start_epoch = None, int(b.get("start_epoch", -1))
        self._state_path = b.get("state_path") or None
        self._n_params = int(plan.get("n_params") or sum(l["n_params"] for l in plan["layers"]))
        self._opt_kind = next(iter(training_cfg["optimizer"])) if isinstance(training_cfg.get("optimizer"), dict) else "?"
        if b.get("init_state_from"):
            from ..utils.state import load_state

            state = load_state(b["init_state_from"], self._n_params)
            if start_epoch < 0:
                start_epoch = int(state["meta"].get("epochs", 0))
        self._cluster = core.LocalCluster(json.dumps(plan), xs, ys, x_size, y_size,
                                          wire="f16" if b.get("wire_dtype") == "f16" else "f32",
                                          sparse=sparse, sparse_r=ser["sparse_capable"]["r"] if sparse else 0.0,
                                          leaky_relu_exact=b.get("leaky_relu_exact", True),
                                          switch_resets_progress=b.get("switch_resets_progress", False),
                                          init_m=None if state is None else np.ascontiguousarray(state["m"], dtype=np.float32),
                                          init_v=None if state is None else np.ascontiguousarray(state["v"], dtype=np.float32),
                                          init_b1t=1.0 if state is None else float(state["adam_pows"][0]),
                                          init_b2t=1.0 if state is None else float(state["adam_pows"][1]),
                                          start_epoch=max(0, start_epoch),
                                          checkpoint_every=int(b.get("checkpoint_every", 0) or 0) if b.get("checkpoint_path") else 0)
        self._plan, self._ckpt_pattern = plan, b.get("checkpoint_path") or None
        self._cluster.start()
        self._done = False

    def stop(self):
        self._cluster.request_stop()

    def events(self):
        while not self._done:
            ev = self._cluster.next_event(200)
            if ev is None:
                continue
            if ev["kind"] == "checkpoint":       # the leading worker took a copy of the model and its optimizer state
                self._write_checkpoints()
                continue
            if ev["kind"] == "complete":
                self._write_checkpoints()
                self._done = True
            yield ev

    def _write_checkpoints(self):
        """Periodic checkpoints (`b200.checkpoint_path` / `checkpoint_every`): weights in the reference's layout plus the
        optimizer-state sidecar, the files GPU ranks write; the sidecar is complete before the weights file appears."""
        from ..utils.state import checkpoint_paths, layers_from_plan, save_state, save_tensors, weight_tensors

        while self._ckpt_pattern:
            c = self._cluster.pop_checkpoint()
            if c is None:
                break
            path, side = checkpoint_paths(self._ckpt_pattern, int(c["epochs"]))
            save_state(side, c["m"], c["v"], np.asarray(c["adam_pows"], dtype=np.float32), optimizer=self._opt_kind,
                       epochs=int(c["epochs"]), n_params=self._n_params)
            save_tensors(path, weight_tensors(layers_from_plan(self._plan), np.asarray(c["params"], dtype=np.float32)))

    def result(self):
        self._cluster.join()
        if self._state_path:
            from ..utils.state import save_state

            st = self._cluster.final_state()
            save_state(self._state_path, st["m"], st["v"], np.asarray(st["adam_pows"], dtype=np.float32),
                       optimizer=self._opt_kind, epochs=int(st["epochs"]), n_params=self._n_params)
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
