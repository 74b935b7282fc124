"""Strategy builders, ``orchestrate`` and the session objects of the ``orchestra`` package
(orchestra-py/src/training.rs:51-301, orchestra-py/src/session.rs:49-306)."""
from __future__ import annotations

import json
import sys
import time
from typing import Any, Sequence

from . import _api as A


def _addrs(addrs: Any) -> list[str]:
    if isinstance(addrs, str) or not isinstance(addrs, (list, tuple)):
        raise TypeError("addrs must be a list of strings")
    out = []
    for a in addrs:
        if not isinstance(a, str):
            raise TypeError("addrs must be a list of strings")
        out.append(a)
    return out


def _need(obj: Any, classes: tuple, what: str):
    if not isinstance(obj, classes):
        raise TypeError(f"{what} must be one of: {', '.join(c.__name__ for c in classes)}")
    return obj


class PyTrainingConfig:
    """The training half of a run: what ``training.json`` describes, plus the dataset object."""

    def __init__(self, cfg: dict, dataset):
        self._cfg = cfg
        self.dataset = dataset

    def to_config(self, with_data: bool = True) -> dict:
        cfg = dict(self._cfg)
        cfg["dataset"] = self.dataset.to_config(with_data)
        if not with_data and isinstance(self.dataset, A.InlineDataset):
            rows = self.dataset.samples.size // self.dataset.x_size
            cfg["dataset"]["src"]["inline"]["rows"] = int(rows)
        return cfg

    def to_json(self, with_data: bool = True) -> str:
        return json.dumps(self.to_config(with_data))

    def __repr__(self):
        return f"PyTrainingConfig({json.dumps(self._cfg)})"


def _common(addrs, dataset, optimizer, loss_fn, max_epochs, batch_size, serializer, offline_epochs, seed,
            early_stopping_tolerance, b200) -> dict:
    _need(dataset, (A.InlineDataset, A.LocalDataset), "dataset")
    _need(optimizer, (A.GradientDescent, A.GradientDescentWithMomentum, A.Adam), "optimizer")
    _need(loss_fn, (A.Mse, A.CrossEntropy), "loss_fn")
    if serializer is not None:
        _need(serializer, (A.BaseSerializer, A.SparseSerializer), "serializer")
    A._positive_int(max_epochs, "max_epochs")
    A._positive_int(batch_size, "batch_size")
    if isinstance(offline_epochs, bool) or not isinstance(offline_epochs, int) or offline_epochs < 0:
        raise ValueError("offline_epochs must be a non-negative integer")
    if seed is not None and (isinstance(seed, bool) or not isinstance(seed, int) or seed < 0):
        raise ValueError("seed must be a non-negative integer")
    if early_stopping_tolerance is not None:
        t = A._float(early_stopping_tolerance, "early_stopping_tolerance")
        if t <= 0.0 or t != t:  # convert.rs:31-41 rejects zero and negative tolerances
            raise ValueError("early_stopping_tolerance must be a positive number")
    cfg = {
        "addrs": _addrs(addrs),
        "serializer": (serializer or A.BaseSerializer()).to_config(),
        "optimizer": optimizer.to_config(),
        "loss_fn": loss_fn.to_config(),
        "batch_size": batch_size,
        "max_epochs": max_epochs,
        "offline_epochs": offline_epochs,
        "seed": seed,
        "early_stopping": None if early_stopping_tolerance is None else {"tolerance": float(early_stopping_tolerance)},
    }
    if b200:
        cfg["b200"] = dict(b200)
    return cfg


def parameter_server(addrs, nservers, dataset, optimizer, loss_fn, sync, store, max_epochs, batch_size,
                     serializer=None, offline_epochs=0, seed=None, early_stopping_tolerance=None,
                     b200: dict | None = None) -> PyTrainingConfig:
    """Parameter-server strategy: ``nservers`` of ``addrs`` own the (sharded) parameters."""
    cfg = _common(addrs, dataset, optimizer, loss_fn, max_epochs, batch_size, serializer, offline_epochs, seed,
                  early_stopping_tolerance, b200)
    _need(sync, (A.BarrierSync, A.NonBlockingSync), "sync")
    _need(store, (A.BlockingStore, A.WildStore), "store")
    cfg["algorithm"] = {"parameter_server": {"nservers": A._positive_int(nservers, "nservers"),
                                             "synchronizer": sync.to_config(), "store": store.to_config()}}
    return PyTrainingConfig(cfg, dataset)


def all_reduce(addrs, dataset, optimizer, loss_fn, max_epochs, batch_size, serializer=None, offline_epochs=0,
               seed=None, early_stopping_tolerance=None, b200: dict | None = None) -> PyTrainingConfig:
    """Ring all-reduce strategy: every address is a worker."""
    cfg = _common(addrs, dataset, optimizer, loss_fn, max_epochs, batch_size, serializer, offline_epochs, seed,
                  early_stopping_tolerance, b200)
    cfg["algorithm"] = "all_reduce"
    return PyTrainingConfig(cfg, dataset)


def strategy_switch(addrs, nservers, dataset, optimizer, loss_fn, sync, store, max_epochs, batch_size,
                    serializer=None, offline_epochs=0, seed=None, early_stopping_tolerance=None,
                    b200: dict | None = None) -> PyTrainingConfig:
    """Starts as all-reduce; once the tracked metric plateaus, ``nservers`` workers become servers."""
    cfg = _common(addrs, dataset, optimizer, loss_fn, max_epochs, batch_size, serializer, offline_epochs, seed,
                  early_stopping_tolerance, b200)
    _need(sync, (A.BarrierSync, A.NonBlockingSync), "sync")
    _need(store, (A.BlockingStore, A.WildStore), "store")
    cfg["algorithm"] = {"strategy_switch": {"nservers": A._positive_int(nservers, "nservers"),
                                            "synchronizer": sync.to_config(), "store": store.to_config()}}
    return PyTrainingConfig(cfg, dataset)


class TrainedModel:
    """Result of a run: flat parameters in model order plus the per-epoch loss history."""

    def __init__(self, params, model_cfg: dict, input_size: int, loss_history: list[float], stop_reason: str,
                 metrics: dict | None = None):
        self._params = params
        self._model_cfg = model_cfg
        self._input_size = input_size
        self._loss_history = list(loss_history)
        self.stop_reason = stop_reason
        self._metrics = metrics or {}

    def weights(self) -> list[float]:
        return [float(v) for v in self._params]

    def weights_array(self):
        """The same parameters as a float32 numpy array (no copy per element)."""
        return self._params

    def loss_history(self) -> list[float]:
        return list(self._loss_history)

    def metrics(self) -> dict:
        """Device-timed per-step records collected by the ranks (additive to the reference's API)."""
        return dict(self._metrics)

    def save_safetensors(self, path) -> None:
        from . import _orchestra as core
        import os

        core.save_safetensors(os.fspath(path), json.dumps(self._model_cfg), self._input_size, self._params)


class _Progress:
    """Per-epoch mean loss over the workers that reported it (session.rs:115-153), one line per epoch."""

    def __init__(self, max_epochs: int, workers: int, quiet: bool):
        self.max_epochs, self.workers, self.quiet = max_epochs, workers, quiet
        self.per_epoch: dict[int, list[float]] = {}
        self.next_epoch_of: dict[int, int] = {}
        self.history: list[float] = []
        self.live = workers

    def worker_left(self):
        self.live = max(1, self.live - 1)
        self._flush()

    def add(self, worker: int, losses: Sequence[float]):
        for l in losses:
            e = self.next_epoch_of.get(worker, 0)
            self.next_epoch_of[worker] = e + 1
            self.per_epoch.setdefault(e, []).append(float(l))
        self._flush()

    def _flush(self, final: bool = False):
        while True:
            e = len(self.history)
            got = self.per_epoch.get(e)
            if not got or (len(got) < self.live and not final):
                return
            mean = sum(got) / len(got)
            self.history.append(mean)
            if not self.quiet:
                print(f"epoch {e + 1}/{self.max_epochs} avg_loss={mean:.6f}", file=sys.stderr)


class Session:
    """A running training session (orchestra-py/src/session.rs:191-306)."""

    def __init__(self, handle, model_cfg: dict, training: PyTrainingConfig):
        self._h = handle
        self._model_cfg = model_cfg
        self._training = training
        self._result: TrainedModel | None = None

    def stop(self) -> None:
        """Ask every worker to stop at its next round boundary."""
        self._h.stop()

    def events(self):
        """Iterate raw training events (dicts) until the run completes."""
        return self._h.events()

    def wait(self, quiet: bool | None = None) -> TrainedModel:
        if self._result is not None:
            return self._result
        cfg = self._training._cfg
        if quiet is None:
            quiet = not sys.stderr.isatty() and bool(int(__import__("os").environ.get("ONO_QUIET", "1")))
        prog = _Progress(cfg["max_epochs"], self._h.n_workers, quiet)
        stop_reason = "max_epochs"
        error = None
        for ev in self._h.events():
            k = ev["kind"]
            if k == "losses":
                prog.add(ev["worker"], ev["losses"])
            elif k == "upgraded":
                prog.worker_left()
            elif k == "error":
                error = ev.get("text") or "worker error"
            elif k == "complete":
                stop_reason = ev.get("text") or stop_reason
        prog._flush(final=True)
        if error is not None and stop_reason == "error":
            if hasattr(self._h, "close"):
                self._h.close()
            raise RuntimeError(f"training failed: {error}")
        params, metrics = self._h.result()
        self._result = TrainedModel(params, self._model_cfg, self._training.dataset.x_size, prog.history, stop_reason,
                                    metrics)
        return self._result


def orchestrate(model: A.Sequential, training: PyTrainingConfig) -> Session:
    """Validate both configs, assign roles, start the run and return its session."""
    if not isinstance(model, A.Sequential):
        raise TypeError("model must be a Sequential")
    if not isinstance(training, PyTrainingConfig):
        raise TypeError("training must come from parameter_server(), all_reduce() or strategy_switch()")
    from oxidized_neural_orchestra_b200.runtime.session import start_session

    model_cfg = model.to_config()
    handle = start_session(model_cfg, training.to_config(with_data=False), training.dataset)
    return Session(handle, model_cfg, training)
