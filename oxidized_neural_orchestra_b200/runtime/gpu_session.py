"""Starting GPU ranks for a session.

Three ways a run reaches its GPUs:

* the calling process already belongs to a ``torch.distributed`` group of one process per GPU
  (``torchrun``): every process calls ``orchestrate`` with the same arguments and becomes the rank at
  its position in ``addrs`` (SPMD);
* a single ``gpu:<i>`` address: the rank runs inside the calling process;
* several ``gpu:<i>`` addresses from a plain process: one child process per GPU is launched
  (``runtime/launch.py``) and rank 0 streams the events back;
* ``host:port`` addresses: node processes that are already listening (``runtime/node.py``).
"""
from __future__ import annotations

import json
import os
import queue
import threading

import numpy as np
import torch
import torch.distributed as dist

from orchestra import _orchestra as core


class GpuHandle:
    """Run handle over a rank running in a thread of this process."""

    def __init__(self, plan: dict, rank: int, world: int, device, xs, ys, group=None):
        self.n_workers = len(plan["workers"])
        self._q: queue.Queue = queue.Queue()
        self._stop = threading.Event()
        self._err: BaseException | None = None
        self._result = None
        self._done = False

        def body():
            try:
                torch.cuda.set_device(device)
                from .gpu_run import run
                from .gpu_worker import GpuRank

                r = GpuRank(plan, rank, world, device, xs, ys, self._q.put, self._stop, group)
                self._result = run(r)
            except BaseException as e:  # surfaced by events()/result()
                self._err = e
                self._q.put({"kind": "error", "worker": 0, "losses": [], "text": f"{type(e).__name__}: {e}"})
                self._q.put({"kind": "complete", "worker": 0, "losses": [], "text": "error"})

        self._t = threading.Thread(target=body, name=f"ono-gpu-rank-{rank}", daemon=True)
        self._t.start()

    def stop(self):
        self._stop.set()

    def events(self):
        while not self._done:
            ev = self._q.get()
            if ev["kind"] == "complete":
                self._done = True
            yield ev

    def result(self):
        self._t.join()
        if self._err is not None:
            raise RuntimeError(f"GPU rank failed: {self._err}") from self._err
        params = self._result["params"]
        if params is None:
            params = np.zeros(0, dtype=np.float32)
        return params, self._result["metrics"]


def partition_for(plan: dict, rank: int, xs: np.ndarray, ys: np.ndarray, x_size: int, y_size: int):
    for w in plan["workers"]:
        if w["rank"] == rank:
            b, e = w["partition"]
            return xs[b * x_size:e * x_size], ys[b * y_size:e * y_size]
    return xs[:0], ys[:0]


def start_gpu_session(model_cfg: dict, training_cfg: dict, dataset, kind: str):
    from .session import load_dataset_arrays

    addrs = training_cfg["addrs"]
    plan = json.loads(core.adapt_configs(json.dumps(model_cfg), json.dumps(training_cfg)))
    if kind == "tcp":
        from .node import start_remote_session

        return start_remote_session(plan, model_cfg, training_cfg, dataset)
    if not torch.cuda.is_available():
        raise RuntimeError("gpu:<i> addresses need CUDA devices; use cpu:<i> addresses for CPU ranks")
    if dist.is_initialized():
        world, rank = dist.get_world_size(), dist.get_rank()
        if world != len(addrs):
            raise ValueError(f"{len(addrs)} addresses for a process group of {world} ranks")
        local = int(os.environ.get("LOCAL_RANK", rank))
        device = torch.device("cuda", local)
    elif len(addrs) == 1:
        world, rank = 1, 0
        device = torch.device("cuda", int(addrs[0].split(":", 1)[1]))
    else:
        from .launch import start_spawned_session

        return start_spawned_session(plan, model_cfg, training_cfg, dataset)
    xs, ys = load_dataset_arrays(dataset)
    px, py = partition_for(plan, rank, xs, ys, dataset.x_size, dataset.y_size)
    return GpuHandle(plan, rank, world, device, px, py)
