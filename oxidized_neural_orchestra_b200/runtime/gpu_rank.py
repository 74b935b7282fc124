"""One GPU rank of a run: worker, parameter server, or both, decided by the plan it is handed.

Counterpart of the reference's role runtimes (worker/src/workers/{all_reduce,parameter_server}.rs,
parameter_server/src/service/pserver.rs, node/src/router.rs:166-341) rebuilt around HBM-resident
flat buffers in a symmetric NVLink window and fused kernels:

    per mini-batch   H2D of the batch (pinned host memory, copy stream) -> CUDA graph of
                     {gather/cast, forward GEMMs, fused softmax-loss, dgrad/wgrad GEMMs, bias grads,
                      [round cadence: local SGD + residual accumulate]}
    per sync point   one fused kernel: reduce-scatter of gradients into the owners + average +
                     optimizer + all-gather of fresh parameters (ownership table = strategy)

Ranks run SPMD: every rank derives the same plan and applies the same policy to the same gathered
losses, so stop / early-stop / switch decisions need no messaging beyond one small all-gather per round.
"""
from __future__ import annotations

import ctypes as C
import json
import threading
import time

import numpy as np
import torch
import torch.distributed as dist

from orchestra import _orchestra as core

from ..models.engine import GpuEngine
from ..ops import _lib
from ..ops import elementwise as ew
from ..parallel import sync as S
from ..parallel.symmetric import SymmetricWindow, WindowLayout

ACT_NAME = {"sigmoid": "sigmoid", "tanh": "tanh", "relu": "relu", "re_l_u": "relu"}


def engine_layers_from_plan(plan: dict) -> list[dict]:
    """LayerSpec documents -> the engine's layer descriptions."""
    out = []
    for l in plan["layers"]:
        (kind, body), = l["spec"].items()
        act = body.get("act_fn")
        if act is None:
            a = None
        elif isinstance(act, str):
            a = (act, 0.0)
        else:
            (an, ab), = act.items()
            a = (ACT_NAME[an], float(ab.get("amp", ab.get("slope", 0.0))))
        if kind == "dense":
            out.append({"kind": "dense", "in": body["dim"][0], "out": body["dim"][1], "act": a})
        elif kind == "conv":
            out.append({"kind": "conv", "input_dim": body["input_dim"], "kernel_dim": body["kernel_dim"],
                        "stride": body["stride"], "padding": body["padding"], "act": a})
        else:
            out.append({"kind": "pool", "input_dim": body["input_dim"], "filter_size": body["filter_size"],
                        "stride": body["stride"], "padding": body["padding"], "act": a})
    return out


def optimizer_cfg(spec: dict) -> S.OptimizerCfg:
    (name, b), = spec.items()
    lr = b.get("learning_rate", b.get("lr"))
    if name == "gradient_descent":
        return S.OptimizerCfg("sgd", lr)
    if name == "gradient_descent_with_momentum":
        return S.OptimizerCfg("momentum", lr, mu=b.get("momentum", b.get("mu", 0.0)))
    return S.OptimizerCfg("adam", lr, b1=b.get("beta1", b.get("b1", 0.9)), b2=b.get("beta2", b.get("b2", 0.999)),
                          eps=b.get("epsilon", b.get("eps", 1e-8)))


def resolve_seed(plan: dict, rank: int, world: int, device=None, group=None) -> int:
    """The run's seed, the same on every rank. A plan without a seed (the public API's default) gets one drawn by
    rank 0 and broadcast: initial parameters are generated per rank from (seed, element index), so ranks that each
    picked their own would start from different models."""
    if plan.get("seed") is not None:
        return int(plan["seed"])
    seed = int.from_bytes(__import__("os").urandom(4), "little") if rank == 0 else 0
    if world > 1 and dist.is_initialized():
        box = [seed]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group,
                                   device=device)
        seed = int(box[0])
    return seed


def snap_ranges(ranges_per_rank: list[list[tuple[int, int]]], n_pad: int) -> list[list[tuple[int, int]]]:
    """Move every interior boundary down to a multiple of 4 elements (the kernels work on float4), the
    same rule on both sides of a boundary so the ranges still partition ``[0, n_pad)``."""
    out = []
    n_true_end = max((e for rs in ranges_per_rank for _, e in rs), default=0)
    for rs in ranges_per_rank:
        cur = []
        for b, e in rs:
            b2 = b // 4 * 4
            e2 = n_pad if e == n_true_end else e // 4 * 4
            if e2 > b2:
                cur.append((b2, e2))
        out.append(cur)
    return out


def snap_to_row_blocks(ranges_per_rank, plan_layers, engine_layers, n, n_pad, rows=128):
    """Move every interior ownership boundary down to a multiple of ``rows`` rows of the weight matrix it falls into
    (or to the start of that layer's bias block), so that a weight-gradient tile pushed by a GEMM epilogue never
    straddles two owners. The same rule applies to both sides of a boundary, so the ranges still partition the vector."""
    marks = []                                     # (begin, end, row_len) of weight blocks, (begin, end, 0) of biases
    for pl, l in zip(plan_layers, engine_layers):
        if l["kind"] != "dense":
            continue
        w0 = pl["offset"]
        marks.append((w0, w0 + l["in"] * l["out"], l["out"]))
        marks.append((w0 + l["in"] * l["out"], w0 + l["in"] * l["out"] + l["out"], 0))

    def snap(b):
        if b >= n:
            return n_pad
        for lo, hi, row in marks:
            if lo <= b < hi:
                return lo + ((b - lo) // (rows * row)) * rows * row if row else lo
        return b

    out = []
    for rs in ranges_per_rank:
        cur = []
        for b, e in rs:
            b2, e2 = (snap(b) if b else 0), snap(e)
            if e2 > b2:
                cur.append((b2, e2))
        out.append(cur)
    return out


class BatchFeeder:
    """Stages mini-batches from pinned host memory to the device on a copy stream, one step ahead.

    The dataset partition stays in (pinned) host memory, as on the reference's workers; every step's inputs
    cross PCIe inside the timed region: the host sends the shuffled row indices of the next batch, and a gather
    kernel on the copy stream pulls exactly those rows out of host memory while the GPU works on the current batch.
    """

    def __init__(self, xs: np.ndarray, ys: np.ndarray, x_size: int, y_size: int, batch: int, device, seed: int,
                 device_resident: bool = False):
        self.rows = xs.size // x_size
        self.x_size, self.y_size, self.batch = x_size, y_size, batch
        self.device = device
        self.seed = seed
        self.host_x = torch.from_numpy(np.ascontiguousarray(xs.reshape(self.rows, x_size)))
        self.host_y = torch.from_numpy(np.ascontiguousarray(ys.reshape(self.rows, y_size)))
        self.device_resident = device_resident
        self.nslots = 2
        if device_resident:
            self.dev_all_x = self.host_x.to(device)
            self.dev_all_y = self.host_y.to(device)
        else:
            self.host_x, self.host_y = self.host_x.pin_memory(), self.host_y.pin_memory()
            self.pin_idx = [torch.empty(batch, dtype=torch.int32).pin_memory() for _ in range(self.nslots)]
            self.dev_idx = [torch.zeros(batch, dtype=torch.int32, device=device) for _ in range(self.nslots)]
        self.dev_x = [torch.zeros(batch, x_size, device=device) for _ in range(self.nslots)]
        self.dev_y = [torch.zeros(batch, y_size, device=device) for _ in range(self.nslots)]
        self.copy_stream = torch.cuda.Stream(device=device)
        self.ready = [torch.cuda.Event() for _ in range(self.nslots)]
        self.consumed = [torch.cuda.Event() for _ in range(self.nslots)]
        self.h2d_bytes_per_step = batch * (x_size + y_size) * 4
        self._perm = None
        self._epoch = -1

    def steps_per_epoch(self) -> int:
        return (self.rows + self.batch - 1) // self.batch

    def _indices(self, epoch: int, step: int) -> torch.Tensor:
        epoch += getattr(self, "epoch_offset", 0)
        if epoch != self._epoch:
            g = torch.Generator()
            g.manual_seed((self.seed * 1000003 + epoch) & 0x7FFFFFFFFFFFFFFF)
            self._perm = torch.randperm(self.rows, generator=g)
            self._epoch = epoch
        lo = step * self.batch
        return self._perm[lo:min(self.rows, lo + self.batch)]

    def stage(self, slot: int, epoch: int, step: int) -> int:
        """Gather the batch on the host and start its H2D copy. Returns the number of rows."""
        idx = self._indices(epoch, step)
        n = idx.numel()
        if self.device_resident:
            with torch.cuda.stream(self.copy_stream):
                self.copy_stream.wait_event(self.consumed[slot])
                di = idx.to(self.device, non_blocking=True)
                torch.index_select(self.dev_all_x, 0, di, out=self.dev_x[slot][:n])
                torch.index_select(self.dev_all_y, 0, di, out=self.dev_y[slot][:n])
                self.ready[slot].record(self.copy_stream)
            return n
        # The dataset partition is pinned: the gather kernel reads the batch's rows straight out of host memory over
        # PCIe on the copy stream (host-to-device copy and gather in one pass), so the host thread only ships the index
        # vector and never touches the rows themselves.
        self.consumed[slot].synchronize()  # the slot's index buffer is free again
        self.pin_idx[slot][:n].copy_(idx)
        with torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(self.consumed[slot])
            self.dev_idx[slot][:n].copy_(self.pin_idx[slot][:n], non_blocking=True)
            ew.rows(self.host_x, idx=self.dev_idx[slot], n_rows=n, dst=self.dev_x[slot], stream=self.copy_stream)
            ew.rows(self.host_y, idx=self.dev_idx[slot], n_rows=n, dst=self.dev_y[slot], stream=self.copy_stream)
            self.ready[slot].record(self.copy_stream)
        return n
