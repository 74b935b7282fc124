"""A CPU rank in its own process: the host-memory twin of the GPU rank.

Local training is the C++ oracle's ``RoundTrainer``; the exchange uses ``torch.distributed`` (gloo)
with the same ownership-table semantics as the fused GPU kernel: sum the workers' residuals, the owner
of each range averages and applies the optimizer, fresh parameters reach every rank. It lets the whole
multi-process control flow (roles, rounds, early stop, stop requests, strategy switch, final gather)
run and be tested on machines without a GPU.
"""
from __future__ import annotations

import json
import time

import numpy as np
import torch
import torch.distributed as dist

from orchestra import _orchestra as core


def _opt_json(spec: dict) -> str:
    return json.dumps(spec)


class CpuRank:
    def __init__(self, plan: dict, rank: int, world: int, xs: np.ndarray, ys: np.ndarray, emit, stop_event, group=None):
        self.plan, self.rank, self.world, self.group = plan, rank, world, group
        self.emit, self.stop_event = emit, stop_event
        self.n = plan["n_params"]
        self.b200 = plan["b200"]
        self.algorithm = plan["algorithm"]
        from .gpu_rank import resolve_seed

        self.seed = resolve_seed(plan, rank, world, None, group)      # one seed for every rank, drawn by rank 0 if the plan has none
        self.worker_ranks = [w["rank"] for w in plan["workers"]]
        self.sync_workers = list(self.worker_ranks)
        self.widx = self.worker_ranks.index(rank) if rank in self.worker_ranks else None
        wspec = plan["workers"][self.widx if self.widx is not None else 0]["spec"]
        self.trainer_spec = wspec["trainer"]
        self.max_epochs, self.offline = self.trainer_spec["max_epochs"], self.trainer_spec["offline_epochs"]
        self.x_size, self.y_size = self.trainer_spec["dataset"]["x_size"], self.trainer_spec["dataset"]["y_size"]
        self.xs, self.ys = np.ascontiguousarray(xs, dtype=np.float32), np.ascontiguousarray(ys, dtype=np.float32)
        self.exact = self.b200.get("leaky_relu_exact", True)
        self.trainer = core.RoundTrainer(json.dumps(self.trainer_spec), self.xs, self.ys, self.exact) if self.widx is not None else None
        self.C = np.concatenate([core.param_gen_fill(json.dumps(l["param_gen"]), self.seed) for l in plan["layers"] if l["param_gen"]])
        self.W = self.C.copy()
        self.R = np.zeros_like(self.C)
        self.policy = core.SessionPolicy(len(self.worker_ranks))
        if plan.get("early_stopping"):
            self.policy.enable_early_stopping(plan["early_stopping"]["window"], plan["early_stopping"]["tolerance"])
        self.grad_norm_switch = False
        if plan.get("switch"):
            self.policy.enable_switch(plan["switch"]["window"], plan["switch"]["threshold"])
            # the switch may watch the norm of the averaged gradient instead of the losses
            # (orchestrator/src/sessions/switch_tracker.rs:48-62 applied to a different series)
            self.grad_norm_switch = plan["switch"].get("metric", "loss") == "grad_norm"
            self.policy.set_switch_on_metric(self.grad_norm_switch)
        self.last_norm = None
        self.switched = False
        self.stop_reason = "max_epochs"
        if self.algorithm == "parameter_server":
            sp = plan["servers"][0]["spec"]
            owners = {s["rank"]: [tuple(r) for r in s["ranges"]] for s in plan["servers"]}
            self._set_ownership([owners.get(r, []) for r in range(world)], self.worker_ranks, sp)
        else:
            from ..parallel.sync import even_ranges

            self._set_ownership(even_ranges(self.n, list(range(world)), world, align=1), self.worker_ranks,
                                {"optimizer": self.trainer_spec["optimizer"], "synchronizer": {"barrier": {}}, "store": "blocking"})

    def _set_ownership(self, ranges, workers, server_spec):
        self.own = ranges
        self.sync_workers = list(workers)
        self.async_mode = server_spec["synchronizer"] == "non_blocking" or server_spec["store"] == "wild"
        self.wild = server_spec["store"] == "wild"
        self.opts = [core.Optimizer(_opt_json(server_spec["optimizer"]), e - b) for b, e in ranges[self.rank]]

    def _all_reduce(self, arr: np.ndarray) -> np.ndarray:
        if self.world == 1:
            return arr
        t = torch.from_numpy(arr)
        dist.all_reduce(t, group=self.group)
        return t.numpy()

    def _sync(self):
        """Residual -> owners -> parameters everywhere (same contract as the fused GPU kernel)."""
        mine = self.R if self.rank in self.sync_workers else np.zeros_like(self.R)
        if self.b200.get("wire_dtype") == "f16":
            mine = core.f16_round_trip(mine)
        nw = len(self.sync_workers)
        if self.async_mode:
            # each push is applied on its own, in rank order (non_blocking.rs:21-31); the blocking store
            # still divides by the number of workers, the wild store does not (wild/shard.rs:43-58)
            table = np.zeros((self.world, self.n), dtype=np.float32)
            table[self.rank] = mine
            table = self._all_reduce(table)
            for wr in self.sync_workers:
                g = table[wr] if self.wild else table[wr] / nw
                for k, (b, e) in enumerate(self.own[self.rank]):
                    self.C[b:e] = self.opts[k].step(self.C[b:e], g[b:e])
        else:
            total = self._all_reduce(mine.copy())
            avg = total / nw
            self.last_norm = float(np.sqrt(np.sum(avg.astype(np.float64) ** 2)))     # every rank holds the same vector
            for k, (b, e) in enumerate(self.own[self.rank]):
                self.C[b:e] = self.opts[k].step(self.C[b:e], avg[b:e])
        fresh = np.zeros_like(self.C)
        for b, e in self.own[self.rank]:
            fresh[b:e] = self.C[b:e]
        self.C = self._all_reduce(fresh)
        self.W = self.C.copy()
        self.R[:] = 0.0

    def _exchange(self, vec):
        v = torch.tensor(vec, dtype=torch.float64)
        if self.world == 1:
            return v.numpy().reshape(1, -1)
        out = [torch.empty_like(v) for _ in range(self.world)]
        dist.all_gather(out, v, group=self.group)
        return torch.stack(out).numpy()

    def _decide(self, losses):
        nl = self.offline + 1
        vec = [float("nan")] * nl + [1.0 if self.stop_event.is_set() else 0.0]
        for i, l in enumerate(losses[:nl]):
            vec[i] = l
        table = self._exchange(vec)
        decision = 0
        for wi, wr in enumerate(self.worker_ranks):
            if wr not in self.sync_workers:
                continue
            ls = [float(x) for x in table[wr, :nl] if not np.isnan(x)]
            if not ls:
                continue
            if any(not np.isfinite(x) for x in ls):
                if self.rank == 0:
                    self.emit({"kind": "error", "worker": wi, "losses": [], "text": "worker reported a non-finite loss"})
                self.stop_reason = "error"
                return 1
            if self.rank == 0:
                self.emit({"kind": "losses", "worker": wi, "losses": ls, "text": ""})
            d = self.policy.on_losses(wi, ls)
            decision = max(decision, d) if d != 2 else (decision or 2)
        if table[:, nl].max() > 0:
            self.stop_reason = "stopped"
            return 1
        if decision == 1:
            self.stop_reason = "early_stopping"
        return decision

    def _switch(self):
        acts = self.plan["switch"]["post_actions"]
        promoted = [a["rank"] for a in acts if a["action"] == "upgrade"]
        remaining = [a["rank"] for a in acts if a["action"] == "switch"]
        if self.rank == 0:
            self.emit({"kind": "switch", "worker": 0, "losses": [], "text": ""})
        epochs_done = self.trainer.epochs_done if self.trainer is not None else 0
        for pr in promoted:
            box = [(self.xs, self.ys)] if self.rank == pr else [None]
            if self.world > 1:
                dist.broadcast_object_list(box, src=pr, group=self.group)
            px, py = box[0]
            rows = px.size // self.x_size
            if self.rank in remaining:
                lo, hi = core.dataset_partitions(rows, len(remaining))[remaining.index(self.rank)]
                self.xs = np.concatenate([self.xs, px[lo * self.x_size:hi * self.x_size]])
                self.ys = np.concatenate([self.ys, py[lo * self.y_size:hi * self.y_size]])
            self.policy.worker_left(self.worker_ranks.index(pr))
        ranges = [[] for _ in range(self.world)]
        spec = None
        for a in acts:
            if a["action"] == "upgrade":
                ranges[a["rank"]] = [tuple(x) for x in a["ranges"]]
                spec = a["spec"]
        if self.rank in promoted:
            self.trainer, self.widx = None, None
        elif self.rank in remaining:
            ts = next(a["trainer_spec"] for a in acts if a["action"] == "switch")
            self.trainer = core.RoundTrainer(json.dumps(ts), self.xs, self.ys, self.exact)
            self._epoch_base = 0 if self.b200.get("switch_resets_progress") else epochs_done
        self._set_ownership(ranges, remaining, spec)
        self.switched = True
        if self.rank == 0:
            for pr in promoted:
                self.emit({"kind": "upgraded", "worker": self.worker_ranks.index(pr), "losses": [], "text": ""})

    def run(self) -> dict:
        epoch = 0
        t0 = time.perf_counter()
        rounds = 0
        while epoch < self.max_epochs:
            nep = min(self.max_epochs - epoch, self.offline + 1)
            losses = []
            if self.trainer is not None:
                # the trainer counts its own epochs; after a switch that carries progress it starts at 0
                # again, so the remaining budget is enforced here
                self.W, self.R, losses, _ = self.trainer.train(self.W, self.R)
                losses = list(losses)[:nep]
            self._sync()
            rounds += 1
            epoch += nep
            decision = self._decide(losses)
            if decision == 1:
                break
            if decision == 0 and self.grad_norm_switch and not self.switched and self.last_norm is not None:
                decision = int(self.policy.on_metric(self.last_norm))
            if decision == 2 and self.algorithm == "strategy_switch" and not self.switched:
                self._switch()
        if self.rank == 0:
            pass
        self.emit({"kind": "complete", "worker": 0, "losses": [], "text": self.stop_reason})
        return {"params": self.C.copy() if self.rank == 0 else None,
                "metrics": {"rounds": rounds, "wall_s": time.perf_counter() - t0, "switched": self.switched}}
