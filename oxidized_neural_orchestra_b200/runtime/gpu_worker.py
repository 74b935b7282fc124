"""The SPMD training loop of one GPU rank (see gpu_rank.py for the pieces it is made of)."""
from __future__ import annotations

import ctypes as C
import json
import math
import os
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
from .gpu_rank import (BatchFeeder, engine_layers_from_plan, optimizer_cfg, resolve_seed, snap_ranges,
                       snap_to_row_blocks)


def _up(n, m=16):
    return (n + m - 1) // m * m


class GpuRank:
    def __init__(self, plan: dict, rank: int, world: int, device: torch.device, xs: np.ndarray, ys: np.ndarray,
                 emit, stop_event: threading.Event, group=None, warmup_steps: int = 0):
        self.plan, self.rank, self.world, self.dev, self.group = plan, rank, world, device, group
        self.emit, self.stop_event = emit, stop_event
        b = plan["b200"]
        self.b200 = b
        self.cadence = b.get("sync_every", "round")
        self.tile = b.get("tile_dtype", "tf32")
        self.algorithm = plan["algorithm"]
        self.n = plan["n_params"]
        self.n_pad = _up(self.n, 16)
        self.seed = resolve_seed(plan, rank, world, device, group)
        self.x_size = plan["layers"][0]["input_size"]
        self.y_size = plan["layers"][-1]["output_size"]
        self.worker_ranks = [w["rank"] for w in plan["workers"]]
        self.widx = self.worker_ranks.index(rank) if rank in self.worker_ranks else None
        self.server_ranks = [s["rank"] for s in plan["servers"]]
        self.warmup_steps = warmup_steps
        self.launches_per_step = 0
        self.step_events: list[torch.cuda.Event] = []
        self.step_wall: list[float] = []
        self.switched = False
        self.use_nvls = False
        self.push_active = self.stage_active = self.wire16_push = self.apply_active = False
        self.wire_copies, self.wire_transport = None, "staged"
        self.pull_staged, self.pull_plan = False, None
        self.buckets, self.bucket_after, self.stage_buckets, self.stage_after = [], {}, [], {}
        self.stream = torch.cuda.Stream(device=device)
        self.comm_stream = torch.cuda.Stream(device=device)
        # the staged gradient push may spread its transfers over several streams (one copy engine each), by destination;
        # one stream is the default: two and three measured 2 % slower on four GPUs (4.71 / 4.74 ms against 4.63 ms per step)
        self.push_streams = [self.comm_stream] + [torch.cuda.Stream(device=device)
                                                  for _ in range(max(0, int(os.environ.get("ONO_PUSH_STREAMS", "1")) - 1))]
        wspec = plan["workers"][self.widx if self.widx is not None else 0]["spec"]
        self.trainer = wspec["trainer"]
        self.max_epochs = self.trainer["max_epochs"]
        self.offline = self.trainer["offline_epochs"]
        self.loss_kind = self.trainer["loss_fn"]
        self.local_lr = optimizer_cfg(self.trainer["optimizer"]).lr
        if self.algorithm == "parameter_server":
            self.opt = optimizer_cfg(plan["servers"][0]["spec"]["optimizer"])
            sp = plan["servers"][0]["spec"]
            self.async_ps = sp["synchronizer"] == "non_blocking" or sp["store"] == "wild"
            self.wild = sp["store"] == "wild"
        else:
            self.opt = optimizer_cfg(self.trainer["optimizer"])
            self.async_ps = self.wild = False
        self._alloc_window()
        self._init_params()
        self._build_engine(xs, ys)
        self._policy()
        self._set_ownership_initial()

    # ------------------------------------------------------------------------------------------
    def _alloc_window(self):
        lay = WindowLayout()
        lay.add("params", self.n_pad, torch.float32)
        lay.add("grads", self.n_pad, torch.float32)
        # Compressed gradient wire of the reference's cadence (comms/src/handles/compressor.rs:71-118,
        # worker/src/middlewares/server_cluster.rs:85-104, comms/src/sparse/protocol.rs:57-86): what a rank sends this
        # round leaves `grads` (its residual keeps the rest) and is published in its window as 16-bit values: the dense
        # `wire16` region and, with the sparse serializer, an ascending (index, f16) list that owners read instead
        # whenever it is the smaller encoding (at most a third of the entries: 6 bytes per pair against 2 per element).
        ser = self.plan.get("serializer", "base")
        self.sparse_r = float(ser["sparse_capable"]["r"]) if isinstance(ser, dict) else None
        wd_round = self.b200.get("wire_dtype", "auto")
        self.compress = self.cadence == "round" and (wd_round in ("f16", "bf16") or self.sparse_r is not None)
        self.cwire = "bf16" if wd_round == "bf16" else "f16"
        if self.compress:
            lay.add("wire16", self.n_pad, torch.bfloat16 if self.cwire == "bf16" else torch.float16)
            if self.sparse_r is not None:
                self.sp_cap = max(16, self.n_pad // 3)
                lay.add("sp_idx", self.sp_cap, torch.int32)
                lay.add("sp_val", self.sp_cap, torch.float16)
                lay.add("sp_cnt", 64, torch.int32)
        # Gradient wire between GPUs. The reference always ships gradients as f16 (comms/src/handles/compressor.rs:104-118,
        # decoded at comms/src/handles/worker.rs:84-101). In step cadence the default here is a bf16 wire (f32 range, so
        # the small gradients of a loss normalised by batch x outputs do not underflow); "f16" gives the reference's
        # format, "f32" the uncompressed wire. One GPU has no wire: its gradients stay f32.
        wd = self.b200.get("wire_dtype", "auto")
        self.wire16 = None
        gp = self.b200.get("grad_push", "auto")
        if self.cadence == "step" and self.world > 1 and wd != "f32" and gp != "reduce":
            self.wire16 = "f16" if wd == "f16" else "bf16"
        lays = engine_layers_from_plan(self.plan)
        dense_only = all(l["kind"] == "dense" for l in lays)
        ar_mode = self.b200.get("allreduce", "auto")
        # 16-bit push (the default data path of a dense model on several GPUs): the weight-gradient GEMMs store their
        # tiles as 16-bit values straight into the slab that the owner of those rows keeps for this rank, so the
        # reduce-scatter rides on backward and the owner reduces `world` local slabs. Slab q of a window holds rank q's
        # gradients, indexed like the flat parameter vector.
        # transport of the pushed tiles: "staged" = local 16-bit gradient vector + copy-engine transfers that overlap with
        # backward (default); "direct" = the epilogues' TMA stores target the owner's window themselves
        self.wire_transport = "direct" if gp == "direct" else "staged"
        self.push16 = (self.wire16 is not None and gp in ("auto", "on", "direct") and dense_only and not self.async_ps and
                       ar_mode in ("auto", "twoshot", "nvls"))
        if self.wire16 is not None:
            self.nslabs = self.world if self.push16 else 1
            lay.add("slab16", self.nslabs * self.n_pad, torch.float16 if self.wire16 == "f16" else torch.bfloat16)
        # f32 gradient push (opt-in, "reduce"): the weight-gradient GEMMs add their output tiles into the f32 accumulator
        # of the rank that owns those rows with TMA reduce-adds
        aligned = dense_only and all(l["out"] % 4 == 0 for l in lays) and all(pl["offset"] % 4 == 0 for pl in self.plan["layers"])
        forced_single = os.environ.get("ONO_PUSH_SINGLE", "0") == "1"
        self.push = (self.cadence == "step" and not self.push16 and gp in ("on", "reduce") and aligned and
                     (self.world > 1 or forced_single))
        if self.push:
            lay.add("acc", self.n_pad, torch.float32)
        # the ring all-reduce (the reference's algorithm, worker/src/middlewares/worker_ring.rs:112-204) circulates chunks
        # through an accumulation window of its own
        # Staged reduce-scatter (step cadence, several GPUs): while backward runs, a few SMs copy the peers' finished
        # gradient ranges this rank owns into local staging buffers (bulk async copies through shared memory), and the
        # fused optimizer kernel afterwards reads every worker's gradient from local HBM instead of over NVLink.
        self.stage = (self.cadence == "step" and self.b200.get("grad_stage", "auto") == "on" and self.world > 1 and
                      not self.push and self.wire16 is None)
        if self.stage:
            lay.add("stage_ready", self.world * _lib.STAGE_BUCKETS, torch.int32)
        # Staged parameter pull (opt-in: `param_pull: "staged"`; bf16 tiles, every rank an owner): owners publish their fresh
        # shadow slices with copy engines at the start of the next step, layer by layer, and announce each layer in the
        # consumers' flag tables; the forward GEMM of a layer waits (bounded) for its flags, so the pull hides behind the
        # layers before it. On 2 GPUs it measured slower than the pull from the fused kernel (8 x 8192 MLP: 4.12 ms
        # against 3.94 ms per step: the transfers share the copy engines with the gradient push and delay it), so the
        # fused kernel stays the default.
        self.pull_wanted = (self.push16 and self.wire_transport == "staged" and self.tile == "bf16" and
                            self.b200.get("param_pull", "auto") == "staged")
        if self.pull_wanted:
            lay.add("pull_ready", self.world * _lib.STAGE_BUCKETS, torch.int32)
        self.ring_wanted = self.b200.get("allreduce") == "ring" and self.algorithm != "parameter_server"
        if self.ring_wanted:
            lay.add("ring_acc", self.n_pad, torch.float32)
        if self.tile == "bf16":
            lay.add("params_bf16", self.n_pad, torch.bfloat16)
        needs_async = self.async_ps
        if self.algorithm == "strategy_switch":
            for a in self.plan["switch"]["post_actions"]:
                if a["action"] == "upgrade":
                    needs_async = a["spec"]["synchronizer"] == "non_blocking" or a["spec"]["store"] == "wild"
        if needs_async:
            lay.add("m", self.n_pad, torch.float32)
            lay.add("v", self.n_pad, torch.float32)
            lay.add("locks", _lib.MAX_RANGES * 512, torch.int32)
        self.layout = lay
        self.win = SymmetricWindow(lay.size, self.dev, self.group)
        self.C = lay.tensor(self.win, "params")
        self.G = lay.tensor(self.win, "grads")
        self.grad_region = "grads"
        if self.compress:
            self.wire16_t = lay.tensor(self.win, "wire16")
            self.wire = None                      # f32 form of the wire, only for the exchanges that read a local buffer
            self.wire_thr = torch.zeros(1, device=self.dev)
            self.wire_sent = torch.zeros(1, dtype=torch.int64, device=self.dev)
            self.wire_bytes = torch.zeros(1, dtype=torch.int64, device=self.dev)     # read from peers by this rank's lifts
            self.wire_rounds = 0
            if self.sparse_r is not None:
                self.sp_idx, self.sp_val = lay.tensor(self.win, "sp_idx"), lay.tensor(self.win, "sp_val")
                self.sp_cnt = lay.tensor(self.win, "sp_cnt")
                self.sp_acc = torch.zeros(self.n_pad, device=self.dev)
                self.sp_scratch = torch.zeros((self.n_pad + 1023) // 1024, dtype=torch.int32, device=self.dev)
                self.sp_tick = torch.zeros(1, device=self.dev)
        self.shadow = lay.tensor(self.win, "params_bf16") if self.tile == "bf16" else None
        if needs_async:
            self.m_win, self.v_win = lay.tensor(self.win, "m"), lay.tensor(self.win, "v")
        z = lambda n, dt=torch.float32: torch.zeros(n, dtype=dt, device=self.dev)
        self.m_loc, self.v_loc = z(self.n_pad), z(self.n_pad)
        self.adam_pows = torch.ones(2, device=self.dev)
        self.epoch_words = torch.zeros(1024, dtype=torch.int32, device=self.dev)
        self.sync_status = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.sumsq = torch.zeros(1, dtype=torch.float64, device=self.dev)
        if self.stage:
            self.stage_buf = [None if q == self.rank else torch.zeros(self.n_pad, device=self.dev) for q in range(self.world)]
            self.stage_step = torch.zeros(1, dtype=torch.int32, device=self.dev)
            self.stage_sms = max(1, min(int(os.environ.get("ONO_STAGE_SMS", "8")), 32))

    def _init_params(self):
        """Every rank generates the whole vector from the per-layer generators: the same Philox
        counters give the same values everywhere (replicas identical by construction)."""
        with torch.cuda.stream(self.stream):
            for l in self.plan["layers"]:
                pg = l["param_gen"]
                if pg is None:
                    continue
                dst = self.C[l["offset"]:l["offset"] + l["n_params"]]
                (kind, body), = pg.items()
                if kind == "const":
                    dst.fill_(body["value"])
                elif kind == "inline":
                    dst.copy_(torch.tensor(body["params"], dtype=torch.float32))
                else:
                    (dn, db), = body["distribution"].items()
                    fi, fo = db.get("fan_in", 1), db.get("fan_out", 0)
                    if dn == "uniform":
                        k, a, bb = "uniform", db["low"], db["high"]
                    elif dn == "uniform_inclusive":
                        k, a, bb = "uniform_inclusive", db["low"], db["high"]
                    elif dn == "normal":
                        k, a, bb = "normal", db["mean"], db["std_dev"]
                    elif dn == "xavier_uniform":
                        r = math.sqrt(6.0 / (fi + fo)); k, a, bb = "uniform_inclusive", -r, r
                    elif dn == "lecun_uniform":
                        r = math.sqrt(3.0 / fi); k, a, bb = "uniform_inclusive", -r, r
                    elif dn == "kaiming":
                        k, a, bb = "normal", 0.0, math.sqrt(2.0 / fi)
                    elif dn == "xavier":
                        k, a, bb = "normal", 0.0, math.sqrt(2.0 / (fi + fo))
                    else:
                        k, a, bb = "normal", 0.0, math.sqrt(1.0 / fi)
                    ew.philox_init(dst, seed=self.seed, index_offset=body.get("index_offset", l["offset"]), kind=k,
                                   a=a, b=bb, stream=self.stream)
            if self.shadow is not None:
                self.shadow.copy_(self.C)
        self.stream.synchronize()

    def _build_engine(self, xs, ys):
        self.engine = None
        self.feeder = None
        if self.widx is None:
            return
        layers = engine_layers_from_plan(self.plan)
        B = self.trainer["batch_size"]
        if self.cadence == "step":
            self.W, self.g = self.C, self.G
        else:
            self.W = self.C.clone()
            self.g = torch.zeros_like(self.C)
        from ..models.conv_engine import make_engine

        self.engine = make_engine(layers, batch_size=B, tile_dtype=self.tile, loss=self.loss_kind, params=self.W,
                                  grads=self.g, params_bf16=self.shadow,
                                  leaky_relu_exact=self.b200.get("leaky_relu_exact", True),
                                  bias_from_shadow=self.cadence == "step")
        self.feeder = BatchFeeder(xs, ys, self.x_size, self.y_size, B, self.dev, self.seed,
                                  device_resident=self.b200.get("data", "host") == "device")
        self.loss_pin = [torch.zeros(1, dtype=torch.float64).pin_memory() for _ in range(2)]
        self.loss_evt = [torch.cuda.Event() for _ in range(2)]
        self.graphs: dict = {}
        self.warm: set = set()
        with torch.cuda.stream(self.stream):
            from ..ops.gemm import _workspace

            _workspace(self.dev, self.stream)       # the training stream's split-K slabs exist before the first (timed) step
            self.engine.refresh(stream=self.stream)
        self.stream.synchronize()

    def _policy(self):
        p = core.SessionPolicy(len(self.worker_ranks))
        es = self.plan.get("early_stopping")
        if es:
            p.enable_early_stopping(es["window"], es["tolerance"])
        sw = self.plan.get("switch")
        if sw:
            p.enable_switch(sw["window"], sw["threshold"])
            p.set_switch_on_metric(sw.get("metric", "loss") == "grad_norm")
        self.policy = p
        self.grad_norm_switch = bool(sw) and sw.get("metric", "loss") == "grad_norm"

    # ------------------------------------------------------------------------------------------
    # ownership table = strategy
    # ------------------------------------------------------------------------------------------
    def _set_ownership_initial(self):
        W = self.world
        if self.algorithm == "parameter_server":
            owners = {s["rank"]: [tuple(r) for r in s["ranges"]] for s in self.plan["servers"]}
            # Few owners for many workers: each owner would pull (N-1) shards over its own links, while
            # the switch-side reduction delivers one reduced shard. Worth it when owners < N - 1.
            pref = self.b200.get("allreduce", "auto")
            n_owners = len(owners)
            self.use_nvls = pref == "nvls" or (pref == "auto" and n_owners < W - 1)
            self._set_ownership([owners.get(r, []) for r in range(W)], self.worker_ranks, self.opt,
                                "async" if self.async_ps else "fused", self.wild)
            return
        mode = self.b200.get("allreduce", "auto")
        if mode == "auto":
            if self.n_pad * 4 <= 256 * 1024 and W > 1:
                mode = "oneshot"
            else:
                # With every rank an owner, peer loads move (N-1)/N of the vector per GPU and direction,
                # the in-switch reduction a full vector outbound: plain P2P is the better two-shot.
                mode = "twoshot"
        if mode in ("oneshot", "ring"):      # every rank ends the exchange with the whole updated vector
            ranges = [[(0, self.n_pad)] for _ in range(W)]
        else:
            ranges = S.even_ranges(self.n_pad, list(range(W)), W)
        kind = {"oneshot": "oneshot", "twoshot": "fused", "nvls": "fused", "ring": "ring", "nccl": "nccl"}[mode]
        self.use_nvls = mode == "nvls"
        self._set_ownership(ranges, self.worker_ranks, self.opt, kind, False)

    def _snap_to_row_blocks(self, ranges):
        return snap_to_row_blocks(ranges, self.plan["layers"], engine_layers_from_plan(self.plan), self.n, self.n_pad)

    def _build_push(self):
        """Per layer: the (row range, destination view) pieces of its weight gradient and the destination of its bias
        gradient, each a view of the owner's accumulator region (a peer's window unless this rank owns it)."""
        acc_off = self.layout.offset("acc") // 4
        local = self.layout.tensor(self.win, "acc")

        def view(owner, begin, rows, cols):
            if owner == self.rank or self.win.handle is None:
                return local[begin:begin + rows * cols].view(rows, cols)
            return self.win.handle.get_buffer(owner, (rows, cols), torch.float32, acc_off + begin)

        w, b = {}, {}
        for li, pl in enumerate(self.engine.plans):
            i, o = pl.in_features, pl.out_features
            pieces = []
            for owner, rs in enumerate(self.own):
                for lo, hi in rs:
                    a0, a1 = max(lo, pl.w_off), min(hi, pl.w_off + i * o)
                    if a1 > a0:
                        r0, r1 = (a0 - pl.w_off) // o, (a1 - pl.w_off) // o
                        assert (a0 - pl.w_off) % o == 0 and (a1 - pl.w_off) % o == 0 and r0 % 8 == 0
                        pieces.append((r0, r1, view(owner, a0, r1 - r0, o)))
                    if lo <= pl.b_off < hi:
                        b[li] = view(owner, pl.b_off, 1, o).view(-1)
            w[li] = sorted(pieces, key=lambda t: t[0])
        return {"w": w, "b": b}

    def _all_ranks_agree(self, mine: bool) -> bool:
        """True when every rank says yes (ranks without an engine always do)."""
        if self.world == 1:
            return mine
        flag = torch.tensor([1.0 if mine else 0.0], device=self.dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        return bool(flag.item() > 0)

    def _plan_pre_reduce(self) -> None:
        """Ranks that own nothing take a part of every owner's share to sum (see ``parallel.sync.pre_reduce_plan``)."""
        plan_ = S.pre_reduce_plan(self.own, _lib.MAX_RANGES)
        if plan_ is not None:
            self.reduce_at, self.finish_at, self.fwd_to = plan_

    def _stripe(self, ranges):
        """Equal shares laid out as one slice of every layer per owner instead of one contiguous run of layers.

        Backward produces gradients layer by layer, last layer first. With contiguous shares the rank that owns the last
        layers ships nothing until backward reaches the first layers and then everything at once, behind the end of
        backward; with a slice of every layer per owner each rank ships the same fraction after every layer and only the
        first layer's slice is left when backward ends. Who owns how much does not change (the shares were equal), so the
        strategy is the same; only applied when the shares are (nearly) equal and the layer count fits the range table."""
        owners = [r for r, rs in enumerate(ranges) if rs]
        sizes = [sum(e - b for b, e in ranges[r]) for r in owners]
        blocks = [(l["offset"], l["offset"] + l["n_params"]) for l in self.plan["layers"] if l["n_params"] > 0]
        if len(owners) < 2 or len(blocks) > _lib.MAX_RANGES or max(sizes) - min(sizes) > 1024:
            return ranges
        out = [[] for _ in ranges]
        k = len(owners)
        for bi, (b, e) in enumerate(blocks):
            end = self.n_pad if bi == len(blocks) - 1 else e
            cuts = [b] + [max(b, min(end, (b + (end - b) * j // k) // 64 * 64)) for j in range(1, k)] + [end]
            for j, r in enumerate(owners):
                if cuts[j + 1] > cuts[j]:
                    out[r].append((cuts[j], cuts[j + 1]))
        return out

    def _build_wire16(self):
        """Where this rank's 16-bit gradients go, per layer.

        ``w[l]``: (row range, destination matrix) pieces of the weight gradient (None for a layer whose rows are not
        16-byte aligned as 16-bit values: its gradient is computed in f32 locally and cast); ``cast[l]``: (f32 source,
        16-bit destination) pairs for the bias gradient and for such unaligned layers.

        Staged transport (default): every destination is slab `rank` of this rank's OWN window; ``self.wire_copies[l]``
        then lists the (destination address in the owner's window, local source address, bytes) transfers that carry
        the ranges other ranks own, issued on the communication stream as copy-engine transfers as soon as layer l's
        gradients exist. Direct transport: the destinations are views of slab `rank` in the owners' windows and the
        GEMM epilogues store over NVLink themselves (one GEMM per owner and layer)."""
        dt = torch.float16 if self.wire16 == "f16" else torch.bfloat16
        slab0 = self.layout.offset("slab16")
        slab_elems0 = slab0 // 2 + self.rank * self.n_pad
        local = self.layout.tensor(self.win, "slab16")
        direct_transport = self.wire_transport == "direct"

        def flat(owner, begin, count):
            if owner == self.rank or self.win.handle is None or not direct_transport:
                return local[self.rank * self.n_pad + begin:self.rank * self.n_pad + begin + count]
            return self.win.handle.get_buffer(owner, (count,), dt, slab_elems0 + begin)

        w, cast, copies = {}, {}, {}
        for li, pl in enumerate(self.engine.plans):
            i, o = pl.in_features, pl.out_features
            aligned = o % 8 == 0 and pl.w_off % 8 == 0
            pieces, casts, cps = [], [], []
            for owner, rs in enumerate(self.own if direct_transport else self.reduce_at):    # staged: whoever sums the range
                for lo, hi in rs:
                    a0, a1 = max(lo, pl.w_off), min(hi, pl.b_off + o)      # the layer's whole block: weights then bias
                    if a1 > a0 and owner != self.rank and not direct_transport:
                        off = 2 * (self.rank * self.n_pad + a0)
                        cps.append((self.win.ptrs[owner] + slab0 + off, self.win.ptrs[self.rank] + slab0 + off, 2 * (a1 - a0), owner))
                    a0, a1 = max(lo, pl.w_off), min(hi, pl.w_off + i * o)
                    if a1 > a0 and direct_transport:
                        if aligned:
                            assert (a0 - pl.w_off) % o == 0 and (a1 - pl.w_off) % o == 0, "ownership must follow whole rows"
                            r0, r1 = (a0 - pl.w_off) // o, (a1 - pl.w_off) // o
                            pieces.append((r0, r1, flat(owner, a0, (r1 - r0) * o).view(r1 - r0, o)))
                        else:
                            casts.append((self.G[a0:a1], flat(owner, a0, a1 - a0)))
                    b0, b1 = max(lo, pl.b_off), min(hi, pl.b_off + o)
                    if b1 > b0 and direct_transport:
                        casts.append((self.G[b0:b1], flat(owner, b0, b1 - b0)))
            if not direct_transport:
                if aligned:
                    pieces = [(0, i, flat(self.rank, pl.w_off, i * o).view(i, o))]
                else:
                    casts.append((self.G[pl.w_off:pl.w_off + i * o], flat(self.rank, pl.w_off, i * o)))
                casts.append((self.G[pl.b_off:pl.b_off + o], flat(self.rank, pl.b_off, o)))
            w[li] = sorted(pieces, key=lambda t: t[0]) if aligned else None
            cast[li] = casts
            copies[li] = cps
        # (a rank with nothing to ship must not touch the communication stream: under graph capture a stream that was never
        # forked from the capturing one cannot be joined)
        self.wire_copies = copies if any(copies.values()) else None
        return {"f16": self.wire16 == "f16", "w": w, "cast": cast}

    def _build_pull(self):
        """Per layer (forward order): the copy-engine transfers that publish this rank's slices of the layer's bf16 shadow
        in every peer's window, and the gate the layer's forward GEMM waits on (one flag per owner, set to the step number
        once that owner's slices of the layer have been delivered)."""
        lay, win = self.layout, self.win
        sh0 = lay.offset("params_bf16")
        plan = []
        for li, pl in enumerate(self.engine.plans):
            lo_l, hi_l = pl.w_off, pl.b_off + pl.out_features
            cps = []
            for b, e in self.own[self.rank]:
                a0, a1 = max(b, lo_l), min(e, hi_l)
                if a1 > a0:
                    for q in range(self.world):
                        if q != self.rank:
                            cps.append((win.ptrs[q] + sh0 + 2 * a0, win.ptrs[self.rank] + sh0 + 2 * a0, 2 * (a1 - a0)))
            plan.append(cps)
        self.pull_plan = plan
        if getattr(self, "pull_step", None) is None:
            self.pull_step = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.pull_flag_arr = (C.c_void_p * self.world)(*win.peer_ptrs(lay.offset("pull_ready")))
        ready = lay.tensor(win, "pull_ready")
        mask = (1 << self.world) - 1
        self.engine.gates = {li: (ready[li:], self.pull_step, _lib.STAGE_BUCKETS, mask) for li in range(len(plan))}

    def pull_publish(self, stream) -> int:
        """Start of a step: advance the step number, then (communication stream, ordered after it) ship every layer's
        fresh slices to the peers and announce the layer. Returns the number of launches and transfers."""
        lib = _lib.load()
        _lib.check(lib.ono_stage_tick(self.pull_step.data_ptr(), _lib.stream_ptr(stream)), "ono_stage_tick")
        ev = torch.cuda.Event()
        ev.record(stream)
        self.comm_stream.wait_event(ev)
        cs = _lib.stream_ptr(self.comm_stream)
        n = 1
        for li, cps in enumerate(self.pull_plan):
            for dst, src, nbytes in cps:
                _lib.check(lib.ono_copy_async(dst, src, nbytes, cs), "ono_copy_async")
            _lib.check(lib.ono_stage_signal(self.pull_flag_arr, self.world, self.rank, li, self.pull_step.data_ptr(), cs),
                       "ono_stage_signal")
            n += len(cps) + 1
        return n

    def wire_ship(self, l: int, stream) -> int:
        """Ship layer l's finished 16-bit gradients to their owners: copy-engine transfers on the communication stream,
        ordered after the kernels that produced them. Returns the number of transfers."""
        cps = self.wire_copies.get(l) if self.wire_copies else None
        if not cps:
            return 0
        ev = torch.cuda.Event()
        ev.record(stream)
        lib, k = _lib.load(), len(self.push_streams)
        for cs in {self.push_streams[owner % k] for _, _, _, owner in cps}:
            cs.wait_event(ev)
        for dst, src, nbytes, owner in cps:
            _lib.check(lib.ono_copy_async(dst, src, nbytes, _lib.stream_ptr(self.push_streams[owner % k])), "ono_copy_async")
        return len(cps)

    def push_streams_used(self):
        """The streams the staged gradient push issues transfers on (the step joins them before the exchange)."""
        if not self.wire_copies:
            return []
        k = len(self.push_streams)
        return list({self.push_streams[owner % k] for cps in self.wire_copies.values() for _, _, _, owner in cps})

    def _build_apply(self, opt, n_workers: int, wild: bool):
        """Layers whose weight-gradient GEMM applies the optimizer itself, and the ranges left to the fused kernel."""
        e = self.engine
        kind = {"sgd": "sgd", "momentum": "momentum", "adam": "adam"}[opt.kind]
        cand = []
        # Only where the GEMM takes the form that moves the master / state / shadow tiles with TMA (bf16 CTA pairs on
        # 256-column tiles, SGD or momentum, a batch that fits the two-stage operand ring): 8192 x 8192 x 512 takes 0.27 ms
        # that way against 0.35 ms for the plain GEMM plus the separate pass. The register form (tf32 tiles, Adam) is
        # faster than its two separate kernels in isolation but slower inside the step (wide MLP, Adam: 1.20 ms against
        # 1.08 ms per step), so those layers keep the separate fused pass.
        B = self.trainer["batch_size"]
        sms = _lib.load().ono_num_sms()
        for li, pl in enumerate(e.plans):
            i, o = pl.in_features, pl.out_features
            tma_form = (e.bf16 and opt.kind in ("sgd", "momentum") and i >= 256 and B <= 2048 and o % 8 == 0 and
                        -(-i // 128) * -(-o // 256) >= sms * 3 // 4 and
                        (e.w_copy_needed[li] or self.shadow is None or (self.shadow.data_ptr() + 2 * pl.w_off) % 16 == 0))
            if os.environ.get("ONO_WGRAD_APPLY") == "force":      # every layer either form can take (tests of both forms)
                tma_form = o % 4 == 0 and i * o >= 1 << 16
            if tma_form and (self.C.data_ptr() + 4 * pl.w_off) % 16 == 0:
                cand.append((i * o, li))
        cand.sort(reverse=True)

        def rest_of(chosen):
            cuts = sorted((e.plans[li].w_off, e.plans[li].w_off + e.plans[li].in_features * e.plans[li].out_features)
                          for li in chosen)
            out, at = [], 0
            for b, en in cuts:
                if b > at:
                    out.append((at, b))
                at = en
            if at < self.n_pad:
                out.append((at, self.n_pad))
            return out

        chosen = [li for _, li in cand]
        while chosen and len(rest_of(chosen)) > _lib.MAX_RANGES:
            chosen.pop()                                    # the smallest layer goes back to the fused kernel
        plan = {}
        for li in chosen:
            pl = e.plans[li]
            i, o = pl.in_features, pl.out_features
            sl = slice(pl.w_off, pl.w_off + i * o)
            shadow = None
            if e.bf16 and not e.w_copy_needed[li] and self.shadow is not None:
                shadow = self.shadow[sl].view(i, o)
            plan[li] = dict(p=self.C[sl].view(i, o), m=self.m_loc[sl].view(i, o), v=self.v_loc[sl].view(i, o), p_bf16=shadow,
                            kind=kind, lr=opt.lr, mu=opt.mu, b1=opt.b1, b2=opt.b2, eps=opt.eps,
                            grad_scale=1.0 if wild else 1.0 / max(1, n_workers), adam_pows=self.adam_pows)
        return plan, rest_of(chosen)

    def _set_ownership(self, ranges, workers, opt, mode, wild):
        W = self.world
        dense_engine = self.engine is not None and isinstance(self.engine, GpuEngine)
        can = mode == "fused" and (dense_engine or self.engine is None)
        self.push_active = bool(self.push) and self._all_ranks_agree(can) if self.push else False
        self.wire16_push = bool(self.push16) and self._all_ranks_agree(can) if self.push16 else False
        self.wire_copies = None
        if self.wire16_push and self.wire_transport == "staged" and self.b200.get("shard_layout", "striped") == "striped":
            ranges = self._stripe(ranges)
        if self.push_active or (self.wire16_push and self.wire_transport == "direct"):
            ranges = self._snap_to_row_blocks(ranges)
        self.own = snap_ranges(ranges, self.n_pad)
        # who sums the 16-bit slabs of which range: the owners themselves, unless ranks that own nothing take a part of it
        self.reduce_at, self.finish_at, self.fwd_to = self.own, None, {}
        pre = self.b200.get("pre_reduce", "auto")
        if self.wire16_push and self.wire_transport == "staged" and mode == "fused" and (pre == "on" or (pre == "auto" and W >= 4)):
            # (on two GPUs the forwarded f32 sums weigh more than the 16-bit slabs they save: measured slower there)
            self._plan_pre_reduce()
        self.buckets, self.bucket_after = [], {}
        self.stage_buckets, self.stage_after, self.stage_active = [], {}, False
        if self.engine is not None:
            self.engine.max_ctas = 0            # only the overlap modes below leave SMs to communication kernels
            if dense_engine:
                self.engine.push = self.engine.wire16 = self.engine.apply_plan = None
        # One GPU that owns every layer: the weight-gradient GEMMs apply the optimizer in their epilogues and the fused
        # kernel afterwards only handles what is left (biases, layers whose rows are not 16-byte aligned)
        self.apply_active = False
        if (W == 1 and dense_engine and self.cadence == "step" and mode in ("fused", "oneshot") and not self.grad_norm_switch
                and not self.push_active and not self.compress
                and self.b200.get("wgrad_apply", "auto") != "off" and os.environ.get("ONO_WGRAD_APPLY", "1") != "0"):
            plan_, rest = self._build_apply(opt, len(workers), wild)
            if plan_:
                self.engine.apply_plan = plan_
                self.own = [rest]
                self.apply_active = True
        self.sync_workers = list(workers)
        self.sync_mode = mode
        self.sync_opt = opt
        n4 = self.n_pad // 4
        # two resident 512-thread blocks per SM at most: blocks of different ranks wait on one another,
        # so the whole grid must be co-resident (the same count on every rank)
        self.nblocks = int(min(2 * _lib.load().ono_num_sms(), max(1, -(-n4 // (512 * 2)))))
        wmask = sum(1 << r for r in workers)
        allmask = (1 << W) - 1
        lay, win = self.layout, self.win
        dest = set(workers) | {0}
        # f32 parameters travel to other ranks only if somebody reads them there: with bf16 tiles in
        # step cadence every consumer reads the bf16 shadow, and the owner keeps the only f32 master
        engines_need_f32 = self.cadence != "step" or self.tile != "bf16" or (
            self.engine is not None and self.engine.needs_f32_params)
        if W > 1 and self.tile == "bf16" and self.cadence == "step":
            flag = torch.tensor([1.0 if engines_need_f32 else 0.0], device=self.dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.group)
            engines_need_f32 = bool(flag.item() > 0)
        self.f32_everywhere = engines_need_f32
        n_layers = len([l for l in self.plan["layers"] if l["n_params"] > 0])
        self.pull_staged = bool(self.pull_wanted and self.wire16_push and mode == "fused" and not engines_need_f32 and
                                all(len(rs) > 0 for rs in self.own) and set(workers) == set(range(W)) and
                                n_layers <= _lib.STAGE_BUCKETS and self.engine is not None)
        self.pull_staged = self._all_ranks_agree(self.pull_staged) if self.pull_wanted else False
        self.pull_plan = None
        if self.engine is not None and isinstance(self.engine, GpuEngine):
            self.engine.gates = None
        if mode in ("fused", "oneshot"):
            s = _lib.OnoSync()
            oneshot = mode == "oneshot"
            pf = [p if (r in dest and not oneshot and engines_need_f32) or r == self.rank else None
                  for r, p in enumerate(win.peer_ptrs(lay.offset("params")))]
            if self.tile == "bf16":
                pb = [p if (r in dest and not oneshot) or r == self.rank else None
                      for r, p in enumerate(win.peer_ptrs(lay.offset("params_bf16")))]
            else:
                pb = [None] * W
            if self.pull_staged:       # the fused kernel refreshes this rank's own copies only; the pull travels separately
                pf = [p if r == self.rank else None for r, p in enumerate(pf)]
                pb = [p if r == self.rank else None for r, p in enumerate(pb)]
            nvls = self.use_nvls and win.mc_ptr != 0 and W > 1
            algo = 1 if nvls else 0
            g_region = self.grad_region
            g_dtype = 0
            stage_active = bool(self.stage) and not self.push_active and not self.compress and mode == "fused"
            self.stage_active = stage_active
            if self.push_active:
                # gradients arrive already summed in this rank's accumulator: nothing to reduce over the wires, the
                # kernel averages, applies the optimizer, zeroes the accumulator and distributes the parameters
                # (through the switch's multicast when there is one)
                g_region, wmask = "acc", 1 << self.rank
                algo = 2 if (win.mc_ptr != 0 and W > 2) else 0
            g_ptrs = win.peer_ptrs(lay.offset(g_region))
            if stage_active:
                # every worker's gradient is read from this GPU's memory: its own window, or the staged copy of a peer's
                g_ptrs = [g_ptrs[q] if q == self.rank else self.stage_buf[q].data_ptr() for q in range(W)]
                algo = 2 if (win.mc_ptr != 0 and W > 2) else 0
            if self.compress and self.sparse_r is not None:
                # sparse wire: every sender's selection is lifted into this rank's own f32 accumulator first (see
                # _launch_sync); the fused kernel then averages it, applies the optimizer and clears it
                g_ptrs = [self.sp_acc.data_ptr()] * W
                wmask, algo = 1 << self.rank, (2 if algo == 1 else algo)
            elif self.compress:
                g_dtype = 1 if self.cwire == "bf16" else 2
                g_ptrs = win.peer_ptrs(lay.offset("wire16"))
            if self.wire16 is not None:
                g_dtype = 2 if self.wire16 == "f16" else 1
                slab0 = lay.offset("slab16")
                if self.wire16_push:
                    # slab q of this rank's own window holds what worker q's GEMMs stored here during backward
                    g_ptrs = [win.ptrs[self.rank] + slab0 + 2 * q * self.n_pad for q in range(W)]
                    algo = 2 if (win.mc_ptr != 0 and W > 2) else 0
                else:
                    # pull form: every worker casts its gradient into slab 0 of its own window, owners read the peers'
                    g_ptrs = win.peer_ptrs(slab0)
            S.fill_sync(s, nranks=W, rank=self.rank, n=self.n_pad, nblocks=self.nblocks, algo=algo,
                        g_ptrs=g_ptrs, p_f32_ptrs=pf, p_bf16_ptrs=pb,
                        flag_ptrs=win.flag_ptrs, worker_mask=wmask, member_mask=allmask, n_workers=len(workers),
                        opt=opt, divide=not wild, timeout_ns=10_000_000_000,
                        g_mc=(win.mc(lay.offset(("wire16" if self.compress else "slab16") if g_dtype else g_region)) or None)
                        if algo == 1 else None,
                        p_mc_f32=(win.mc(lay.offset("params")) or None) if (engines_need_f32 and not self.pull_staged) else None,
                        p_mc_bf16=(win.mc(lay.offset("params_bf16")) or None) if (self.tile == "bf16" and not self.pull_staged) else None)
            local = dict(p_master=self.C.data_ptr(), m=self.m_loc.data_ptr(), v=self.v_loc.data_ptr(), state_off=0,
                         adam_pows=self.adam_pows.data_ptr(), epoch=self.epoch_words.data_ptr(),
                         sumsq=self.sumsq.data_ptr() if self.grad_norm_switch else None, status=self.sync_status.data_ptr())
            self.sync_struct2, self.fwd_copies = None, []
            if self.fwd_to:
                # first launch: owners update the part they reduce themselves, their partners forward f32 sums of theirs;
                # second launch: the owners finish the forwarded parts from their own f32 gradient vector
                # (the partner writes its sums into its OWN f32 gradient vector and a copy engine carries them to the owner
                # between the two launches: stores issued by SMs over NVLink reached ~320 GB/s here, the copy engine 770)
                f32_ptrs = win.peer_ptrs(lay.offset(self.grad_region))
                mine = self.rank in self.fwd_to
                S.fill_local(s.loc[self.rank], ranges=self.reduce_at[self.rank], fwd=f32_ptrs[self.rank] if mine else None, **local)
                self.fwd_copies = [(f32_ptrs[self.fwd_to[self.rank]] + 4 * b, f32_ptrs[self.rank] + 4 * b, 4 * (e - b))
                                   for b, e in self.reduce_at[self.rank]] if mine else []
                s2 = _lib.OnoSync()
                S.fill_sync(s2, nranks=W, rank=self.rank, n=self.n_pad, nblocks=self.nblocks, algo=algo, g_ptrs=f32_ptrs,
                            p_f32_ptrs=pf, p_bf16_ptrs=pb, flag_ptrs=win.flag_ptrs, worker_mask=1 << self.rank,
                            member_mask=allmask, n_workers=len(workers), opt=opt, divide=not wild, timeout_ns=10_000_000_000,
                            p_mc_f32=(win.mc(lay.offset("params")) or None) if engines_need_f32 else None,
                            p_mc_bf16=(win.mc(lay.offset("params_bf16")) or None) if self.tile == "bf16" else None)
                S.fill_local(s2.loc[self.rank], ranges=self.finish_at[self.rank], **local)
                self.sync_struct2 = s2
            else:
                S.fill_local(s.loc[self.rank], ranges=self.own[self.rank], **local)
            s.g_dtype = g_dtype
            if self.compress and self.sparse_r is not None:
                s.zero_grad = 1
            if self.push_active:
                s.zero_grad = 1
                if self.engine is not None:
                    self.engine.push = self._build_push()
            if self.wire16_push and self.engine is not None:
                self.engine.wire16 = self._build_wire16()
            if self.pull_staged:
                self._build_pull()
            self.sync_struct = s
            self._build_buckets()
            self._build_stage(workers)
        elif mode == "async":
            a = _lib.OnoPsAsync()
            a.nranks, a.rank, a.nblocks = W, self.rank, self.nblocks
            for r in range(W):
                a.master[r] = win.peer_ptrs(lay.offset("params"))[r]
                a.m[r] = win.peer_ptrs(lay.offset("m"))[r]
                a.v[r] = win.peer_ptrs(lay.offset("v"))[r]
                a.state_off[r] = 0
                a.locks[r] = None if wild else win.peer_ptrs(lay.offset("locks"))[r]
                a.n_ranges[r] = len(self.own[r])
                for i, (b, e) in enumerate(self.own[r]):
                    a.ranges[r][i].begin, a.ranges[r][i].end = b, e
            a.n_workers, a.divide = len(workers), int(not wild)
            a.kind = S.OPT_KIND[opt.kind]
            a.lr, a.mu, a.b1, a.b2, a.eps = opt.lr, opt.mu, opt.b1, opt.b2, opt.eps
            a.adam_pows = self.adam_pows.data_ptr()
            a.status = self.sync_status.data_ptr()
            a.timeout_ns = 10_000_000_000
            self.async_struct = a
        elif mode == "ring":
            if "ring_acc" not in lay.regions:
                raise RuntimeError("ring all-reduce needs its accumulation window (set b200.allreduce before start)")
            if set(workers) != set(range(W)):
                raise RuntimeError("ring all-reduce needs every rank to be a worker")
            r = _lib.OnoRing()
            r.nranks, r.rank, r.n = W, self.rank, self.n_pad
            r.nblocks = int(min(_lib.load().ono_num_sms(), max(1, self.n_pad // 4 // W // 512)))
            for q in range(W):
                r.acc[q] = win.peer_ptrs(lay.offset("ring_acc"))[q]
                r.flags[q] = win.flag_ptrs[q] + 4096 * 4        # the second half of the flag pad
            self.ring_epoch = getattr(self, "ring_epoch", None)
            if self.ring_epoch is None:
                self.ring_epoch = torch.zeros(1024, dtype=torch.int32, device=self.dev)
            r.epoch = self.ring_epoch.data_ptr()
            r.p, r.m, r.v = self.C.data_ptr(), self.m_loc.data_ptr(), self.v_loc.data_ptr()
            r.adam_pows = self.adam_pows.data_ptr()
            r.p_bf16 = self.shadow.data_ptr() if self.shadow is not None else None
            r.kind = S.OPT_KIND[opt.kind]
            r.lr, r.mu, r.b1, r.b2, r.eps = opt.lr, opt.mu, opt.b1, opt.b2, opt.eps
            r.status, r.timeout_ns = self.sync_status.data_ptr(), 10_000_000_000
            self.ring_struct = r

    def _build_buckets(self) -> None:
        """Split the fused synchronisation into per-layer buckets, in backward order, so that a bucket
        can run on the communication stream as soon as its layers' gradients exist while the layers
        below are still in backward (the reference exchanges only after the whole round:
        worker/src/workers/all_reduce.rs:114-133).

        A float4 group that straddles two layers goes with the lower layer, whose gradient is the last
        of the two to be produced."""
        import os

        self.buckets = []           # [(launch_after_layer, OnoSync)] in launch order
        self.bucket_after: dict[int, list] = {}
        # Opt-in (ONO_OVERLAP=1): measured slower than the single fused launch at 1, 2, 4 and 8 B200s. Peer loads are
        # issued per thread, and NVLink throughput grows with the number of SMs issuing them (about 4-5 GB/s per SM):
        # 16 / 32 SMs left to the bucket kernels moved gradients at roughly 70 / 140 GB/s on 4 GPUs, against 650 GB/s
        # when the fused kernel owns the whole GPU after backward.
        if (self.sync_mode != "fused" or self.cadence != "step" or os.environ.get("ONO_OVERLAP", "0") == "0"):
            return
        # The persistent GEMM (one CTA per SM, all of its shared memory and most registers) and a 512-thread
        # synchronisation block do not fit on one SM together, so the SMs are split: `comm_sms` of them are left to the
        # bucket kernels, the GEMMs run on the rest.
        comm_sms = max(1, min(int(os.environ.get("ONO_OVERLAP_SMS", "24")), _lib.load().ono_num_sms() // 2))
        if self.engine is not None:
            self.engine.max_ctas = _lib.load().ono_num_sms() - comm_sms
        up4 = lambda x: (x + 3) // 4 * 4
        layers = [l for l in self.plan["layers"] if l["n_params"] > 0]
        min_elems = 4 << 20
        sms = _lib.load().ono_num_sms()
        pending_end = self.n_pad
        cur_end = None
        for idx in range(len(layers) - 1, -1, -1):
            l = layers[idx]
            begin = 0 if idx == 0 else up4(l["offset"])
            if cur_end is None:
                cur_end = pending_end
            if cur_end - begin >= min_elems or idx == 0:
                if cur_end > begin:
                    s = _lib.OnoSync.from_buffer_copy(self.sync_struct)
                    mine = []
                    for b, e in self.own[self.rank]:
                        lo, hi = max(b, begin), min(e, cur_end)
                        if hi > lo:
                            mine.append((lo, hi))
                    loc = s.loc[self.rank]
                    loc.n_ranges = len(mine)
                    for i, (b, e) in enumerate(mine):
                        loc.ranges[i].begin, loc.ranges[i].end = b, e
                    # one block per SM at most: these kernels share the SMs with the running GEMMs
                    owners = max(1, sum(1 for r in self.own if r))
                    s.nblocks = int(min(comm_sms, max(1, -(-((cur_end - begin) // 4 // owners) // (512 * 2)))))
                    entry = (l["index"], s)
                    self.buckets.append(entry)
                    self.bucket_after.setdefault(l["index"], []).append(s)
                pending_end = begin
                cur_end = None

    def _bucket_ranges(self, min_elems: int = 4 << 20):
        """(layer index after which the bucket is complete, begin, end) in backward order: whole layers grouped until a
        bucket holds at least `min_elems` parameters; a float4 group straddling two layers goes with the lower layer."""
        up4 = lambda x: (x + 3) // 4 * 4
        layers = [l for l in self.plan["layers"] if l["n_params"] > 0]
        out, pending_end, cur_end = [], self.n_pad, None
        for idx in range(len(layers) - 1, -1, -1):
            l = layers[idx]
            begin = 0 if idx == 0 else up4(l["offset"])
            if cur_end is None:
                cur_end = pending_end
            if cur_end - begin >= min_elems or idx == 0:
                if cur_end > begin:
                    out.append((l["index"], begin, cur_end))
                pending_end, cur_end = begin, None
        return out

    def _build_stage(self, workers) -> None:
        """Per bucket: the pull of the peers' gradient ranges this rank owns (launched on the communication stream once
        the peers have announced the bucket) and the announcement of this rank's own gradients."""
        self.stage_buckets, self.stage_after = [], {}
        if not self.stage_active:
            return
        if self.engine is not None:
            self.engine.max_ctas = _lib.load().ono_num_sms() - self.stage_sms
        buckets = self._bucket_ranges()
        while len(buckets) > _lib.STAGE_BUCKETS:                      # merge neighbours until the flag table suffices
            buckets = [(buckets[i + 1][0] if i + 1 < len(buckets) else buckets[i][0],
                        buckets[i + 1][1] if i + 1 < len(buckets) else buckets[i][1], buckets[i][2])
                       for i in range(0, len(buckets), 2)]
        g_peer = self.win.peer_ptrs(self.layout.offset(self.grad_region))
        ready = self.layout.tensor(self.win, "stage_ready")
        self.stage_flag_arr = (C.c_void_p * self.world)(*self.win.peer_ptrs(self.layout.offset("stage_ready")))
        for k, (layer, begin, end) in enumerate(buckets):
            mine = []
            for b, e in self.own[self.rank]:
                lo, hi = max(b, begin), min(e, end)
                if hi > lo:
                    mine.append((lo, hi))
            pull = None
            if mine:
                pull = _lib.OnoStagePull()
                pull.nranks, pull.rank, pull.nblocks, pull.bucket = self.world, self.rank, self.stage_sms, k
                for q in range(self.world):
                    pull.src[q] = g_peer[q] if (q in workers and q != self.rank) else None
                    pull.dst[q] = self.stage_buf[q].data_ptr() if q != self.rank else None
                pull.n_ranges = len(mine)
                for i, (b, e) in enumerate(mine):
                    pull.ranges[i].begin, pull.ranges[i].end = b, e
                pull.ready, pull.step = ready.data_ptr(), self.stage_step.data_ptr()
                pull.status, pull.timeout_ns = self.sync_status.data_ptr(), 10_000_000_000
            self.stage_buckets.append((layer, k, pull))
            self.stage_after.setdefault(layer, []).append((k, pull))

    def stage_tick(self, stream) -> int:
        _lib.check(_lib.load().ono_stage_tick(self.stage_step.data_ptr(), _lib.stream_ptr(stream)), "ono_stage_tick")
        return 1

    def stage_signal(self, k: int, stream) -> int:
        _lib.check(_lib.load().ono_stage_signal(self.stage_flag_arr, self.world, self.rank, k, self.stage_step.data_ptr(),
                                                _lib.stream_ptr(stream)), "ono_stage_signal")
        return 1

    def stage_pull(self, pull, stream) -> int:
        if pull is None:
            return 0
        _lib.check(_lib.load().ono_stage_pull(C.byref(pull), _lib.stream_ptr(stream)), "ono_stage_pull")
        return 1

    def _launch_sync(self, g_tensor: torch.Tensor, stream) -> int:
        """One synchronisation of `g_tensor` (the window's gradient region) into the parameters."""
        n = 0
        if self.compress and g_tensor is self.G:
            from ..ops import compress as cp

            fused = self.sync_mode in ("fused", "oneshot")
            sparse = self.sparse_r is not None
            if not fused and self.wire is None:
                self.wire = torch.zeros(self.n_pad, device=self.dev)
            if self.widx is not None:
                thr = None
                if sparse:
                    thr = cp.sparse_threshold(self.G[:self.n], self.sparse_r, self.seed + self.wire_rounds, out=self.wire_thr,
                                              stream=stream)
                    n += 1
                    if fused:     # the (index, f16) list of the selection, before the mask takes it out of the residual
                        cp.sparse_compact(self.G, thr, self.sp_cap, zero_sent=False, stream=stream,
                                          out=(self.sp_idx, self.sp_val, self.sp_cnt[:1]), scratch=self.sp_scratch)
                        n += 3
                cp.wire_mask(self.G, None if fused else self.wire, thr, self.wire_sent, wire16=self.wire16_t if fused else None,
                             stream=stream)
                n += 1
            self.wire_rounds += 1
            if fused and sparse:
                if self.world > 1:      # every sender's list is complete before anyone reads it
                    with torch.cuda.stream(stream):
                        dist.all_reduce(self.sp_tick, group=self.group)
                lay, win = self.layout, self.win
                idx_p, val_p = win.peer_ptrs(lay.offset("sp_idx")), win.peer_ptrs(lay.offset("sp_val"))
                cnt_p, w16_p = win.peer_ptrs(lay.offset("sp_cnt")), win.peer_ptrs(lay.offset("wire16"))
                for q in self.sync_workers:
                    for b, e in self.own[self.rank]:
                        cp.sparse_lift_range(self.sp_acc, b, min(e, self.n_pad), idx_p[q], val_p[q], cnt_p[q], self.sp_cap, w16_p[q],
                                             self.cwire == "f16", self.wire_bytes if q != self.rank else None, stream=stream)
                        n += 1
            g_tensor = self.wire if not fused else self.G
        if self.sync_opt.kind == "adam" and not self.apply_active:   # with the optimizer in the GEMM epilogues the step ticks first
            ew.adam_tick(self.adam_pows, self.sync_opt.b1, self.sync_opt.b2, stream=stream)
            n += 1
        if (self.wire16 is not None and not self.wire16_push and self.sync_mode in ("fused", "oneshot")
                and self.widx is not None and self.rank in self.sync_workers):
            # 16-bit wire, pull form: this worker's gradient goes to slab 0 of its own window as 16-bit values
            ew.cast16(g_tensor, self.layout.tensor(self.win, "slab16")[:self.n_pad], f16=self.wire16 == "f16", stream=stream)
            n += 1
        if self.sync_mode in ("fused", "oneshot"):
            S.launch_sync(self.sync_struct, stream=stream)
            n += 1
            if getattr(self, "sync_struct2", None) is not None:
                lib, sp = _lib.load(), _lib.stream_ptr(stream)
                for dst, src, nbytes in self.fwd_copies:       # a partner's sums travel to their owner; owners have none
                    _lib.check(lib.ono_copy_async(dst, src, nbytes, sp), "ono_copy_async")
                S.launch_sync(self.sync_struct2, stream=stream)
                n += 1 + len(self.fwd_copies)
        elif self.sync_mode == "async":
            if self.widx is not None and self.rank in self.sync_workers:
                a = self.async_struct
                a.g = g_tensor.data_ptr()
                a.p_local_f32 = self.W.data_ptr()
                a.p_local_bf16 = self.shadow.data_ptr() if self.shadow is not None else None
                _lib.check(_lib.load().ono_ps_async_step(C.byref(a), _lib.stream_ptr(stream)), "ono_ps_async_step")
                n += 1
        elif self.sync_mode == "ring":
            self.ring_struct.g = g_tensor.data_ptr()
            _lib.check(_lib.load().ono_ring_allreduce(C.byref(self.ring_struct), _lib.stream_ptr(stream)), "ono_ring_allreduce")
            n += 1
        elif self.sync_mode == "nccl":
            with torch.cuda.stream(stream):
                if self.world > 1:
                    dist.all_reduce(g_tensor, group=self.group)
            ew.optim_step(self.C, g_tensor, kind=self.sync_opt.kind, lr=self.sync_opt.lr, mu=self.sync_opt.mu,
                          b1=self.sync_opt.b1, b2=self.sync_opt.b2, eps=self.sync_opt.eps, m=self.m_loc,
                          v=self.v_loc, adam_pows=self.adam_pows, grad_scale=1.0 / len(self.sync_workers),
                          p_bf16=self.shadow, stream=stream)
            n += 2
        return n
