"""Round / step loops of a GPU rank, graph capture, loss exchange and the strategy switch."""
from __future__ import annotations

import time

import numpy as np
import torch
import torch.distributed as dist

from ..ops import elementwise as ew
from ..parallel import sync as S
from .gpu_rank import BatchFeeder


def _steps_per_epoch(r) -> int:
    """Step cadence: every worker takes the same number of steps per epoch (the minimum over the
    workers' partitions), since each step ends in a collective."""
    counts = []
    for w in r.plan["workers"]:
        if w["rank"] not in r.sync_workers:
            continue
        rows = r.extra_rows.get(w["rank"], 0) + w["partition"][1] - w["partition"][0]
        counts.append(-(-rows // w["spec"]["trainer"]["batch_size"]))
    return max(1, min(counts)) if counts else 0


def _batch_body(r, slot: int, nrows: int, with_sync: bool) -> int:
    """The kernel sequence of one mini-batch on the current stream. Returns the launch count."""
    st = torch.cuda.current_stream()
    f, e = r.feeder, r.engine
    e.loss_sum.zero_()
    n = 1
    if with_sync and r.apply_active and r.sync_opt.kind == "adam":
        # the weight-gradient GEMMs apply Adam in their epilogues: the step's powers must exist before backward
        ew.adam_tick(r.adam_pows, r.sync_opt.b1, r.sync_opt.b2, stream=st)
        n += 1
    if with_sync and r.buckets:
        # bucketed: each layer's gradients are synchronised on the communication stream as soon as
        # they exist, while backward continues below that layer
        if r.sync_opt.kind == "adam":
            ew.adam_tick(r.adam_pows, r.sync_opt.b1, r.sync_opt.b2, stream=st)
            n += 1
        comm = r.comm_stream

        def after_layer(l):
            k = 0
            for bk in r.bucket_after.get(l, ()):
                ev = torch.cuda.Event()
                ev.record(st)
                comm.wait_event(ev)
                S.launch_sync(bk, stream=comm)
                k += 1
            return k

        n += e.step(f.dev_x[slot], f.dev_y[slot], nrows, stream=st, after_layer=after_layer)
        st.wait_stream(comm)
        n += e.refresh(stream=st)
        return n
    if with_sync and r.stage_buckets:
        # staged reduce-scatter: every finished bucket is announced to the peers, and the peers' copies of the ranges
        # this rank owns are pulled into local staging on the communication stream while backward continues
        n += r.stage_tick(st)
        comm = r.comm_stream

        def after_layer_stage(l):
            k = 0
            for bucket, pull in r.stage_after.get(l, ()):
                k += r.stage_signal(bucket, st)
                if pull is not None:
                    ev = torch.cuda.Event()
                    ev.record(st)
                    comm.wait_event(ev)
                    k += r.stage_pull(pull, comm)
            return k

        n += e.step(f.dev_x[slot], f.dev_y[slot], nrows, stream=st, after_layer=after_layer_stage)
        st.wait_stream(comm)
        n += r._launch_sync(r.G, st)
        n += e.refresh(stream=st)
        return n
    ph = r.phase_events if getattr(r, "phase_timing", False) else None

    def mark(name):     # phase boundary: a timed event on the stream and an NVTX range for external profilers
        if ph is None:
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(st)
        if ph and ph[-1][0] != "end":
            torch.cuda.nvtx.range_pop()
        ph.append((name, ev))
        if name != "end":
            torch.cuda.nvtx.range_push(name)

    mark("compute")
    if with_sync and r.pull_staged:
        n += r.pull_publish(st)          # last step's fresh parameters travel while this step's first layers already run
    if with_sync and (r.wire_copies or r.pull_staged):
        # 16-bit gradients leave for their owners layer by layer on the communication stream (copy engines) while the
        # layers below are still in backward; the fused kernel starts once the last transfer has been issued and done
        n += e.step(f.dev_x[slot], f.dev_y[slot], nrows, stream=st,
                    after_layer=(lambda l: r.wire_ship(l, st)) if r.wire_copies else None)
        for cs in (r.push_streams_used() if r.wire_copies else []):
            st.wait_stream(cs)
        if r.pull_staged:
            st.wait_stream(r.comm_stream)
    else:
        n += e.step(f.dev_x[slot], f.dev_y[slot], nrows, stream=st)
    mark("exchange")
    if r.cadence == "round":
        # sequential.rs:129-141: stateless SGD on the working copy, residual += grad
        ew.local_sgd(r.W[:r.n], r.g[:r.n], r.G[:r.n], r.local_lr, p_bf16=r.shadow, stream=st)
        n += 1
    elif with_sync:
        n += r._launch_sync(r.G, st)
    mark("refresh")
    n += e.refresh(stream=st)
    mark("end")
    return n


def run_batch(r, slot: int, nrows: int) -> None:
    """Run one mini-batch: eagerly the first time a (slot, rows) shape is seen, from a CUDA graph after."""
    key = (slot, nrows, r.sync_mode, r.cadence)
    st = r.stream
    st.wait_event(r.feeder.ready[slot])
    # the staged reduce-scatter (experimental) forks onto the communication stream inside the step; it runs uncaptured
    graphable = r.sync_mode != "nccl" and not r.stage_active and not getattr(r, "phase_timing", False)
    with torch.cuda.stream(st):
        if key not in r.warm or not graphable:
            r.launches_per_step = _batch_body(r, slot, nrows, True)
            r.warm.add(key)
        else:
            g = r.graphs.get(key)
            if g is None:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=st):
                    r.launches_per_step = _batch_body(r, slot, nrows, True)
                r.graphs[key] = g
            g.replay()
        r.feeder.consumed[slot].record(st)
        r.loss_pin[slot].copy_(r.engine.loss_sum, non_blocking=True)  # D2H read of the step's result
        r.loss_evt[slot].record(st)
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(st)
    r.step_events.append(ev)
    r.step_wall.append(time.perf_counter())


def server_step(r) -> None:
    """A pure server rank takes part in the synchronisation only."""
    with torch.cuda.stream(r.stream):
        if r.stage_buckets:   # a server-only rank pulls the workers' gradients of the ranges it owns
            r.stage_tick(r.stream)
            for _, _, pull in r.stage_buckets:
                r.stage_pull(pull, r.stream)
            r._launch_sync(r.G, r.stream)
        elif r.buckets:  # the same launches, in the same order, as the workers issue
            if r.sync_opt.kind == "adam":
                ew.adam_tick(r.adam_pows, r.sync_opt.b1, r.sync_opt.b2, stream=r.stream)
            for _, bk in r.buckets:
                S.launch_sync(bk, stream=r.stream)
        else:
            r._launch_sync(r.G, r.stream)
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(r.stream)
    r.step_events.append(ev)
    r.step_wall.append(time.perf_counter())


def exchange(r, values: list[float]) -> np.ndarray:
    """All ranks learn every rank's small vector (losses, stop flag): one tiny all-gather."""
    v = torch.tensor(values, dtype=torch.float64, device=r.dev)
    if r.world == 1:
        return v.cpu().numpy().reshape(1, -1)
    # Issued on the training stream: the collective must not start before this rank's fused kernels
    # have retired, or the two would wait on each other for SM space across ranks.
    with torch.cuda.stream(r.stream):
        out = torch.empty(r.world * len(values), dtype=torch.float64, device=r.dev)
        dist.all_gather_into_tensor(out, v.to(r.dev), group=r.group)
        host = out.cpu()
    return host.numpy().reshape(r.world, -1)


def check_status(r) -> None:
    bad = int(r.sync_status.item())
    if r.engine is not None:
        bad = bad or int(r.engine.status.item())
    if bad:
        raise RuntimeError(f"rank {r.rank}: a kernel wait timed out (status {bad}); a peer is late or gone")


def report_and_decide(r, epoch_losses: list[float]) -> int:
    """Gather this round's losses and the stop flag, emit events (rank 0) and run the shared policy."""
    nl = max(1, r.offline + 1)
    vec = [float("nan")] * nl + [1.0 if r.stop_event.is_set() else 0.0]
    for i, l in enumerate(epoch_losses[:nl]):
        vec[i] = l
    table = exchange(r, vec)
    decision = 0
    stop_req = bool(table[:, nl].max() > 0)
    for wi, wr in enumerate(r.worker_ranks):
        if wr not in r.sync_workers:
            continue
        losses = [float(x) for x in table[wr, :nl] if not np.isnan(x)]
        if not losses:
            continue
        if any(not np.isfinite(x) for x in losses):
            if r.rank == 0:
                r.emit({"kind": "error", "worker": wi, "losses": [], "text": "worker reported a non-finite loss"})
            r.stop_reason = "error"
            return 1
        if r.rank == 0:
            r.emit({"kind": "losses", "worker": wi, "losses": losses, "text": ""})
        d = r.policy.on_losses(wi, losses)
        decision = max(decision, d) if d != 2 else (decision or 2)
    if stop_req:
        r.stop_reason = "stopped"
        return 1
    if decision == 1:
        r.stop_reason = "early_stopping"
    return decision


def do_switch(r) -> None:
    """All-reduce -> parameter server in place: the promoted ranks adopt the ranges they will own
    (every replica already holds the full vector), optimizer state restarts, and their data is
    re-scattered to the remaining workers (node/src/router.rs:305-341, worker/src/builder.rs:165-200)."""
    if not any(a["action"] == "switch" for a in r.plan["switch"]["post_actions"]):
        # every rank would be promoted and nobody would be left to train (as many servers as nodes): the run stays in
        # all-reduce; the same decision on every rank, since all of them read it from the plan
        r.switch_declined = True        # reported in the run's metrics; the test is not repeated
        r.grad_norm_switch = False
        return
    if r.pull_staged:           # the last step's parameters have not been published yet: do it before ownership changes
        with torch.cuda.stream(r.stream):
            r.pull_publish(r.stream)
            r.stream.wait_stream(r.comm_stream)
    torch.cuda.synchronize(r.dev)
    if r.world > 1:
        dist.barrier(group=r.group)
    acts = r.plan["switch"]["post_actions"]
    promoted = [a["rank"] for a in acts if a["action"] == "upgrade"]
    remaining = [a["rank"] for a in acts if a["action"] == "switch"]
    if r.rank == 0:
        r.emit({"kind": "switch", "worker": 0, "losses": [], "text": ""})
        for a in acts:
            if a["action"] == "upgrade":
                r.emit({"kind": "upgrading", "worker": r.worker_ranks.index(a["rank"]), "losses": [], "text": ""})
    # dataset of each promoted rank -> split over the remaining workers, appended to theirs
    for pr in promoted:
        meta = torch.zeros(1, dtype=torch.int64, device=r.dev)
        if r.rank == pr:
            meta[0] = r.feeder.rows
        dist.broadcast(meta, src=pr, group=r.group)
        rows = int(meta.item())
        bx = torch.empty(rows, r.x_size, device=r.dev)
        by = torch.empty(rows, r.y_size, device=r.dev)
        if r.rank == pr:
            bx.copy_(r.feeder.host_x)
            by.copy_(r.feeder.host_y)
        dist.broadcast(bx, src=pr, group=r.group)
        dist.broadcast(by, src=pr, group=r.group)
        if r.rank in remaining:
            k = remaining.index(r.rank)
            from orchestra import _orchestra as core

            lo, hi = core.dataset_partitions(rows, len(remaining))[k]
            f = r.feeder
            xs = np.concatenate([f.host_x.numpy().reshape(-1), bx[lo:hi].cpu().numpy().reshape(-1)])
            ys = np.concatenate([f.host_y.numpy().reshape(-1), by[lo:hi].cpu().numpy().reshape(-1)])
            r.feeder = BatchFeeder(xs, ys, r.x_size, r.y_size, f.batch, r.dev, r.seed, f.device_resident)
        for k, wr in enumerate(remaining):
            lo, hi = __import__("orchestra")._orchestra.dataset_partitions(rows, len(remaining))[k]
            r.extra_rows[wr] = r.extra_rows.get(wr, 0) + (hi - lo)
    ranges = [[] for _ in range(r.world)]
    spec = None
    for a in acts:
        if a["action"] == "upgrade":
            ranges[a["rank"]] = [tuple(x) for x in a["ranges"]]
            spec = a["spec"]
    from .gpu_rank import optimizer_cfg

    opt = optimizer_cfg(spec["optimizer"])
    is_async = spec["synchronizer"] == "non_blocking" or spec["store"] == "wild"
    torch.cuda.synchronize(r.dev)
    r.m_loc.zero_(); r.v_loc.zero_(); r.adam_pows.fill_(1.0)   # builder.rs:179-181: state restarts
    if hasattr(r, "m_win"):
        r.m_win.zero_(); r.v_win.zero_()
    r.graphs.clear(); r.warm.clear()
    for pr in promoted:
        r.policy.worker_left(r.worker_ranks.index(pr))
    if r.rank in promoted:
        r.engine, r.feeder, r.widx = None, None, None
    r._set_ownership(ranges, remaining, opt, "async" if is_async else "fused", spec["store"] == "wild")
    r.switched = True
    r.switched_at_step = len(r.step_events)
    if r.world > 1:
        dist.barrier(group=r.group)
    if r.rank == 0:
        for pr in promoted:
            r.emit({"kind": "upgraded", "worker": r.worker_ranks.index(pr), "losses": [], "text": ""})
