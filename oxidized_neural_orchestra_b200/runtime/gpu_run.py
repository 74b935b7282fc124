"""Entry point of a GPU rank's training run: ``run(rank_state)`` drives the loops of gpu_loop.py
to completion and returns the final parameters (rank 0) and the device-timed step records."""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.distributed as dist

from ..utils.trace import MetricsSink, Tracer
from . import gpu_loop as L


def _drain_loss(r, slot: int, pending: list) -> float:
    if not pending[slot]:
        return 0.0
    r.loss_evt[slot].synchronize()
    pending[slot] = False
    return float(r.loss_pin[slot].item())


def _norm_check(r, hist: list) -> int:
    """Feed the per-step global gradient norms gathered since the last check to the switch tracker."""
    if not hist:
        return 0
    with torch.cuda.stream(r.stream):  # ordered after this rank's fused kernels (see gpu_loop.exchange)
        v = torch.stack(hist).reshape(-1)
        if r.world > 1:
            dist.all_reduce(v, group=r.group)
        host = v.cpu().numpy()
    decision = 0
    for x in host:
        if r.policy.on_metric(math.sqrt(max(float(x), 0.0))) == 2:
            decision = 2
    hist.clear()
    return decision


def _bench_hook(r, it: int) -> None:
    """Optional timed window [warmup, warmup + steps) bracketed by synchronize + barrier on both sides
    (set through ONO_BENCH_WARMUP / ONO_BENCH_STEPS; used by the benchmark harness)."""
    if r.bench is None:
        return
    w, k = r.bench
    if it == w or it == w + k:
        torch.cuda.synchronize(r.dev)
        if r.world > 1:
            dist.barrier(group=r.group)
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(r.stream)
        r.bench_events.append(ev)
        r.bench_wall.append(__import__("time").perf_counter())


def _record_epoch(r, tracer, sink, ev_first: int, epoch_first: int, epoch_now: int, losses: list, t_epoch: float) -> None:
    """One metrics record and the device spans of the steps recorded since ``ev_first``."""
    import time

    evs = r.step_events[ev_first:]
    dev_ms, worst = 0.0, 0.0
    if len(evs) >= 2:
        evs[-1].synchronize()
        for a, b in zip(evs[:-1], evs[1:]):
            d = a.elapsed_time(b)
            dev_ms += d
            worst = max(worst, d)
            tracer.device_span("step", a, b, epoch=epoch_first)
    wall = time.perf_counter() - t_epoch
    tracer.events.append({"name": "epoch", "ph": "X", "pid": r.rank, "tid": 0, "ts": (t_epoch - tracer.t0) * 1e6,
                          "dur": wall * 1e6, "args": {"epoch": epoch_first, "losses": losses}}) if tracer.on else None
    phase_ms: dict = {}
    ph = getattr(r, "phase_events", None)
    if ph:
        ph[-1][1].synchronize()
        count: dict = {}
        for (name, a), (_, b) in zip(ph[:-1], ph[1:]):
            if name == "end":
                continue
            phase_ms[name] = phase_ms.get(name, 0.0) + a.elapsed_time(b)
            count[name] = count.get(name, 0) + 1
            tracer.device_span(name, a, b, epoch=epoch_first)
        phase_ms = {k: v / count[k] for k, v in phase_ms.items()}
        r.phase_ms_last = phase_ms
        ph.clear()
    steps = max(0, len(evs) - 1)
    rows = steps * int(getattr(r.engine, "B", 0) or 0)
    sink.write(epoch=epoch_now, epochs_in_record=max(1, epoch_now - epoch_first), loss=(losses[-1] if losses else None),
               steps=steps, device_ms=dev_ms, max_step_ms=worst, wall_s=wall,
               samples_per_sec=(rows / (dev_ms / 1e3) if dev_ms > 0 else None),
               epochs_per_sec=(max(1, epoch_now - epoch_first) / wall if wall > 0 else None),
               strategy=("parameter_server" if r.switched else r.algorithm), sync_mode=r.sync_mode,
               **({"phase_ms": phase_ms} if phase_ms else {}),
               h2d_bytes_per_step=(r.feeder.h2d_bytes_per_step if r.feeder is not None else 0))


def _state_tensors(r):
    """Where this rank keeps the optimizer moments of the ranges it owns (asynchronous PS: in the window)."""
    if r.sync_mode == "async" and hasattr(r, "m_win"):
        return r.m_win, r.v_win
    return r.m_loc, r.v_loc


def _load_state(r, path: str) -> int:
    """Copy a saved optimizer state into this rank's buffers; returns the number of epochs the file records."""
    from ..utils.state import load_state

    st = load_state(path, r.n)
    targets = [(r.m_loc, "m"), (r.v_loc, "v")]
    if hasattr(r, "m_win"):
        targets += [(r.m_win, "m"), (r.v_win, "v")]
    with torch.cuda.stream(r.stream):
        for dst, k in targets:
            dst[:r.n].copy_(torch.from_numpy(st[k].copy()).to(r.dev))
        r.adam_pows.copy_(torch.from_numpy(st["adam_pows"].copy()).to(r.dev))
    r.stream.synchronize()
    return int(st["meta"].get("epochs", 0))


def _save_state(r, path: str, epochs: int) -> None:
    """Owners' moments -> rank 0 -> ``path`` (same gather as the final parameters)."""
    from ..utils.state import save_state

    m, v = _state_tensors(r)
    if r.world > 1 and r.sync_mode not in ("oneshot", "ring"):
        both = torch.zeros(2, r.n_pad, device=r.dev)
        for b, e in r.own[r.rank]:
            both[0, b:e] = m[b:e]
            both[1, b:e] = v[b:e]
        dist.all_reduce(both, group=r.group)
        m, v = both[0], both[1]
    if r.rank == 0:
        save_state(path, m[:r.n].cpu().numpy(), v[:r.n].cpu().numpy(), r.adam_pows.cpu().numpy(),
                   optimizer=r.sync_opt.kind, epochs=epochs, n_params=r.n)


def _gather_params(r):
    """The authoritative parameters on rank 0: owners' ranges where ownership is partitioned (session.rs:293-359),
    rank 0's replica otherwise (session.rs:371-412). Collective."""
    if r.world > 1 and r.sync_mode not in ("oneshot", "ring"):
        tmp = torch.zeros_like(r.C)
        for b, e in r.own[r.rank]:
            tmp[b:e] = r.C[b:e]
        dist.all_reduce(tmp, group=r.group)
        return tmp
    return r.C


def _checkpoint(r, epochs_done: int) -> None:
    """Periodic checkpoint: weights in the reference's layout plus the optimizer-state sidecar (collective; rank 0 writes)."""
    from ..utils.state import save_tensors, weight_tensors
    from .gpu_rank import engine_layers_from_plan

    torch.cuda.synchronize(r.dev)
    path = r.b200["checkpoint_path"]
    path = path.replace("{epoch}", str(epochs_done)) if "{epoch}" in path else f"{path}.epoch{epochs_done}"
    base = path[:-len(".safetensors")] if path.endswith(".safetensors") else path
    with torch.cuda.stream(r.stream):
        params = _gather_params(r)
        host = params[:r.n].cpu().numpy() if r.rank == 0 else None
        _save_state(r, base + ".state.safetensors", epochs_done)   # the sidecar is complete before the weights file appears
    if r.rank == 0:
        save_tensors(path, weight_tensors(engine_layers_from_plan(r.plan), host))
    torch.cuda.synchronize(r.dev)


def run(r) -> dict:
    import os

    w, k = os.environ.get("ONO_BENCH_WARMUP"), os.environ.get("ONO_BENCH_STEPS")
    r.bench = (int(w), int(k)) if w is not None and k is not None else None
    r.bench_events, r.bench_wall = [], []
    r.extra_rows = {}
    r.stop_reason = "max_epochs"
    epoch, it = 0, 0
    pending = [False, False]
    norm_hist: list = []
    check_every = int(r.b200.get("switch_check_every", 10))
    r.phase_timing = bool(r.b200.get("phase_timing", False)) and r.engine is not None
    r.phase_events = []
    tracer = r.tracer = Tracer(r.b200.get("trace_path") or None, r.rank)
    sink = MetricsSink(r.b200.get("metrics_path") or None, r.rank)
    tracer.device_anchor(r.stream)
    first_epoch = int(r.b200.get("start_epoch", -1))
    if r.b200.get("init_state_from"):
        recorded = _load_state(r, r.b200["init_state_from"])
        first_epoch = recorded if first_epoch < 0 else first_epoch
    r.first_epoch = max(0, first_epoch)
    ckpt_mark = r.first_epoch // max(1, int(r.b200.get("checkpoint_every", 0) or 1))
    if r.feeder is not None:
        r.feeder.epoch_offset = r.first_epoch       # the shuffle sequence continues where the saved run stopped
    while epoch < r.max_epochs:
        decision = 0
        epoch_losses: list[float] = []
        ev_first, epoch_first, t_epoch = len(r.step_events), epoch, __import__("time").perf_counter()
        if r.cadence == "step":
            steps = L._steps_per_epoch(r)
            total, cnt = 0.0, 0
            staged = [0, 0]
            if r.engine is not None:
                staged[it % 2] = r.feeder.stage(it % 2, epoch, 0)
            for s in range(steps):
                slot = it % 2
                _bench_hook(r, it)
                if r.engine is not None:
                    total += _drain_loss(r, slot, pending)
                    L.run_batch(r, slot, staged[slot])
                    pending[slot] = True
                    cnt += 1
                    if s + 1 < steps:
                        staged[slot ^ 1] = r.feeder.stage(slot ^ 1, epoch, s + 1)
                else:
                    L.server_step(r)
                it += 1
                if r.grad_norm_switch and not r.switched:
                    with torch.cuda.stream(r.stream):
                        norm_hist.append(r.sumsq.clone())
                        r.sumsq.zero_()
                    if len(norm_hist) >= check_every and _norm_check(r, norm_hist) == 2:
                        decision = 2
                        break
            if r.engine is not None:
                total += _drain_loss(r, 0, pending) + _drain_loss(r, 1, pending)
                epoch_losses.append(total / max(1, cnt))
            if decision != 2:
                epoch += 1
        else:
            nep = min(r.max_epochs - epoch, r.offline + 1)
            for e in range(nep):
                if r.engine is None:
                    continue
                steps = r.feeder.steps_per_epoch()
                total, cnt = 0.0, 0
                staged = [0, 0]
                staged[it % 2] = r.feeder.stage(it % 2, epoch + e, 0)
                for s in range(steps):
                    slot = it % 2
                    total += _drain_loss(r, slot, pending)
                    L.run_batch(r, slot, staged[slot])
                    pending[slot] = True
                    cnt += 1
                    if s + 1 < steps:
                        staged[slot ^ 1] = r.feeder.stage(slot ^ 1, epoch + e, s + 1)
                    it += 1
                total += _drain_loss(r, 0, pending) + _drain_loss(r, 1, pending)
                epoch_losses.append(total / max(1, cnt))
            # one exchange per round: residual -> owners -> fresh parameters everywhere
            with torch.cuda.stream(r.stream):
                r._launch_sync(r.G, r.stream)
                if r.engine is not None:
                    if r.sync_mode != "async":
                        r.W.copy_(r.C)
                    if not r.compress:      # with a compressed wire the unsent part stays as the residual
                        r.G.zero_()
                    r.engine.refresh(stream=r.stream)
                ev = torch.cuda.Event(enable_timing=True)
                ev.record(r.stream)
            r.round_events = getattr(r, "round_events", []) + [ev]
            epoch += nep
        if tracer.on or sink.on or r.phase_timing:
            _record_epoch(r, tracer, sink, ev_first, epoch_first, epoch, epoch_losses, t_epoch)
        if decision != 2:
            with tracer.span("report_and_decide", epoch=epoch):
                decision = L.report_and_decide(r, epoch_losses)
        L.check_status(r)
        every = int(r.b200.get("checkpoint_every", 0) or 0)
        if every > 0 and r.b200.get("checkpoint_path") and decision == 0 and (r.first_epoch + epoch) // every > ckpt_mark:
            ckpt_mark = (r.first_epoch + epoch) // every      # a round of several epochs may cross more than one multiple
            _checkpoint(r, r.first_epoch + epoch)
        if decision == 1:
            break
        if decision == 2 and r.algorithm == "strategy_switch" and not r.switched and not getattr(r, "switch_declined", False):
            with tracer.span("strategy_switch", epoch=epoch):
                L.do_switch(r)
            pending = [False, False]
    _bench_hook(r, it)
    torch.cuda.synchronize(r.dev)
    L.check_status(r)
    # final parameters: the owners' ranges are authoritative (session.rs:293-359); all-reduce replicas
    # are identical and rank 0's copy is taken (session.rs:371-412)
    # (with bf16 tiles only the owner of a range holds its up-to-date f32 master, so the owners'
    # ranges are collected whenever ownership is partitioned; one-shot replicates ownership)
    if r.world > 1 and r.sync_mode not in ("oneshot", "ring"):
        tmp = torch.zeros_like(r.C)
        for b, e in r.own[r.rank]:
            tmp[b:e] = r.C[b:e]
        if r.world > 1:
            dist.all_reduce(tmp, group=r.group)
        final = tmp
    else:
        final = r.C
    params = final[:r.n].cpu().numpy() if r.rank == 0 else None
    if r.b200.get("state_path"):
        _save_state(r, r.b200["state_path"], r.first_epoch + epoch)
    ms = []
    evs = r.step_events
    for a, b in zip(evs[:-1], evs[1:]):
        ms.append(a.elapsed_time(b))
    metrics = {
        "step_ms": ms, "steps": len(evs), "step_wall": r.step_wall, "launches_per_step": r.launches_per_step,
        "h2d_bytes_per_step": r.feeder.h2d_bytes_per_step if r.feeder is not None else 0,
        "d2h_bytes_per_step": 8 if r.feeder is not None else 0, "switched": r.switched,
        "switched_at_step": getattr(r, "switched_at_step", None), "switch_declined": bool(getattr(r, "switch_declined", False)),
        "sync_mode": r.sync_mode,
        "nvls": bool(r.use_nvls and r.win.mc_ptr),
        # what travels between GPUs: the 16-bit wire applies to the fused kernels of step cadence
        "wire": (r.wire16 if (r.wire16 is not None and r.sync_mode in ("fused", "oneshot")) else "f32") if r.world > 1 else "none",
        "wire_push": bool(r.wire16_push), "wire_transport": r.wire_transport if r.wire16_push else None,
        "wgrad_apply": bool(r.apply_active), "param_pull": "staged" if r.pull_staged else "kernel",
        "pre_reduce": bool(getattr(r, "fwd_to", None)),
    }
    if r.phase_timing:
        metrics["phase_ms"] = getattr(r, "phase_ms_last", {})     # means over the steps of the last record
    metrics["grad_push"] = bool(r.push_active)
    metrics["grad_stage"] = bool(r.stage_active)
    if r.compress:
        sent = int(r.wire_sent.item())
        metrics["wire"] = (r.cwire + "+sparse") if r.sparse_r is not None else r.cwire
        metrics["wire_sent_fraction"] = sent / max(1, r.wire_rounds * r.n_pad) if r.widx is not None else None
        if r.world > 1 and r.sync_mode in ("fused", "oneshot"):
            # bytes this rank read from its peers per round, against what the dense 16-bit wire moves for the same ranges
            owned = sum(e - b for b, e in r.own[r.rank])
            senders = len([q for q in r.sync_workers if q != r.rank])
            dense = 2 * owned * senders
            got = int(r.wire_bytes.item()) / max(1, r.wire_rounds) if r.sparse_r is not None else dense
            t = torch.tensor([got, dense], dtype=torch.float64, device=r.dev)
            dist.all_reduce(t, group=r.group)
            metrics["wire_bytes_per_round"], metrics["wire_dense16_bytes_per_round"] = float(t[0]), float(t[1])
            metrics["wire_dense32_bytes_per_round"] = 2.0 * float(t[1])
    if len(r.bench_events) == 2:
        metrics["bench_ms"] = r.bench_events[0].elapsed_time(r.bench_events[1])
        metrics["bench_wall_s"] = r.bench_wall[1] - r.bench_wall[0]
        if r.world > 1:  # the slowest rank defines the time
            t = torch.tensor([metrics["bench_ms"], metrics["bench_wall_s"]], dtype=torch.float64, device=r.dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=r.group)
            metrics["bench_ms"], metrics["bench_wall_s"] = float(t[0]), float(t[1])
    tracer.write()
    r.result = {"params": params, "metrics": metrics}
    # every process closes its own event stream (the other events come from rank 0 only)
    r.emit({"kind": "complete", "worker": 0, "losses": [], "text": r.stop_reason})
    return {"params": params, "metrics": metrics}
