#!/usr/bin/env python
"""Headline benchmark: samples/sec of the flagship training step on N B200s of one node.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched once per GPU by torchrun)
    python bench.py --impl reference ...                      (the reference itself, if installable)

Flagship = the deep dense MLP named by the baseline configs: 8 layers of width 8192 (GELU) + a
1000-class head, input N(0,1) of width 8192, f32 master weights with bf16 tensor-core tiles, SGD with
momentum 0.9, batch 512 per GPU (weak scaling), parameter server with the flat parameter vector split
evenly over min(4, N) server ranks that also train (every GPU is a worker). Random-init weights and
synthetic data of that shape. Other configs: ``--config mlp|wide|cnn`` (see CONFIGS).

Two measurements, both through the public API (``orchestra.orchestrate(...).wait()``):
  value  device-timed K steps with the dataset resident in HBM (inputs gathered on the device)
  e2e    the same run with the dataset in pinned host memory: every step's inputs cross PCIe inside
         the timed region and the step's loss is read back to the host
The reference publishes no number for this configuration (its figures are CPU runs of LeNet-5 / Nielsen), so
``vs_baseline`` is measured in the same invocation: the NCCL + cuBLAS arm (``baseline/torch_nccl.py``: the same model,
strategy, batch and wire width written with library calls only) runs right after ours with the same N, K and W, and
``vs_baseline`` = our value / that arm's value (``baseline`` holds its numbers; ``--no-baseline`` skips it).
Timing: CUDA events on the training stream, after W warm-up steps, with synchronize + barrier on both
sides, max over ranks. Every step reads inputs (8 MB+ activations) and 2.7 GB of weights/gradients,
far above the 126 MB L2, so no explicit L2 flush is needed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    # name: (x_size, hidden layers [(width, act)], classes, tile, optimizer, per-gpu batch, strategy)
    "deep": dict(x=8192, hidden=[(8192, "gelu")] * 8, classes=1000, tile="bf16", opt=("momentum", 0.01, 0.9),
                 batch=512, strategy="ps4", init="kaiming", data="normal",
                 model="deep-mlp-8x8192-gelu-1000 (545M params)"),
    "wide": dict(x=784, hidden=[(4096, "relu")] * 3, classes=10, tile="tf32", opt=("adam", 1e-3), batch=1024,
                 strategy="ar", init="kaiming", data="uniform", model="wide-mlp-784-4096x3-10"),
    "mlp": dict(x=784, hidden=[(128, "relu")], classes=10, tile="tf32", opt=("sgd", 0.01), batch=32, strategy="ar",
                init="xavier_uniform", data="uniform", model="mlp-784-128-10"),
    # conv entries: (filters, kernel, stride, padding), all ReLU; global batch 2048 over 6 workers = 342 per worker
    "cnn": dict(x=784, conv_input=(1, 28, 28), conv=[(32, 3, 1, 1), (64, 3, 2, 1), (64, 3, 2, 1)], hidden=[(128, "relu")],
                classes=10, tile="tf32", opt=("adam", 1e-3), batch=342, strategy="ps2", init="kaiming", data="uniform",
                model="cnn-3conv-2dense-28x28"),
}
SWITCH = {"metric": "grad_norm", "window": 50, "threshold": 1e-2}


def reference_arm() -> None:
    why = ("the reference is a Rust workspace whose Python module builds with maturin + cargo; neither a Rust "
           "toolchain nor vendored crates exist offline (pip install: \"No module named 'maturin'\")")
    if os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "orchestra")):
        why = "baseline/_ref holds no built extension module (no Rust toolchain offline)"
    print(json.dumps({"impl": "reference", "unavailable": why}))


def build_run(cfg: dict, n_gpus: int, steps_total: int, data_mode: str, seed: int = 0):
    import numpy as np

    import orchestra
    from orchestra import Sequential
    from orchestra.activations import GELU, ReLU, Softmax
    from orchestra.arch import Dense
    from orchestra.datasets import InlineDataset
    from orchestra.initialization import Kaiming, XavierUniform
    from orchestra.loss_fns import CrossEntropy
    from orchestra.optimizers import Adam, GradientDescent, GradientDescentWithMomentum
    from orchestra.store import BlockingStore
    from orchestra.sync import BarrierSync

    init = Kaiming() if cfg["init"] == "kaiming" else XavierUniform()
    act = {"gelu": GELU, "relu": lambda: ReLU(0.0)}
    layers = []
    if cfg.get("conv"):
        from orchestra.arch import Conv2d
        c, h, w_ = cfg["conv_input"]
        for f, k, s, p in cfg["conv"]:
            layers.append(Conv2d((c, h, w_), (f, c, k), s, p, init, ReLU(0.0)))
            c, h, w_ = f, (h + 2 * p - k) // s + 1, (w_ + 2 * p - k) // s + 1
    layers += [Dense(w, init, act[a]()) for w, a in cfg["hidden"]] + [Dense(cfg["classes"], init, Softmax())]
    model = Sequential(layers)
    B = cfg["batch"]
    steps_per_epoch = 8
    rows = n_gpus * B * steps_per_epoch
    rng = np.random.default_rng(seed)
    if cfg["data"] == "normal":
        xs = rng.standard_normal((rows, cfg["x"]), dtype=np.float32)
    else:
        xs = rng.random((rows, cfg["x"]), dtype=np.float32)
    ys = np.zeros((rows, cfg["classes"]), dtype=np.float32)
    ys[np.arange(rows), rng.integers(0, cfg["classes"], rows)] = 1.0
    ds = InlineDataset(xs, ys, cfg["x"], cfg["classes"])
    o = cfg["opt"]
    opt = {"sgd": lambda: GradientDescent(o[1]), "momentum": lambda: GradientDescentWithMomentum(o[1], o[2]),
           "adam": lambda: Adam(o[1])}[o[0]]()
    epochs = -(-steps_total // steps_per_epoch)
    addrs = [f"gpu:{i}" for i in range(n_gpus)]
    b200 = {"sync_every": "step", "tile_dtype": cfg["tile"], "data": data_mode, "sharding": "even", "colocate": True}
    if cfg.get("grad_push"):
        b200["grad_push"] = cfg["grad_push"]
    if cfg.get("grad_stage"):
        b200["grad_stage"] = cfg["grad_stage"]
    if cfg.get("pre_reduce"):
        b200["pre_reduce"] = cfg["pre_reduce"]
    if cfg.get("phase_timing"):
        b200["phase_timing"] = True
    if cfg.get("wire"):
        b200["wire_dtype"] = cfg["wire"]
    strat = cfg["strategy"]
    if strat.startswith("ps") or strat.startswith("ss"):
        ns = min(int(strat[2:] or 2), n_gpus)
        if strat.startswith("ss"):
            b200.update(switch_metric=SWITCH["metric"], switch_window=SWITCH["window"], switch_threshold=SWITCH["threshold"])
        fn = orchestra.parameter_server if strat.startswith("ps") else orchestra.strategy_switch
        training = fn(addrs, ns, ds, opt, CrossEntropy(), BarrierSync(), BlockingStore(), max_epochs=epochs, batch_size=B,
                      seed=seed, b200=b200)
        par = f"{strat[:2]}(servers={ns},colocated)+dp{n_gpus}"
    else:
        training = orchestra.all_reduce(addrs, ds, opt, CrossEntropy(), max_epochs=epochs, batch_size=B, seed=seed,
                                        b200=b200)
        par = f"dp{n_gpus}"
    return model, training, par


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc, self.lines = None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        time.sleep(0.1)
        sm, mx, reasons = [], [], set()
        for ln in list(self.lines):
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9 or f[0] != "0":
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        busy = sorted(sm)[len(sm) // 2:] if sm else []
        return {"sm_mhz": busy[len(busy) // 2] if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--config", default="deep", choices=sorted(CONFIGS))
    ap.add_argument("--push", default=None, choices=("on", "off", "auto", "direct", "reduce"),
                    help="gradient push: auto/on = 16-bit tiles + copy engines, direct = epilogue stores into the owner's window, "
                         "reduce = f32 reduce-adds, off = the fused kernel pulls")
    ap.add_argument("--pre-reduce", default=None, choices=("auto", "on", "off"),
                    help="fewer owners than ranks: ranks that own nothing sum a part of each owner's share (default auto)")
    ap.add_argument("--stage", default=None, choices=("on", "off", "auto"), help="staged reduce-scatter during backward")
    ap.add_argument("--phases", action="store_true",
                    help="diagnostic: run the steps uncaptured with CUDA events around compute / exchange / refresh and add "
                         "their mean durations (phase_ms) to the line; such a line is not a benchmark value")
    ap.add_argument("--strategy", default=None, help="override the config's strategy: ar | psN | ssN (N server ranks)")
    ap.add_argument("--switch-window", type=int, default=None, help="strategy switch: window (steps) of the gradient-norm test")
    ap.add_argument("--switch-threshold", type=float, default=None, help="strategy switch: relative-change threshold")
    ap.add_argument("--no-baseline", action="store_true", help="do not run the NCCL + cuBLAS arm after ours (vs_baseline: null)")
    ap.add_argument("--wire", default=None, choices=("auto", "f32", "f16", "bf16"), help="gradient wire between GPUs")
    args = ap.parse_args()
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:      # one line per job, also when launched once per GPU
            reference_arm()
        return
    import torch
    import torch.distributed as dist

    from orchestra import orchestrate

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))))
    cfg = dict(CONFIGS[args.config])
    if args.strategy:
        cfg["strategy"] = args.strategy
    if args.push:
        cfg["grad_push"] = args.push
    if args.stage:
        cfg["grad_stage"] = args.stage
    if args.pre_reduce:
        cfg["pre_reduce"] = args.pre_reduce
    if args.phases:
        cfg["phase_timing"] = True
    if args.wire:
        cfg["wire"] = args.wire
    if args.switch_window:
        SWITCH["window"] = args.switch_window
    if args.switch_threshold is not None:
        SWITCH["threshold"] = args.switch_threshold
    W, K = max(3, args.warmup), args.steps
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import torch_nccl
    st = cfg["strategy"]
    nccl_args = (cfg, args.config, st[:2], int(st[2:] or 2) if st != "ar" else 1, K, W, SWITCH)
    nccl_wire = "f32" if cfg.get("wire") == "f32" else "bf16"
    if args.impl == "nccl":
        torch_nccl.main(*nccl_args, ClockSampler, nccl_wire)
        if world > 1:
            dist.destroy_process_group()
        return
    os.environ["ONO_BENCH_WARMUP"], os.environ["ONO_BENCH_STEPS"] = str(W), str(K)
    results = {}
    clocks = None
    for mode in ("device", "host"):
        model, training, par = build_run(cfg, world, W + K, mode)
        sampler = ClockSampler() if (rank == 0 and mode == "device") else None
        if sampler:
            sampler.start()
        trained = orchestrate(model, training).wait(quiet=True)
        if sampler:
            clocks = sampler.stop()
        results[mode] = trained.metrics()
        del trained
        torch.cuda.empty_cache()
    if world > 1:
        dist.barrier()
    out = None
    if rank == 0:
        m, e = results["device"], results["host"]
        gb = cfg["batch"] * world
        value = gb * K / (m["bench_ms"] / 1e3)
        e2e = gb * K / e["bench_wall_s"]
        # parameters + gradients + optimizer state touched by every step, against the 126 MB L2
        widths = [cfg["x"] if not cfg.get("conv") else 3136] + [w for w, _ in cfg["hidden"]] + [cfg["classes"]]
        n_par = sum(a * b + b for a, b in zip(widths[:-1], widths[1:]))
        ws_mb = n_par * 4 * 3 / 1e6
        l2_note = (f"per-step working set (~{ws_mb:.0f} MB of weights, gradients and optimizer state) exceeds the 126 MB L2"
                   if ws_mb > 126 else
                   f"per-step working set (~{ws_mb:.0f} MB) fits in L2: steady-state training loop, no flush between steps")
        out = {
            "metric": "samples/sec (device-timed, max over ranks)", "value": value, "unit": "samples/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": m["bench_ms"] / K, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None,
            "dtype": "bf16" if cfg["tile"] == "bf16" else "tf32", "data": "synthetic",
            "config": {"model": cfg["model"], "global_batch": gb, "seq_len": None, "parallelism": par,
                       "optimizer": cfg["opt"][0], "l2": l2_note,
                       "sync": m["sync_mode"], "wire": m.get("wire"), "wire_push": bool(m.get("wire_push", False)),
                       "wire_transport": m.get("wire_transport"), "param_pull": m.get("param_pull"),
                       "pre_reduce": bool(m.get("pre_reduce", False)),
                       "wgrad_apply": bool(m.get("wgrad_apply", False)),
                       "grad_push": bool(m.get("grad_push", False)), "grad_stage": bool(m.get("grad_stage", False))},
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "samples/s", "h2d_bytes_per_step": e["h2d_bytes_per_step"],
                    "d2h_bytes_per_step": e["d2h_bytes_per_step"], "ms_per_step": e["bench_wall_s"] * 1e3 / K,
                    "device_ms_per_step": e["bench_ms"] / K},
            "gpu_launches": int(m["launches_per_step"]) * K,
        }
        if cfg["strategy"].startswith("ss"):
            # the two phases of the strategy switch, from the per-step CUDA events of the device-resident run: all-reduce
            # before the promoted ranks became servers, parameter server after (steps next to the switch itself left out)
            sm, at = m.get("step_ms") or [], m.get("switched_at_step")
            out["switch"] = {"metric": SWITCH["metric"], "window": SWITCH["window"], "threshold": SWITCH["threshold"],
                             "switched_at_step": at, "declined": bool(m.get("switch_declined", False))}
            if at and len(sm) > at + 6 and at > 8:
                pre, post = sm[5:at - 2], sm[at + 3:]
                workers_after = world - min(int(cfg["strategy"][2:] or 2), world)
                out["switch"].update(pre_ms_per_step=sum(pre) / len(pre), post_ms_per_step=sum(post) / len(post),
                                     pre_samples_per_s=gb / (sum(pre) / len(pre) / 1e3),
                                     post_samples_per_s=cfg["batch"] * workers_after / (sum(post) / len(post) / 1e3))
        if m.get("phase_ms"):
            out["phase_ms"] = m["phase_ms"]
            out["config"]["phase_timing"] = "steps ran uncaptured with per-phase events: diagnostic line, not a benchmark value"
    # The comparison arm runs after our numbers are final. It is library code driven by this script: if it fails or does
    # not finish within its deadline, our line is printed without the comparison and the job still ends cleanly.
    if not args.no_baseline and not args.phases:
        def give_up():
            if rank == 0:
                out["baseline_error"] = "the NCCL + cuBLAS arm did not finish within its deadline"
                print(json.dumps(out), flush=True)
            os._exit(0)

        timer = threading.Timer(float(os.environ.get("ONO_BASELINE_DEADLINE_S", "240")), give_up)
        timer.daemon = True
        timer.start()
        base = None
        try:
            base = torch_nccl.measure(*nccl_args, None, nccl_wire)       # every rank takes part; rank 0 gets the line
        except Exception as exc:        # noqa: BLE001 - whatever the library arm raises must not cost our own result
            if rank == 0:
                out["baseline_error"] = f"{type(exc).__name__}: {exc}"[:300]
        timer.cancel()
        if rank == 0 and base:
            out["vs_baseline"] = out["value"] / base["value"]
            out["baseline"] = {"impl": base["impl"], "what": "same model / strategy / batch / wire with NCCL + cuBLAS (baseline/torch_nccl.py), "
                               "run in this invocation right after ours", "value": base["value"], "ms_per_step": base["ms_per_step"],
                               "e2e_value": base["e2e"]["value"], "e2e_ratio": out["e2e"]["value"] / base["e2e"]["value"],
                               "cuda_graph": base["config"]["cuda_graph"], "wire": base["config"]["wire"]}
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
