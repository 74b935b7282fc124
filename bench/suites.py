#!/usr/bin/env python
"""Strategy benchmark suites over the public API, in the spirit of the reference's harness
(benchmarks/run_issue_benchmarks.py:64-229, benchmarks/issue/{suites,runner,metrics,results}.py).

    python bench/suites.py [--suite strategies|scalability|offline|published] [--model lenet5|nielsen|both]
                           [--nodes gpu|cpu] [--rows 4096] [--epochs 4] [--repeats 1] [--out bench/results]

Every run trains LeNet-5 or the Nielsen network on seeded MNIST-shaped synthetic data (class prototypes plus
noise) through ``orchestrate(...).wait()`` and records, like the reference (benchmarks/issue/metrics.py:11-32):
``train_seconds`` (wall clock of ``wait``), ``samples_per_sec = samples * epochs / train_seconds``,
``epochs_per_sec``, ``final_loss``, ``accuracy`` on a held-out set (evaluated with a plain PyTorch restatement
of the model loaded from the trained weights, as benchmarks/issue/models.py:138-154 does), ``loss_per_sec`` and
``accuracy_per_sec``. Results go to ``<out>/history.jsonl`` (one record per repeat) and ``<out>/summary.md``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "examples"))


def make_data(rows: int, seed: int):
    rng = np.random.default_rng(seed)
    proto = rng.random((10, 784), dtype=np.float32)
    def draw(n):
        labels = rng.integers(0, 10, n)
        xs = np.clip(proto[labels] + 0.35 * rng.standard_normal((n, 784), dtype=np.float32), 0, 1).astype(np.float32)
        return xs, labels
    xtr, ltr = draw(rows)
    xte, lte = draw(max(256, rows // 8))
    return xtr, np.eye(10, dtype=np.float32)[ltr], xte, lte


def torch_accuracy(model_name: str, weights: np.ndarray, xs: np.ndarray, labels: np.ndarray) -> float:
    """Plain PyTorch restatement of the two models, fed with the flat parameter vector (layout: per layer W then b;
    dense W is [in, out], conv W is [F, C, k, k])."""
    import torch
    import torch.nn.functional as F

    w = torch.from_numpy(np.asarray(weights, dtype=np.float32))
    off = 0

    def take(*shape):
        nonlocal off
        n = int(np.prod(shape))
        t = w[off:off + n].view(*shape)
        off += n
        return t

    x = torch.from_numpy(xs).view(-1, 1, 28, 28)
    # the reference pads pooling inputs with zeros that compete in the max; neither model pads its pools
    if model_name == "nielsen":
        k, b = take(20, 1, 5, 5), take(20)
        a = F.max_pool2d(F.conv2d(x, k, b), 2, 2).flatten(1)
        a = torch.sigmoid(a @ take(20 * 12 * 12, 100) + take(100))
        z = a @ take(100, 10) + take(10)
    else:
        k, b = take(6, 1, 5, 5), take(6)
        a = F.max_pool2d(torch.tanh(F.conv2d(x, k, b, padding=2)), 2, 2)
        k, b = take(16, 6, 5, 5), take(16)
        a = F.max_pool2d(torch.tanh(F.conv2d(a, k, b)), 2, 2).flatten(1)
        a = torch.tanh(a @ take(400, 120) + take(120))
        a = torch.tanh(a @ take(120, 84) + take(84))
        z = a @ take(84, 10) + take(10)
    assert off == w.numel(), (off, w.numel())
    return float((z.argmax(1).numpy() == labels).mean())


def suites(kind: str, n_nodes: int):
    """(label, strategy, workers, servers, extra) tuples; the reference's suites use 3/5/7 workers and 2 servers
    (benchmarks/issue/suites.py:148-178), capped here by the nodes available."""
    cap = lambda w: max(1, min(w, n_nodes))
    if kind == "strategies":
        return [("all_reduce", "ar", cap(5), 0, {}), ("ps_blocking", "ps", cap(5), min(2, cap(5)), {}),
                ("ps_non_blocking", "ps_async", cap(5), min(2, cap(5)), {}), ("strategy_switch", "ss", cap(5), min(2, cap(5)), {})]
    if kind == "scalability":
        return [(f"all_reduce_{w}w", "ar", w, 0, {}) for w in sorted({cap(1), cap(3), cap(5), cap(7)})] + \
               [(f"ps_{w}w_2s", "ps", w, min(2, w), {}) for w in sorted({cap(3), cap(5)})]
    if kind == "offline":
        return [(f"all_reduce_offline{e}", "ar", cap(3), 0, {"offline_epochs": e}) for e in (0, 1, 4)]
    if kind == "published":
        # the throughput rows the reference publishes (benchmarks/README.md:80-85 execution speed, :116-125 scalability):
        # 4 000 samples, 8 epochs, plain SGD; servers are separate nodes, so a PS row uses workers + 2 nodes
        rows = [("AR 3w offline 0 b64", "ar", 3, 0, {}), ("AR 3w offline 4 b64", "ar", 3, 0, {"offline_epochs": 4}),
                ("AR 3w offline 0 b256", "ar", 3, 0, {"batch": 256}), ("AR 5w", "ar", 5, 0, {}), ("AR 7w", "ar", 7, 0, {}),
                ("PS blocking 3w+2s", "ps", 3, 2, {"pure_servers": True}), ("PS blocking 5w+2s", "ps", 5, 2, {"pure_servers": True})]
        return [r for r in rows if r[2] + (r[3] if r[4].get("pure_servers") else 0) <= n_nodes]
    raise SystemExit(f"unknown suite {kind}")


# samples/s the reference publishes for the rows of the `published` suite (benchmarks/README.md:80-85,116-125; CPU
# containers on one ~8-core host)
PUBLISHED = {
    ("lenet5", "AR 3w offline 0 b64"): 9675, ("lenet5", "AR 3w offline 4 b64"): 9827, ("lenet5", "AR 3w offline 0 b256"): 8928,
    ("nielsen", "AR 3w offline 0 b64"): 8353, ("nielsen", "AR 3w offline 4 b64"): 8527, ("nielsen", "AR 3w offline 0 b256"): 7721,
    ("lenet5", "AR 5w"): 10012, ("lenet5", "AR 7w"): 10899, ("lenet5", "PS blocking 3w+2s"): 9970, ("lenet5", "PS blocking 5w+2s"): 11356,
    ("nielsen", "AR 5w"): 8404, ("nielsen", "AR 7w"): 8605, ("nielsen", "PS blocking 3w+2s"): 8227, ("nielsen", "PS blocking 5w+2s"): 8920,
}


class NodeProcesses:
    """`n` native node processes (`bin/ono-node`, one CPU rank each) listening on loopback ports: the deployment the
    reference's numbers come from (one node per container on one host, its README "benchmarks"), minus the containers."""

    def __init__(self, n: int):
        import socket
        import subprocess

        exe = os.path.join(ROOT, "bin", "ono-node")
        if not os.path.exists(exe):
            raise SystemExit("bin/ono-node is missing: python -m oxidized_neural_orchestra_b200.build")
        self.procs, self.addrs = [], []
        env = dict(os.environ, ONO_LOG="warn", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
        for _ in range(n):
            with socket.socket() as sk:
                sk.bind(("127.0.0.1", 0))
                port = sk.getsockname()[1]
            self.procs.append(subprocess.Popen([exe, "--port", str(port), "--device", "cpu"], env=env))
            self.addrs.append(f"127.0.0.1:{port}")
        deadline = time.time() + 60
        for a in self.addrs:
            host, port = a.rsplit(":", 1)
            while True:
                try:
                    socket.create_connection((host, int(port)), timeout=0.5).close()
                    break
                except OSError:
                    if time.time() > deadline:
                        self.close()
                        raise SystemExit(f"node {a} did not start listening")
                    time.sleep(0.05)

    def close(self):
        for p in self.procs:
            p.kill()
        for p in self.procs:
            p.wait(timeout=30)


def run_one(model_name, label, strategy, workers, servers, extra, prefix, data, epochs, batch):
    if prefix == "tcp":
        extra = dict(extra)
        n = workers + (servers if extra.get("pure_servers") else 0)
        nodes = NodeProcesses(n)
        try:
            return run_one(model_name, label, strategy, workers, servers, dict(extra, _addrs=nodes.addrs), "node", data, epochs, batch)
        finally:
            nodes.close()
    return _run_one(model_name, label, strategy, workers, servers, extra, prefix, data, epochs, batch)


def _run_one(model_name, label, strategy, workers, servers, extra, prefix, data, epochs, batch):
    import orchestra
    from mnist_models import lenet5, nielsen
    from orchestra import orchestrate
    from orchestra.datasets import InlineDataset
    from orchestra.loss_fns import CrossEntropy
    from orchestra.optimizers import GradientDescent
    from orchestra.store import BlockingStore
    from orchestra.sync import BarrierSync, NonBlockingSync

    xtr, ytr, xte, lte = data
    extra = dict(extra)
    pure = extra.pop("pure_servers", False)
    batch = extra.pop("batch", batch)
    lr = extra.pop("lr", 0.5)
    addrs = extra.pop("_addrs", None) or [f"{prefix}:{i}" for i in range(workers + (servers if pure else 0))]
    ds = InlineDataset(xtr, ytr, 784, 10)
    wire = extra.pop("wire", None)
    common = dict(max_epochs=epochs, batch_size=batch, seed=42, **extra)
    b200 = {"colocate": True} if (prefix == "gpu" and not pure) else None
    if wire:        # the reference always ships gradients as f16 (comms/src/handles/compressor.rs:104-118)
        b200 = dict(b200 or {}, wire_dtype=wire)
    opt, loss = GradientDescent(lr), CrossEntropy()   # the loss is normalised by batch x classes (cross_entropy.rs:35-47)
    if strategy == "ar":
        cfg = orchestra.all_reduce(addrs, ds, opt, loss, **(dict(common, b200=b200) if b200 else common))
    else:
        sync = NonBlockingSync() if strategy == "ps_async" else BarrierSync()
        fn = orchestra.strategy_switch if strategy == "ss" else orchestra.parameter_server
        kw = dict(common, b200=b200) if b200 and servers >= workers else (dict(common, b200=b200) if b200 else common)
        if prefix == "cpu" and servers >= workers and not pure:
            return None                      # the reference needs at least one pure worker
        cfg = fn(addrs, servers, ds, opt, loss, sync, BlockingStore(), **kw)
    model = {"lenet5": lenet5, "nielsen": nielsen}[model_name]()
    t0 = time.perf_counter()
    trained = orchestrate(model, cfg).wait(quiet=True)
    secs = time.perf_counter() - t0
    hist = trained.loss_history()
    acc = torch_accuracy(model_name, trained.weights_array(), xte, lte)
    done = len(hist)
    met = trained.metrics() or {}
    # device time of the training steps alone (CUDA events; GPU ranks): the wall clock above also holds the start-up
    # of one process per GPU, which the reference's figure (nodes already running) does not
    step_ms = met.get("step_ms") or []
    dev_s = sum(step_ms) / 1e3 if step_ms else None
    return {"device_seconds": dev_s,
            "samples_per_sec_device": (len(xtr) * done / dev_s * (len(step_ms) / (len(step_ms) + 1.0))) if dev_s else None,
            "batch": batch, "nodes": len(addrs), "suite_label": label, "model": model_name, "strategy": strategy, "workers": workers, "servers": servers,
            "backend": prefix, "epochs": done, "samples": len(xtr), "train_seconds": secs,
            "samples_per_sec": len(xtr) * done / secs, "epochs_per_sec": done / secs, "final_loss": hist[-1] if hist else None,
            "accuracy": acc, "loss_per_sec": (hist[0] - hist[-1]) / secs if len(hist) > 1 else 0.0,
            "accuracy_per_sec": acc / secs, "switched": bool(trained.metrics().get("switched", False)), **extra}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--suite", default="strategies")
    ap.add_argument("--model", default="both", choices=("lenet5", "nielsen", "both"))
    ap.add_argument("--nodes", default=None, choices=("gpu", "cpu", "tcp"),
                    help="gpu: one rank per local GPU; cpu: in-process rank threads; tcp: one native ono-node process per node on "
                         "loopback ports (the reference's deployment without the containers)")
    ap.add_argument("--rows", type=int, default=4096)
    ap.add_argument("--epochs", type=int, default=4)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--repeats", type=int, default=1)
    ap.add_argument("--wire", default=None, choices=("f16", "bf16", "f32"), help="gradient wire (b200.wire_dtype); the reference's is f16")
    ap.add_argument("--only", default="", help="comma-separated substrings: run only the suite rows whose label contains one of them")
    ap.add_argument("--out", default=os.path.join(ROOT, "bench", "results"))
    a = ap.parse_args()
    import torch

    prefix = a.nodes or ("gpu" if torch.cuda.is_available() else "cpu")
    n_nodes = torch.cuda.device_count() if prefix == "gpu" else 7
    if a.suite == "published" and a.rows == 4096 and a.epochs == 4:
        a.rows, a.epochs = 4000, 8               # the reference's budget for these rows
    os.makedirs(a.out, exist_ok=True)
    data = make_data(a.rows, 42)
    records = []
    with open(os.path.join(a.out, "history.jsonl"), "a") as hist:
        for model_name in (("lenet5", "nielsen") if a.model == "both" else (a.model,)):
            for label, strategy, workers, servers, extra in suites(a.suite, n_nodes):
                if a.only and not any(k in label for k in a.only.split(",")):
                    continue
                for rep in range(a.repeats):
                    if a.suite == "published":      # the models' recipes: benchmarks/issue/suites.py:148-178
                        extra = dict(extra, lr=0.05 if model_name == "lenet5" else 0.1)
                    if a.wire:
                        extra = dict(extra, wire=a.wire)
                    rec = run_one(model_name, label, strategy, workers, servers, extra, prefix, data, a.epochs, a.batch)
                    if rec is None:
                        continue
                    rec.update(suite=a.suite, repeat=rep, time=time.time())
                    hist.write(json.dumps(rec) + "\n")
                    hist.flush()
                    records.append(rec)
                    print(f"{model_name:8s} {label:22s} {rec['samples_per_sec']:12.0f} samples/s  loss {rec['final_loss']:.5f}  "
                          f"acc {rec['accuracy']:.3f}", file=sys.stderr)
    if a.suite == "published":
        with open(os.path.join(a.out, f"published_{prefix}.md"), "w") as f:
            f.write(f"# The reference's published throughput rows on `{prefix}` nodes ({a.rows} samples, {a.epochs} epochs, SGD)\n\n"
                    "samples/s = samples x epochs / wall seconds of `orchestrate(...).wait()` (the reference's definition); "
                    "`device` = the same count over the CUDA-event time of the training steps (GPU ranks only).\n\n"
                    "| model | run | nodes | batch | samples/s (wall) | samples/s (device) | reference, published | wall / published | final loss | accuracy |\n"
                    "|---|---|---|---|---|---|---|---|---|---|\n")
            for r in records:
                pub = PUBLISHED.get((r["model"], r["suite_label"]))
                dev = f"{r['samples_per_sec_device']:.0f}" if r.get("samples_per_sec_device") else "-"
                f.write(f"| {r['model']} | {r['suite_label']} | {r['nodes']} | {r['batch']} | {r['samples_per_sec']:.0f} | {dev} | "
                        f"{pub if pub else '-'} | {(r['samples_per_sec'] / pub):.2f}x | {r['final_loss']:.5f} | {r['accuracy']:.3f} |\n"
                        if pub else "")
    with open(os.path.join(a.out, "summary.md"), "w") as f:
        f.write(f"# Suite `{a.suite}` on `{prefix}` nodes ({a.rows} samples, {a.epochs} epochs, batch {a.batch})\n\n")
        f.write("| model | run | workers | servers | samples/s | epochs/s | final loss | accuracy | switched |\n|---|---|---|---|---|---|---|---|---|\n")
        for r in records:
            f.write(f"| {r['model']} | {r['suite_label']} | {r['workers']} | {r['servers']} | {r['samples_per_sec']:.0f} | "
                    f"{r['epochs_per_sec']:.3f} | {r['final_loss']:.5f} | {r['accuracy']:.3f} | {r['switched']} |\n")
    print(json.dumps({"suite": a.suite, "runs": len(records), "out": a.out}))


if __name__ == "__main__":
    main()
