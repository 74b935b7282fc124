#!/usr/bin/env python
"""Train LeNet-5 or the Nielsen network the way the reference's driver does (orchestra-py/local.py:1-76).

    NODES=gpu:0,gpu:1 SERVERS=1 python examples/local.py                       # synthetic MNIST-shaped data
    SAMPLES_PATH=train_x.bin LABELS_PATH=train_y.bin python examples/local.py  # packed f32 (or .csv/.tsv)

Environment: NODES (comma-separated addresses: gpu:<i>, cpu:<i> or host:port of listening nodes; default the
local GPUs, or three CPU ranks without a GPU), SERVERS (parameter servers; 0 = ring all-reduce), MODEL
(lenet5|nielsen), EPOCHS, BATCH, SAMPLES_PATH, LABELS_PATH, SAFETENSORS_PATH, EARLY_STOPPING_TOLERANCE.
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import orchestra  # noqa: E402
from orchestra import orchestrate  # noqa: E402
from orchestra.datasets import InlineDataset, LocalDataset  # noqa: E402
from orchestra.loss_fns import CrossEntropy  # noqa: E402
from orchestra.optimizers import GradientDescent  # noqa: E402
from orchestra.store import BlockingStore  # noqa: E402
from orchestra.sync import BarrierSync  # noqa: E402

from mnist_models import lenet5, nielsen  # noqa: E402


def default_nodes():
    try:
        import torch

        n = torch.cuda.device_count()
    except Exception:
        n = 0
    return [f"gpu:{i}" for i in range(n)] if n else ["cpu:0", "cpu:1", "cpu:2"]


def main():
    nodes = os.environ["NODES"].split(",") if os.environ.get("NODES") else default_nodes()
    servers = int(os.environ.get("SERVERS", "0"))
    epochs, batch = int(os.environ.get("EPOCHS", "4")), int(os.environ.get("BATCH", "64"))
    model = {"lenet5": lenet5, "nielsen": nielsen}[os.environ.get("MODEL", "lenet5")]()
    if os.environ.get("SAMPLES_PATH"):
        ds = LocalDataset(os.environ["SAMPLES_PATH"], os.environ["LABELS_PATH"], 784, 10)
    else:
        rng = np.random.default_rng(42)
        rows = int(os.environ.get("ROWS", "4096"))
        labels = rng.integers(0, 10, rows)
        proto = rng.random((10, 784), dtype=np.float32)           # one blurry prototype per class
        xs = np.clip(proto[labels] + 0.3 * rng.standard_normal((rows, 784), dtype=np.float32), 0, 1)
        ds = InlineDataset(xs, np.eye(10, dtype=np.float32)[labels], 784, 10)
    tol = os.environ.get("EARLY_STOPPING_TOLERANCE")
    common = dict(max_epochs=epochs, batch_size=batch, seed=42, early_stopping_tolerance=float(tol) if tol else None)
    opt, loss = GradientDescent(0.05), CrossEntropy()
    if servers > 0:
        cfg = orchestra.parameter_server(nodes, servers, ds, opt, loss, BarrierSync(), BlockingStore(), **common,
                                         b200={"colocate": all(n.startswith("gpu:") for n in nodes)})
    else:
        cfg = orchestra.all_reduce(nodes, ds, opt, loss, **common)
    trained = orchestrate(model, cfg).wait()
    hist = trained.loss_history()
    print(f"epochs={len(hist)} first_loss={hist[0]:.5f} last_loss={hist[-1]:.5f} params={len(trained.weights_array())}")
    out = os.environ.get("SAFETENSORS_PATH")
    if out:
        trained.save_safetensors(out)
        print("saved", out)


if __name__ == "__main__":
    main()
