#!/usr/bin/env python
"""Checkpoint and resume: train for a few epochs with periodic checkpoints, then start a second run from the last
checkpoint (weights + optimizer state + shuffle position) and carry on.

    python examples/resume.py                      # all local GPUs (three CPU ranks without a GPU), Nielsen network on synthetic MNIST-shaped data
    EPOCHS=6 EVERY=2 OUT=/tmp/ck python examples/resume.py

The reference exports final weights only (orchestrator/src/sessions/trained_model.rs:36-121); the optimizer-state
sidecar and the periodic checkpoints are additions of the `b200` block (`checkpoint_path`, `checkpoint_every`,
`init_from`, `init_state_from`)."""
import os
import sys
import tempfile

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import orchestra  # noqa: E402
from orchestra import orchestrate  # noqa: E402
from orchestra.datasets import InlineDataset  # noqa: E402
from orchestra.loss_fns import CrossEntropy  # noqa: E402
from orchestra.optimizers import Adam  # noqa: E402

from mnist_models import nielsen  # noqa: E402


def main() -> int:
    import torch

    gpu = torch.cuda.is_available()
    nodes = [f"gpu:{i}" for i in range(torch.cuda.device_count())] if gpu else [f"cpu:{i}" for i in range(3)]
    epochs, every = int(os.environ.get("EPOCHS", "4")), int(os.environ.get("EVERY", "2"))
    out = os.environ.get("OUT") or tempfile.mkdtemp(prefix="ono-ck-")
    os.makedirs(out, exist_ok=True)
    rng = np.random.default_rng(42)
    rows = 4096 if gpu else 1024
    labels = rng.integers(0, 10, rows)
    proto = rng.random((10, 784), dtype=np.float32)
    xs = np.clip(proto[labels] + 0.3 * rng.standard_normal((rows, 784), dtype=np.float32), 0, 1)
    ds = InlineDataset(xs, np.eye(10, dtype=np.float32)[labels], 784, 10)

    def cfg(n_epochs, **b200):
        return orchestra.all_reduce(nodes, ds, Adam(1e-3), CrossEntropy(), max_epochs=n_epochs, batch_size=64, seed=42,
                                    b200={**({"sync_every": "step"} if gpu else {}), **b200})

    pattern = os.path.join(out, "nielsen_{epoch}.safetensors")
    first = orchestrate(nielsen(), cfg(epochs, checkpoint_path=pattern, checkpoint_every=every)).wait()
    last = (epochs // every) * every
    weights = pattern.replace("{epoch}", str(last))
    state = weights[:-len(".safetensors")] + ".state.safetensors"
    print(f"first run: loss {first.loss_history()[-1]:.5f}; resuming from {weights}")
    second = orchestrate(nielsen(), cfg(epochs, init_from=weights, init_state_from=state)).wait()
    print(f"second run: loss {second.loss_history()[0]:.5f} -> {second.loss_history()[-1]:.5f}")
    second.save_safetensors(os.path.join(out, "nielsen_final.safetensors"))
    return 0


if __name__ == "__main__":
    sys.exit(main())
