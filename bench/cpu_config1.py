#!/usr/bin/env python
"""The CPU-capable baseline configuration, timed on the C++ engine with in-process CPU ranks:

MLP 784 -> 128 (ReLU) -> 10 (softmax cross-entropy), f32, Xavier-uniform init seed 0, SGD lr 0.01, batch 32, one epoch,
ring all-reduce over 3 workers, 60 000 seeded synthetic samples (pixels ~U[0,1], labels uniform in 0..9).

    python bench/cpu_config1.py [--workers 3] [--samples 60000]

samples/s = samples x epochs / wall seconds of ``orchestrate(...).wait()``, the reference harness's definition
(benchmarks/issue/metrics.py:20-23). Needs no GPU.
"""
import argparse
import json
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workers", type=int, default=3)
    ap.add_argument("--samples", type=int, default=60000)
    a = ap.parse_args()
    import orchestra
    from orchestra import Sequential, orchestrate
    from orchestra.activations import ReLU, Softmax
    from orchestra.arch import Dense
    from orchestra.datasets import InlineDataset
    from orchestra.initialization import XavierUniform
    from orchestra.loss_fns import CrossEntropy
    from orchestra.optimizers import GradientDescent

    rng = np.random.default_rng(0)
    xs = rng.random((a.samples, 784), dtype=np.float32)
    ys = np.eye(10, dtype=np.float32)[rng.integers(0, 10, a.samples)]
    model = Sequential([Dense(128, XavierUniform(), ReLU(0.0)), Dense(10, XavierUniform(), Softmax())])
    cfg = orchestra.all_reduce([f"cpu:{i}" for i in range(a.workers)], InlineDataset(xs, ys, 784, 10), GradientDescent(0.01),
                               CrossEntropy(), max_epochs=1, batch_size=32, seed=0)
    t0 = time.perf_counter()
    trained = orchestrate(model, cfg).wait(quiet=True)
    secs = time.perf_counter() - t0
    print(json.dumps({"config": "mlp-784-128-10, ring all-reduce, CPU ranks", "workers": a.workers, "samples": a.samples, "epochs": 1,
                      "train_seconds": secs, "samples_per_sec": a.samples / secs, "final_loss": trained.loss_history()[-1],
                      "cpus": os.cpu_count()}))


if __name__ == "__main__":
    main()
