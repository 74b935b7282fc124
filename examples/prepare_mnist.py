#!/usr/bin/env python
"""Turn the standard MNIST IDX files into the packed little-endian f32 files the trainers read.

    python examples/prepare_mnist.py train-images-idx3-ubyte.gz train-labels-idx1-ubyte.gz out_dir [--limit N]

Writes ``out_dir/mnist_x.bin`` (rows of 784 pixels scaled to [0, 1]) and ``out_dir/mnist_y.bin`` (one-hot rows of 10),
the format of the reference's datasets (orchestrator/src/dataset_format.rs:12-155, benchmarks/issue/runner.py:70-77):

    SAMPLES_PATH=out_dir/mnist_x.bin LABELS_PATH=out_dir/mnist_y.bin python examples/local.py

(The reference fetches a zip from the network in scripts/download_mnist.py; this script only converts files you have.)
"""
import gzip
import os
import struct
import sys

import numpy as np


def read_idx(path: str) -> np.ndarray:
    op = gzip.open if path.endswith(".gz") else open
    with op(path, "rb") as f:
        magic, = struct.unpack(">I", f.read(4))
        ndim = magic & 0xFF
        if (magic >> 8) != 0x08:
            raise ValueError(f"{path}: not an unsigned-byte IDX file")
        dims = struct.unpack(">" + "I" * ndim, f.read(4 * ndim))
        return np.frombuffer(f.read(), dtype=np.uint8).reshape(dims)


def main():
    if len(sys.argv) < 4:
        raise SystemExit(__doc__)
    images, labels, out = sys.argv[1:4]
    limit = int(sys.argv[sys.argv.index("--limit") + 1]) if "--limit" in sys.argv else None
    x, y = read_idx(images), read_idx(labels)
    if limit:
        x, y = x[:limit], y[:limit]
    if x.shape[0] != y.shape[0]:
        raise SystemExit("images and labels differ in count")
    os.makedirs(out, exist_ok=True)
    (x.reshape(x.shape[0], -1).astype("<f4") / 255.0).tofile(os.path.join(out, "mnist_x.bin"))
    np.eye(10, dtype="<f4")[y].tofile(os.path.join(out, "mnist_y.bin"))
    print(f"{x.shape[0]} samples -> {out}/mnist_x.bin, {out}/mnist_y.bin")


if __name__ == "__main__":
    main()
