"""Optimizer-state sidecar of a checkpoint.

The reference exports final weights only (orchestrator/src/sessions/trained_model.rs:36-121): no optimizer state,
no resume; at a strategy switch the state is reset (worker/src/builder.rs:179-181). Here a run can additionally
write ``<name>.state.safetensors`` (``b200.state_path``) and a later run can start from it
(``b200.init_state_from``, together with ``b200.init_from`` for the weights), which continues momentum / Adam
exactly where the first run stopped.

The file is a safetensors container (8-byte little-endian header length, JSON header, raw little-endian data):
``optimizer.m`` and ``optimizer.v`` F32 ``[n_params]`` in the flat parameter order of the weights file,
``optimizer.adam_pows`` F32 ``[2]`` (running b1^t, b2^t), and string metadata (optimizer kind, epochs done).
"""
from __future__ import annotations

import json
import struct

import numpy as np


def weight_tensors(engine_layers: list[dict], params: np.ndarray) -> list:
    """(name, array) pairs of a weights checkpoint in the reference's layout
    (orchestrator/src/sessions/trained_model.rs:36-121): for layer i in model order ``layer_{i}.weight`` F32 [in, out]
    (dense) / [F, C, K, K] (conv) / [0] (max-pool), then ``layer_{i}.bias`` F32 [out] / [F] / [0]; the data are consecutive
    slices of the flat parameter vector."""
    out, off = [], 0
    shapes = []
    for l in engine_layers:
        if l["kind"] == "dense":
            shapes.append(((l["in"], l["out"]), (l["out"],)))
        elif l["kind"] == "conv":
            f, c, k = l["kernel_dim"]
            shapes.append(((f, c, k, k), (f,)))
        else:
            shapes.append(((0,), (0,)))
    total = sum(int(np.prod(w)) + int(np.prod(b)) for w, b in shapes)
    if total != params.shape[0]:
        raise ValueError(f"model layout covers {total} parameters, the vector has {params.shape[0]}")
    for i, l in enumerate(engine_layers):
        if l["kind"] == "dense":
            wshape, bshape = (l["in"], l["out"]), (l["out"],)
        elif l["kind"] == "conv":
            f, c, k = l["kernel_dim"]
            wshape, bshape = (f, c, k, k), (f,)
        else:
            wshape, bshape = (0,), (0,)
        for name, shape in ((f"layer_{i}.weight", wshape), (f"layer_{i}.bias", bshape)):
            n = int(np.prod(shape))
            out.append((name, np.ascontiguousarray(params[off:off + n], dtype="<f4").reshape(shape)))
            off += n
    return out


def layers_from_plan(plan: dict) -> list[dict]:
    """The layer descriptions ``weight_tensors`` needs, straight from a plan's LayerSpec documents."""
    out = []
    for l in plan["layers"]:
        (kind, body), = l["spec"].items()
        if kind == "dense":
            out.append({"kind": "dense", "in": body["dim"][0], "out": body["dim"][1]})
        elif kind == "conv":
            out.append({"kind": "conv", "kernel_dim": body["kernel_dim"]})
        else:
            out.append({"kind": "pool"})
    return out


def checkpoint_paths(pattern: str, epochs_done: int) -> tuple[str, str]:
    """Weights file and state sidecar of a periodic checkpoint: ``{epoch}`` in the pattern is replaced, else
    ``.epoch<N>`` is appended; the sidecar sits beside the weights as ``<base>.state.safetensors``."""
    path = pattern.replace("{epoch}", str(epochs_done)) if "{epoch}" in pattern else f"{pattern}.epoch{epochs_done}"
    base = path[:-len(".safetensors")] if path.endswith(".safetensors") else path
    return path, base + ".state.safetensors"


def save_tensors(path: str, tensors: list, meta: dict | None = None, sort: bool = True) -> None:
    """Write (name, f32 array) pairs as a safetensors file (no metadata block unless ``meta`` is given). Entries are
    laid out in name order, like the core exporter (csrc/core/codec.cpp) and the reference's, so the files are equal
    byte for byte. The file appears under its final name only when complete (temporary file, fsync, rename): a crash
    during a periodic checkpoint leaves the previous file in place, never a truncated one."""
    import os

    if sort:
        tensors = sorted(tensors, key=lambda nt: nt[0])
    header: dict = {}
    if meta is not None:
        header["__metadata__"] = {k: str(val) for k, val in meta.items()}
    off = 0
    for name, t in tensors:
        header[name] = {"dtype": "F32", "shape": list(t.shape), "data_offsets": [off, off + t.nbytes]}
        off += t.nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, t in tensors:
            f.write(t.tobytes())
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def save_state(path: str, m: np.ndarray, v: np.ndarray, adam_pows: np.ndarray, **meta) -> None:
    save_tensors(path, [("optimizer.m", np.ascontiguousarray(m, dtype="<f4")), ("optimizer.v", np.ascontiguousarray(v, dtype="<f4")),
                        ("optimizer.adam_pows", np.ascontiguousarray(adam_pows, dtype="<f4"))], meta, sort=False)


def load_state(path: str, n_params: int) -> dict:
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        if hlen > (1 << 26):
            raise ValueError(f"{path}: implausible header length {hlen}")
        header = json.loads(f.read(hlen))
        data = f.read()
    out: dict = {"meta": header.get("__metadata__", {})}
    for name in ("optimizer.m", "optimizer.v", "optimizer.adam_pows"):
        e = header.get(name)
        if e is None or e.get("dtype") != "F32":
            raise ValueError(f"{path}: no F32 tensor {name}")
        b, en = e["data_offsets"]
        arr = np.frombuffer(data[b:en], dtype="<f4").reshape(e["shape"])
        out[name.split(".", 1)[1]] = arr
    if out["m"].shape != (n_params,) or out["v"].shape != (n_params,) or out["adam_pows"].shape != (2,):
        raise ValueError(f"{path}: state of {out['m'].shape[0]} parameters does not fit a model of {n_params}")
    return out
