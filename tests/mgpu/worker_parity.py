"""SPMD body of the multi-GPU parity test: run under torchrun, one process per GPU.

Every rank trains the same small MLP through the public API on `gpu:<i>` addresses with each strategy
and fused-kernel variant, and rank 0 compares the result with the in-process CPU oracle run of the same
configuration (one batch per worker and epoch, so batch order cannot differ)."""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import orchestra  # noqa: E402
from orchestra import Sequential, orchestrate  # noqa: E402
from orchestra.activations import ReLU, Softmax, Tanh  # noqa: E402
from orchestra.arch import Dense  # noqa: E402
from orchestra.datasets import InlineDataset  # noqa: E402
from orchestra.initialization import XavierUniform  # noqa: E402
from orchestra.loss_fns import CrossEntropy  # noqa: E402
from orchestra.optimizers import Adam, GradientDescent, GradientDescentWithMomentum  # noqa: E402
from orchestra.store import BlockingStore, WildStore  # noqa: E402
from orchestra.sync import BarrierSync, NonBlockingSync  # noqa: E402


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    rng = np.random.default_rng(0)
    rows = 48 * world
    xs = rng.random((rows, 200), dtype=np.float32)
    ys = np.eye(10, dtype=np.float32)[rng.integers(0, 10, rows)]
    model = Sequential([Dense(300, XavierUniform(), Tanh()), Dense(120, XavierUniform(), ReLU(0.0)),
                        Dense(10, XavierUniform(), Softmax())])
    ds = lambda: InlineDataset(xs, ys, 200, 10)
    gpu = [f"gpu:{i}" for i in range(world)]
    cpu = [f"cpu:{i}" for i in range(world)]
    cases = []
    for cadence in ("step", "round"):
        for ar in ("twoshot", "oneshot", "nvls", "ring", "nccl"):
            cases.append((f"ar-{ar}-{cadence}", lambda a, c=cadence, m=ar: orchestra.all_reduce(
                a, ds(), GradientDescentWithMomentum(0.1, 0.9), CrossEntropy(), 6, 48, seed=4,
                b200={"sync_every": c, "allreduce": m})))
        # Adam divides by sqrt(v): tf32 tiles against the f32 oracle drift faster, hence the wider bound
        cases.append((f"ar-adam-{cadence}", lambda a, c=cadence: orchestra.all_reduce(
            a, ds(), Adam(0.002), CrossEntropy(), 6, 48, seed=4, b200={"sync_every": c})))
        cases.append((f"ps-colocated-even-{cadence}", lambda a, c=cadence: orchestra.parameter_server(
            a, max(1, world // 2), ds(), GradientDescentWithMomentum(0.1, 0.9), CrossEntropy(), BarrierSync(),
            BlockingStore(), 6, 48, seed=4, b200={"sync_every": c, "colocate": True, "sharding": "even"})))
    # bf16 tiles in step cadence: only owners keep f32 masters, everyone else consumes the bf16 shadow
    for ar in ("twoshot", "auto"):
        cases.append((f"bf16-ar-{ar}-step", lambda a, m=ar: orchestra.all_reduce(
            a, ds(), GradientDescentWithMomentum(0.1, 0.9), CrossEntropy(), 6, 48, seed=4,
            b200={"sync_every": "step", "tile_dtype": "bf16", "allreduce": m})))
    cases.append(("bf16-ps-colocated-even-step", lambda a: orchestra.parameter_server(
        a, max(1, world // 2), ds(), GradientDescentWithMomentum(0.1, 0.9), CrossEntropy(), BarrierSync(),
        BlockingStore(), 6, 48, seed=4, b200={"sync_every": "step", "tile_dtype": "bf16", "colocate": True,
                                               "sharding": "even"})))
    if world >= 2:
        cases.append(("ps-pure-servers-layer-round", lambda a: orchestra.parameter_server(
            a, 1, ds(), GradientDescent(0.2), CrossEntropy(), BarrierSync(), BlockingStore(), 6, 48, seed=4)))
        cases.append(("ps-async-wild-round", lambda a: orchestra.parameter_server(
            a, 1, ds(), GradientDescent(0.05), CrossEntropy(), NonBlockingSync(), WildStore(), 6, 48, seed=4)))
        cases.append(("switch-round", lambda a: orchestra.strategy_switch(
            a, 1, ds(), Adam(0.002), CrossEntropy(), BarrierSync(), BlockingStore(), 8, 48, seed=4,
            b200={"switch_window": 2, "switch_threshold": 10.0})))
    # gradient push: weight-gradient GEMMs add their tiles into the owner's window over NVLink (needs layer widths that
    # are multiples of 4, hence its own model with 12 classes)
    ys12 = np.eye(12, dtype=np.float32)[rng.integers(0, 12, rows)]
    model12 = Sequential([Dense(384, XavierUniform(), Tanh()), Dense(128, XavierUniform(), ReLU(0.0)),
                          Dense(12, XavierUniform(), Softmax())])
    ds12 = lambda: InlineDataset(xs, ys12, 200, 12)
    push_cases = []
    for tile in ("tf32", "bf16"):
        push_cases.append((f"push-ar-{tile}-step", lambda a, t=tile: orchestra.all_reduce(
            a, ds12(), GradientDescentWithMomentum(0.1, 0.9), CrossEntropy(), 6, 48, seed=4,
            b200={"sync_every": "step", "tile_dtype": t, "grad_push": "on"})))
        push_cases.append((f"push-ps-{tile}-step", lambda a, t=tile: orchestra.parameter_server(
            a, max(1, world // 2), ds12(), GradientDescentWithMomentum(0.1, 0.9), CrossEntropy(), BarrierSync(),
            BlockingStore(), 6, 48, seed=4, b200={"sync_every": "step", "tile_dtype": t, "colocate": True,
                                                   "sharding": "even", "grad_push": "on"})))
    # staged reduce-scatter: peers' gradient ranges copied into local staging during backward
    for tile in ("tf32", "bf16"):
        push_cases.append((f"stage-ar-{tile}-step", lambda a, t=tile: orchestra.all_reduce(
            a, ds12(), GradientDescentWithMomentum(0.1, 0.9), CrossEntropy(), 6, 48, seed=4,
            b200={"sync_every": "step", "tile_dtype": t, "grad_stage": "on"})))
        push_cases.append((f"stage-ps-{tile}-step", lambda a, t=tile: orchestra.parameter_server(
            a, max(1, world // 2), ds12(), GradientDescentWithMomentum(0.1, 0.9), CrossEntropy(), BarrierSync(),
            BlockingStore(), 6, 48, seed=4, b200={"sync_every": "step", "tile_dtype": t, "colocate": True,
                                                   "sharding": "even", "grad_stage": "on"})))
    if world >= 2:
        push_cases.append(("stage-ps-pure-server-step", lambda a: orchestra.parameter_server(
            a, 1, ds12(), GradientDescent(0.2), CrossEntropy(), BarrierSync(), BlockingStore(), 6, 48, seed=4,
            b200={"sync_every": "step", "grad_stage": "on"})))
    report = {}
    ok = True
    only = os.environ.get("ONO_PARITY_ONLY", "")
    for name, make, mdl in [(n, m, model) for n, m in cases] + [(n, m, model12) for n, m in push_cases]:
        if only and only not in name:
            continue
        got = orchestrate(mdl, make(gpu)).wait(quiet=True)
        met = got.metrics()
        if rank == 0:
            ref = orchestrate(mdl, make(cpu)).wait(quiet=True)
            lg, lr = np.array(got.loss_history()), np.array(ref.loss_history())
            same_len = lg.shape == lr.shape
            dl = float(np.abs(lg - lr).max() / max(1e-9, np.abs(lr).max())) if same_len else float("inf")
            dw = float(np.abs(got.weights_array() - ref.weights_array()).max())
            # asynchronous pushes land in a different order on GPUs than in the oracle's rank order
            loose = any(k in name for k in ("async", "adam", "switch", "bf16"))
            # closeness to the oracle is the criterion; Adam's first steps move every weight by ~lr whatever the
            # gradient's size, so its loss need not fall within six steps
            if name.startswith("stage") and not met.get("grad_stage"):
                same_len = False
            if name.startswith("push") and not met.get("grad_push"):
                same_len = False          # the case must really have run with pushed gradients
            good = same_len and dl < (0.3 if loose else 0.05) and dw < (0.2 if loose else 2e-2) and (loose or lg[-1] < lg[0])
            report[name] = {"ok": bool(good), "dloss": dl, "dw": dw, "loss": [float(lg[0]), float(lg[-1])] if same_len else [], "nvls": met.get("nvls"), "mode": met.get("sync_mode"),
                            "switched": met.get("switched"), "push": met.get("grad_push"), "stage": met.get("grad_stage")}
            ok = ok and good
        dist.barrier()
    if rank == 0:
        print("MGPU_REPORT " + json.dumps(report))
        print("MGPU_OK" if ok else "MGPU_FAIL")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
