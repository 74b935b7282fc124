"""NCCL + cuBLAS/cuDNN baseline of the three strategies in plain eager PyTorch (no custom kernel).

This is the comparison arm for the hand-written kernels: the same models, batch sizes, optimizers and
synchronisation cadence (one exchange per step) expressed with library calls only.

  all-reduce          autograd backward -> ``ncclAllReduce`` of the flat gradient -> ``torch`` fused optimizer
                      on every rank (average folded into the gradient with one ``mul_``)
  parameter server    backward -> ``dist.reduce`` of every shard to its server rank -> fused optimizer on the
                      shard (server owns the state) -> ``dist.broadcast`` of the fresh shard to every rank
  strategy switch     all-reduce until the relative change of the global gradient norm stays under the threshold
                      for ``window`` steps (norm via one extra reduction + host read), then parameter server

bf16 tiles are expressed the usual way, with ``torch.autocast`` over f32 master weights; tf32 tiles with
``allow_tf32``. Loss is softmax cross-entropy scaled by 1/(B*C) like the reference's normaliser
(machine_learning/src/arch/loss/cross_entropy.rs:35-47) so that both arms take the same optimizer steps.

Timing follows the same rules as the main benchmark: CUDA events on the compute stream after the warm-up
steps, barrier + synchronize on both sides, max over ranks.
"""
from __future__ import annotations

import json
import math
import os
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F


def _build_model(cfg, dev):
    """Flat f32 parameter/gradient buffers with per-layer views (weights [out,in] for cuBLAS, conv OIHW)."""
    shapes = []
    if cfg.get("conv"):
        c, h, w = cfg["conv_input"]
        for (f, k, s, p) in cfg["conv"]:
            shapes.append(("conv", (f, c, k, k), (f,), s, p))
            h = (h + 2 * p - k) // s + 1
            w = (w + 2 * p - k) // s + 1
            c = f
        fan = c * h * w
    else:
        fan = cfg["x"]
    for width, act in cfg["hidden"]:
        shapes.append(("dense", (width, fan), (width,), act, None))
        fan = width
    shapes.append(("dense", (cfg["classes"], fan), (cfg["classes"],), None, None))
    n = sum(math.prod(s[1]) + math.prod(s[2]) for s in shapes)
    npad = (n + 1023) // 1024 * 1024
    flat = torch.zeros(npad, device=dev)
    grad = torch.zeros(npad, device=dev)
    layers, off = [], 0
    for kind, ws, bs, a, b in shapes:
        nw, nb = math.prod(ws), math.prod(bs)
        W = flat[off:off + nw].view(ws).requires_grad_(True)
        W.grad = grad[off:off + nw].view(ws)
        off += nw
        bb = flat[off:off + nb].view(bs).requires_grad_(True)
        bb.grad = grad[off:off + nb].view(bs)
        off += nb
        fan_in = math.prod(ws[1:])
        with torch.no_grad():
            W.normal_(0, math.sqrt(2.0 / fan_in))
            bb.normal_(0, math.sqrt(2.0 / fan_in))
        layers.append((kind, W, bb, a, b))
    return flat, grad, layers, n


def _forward(cfg, layers, x):
    act = {"relu": F.relu, "gelu": lambda t: F.gelu(t, approximate="tanh"), None: lambda t: t}
    a = x
    if cfg.get("conv"):
        a = a.view(-1, *cfg["conv_input"])
    for kind, W, b, p1, p2 in layers:
        if kind == "conv":
            a = F.relu(F.conv2d(a, W, b, stride=p1, padding=p2))
        else:
            if a.dim() > 2:
                a = a.flatten(1)
            a = act[p1](F.linear(a, W, b))
    return a


def _optimizer(cfg, tensors):
    o = cfg["opt"]
    if o[0] == "adam":
        return torch.optim.Adam(tensors, lr=o[1], fused=True)
    return torch.optim.SGD(tensors, lr=o[1], momentum=o[2] if o[0] == "momentum" else 0.0, fused=True)


def run(cfg, strategy, n_servers, steps, warmup, data_mode, switch=None):
    """One timed run; returns (device ms for ``steps`` steps, wall s, h2d bytes/step, d2h bytes/step, info)."""
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.allow_tf32 = True
    torch.manual_seed(0)
    flat, grad, layers, n = _build_model(cfg, dev)
    if world > 1:
        dist.broadcast(flat, 0)
    B, C = cfg["batch"], cfg["classes"]
    nb = 8
    gen = torch.Generator(device="cpu").manual_seed(1 + rank)
    xs = torch.randn(nb * B, cfg["x"], generator=gen) if cfg["data"] == "normal" else torch.rand(nb * B, cfg["x"], generator=gen)
    ys = torch.randint(0, C, (nb * B,), generator=gen)
    if data_mode == "device":
        xs, ys = xs.to(dev), ys.to(dev)
    else:
        xs, ys = xs.pin_memory(), ys.pin_memory()
    servers = list(range(min(n_servers, world)))
    npad = flat.numel()
    per = (npad // len(servers) + 255) // 256 * 256
    shards = [(s * per, min(npad, (s + 1) * per)) for s in range(len(servers))]
    full_opt = _optimizer(cfg, [flat.detach().requires_grad_(False)])
    full_opt.param_groups[0]["params"][0].grad = grad
    shard_opt = None
    mode = "ps" if strategy == "ps" else "ar"
    norms, calm, switched_at = [], 0, None
    autocast = torch.autocast("cuda", dtype=torch.bfloat16, enabled=cfg["tile"] == "bf16")
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    loss_host = torch.zeros(1).pin_memory()
    t0 = 0.0

    def make_shard_opt():
        mine = [(a, b) for s, (a, b) in zip(servers, shards) if s == rank]
        if not mine:
            return None
        a, b = mine[0]
        p = flat[a:b].detach()
        p.grad = grad[a:b]
        return _optimizer(cfg, [p])

    if mode == "ps":
        shard_opt = make_shard_opt()
    for step in range(warmup + steps):
        if step == warmup:
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            ev0.record()
        i = step % nb
        x, y = xs[i * B:(i + 1) * B], ys[i * B:(i + 1) * B]
        if data_mode != "device":
            x, y = x.to(dev, non_blocking=True), y.to(dev, non_blocking=True)
        grad.zero_()
        with autocast:
            z = _forward(cfg, layers, x)
        loss = F.cross_entropy(z.float(), y, reduction="sum") / (B * C)
        loss.backward()
        if mode == "ar":
            if world > 1:
                dist.all_reduce(grad)
                grad.mul_(1.0 / world)
            if strategy == "ss" and switch and switched_at is None:
                norms.append(float(grad.norm().item()))
                if len(norms) > 1:
                    rel = abs(norms[-1] - norms[-2]) / max(norms[-2], 1e-30)
                    calm = calm + 1 if rel < switch["threshold"] else 0
                if calm >= switch["window"]:
                    mode, switched_at = "ps", step
                    shard_opt = make_shard_opt()
            full_opt.step()
        else:
            if world > 1:
                for s, (a, b) in zip(servers, shards):
                    dist.reduce(grad[a:b], dst=s)
            if shard_opt is not None:
                a, b = [ab for s, ab in zip(servers, shards) if s == rank][0]
                grad[a:b].mul_(1.0 / world)
                shard_opt.step()
            if world > 1:
                for s, (a, b) in zip(servers, shards):
                    dist.broadcast(flat[a:b], src=s)
        if data_mode != "device":
            loss_host.copy_(loss.detach().reshape(1), non_blocking=True)
            torch.cuda.current_stream().synchronize()
    ev1.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    if world > 1:
        dist.barrier()
    ms = torch.tensor([ev0.elapsed_time(ev1), wall], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    h2d = B * cfg["x"] * 4 + B * 8 if data_mode != "device" else 0
    return float(ms[0]), float(ms[1]), h2d, 4 if data_mode != "device" else 0, {"params": n, "switched_at": switched_at}


def main(cfg, name, strategy, n_servers, steps, warmup, switch, clock_sampler):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    sampler = clock_sampler() if rank == 0 else None
    if sampler:
        sampler.start()
    ms, _, _, _, info = run(cfg, strategy, n_servers, steps, warmup, "device", switch)
    clocks = sampler.stop() if sampler else None
    _, wall, h2d, d2h, _ = run(cfg, strategy, n_servers, steps, warmup, "host", switch)
    if rank == 0:
        gb = cfg["batch"] * world
        print(json.dumps({
            "impl": "nccl+cublas", "metric": "samples/sec (device-timed, max over ranks)", "value": gb * steps / (ms / 1e3),
            "unit": "samples/s", "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms / steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16" if cfg["tile"] == "bf16" else "tf32", "data": "synthetic",
            "config": {"model": cfg["model"], "config_name": name, "global_batch": gb, "seq_len": None,
                       "parallelism": f"{strategy}(servers={min(n_servers, world)})+dp{world}", "optimizer": cfg["opt"][0],
                       "switched_at": info["switched_at"]},
            "clocks": clocks,
            "e2e": {"value": gb * steps / wall, "unit": "samples/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": 0}))
