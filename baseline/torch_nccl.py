"""NCCL + cuBLAS/cuDNN baseline of the three strategies in plain PyTorch (no custom kernel).

This is the comparison arm for the hand-written kernels: the same models, batch sizes, optimizers and
synchronisation cadence (one exchange per step) expressed with library calls only, written the way a
careful PyTorch user would write them:

  mixed precision     bf16 configs keep f32 master weights plus a flat bf16 shadow that the layers read; the
                      optimizer refreshes the shadow (no per-step re-cast of the weights by ``autocast``); gradients
                      are bf16. tf32 configs run f32 storage with ``allow_tf32``.
  all-reduce          backward -> one ``ncclAllReduce`` of the flat gradient (bf16 on the wire, like the kernels'
                      default wire; f32 with ``wire="f32"``) -> fused update on every rank
  parameter server    backward -> ONE ``ncclReduceScatter`` over all ranks -> the reduced pieces of a server's shard
                      are collected by that server (grouped point-to-point) -> the server updates its shard (it owns
                      the optimizer state) -> fresh pieces go back and ONE ``ncclAllGather`` publishes the parameters
  strategy switch     all-reduce until the relative change of the global gradient norm stays under the threshold
                      for ``window`` steps (norm via one extra reduction + host read), then parameter server
  CUDA graph          the whole step (forward, backward, collectives, optimizer) is captured once and replayed,
                      unless capture fails or the strategy still has to watch the gradient norm on the host

Loss is softmax cross-entropy scaled by 1/(B*C) like the reference's normaliser
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
    """Flat f32 master, flat compute copy (bf16 shadow, or the master itself) and flat gradient of the compute dtype,
    with per-layer views (weights [out,in] for cuBLAS, conv OIHW)."""
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
    npad = (n + 8191) // 8192 * 8192
    cd = torch.bfloat16 if cfg["tile"] == "bf16" else torch.float32
    master = torch.zeros(npad, device=dev)
    comp = torch.zeros(npad, device=dev, dtype=cd) if cd != torch.float32 else master
    grad = torch.zeros(npad, device=dev, dtype=cd)
    layers, off = [], 0
    for kind, ws, bs, a, b in shapes:
        nw, nb = math.prod(ws), math.prod(bs)
        fan_in = math.prod(ws[1:])
        with torch.no_grad():
            master[off:off + nw + nb].normal_(0, math.sqrt(2.0 / fan_in))
        W = comp[off:off + nw].view(ws).requires_grad_(True)
        W.grad = grad[off:off + nw].view(ws)
        off += nw
        bb = comp[off:off + nb].view(bs).requires_grad_(True)
        bb.grad = grad[off:off + nb].view(bs)
        off += nb
        layers.append((kind, W, bb, a, b))
    if comp is not master:
        comp.copy_(master)
    return master, comp, grad, layers, n


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


class _Update:
    """SGD / momentum / Adam on an f32 master slice from a gradient slice of any float dtype, refreshing the compute
    copy; in-place torch ops only (mixed dtypes promote to f32), usable under CUDA-graph capture."""

    def __init__(self, cfg, master, comp, grad, lo, hi, scale):
        self.kind, self.lr = cfg["opt"][0], cfg["opt"][1]
        self.mu = cfg["opt"][2] if self.kind == "momentum" else 0.0
        self.p, self.c, self.g, self.scale = master[lo:hi], (comp[lo:hi] if comp is not master else None), grad[lo:hi], scale
        self.m = torch.zeros_like(self.p) if self.kind != "sgd" else None
        self.v = torch.zeros_like(self.p) if self.kind == "adam" else None
        self.pows = torch.ones(2, device=master.device)
        self.betas = torch.tensor([0.9, 0.999], device=master.device)
        self.tmp = torch.empty_like(self.p) if self.kind == "adam" else None

    def step(self):
        p, g = self.p, self.g
        if self.kind == "sgd":
            p.add_(g, alpha=-self.lr * self.scale)
        elif self.kind == "momentum":
            self.m.mul_(self.mu).add_(g, alpha=self.scale)
            p.add_(self.m, alpha=-self.lr)
        else:
            b1, b2, eps = 0.9, 0.999, 1e-8
            self.pows.mul_(self.betas)
            self.m.mul_(b1).add_(g, alpha=(1 - b1) * self.scale)
            self.tmp.copy_(g).mul_(self.scale)
            self.v.mul_(b2).addcmul_(self.tmp, self.tmp, value=1 - b2)
            torch.sqrt(self.v, out=self.tmp)
            self.tmp.add_(eps)
            step = self.lr * torch.sqrt(1 - self.pows[1]) / (1 - self.pows[0])
            self.tmp.reciprocal_().mul_(self.m).mul_(step)
            p.sub_(self.tmp)
        if self.c is not None:
            self.c.copy_(p)


def run(cfg, strategy, n_servers, steps, warmup, data_mode, switch=None, wire="bf16", graph=True):
    """One timed run; returns (device ms for ``steps`` steps, wall s, h2d bytes/step, d2h bytes/step, info)."""
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.allow_tf32 = True
    torch.manual_seed(0)
    master, comp, grad, layers, n = _build_model(cfg, dev)
    if world > 1:
        dist.broadcast(master, 0)
        if comp is not master:
            comp.copy_(master)
    B, C = cfg["batch"], cfg["classes"]
    cd = comp.dtype
    nb = 8
    gen = torch.Generator(device="cpu").manual_seed(1 + rank)
    xs = torch.randn(nb * B, cfg["x"], generator=gen) if cfg["data"] == "normal" else torch.rand(nb * B, cfg["x"], generator=gen)
    ys = torch.randint(0, C, (nb * B,), generator=gen)
    if data_mode == "device":
        xs, ys = xs.to(dev), ys.to(dev)
    else:
        xs, ys = xs.pin_memory(), ys.pin_memory()
    npad = master.numel()
    ns = max(1, min(n_servers, world))
    piece = npad // world                       # what one rank holds after the reduce-scatter
    group_sz = world // ns if world % ns == 0 else 0
    # 16-bit wire for f32 gradients: cast, reduce, cast back (what DDP's bf16 compression hook does)
    wire16 = torch.empty(npad, device=dev, dtype=torch.bfloat16) if (wire == "bf16" and grad.dtype == torch.float32 and world > 1) else None
    wbuf = wire16 if wire16 is not None else grad
    rs_out = torch.empty(piece, device=dev, dtype=wbuf.dtype)
    ag_in = torch.empty(piece, device=dev, dtype=cd)
    x_dev = torch.zeros(B, cfg["x"], device=dev)
    y_dev = torch.zeros(B, dtype=torch.long, device=dev)
    loss_dev = torch.zeros(1, device=dev)
    full_upd = _Update(cfg, master, comp, grad, 0, npad, 1.0 / world)
    # parameter server: server s owns pieces [s*group_sz, (s+1)*group_sz) of the reduce-scatter layout
    my_server = rank // group_sz if group_sz else None
    is_server = group_sz and rank % group_sz == 0
    shard_g = torch.empty(piece * group_sz, device=dev, dtype=wbuf.dtype) if is_server else None
    shard_upd = None
    if is_server:
        lo = rank * piece
        shard_upd = _Update(cfg, master, comp, _Shift(shard_g, lo), lo, lo + piece * group_sz, 1.0 / world)

    def exchange_ps():
        """reduce-scatter -> pieces to their server -> shard update -> fresh pieces back -> all-gather."""
        if wire16 is not None:
            wire16.copy_(grad)
        dist.reduce_scatter_tensor(rs_out, wbuf)
        if group_sz > 1:
            ops = []
            if is_server:
                shard_g[:piece].copy_(rs_out)
                for j in range(1, group_sz):
                    ops.append(dist.P2POp(dist.irecv, shard_g[j * piece:(j + 1) * piece], rank + j))
            else:
                ops.append(dist.P2POp(dist.isend, rs_out, my_server * group_sz))
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        elif is_server:
            shard_g.copy_(rs_out)
        if is_server:
            shard_upd.step()
        src = comp
        if group_sz > 1:
            ops = []
            if is_server:
                for j in range(1, group_sz):
                    ops.append(dist.P2POp(dist.isend, src[(rank + j) * piece:(rank + j + 1) * piece], rank + j))
                ag_in.copy_(src[rank * piece:(rank + 1) * piece])
            else:
                ops.append(dist.P2POp(dist.irecv, ag_in, my_server * group_sz))
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        else:
            ag_in.copy_(src[rank * piece:(rank + 1) * piece])
        dist.all_gather_into_tensor(comp, ag_in)

    def exchange_ar():
        if world > 1:
            if wire16 is not None:
                wire16.copy_(grad)
                dist.all_reduce(wire16)
                grad.copy_(wire16)
            else:
                dist.all_reduce(grad)

    state = {"mode": "ps" if (strategy == "ps" and world > 1 and group_sz) else "ar"}

    def body():
        grad.zero_()
        z = _forward(cfg, layers, x_dev.to(cd))
        loss = F.cross_entropy(z.float(), y_dev, reduction="sum") / (B * C)
        loss.backward()
        loss_dev.copy_(loss.detach().reshape(1))
        if state["mode"] == "ar":
            exchange_ar()
            full_upd.step()
        else:
            exchange_ps()

    norms, calm, switched_at = [], 0, None
    watching = strategy == "ss" and switch is not None and world > 1 and group_sz
    graphs: dict = {}
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    loss_host = torch.zeros(1).pin_memory()
    t0 = 0.0
    used_graph = False
    for step in range(warmup + steps):
        if step == warmup:
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            ev0.record()
        i = step % nb
        x_dev.copy_(xs[i * B:(i + 1) * B], non_blocking=True)
        y_dev.copy_(ys[i * B:(i + 1) * B], non_blocking=True)
        key = state["mode"]
        can_graph = graph and not (watching and switched_at is None)
        if can_graph and key not in graphs and step >= 2:
            try:
                g = torch.cuda.CUDAGraph()
                torch.cuda.synchronize()
                with torch.cuda.graph(g):
                    body()
                graphs[key] = g
            except Exception:
                graphs[key] = None
                torch.cuda.synchronize()
        if can_graph and graphs.get(key) is not None:
            graphs[key].replay()
            used_graph = True
        else:
            body()
        if watching and switched_at is None:
            norms.append(float(grad.float().norm().item()) / world)
            if len(norms) > 1:
                rel = abs(norms[-1] - norms[-2]) / max(norms[-2], 1e-30)
                calm = calm + 1 if rel < switch["threshold"] else 0
            if calm >= switch["window"]:
                state["mode"], switched_at = "ps", step
        if data_mode != "device":
            loss_host.copy_(loss_dev, non_blocking=True)
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
    return float(ms[0]), float(ms[1]), h2d, 4 if data_mode != "device" else 0, {
        "params": n, "switched_at": switched_at, "cuda_graph": used_graph, "final_loss": float(loss_dev.item()),
        "wire": ("bf16" if wbuf.dtype == torch.bfloat16 else "f32") if world > 1 else "none"}


def _Shift(buf, lo):
    """A view trick: ``_Update`` slices its gradient with the same [lo, hi) as the master; the server's collected
    gradient shard starts at 0, so hand it an object whose slice [lo:hi] is the whole buffer."""
    class _S:
        def __getitem__(self, sl):
            return buf[sl.start - lo:sl.stop - lo]
    return _S()


def measure(cfg, name, strategy, n_servers, steps, warmup, switch, clock_sampler=None, wire="bf16") -> dict | None:
    """Device-timed and end-to-end runs of the arm; rank 0 gets the result line as a dict."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    sampler = clock_sampler() if (rank == 0 and clock_sampler is not None) else None
    if sampler:
        sampler.start()
    ms, _, _, _, info = run(cfg, strategy, n_servers, steps, warmup, "device", switch, wire)
    clocks = sampler.stop() if sampler else None
    _, wall, h2d, d2h, _ = run(cfg, strategy, n_servers, steps, warmup, "host", switch, wire)
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    gb = cfg["batch"] * world
    return {
        "impl": "nccl+cublas", "metric": "samples/sec (device-timed, max over ranks)", "value": gb * steps / (ms / 1e3),
        "unit": "samples/s", "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms / steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if cfg["tile"] == "bf16" else "tf32", "data": "synthetic",
        "config": {"model": cfg["model"], "config_name": name, "global_batch": gb, "seq_len": None,
                   "parallelism": f"{strategy}(servers={min(n_servers, world)})+dp{world}", "optimizer": cfg["opt"][0],
                   "switched_at": info["switched_at"], "cuda_graph": info["cuda_graph"], "wire": info["wire"]},
        "clocks": clocks,
        "e2e": {"value": gb * steps / wall, "unit": "samples/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": wall * 1e3 / steps},
        "gpu_launches": 0}


def main(cfg, name, strategy, n_servers, steps, warmup, switch, clock_sampler, wire="bf16"):
    line = measure(cfg, name, strategy, n_servers, steps, warmup, switch, clock_sampler, wire)
    if line is not None:
        print(json.dumps(line))
