#!/usr/bin/env python
"""Kernel-level benchmarks (CUDA-event timed, warm-up excluded, max over ranks).

    python bench/kernels.py gemm  [--m 4096 --n 4096 --k 4096 --dtype bf16 --iters 20]
    python bench/kernels.py wgrad [--m 8192 --n 8192 --k 512 --dtype bf16 --opt momentum]   (weight-gradient output forms)
    python bench/kernels.py sync  [--elems 67108864 --opt adam --iters 20]            (1 GPU: fused optimizer pass)
    torchrun --nproc-per-node N bench/kernels.py sweep [--max-bytes 1073741824]        (all-reduce sweep)

``sweep`` is the gradient all-reduce study: f32 buffers from 1 KB to 1 GB (powers of 4) ~N(0,1e-3), each
reduced over the ranks with the average and an SGD step into an equal-sized parameter buffer fused in,
for the ring / one-shot / two-shot / NVLS kernels against ``ncclAllReduce`` + one elementwise kernel.
It reports bus bandwidth ``S/t * 2(n-1)/n`` and the fraction of the NVLink roofline (bytes that must
cross the links per GPU and direction divided by the measured 770 GB/s peer-copy bandwidth).
Inputs larger than L2 are used where the size allows; below that an L2 flush (a 256 MB write) runs
between timed iterations.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

NVLINK_GBS = 770.0


def _time(fn, iters, flush=None, pre=None):
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    tot = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.fill_(1.0)
        if pre is not None:
            pre()
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        tot += s.elapsed_time(e)
    return tot / iters


def cmd_gemm(a):
    from oxidized_neural_orchestra_b200.ops.gemm import gemm

    dt = torch.bfloat16 if a.dtype == "bf16" else torch.float32
    A = torch.randn(a.m, a.k, device="cuda", dtype=dt)
    B = torch.randn(a.n, a.k, device="cuda", dtype=dt)
    out = torch.zeros(a.m, a.n, device="cuda")
    for _ in range(3):
        gemm(A, B, out=out, bn=a.bn, pair=a.pair)
    ms = _time(lambda: gemm(A, B, out=out, bn=a.bn, pair=a.pair), a.iters)
    torch.backends.cuda.matmul.allow_tf32 = True
    Bt = B.t()
    for _ in range(3):
        torch.matmul(A, Bt)
    ref = _time(lambda: torch.matmul(A, Bt), a.iters)
    fl = 2.0 * a.m * a.n * a.k
    print(json.dumps({"kernel": "gemm_tcgen05", "m": a.m, "n": a.n, "k": a.k, "dtype": a.dtype, "pair": a.pair, "ms": ms,
                      "tflops": fl / ms / 1e9, "cublas_ms": ref, "cublas_tflops": fl / ref / 1e9}))


def cmd_wgrad(a):
    """The weight-gradient GEMM dW[in,out] = X^T d (operands as the engines store them: [batch, in] and [batch, out]) in its
    three output forms: f32 store, 16-bit wire store, optimizer applied in the epilogue (master + state + bf16 shadow updated
    in place), the last one against the f32 store followed by the separate fused optimizer pass."""
    from oxidized_neural_orchestra_b200.ops import elementwise as ew
    from oxidized_neural_orchestra_b200.ops.gemm import gemm

    dt = torch.bfloat16 if a.dtype == "bf16" else torch.float32
    M, N, K = a.m, a.n, a.k
    x = (torch.randn(K, M, device="cuda") / 8).to(dt)
    d = (torch.randn(K, N, device="cuda") / 8).to(dt)
    g32 = torch.zeros(M, N, device="cuda")
    g16 = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    p, m, v = torch.randn(M, N, device="cuda"), torch.zeros(M, N, device="cuda"), torch.zeros(M, N, device="cuda")
    sh = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    pows = torch.full((2,), 0.5, device="cuda")
    ap = dict(p=p, m=m, v=v, p_bf16=sh if a.dtype == "bf16" else None, kind=a.opt, lr=1e-3, mu=0.9, adam_pows=pows)
    kw = dict(a_mn_major=True, b_mn_major=True, pair=a.pair)
    forms = {
        "store_f32": lambda: gemm(x, d, out=g32, **kw),
        "store_bf16": lambda: gemm(x, d, out_bf16=g16, **kw),
        "apply": lambda: gemm(x, d, apply=ap, **kw),
        "store_f32+optimizer_pass": lambda: (gemm(x, d, out=g32, **kw),
                                             ew.optim_step(p.view(-1), g32.view(-1), kind=a.opt, lr=1e-3, mu=0.9, m=m.view(-1),
                                                           v=v.view(-1), adam_pows=pows, p_bf16=sh.view(-1) if a.dtype == "bf16" else None)),
    }
    state = {"sgd": 8, "momentum": 16, "adam": 24}[a.opt] + (2 if a.dtype == "bf16" else 0)
    fl = 2.0 * M * N * K
    flush = torch.empty(64 << 20, device="cuda")
    for name, fn in forms.items():
        if a.form and name != a.form:
            continue
        for _ in range(3):
            fn()
        ms = _time(fn, a.iters, flush=flush if M * N * 4 < (256 << 20) else None)
        rec = {"kernel": "gemm_tcgen05 wgrad", "form": name, "m": M, "n": N, "k": K, "dtype": a.dtype, "opt": a.opt, "ms": ms,
               "tflops": fl / ms / 1e9}
        if name == "apply":
            rec["state_GBs"] = state * M * N / ms / 1e6
        print(json.dumps(rec))


def cmd_sync(a):
    from oxidized_neural_orchestra_b200.ops import _lib
    from oxidized_neural_orchestra_b200.ops.elementwise import adam_tick
    from oxidized_neural_orchestra_b200.parallel import sync as S

    n = a.elems
    z = lambda dt=torch.float32: torch.zeros(n, device="cuda", dtype=dt)
    p, g, m, v, pb = z(), z(), z(), z(), z(torch.bfloat16)
    g.normal_(0, 1e-3)
    nblocks = min(2 * _lib.load().ono_num_sms(), max(1, n // 4 // 1024))
    flags = torch.zeros(8192, device="cuda", dtype=torch.int32)
    epoch = torch.zeros(1024, device="cuda", dtype=torch.int32)
    pows = torch.full((2,), 0.5, device="cuda")
    s = _lib.OnoSync()
    S.fill_sync(s, nranks=1, rank=0, n=n, nblocks=nblocks, algo=0, g_ptrs=[g.data_ptr()], p_f32_ptrs=[p.data_ptr()],
                p_bf16_ptrs=[pb.data_ptr() if a.bf16_shadow else None], flag_ptrs=[flags.data_ptr()], worker_mask=1,
                member_mask=1, n_workers=1, opt=S.OptimizerCfg(kind=a.opt, lr=0.01, mu=0.9))
    S.fill_local(s.loc[0], p_master=p.data_ptr(), m=m.data_ptr(), v=v.data_ptr(), state_off=0, adam_pows=pows.data_ptr(),
                 epoch=epoch.data_ptr(), ranges=[(0, n)])
    for _ in range(3):
        S.launch_sync(s)
    ms = _time(lambda: S.launch_sync(s), a.iters)
    per = {"sgd": 12, "momentum": 20, "adam": 28}[a.opt] + (2 if a.bf16_shadow else 0)
    print(json.dumps({"kernel": "sync_kernel(1 rank)", "elems": n, "opt": a.opt, "ms": ms, "GBs": per * n / ms / 1e6,
                      "bytes_per_elem": per}))


def cmd_sync_emulated(a):
    """All ranks of the two-shot reduce-scatter + optimizer + all-gather kernel as ONE cooperative launch on one GPU
    (grid.y = rank, every rank with its own buffers): the cross-rank flag protocol and the peer loads and stores run
    for real, only the wires are missing. Used to profile the multi-rank kernel where ncu may not wrap a multi-process run."""
    from oxidized_neural_orchestra_b200.ops import _lib
    from oxidized_neural_orchestra_b200.parallel import sync as S

    R, n = a.emulate_ranks, a.elems
    torch.manual_seed(0)
    z = lambda dt=torch.float32: torch.zeros(n, device="cuda", dtype=dt)
    wire = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[a.wire]
    g, p, m, v = [z(wire) for _ in range(R)], [z() for _ in range(R)], [z() for _ in range(R)], [z() for _ in range(R)]
    pb = [z(torch.bfloat16) for _ in range(R)] if a.bf16_shadow else [None] * R
    for t in g:
        t.normal_(0, 1e-3)
    nblocks = max(1, min(_lib.load().ono_num_sms() // R, n // 4 // 1024))
    flags = [torch.zeros(nblocks * 8, device="cuda", dtype=torch.int32) for _ in range(R)]
    epoch = [torch.zeros(nblocks, device="cuda", dtype=torch.int32) for _ in range(R)]
    status = torch.zeros(1, device="cuda", dtype=torch.int32)
    pows = torch.full((2,), 0.5, device="cuda")
    s = _lib.OnoSync()
    S.fill_sync(s, nranks=R, rank=0, n=n, nblocks=nblocks, algo=0, g_ptrs=[t.data_ptr() for t in g],
                p_f32_ptrs=[None if a.f32_master_only else t.data_ptr() for t in p],
                p_bf16_ptrs=[None if t is None else t.data_ptr() for t in pb],
                flag_ptrs=[t.data_ptr() for t in flags],
                worker_mask=(1 << R) - 1, member_mask=(1 << R) - 1, n_workers=R, opt=S.OptimizerCfg(kind=a.opt, lr=0.01, mu=0.9))
    s.g_dtype = {"f32": 0, "bf16": 1, "f16": 2}[a.wire]
    ranges = S.even_ranges(n, list(range(R)), R, align=a.range_align)
    for r in range(R):
        S.fill_local(s.loc[r], p_master=p[r].data_ptr(), m=m[r].data_ptr(), v=v[r].data_ptr(), state_off=0,
                     adam_pows=pows.data_ptr(), epoch=epoch[r].data_ptr(), ranges=ranges[r], status=status.data_ptr())
    for _ in range(3):
        S.launch_sync(s, emulated=True)
    ms = _time(lambda: S.launch_sync(s, emulated=True), a.iters)
    assert status.item() == 0
    # owner state + R gradient reads + R parameter writes (f32, and bf16 with the shadow)
    per = ({"sgd": 8, "momentum": 16, "adam": 24}[a.opt] + g[0].element_size() * R + (0 if a.f32_master_only else 4 * R)
           + (2 * R if a.bf16_shadow else 0))
    rec = {"kernel": f"sync_kernel_emulated({R} ranks, one GPU)", "elems": n, "opt": a.opt, "wire": a.wire, "ms": ms,
           "GBs_local_hbm": per * n / ms / 1e6, "blocks_per_rank": nblocks}
    if a.checksum:      # bits of every rank's parameters and optimizer state: equal between runs (fixed summation order)
        import hashlib

        h = hashlib.sha256()
        for t in p + m + v:
            h.update(t.cpu().numpy().tobytes())
        rec["checksum"] = h.hexdigest()
    print(json.dumps(rec))


def cmd_sweep(a):
    from oxidized_neural_orchestra_b200.ops import _lib
    from oxidized_neural_orchestra_b200.parallel import sync as S
    from oxidized_neural_orchestra_b200.parallel.symmetric import SymmetricWindow, WindowLayout

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", local)
    lib = _lib.load()
    maxn = a.max_bytes // 4
    lay = WindowLayout()
    lay.add("g", maxn, torch.float32)
    lay.add("p", maxn, torch.float32)
    lay.add("acc", maxn, torch.float32)
    win = SymmetricWindow(lay.size, dev)
    G, P, ACC = (lay.tensor(win, k) for k in ("g", "p", "acc"))
    epoch = torch.zeros(1024, device=dev, dtype=torch.int32)
    repoch = torch.zeros(1024, device=dev, dtype=torch.int32)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    flush = torch.empty(64 << 20, device=dev)
    sms = lib.ono_num_sms()
    rows = []
    size = max(1024, a.min_bytes)
    while size <= a.max_bytes:
        n = size // 4
        G[:n].normal_(0, 1e-3)
        nblocks = int(min(2 * sms, max(1, -(-(n // 4) // 1024))))
        opt = S.OptimizerCfg(kind="sgd", lr=0.01)
        variants = {}

        def fused(ranges, algo, dest_all):
            s = _lib.OnoSync()
            pf = win.peer_ptrs(lay.offset("p")) if dest_all else [p if r == rank else None for r, p in enumerate(win.peer_ptrs(lay.offset("p")))]
            S.fill_sync(s, nranks=world, rank=rank, n=n, nblocks=nblocks, algo=algo, g_ptrs=win.peer_ptrs(lay.offset("g")),
                        p_f32_ptrs=pf, p_bf16_ptrs=[None] * world, flag_ptrs=win.flag_ptrs, worker_mask=(1 << world) - 1,
                        member_mask=(1 << world) - 1, n_workers=world, opt=opt, timeout_ns=10_000_000_000,
                        g_mc=win.mc(lay.offset("g")) or None, p_mc_f32=win.mc(lay.offset("p")) or None)
            S.fill_local(s.loc[rank], p_master=P.data_ptr(), m=None, v=None, state_off=0, adam_pows=None,
                         epoch=epoch.data_ptr(), ranges=ranges[rank], status=status.data_ptr())
            return lambda: S.launch_sync(s)

        n4 = (n + 3) // 4 * 4
        variants["oneshot"] = fused([[(0, n4)] for _ in range(world)], 0, False)
        if n >= 4 * world:
            variants["twoshot"] = fused(S.even_ranges(n4, list(range(world)), world), 0, True)
            if win.mc_ptr:
                variants["nvls"] = fused(S.even_ranges(n4, list(range(world)), world), 1, True)
            r = _lib.OnoRing()
            r.nranks, r.rank, r.nblocks, r.n = world, rank, int(min(sms, max(1, n // 4 // world // 512))), n
            r.g = G.data_ptr()
            for q in range(world):
                r.acc[q] = win.peer_ptrs(lay.offset("acc"))[q]
                r.flags[q] = win.flag_ptrs[q] + 4096 * 4
            r.epoch, r.p, r.kind, r.lr = repoch.data_ptr(), P.data_ptr(), 0, 0.01
            r.status, r.timeout_ns = status.data_ptr(), 10_000_000_000
            variants["ring"] = lambda: _lib.check(lib.ono_ring_allreduce(C.byref(r), _lib.stream_ptr()), "ring")

        def nccl():
            dist.all_reduce(G[:n])
            P[:n].add_(G[:n], alpha=-0.01 / world)
        variants["nccl+elementwise"] = nccl
        for name, fn in variants.items():
            if name == "oneshot" and size > (8 << 20):
                continue
            iters = 20 if size <= (64 << 20) else 5
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            dist.barrier()
            ms = _time(fn, iters, flush=flush if size < (128 << 20) else None, pre=lambda: G[:n].normal_(0, 1e-3) if name.startswith("nccl") else None)
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
            bus = size / ms / 1e6 * 2 * (world - 1) / world
            link_bytes = size * 2 * (world - 1) / world if name not in ("oneshot",) else size * (world - 1)
            rows.append({"bytes": size, "variant": name, "ms": ms, "bus_GBs": bus,
                         "roofline_frac": (link_bytes / (NVLINK_GBS * 1e6)) / ms if world > 1 else None})
        if int(status.item()):
            raise RuntimeError(f"kernel wait timed out at size {size}")
        size *= 4
    if rank == 0:
        for r_ in rows:
            print(json.dumps(r_))
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=4096); g.add_argument("--n", type=int, default=4096)
    g.add_argument("--k", type=int, default=4096); g.add_argument("--dtype", default="bf16")
    g.add_argument("--bn", type=int, default=0); g.add_argument("--pair", type=int, default=0, choices=(-1, 0, 1), help="CTA pairs: 1 on, -1 off, 0 the library default"); g.add_argument("--iters", type=int, default=20)
    wg = sub.add_parser("wgrad")
    wg.add_argument("--m", type=int, default=8192); wg.add_argument("--n", type=int, default=8192)
    wg.add_argument("--k", type=int, default=512); wg.add_argument("--dtype", default="bf16")
    wg.add_argument("--opt", default="momentum"); wg.add_argument("--pair", type=int, default=0, choices=(-1, 0, 1))
    wg.add_argument("--iters", type=int, default=10)
    wg.add_argument("--form", default="", help="run one output form only: store_f32 | store_bf16 | apply | store_f32+optimizer_pass")
    s = sub.add_parser("sync")
    s.add_argument("--elems", type=int, default=64 << 20); s.add_argument("--opt", default="adam")
    s.add_argument("--bf16-shadow", action="store_true"); s.add_argument("--iters", type=int, default=20)
    s.add_argument("--emulate-ranks", type=int, default=0, help="run R ranks as one cooperative launch on this GPU")
    s.add_argument("--wire", default="f32", choices=("f32", "bf16", "f16"), help="with --emulate-ranks: format of the gradient windows")
    s.add_argument("--f32-master-only", action="store_true", help="with --emulate-ranks: f32 parameters stay with their owner, only "
                   "the bf16 shadow goes to every rank (bf16-tile engines; lets 16-bit windows take the 16-byte path)")
    s.add_argument("--range-align", type=int, default=8, help="with --emulate-ranks: owned ranges are cut at multiples of this many "
                   "elements (8: the kernel's 16-byte path for 16-bit windows; 4: its 8-byte path)")
    s.add_argument("--checksum", action="store_true", help="with --emulate-ranks: print a hash of the resulting state")
    w = sub.add_parser("sweep")
    w.add_argument("--max-bytes", type=int, default=1 << 30)
    w.add_argument("--min-bytes", type=int, default=1024)
    a = ap.parse_args()
    if a.cmd == "sync" and a.emulate_ranks > 1:
        return cmd_sync_emulated(a)
    {"gemm": cmd_gemm, "wgrad": cmd_wgrad, "sync": cmd_sync, "sweep": cmd_sweep}[a.cmd](a)


if __name__ == "__main__":
    main()
