"""Builders for the fused gradient-synchronisation kernels (``csrc/kernels/collectives.cu``).

The *ownership table* is what distinguishes the reference's three strategies on this runtime:

* all-reduce (worker/src/middlewares/worker_ring.rs:82-204): every rank owns ``1/N`` of the flat
  vector (two-shot) or, for small vectors, all of it (one-shot);
* parameter server (parameter_server/src/storage/blocking/store.rs:84-108): only server ranks own
  ranges, either whole layers (the reference's LPT assignment,
  orchestrator/src/configs/adapter.rs:605-687,1189-1202) or an even flat split;
* strategy switch: the table changes in place while parameters stay where they are.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

from ..ops import _lib
from ..ops.elementwise import OPT_KIND


def even_ranges(n: int, owners: list[int], nranks: int, align: int = 4) -> list[list[tuple[int, int]]]:
    """Split ``[0,n)`` evenly (boundaries multiples of ``align``) among ``owners``."""
    out: list[list[tuple[int, int]]] = [[] for _ in range(nranks)]
    units = (n + align - 1) // align
    k = len(owners)
    base, rem = divmod(units, k)
    lo = 0
    for j, r in enumerate(owners):
        cnt = base + (1 if j < rem else 0)
        hi = lo + cnt
        if cnt:
            out[r].append((lo * align, min(hi * align, (n + align - 1) // align * align)))
        lo = hi
    return out


def pre_reduce_plan(own: list[list[tuple[int, int]]], max_ranges: int):
    """Fewer owners than ranks (a parameter server with 4 servers on 8 GPUs): every worker's 16-bit gradients of an
    owner's share converge on that owner, (N-1)/S of the vector through one GPU's links, while the ranks that own nothing
    receive nothing. Those ranks become reducers: each owner keeps 1/(k+1) of every range it owns and hands one such part
    to each of its k idle partners; the workers ship a part's gradients to whoever reduces it, the partner sums the slabs in
    f32 in rank order (first launch of the exchange), a copy engine carries the f32 sums into the owner's f32 gradient
    vector, and the owner finishes those parts from its own memory (second launch). Same sums, same order, same result; the bytes that
    arrive at any one GPU during backward drop by the factor k+1.

    Returns ``(reduce_at, finish_at, fwd_to)``: per rank the ranges whose slabs it sums in the first launch; per owner
    the ranges it finishes in the second; partner rank -> owner rank. ``None`` when the layout does not allow it (no idle
    ranks, idle ranks not a multiple of the owners, a range not cut at multiples of 8, range tables too long)."""
    owners = [r for r, rs in enumerate(own) if rs]
    idle = [r for r, rs in enumerate(own) if not rs]
    if not owners or not idle or len(idle) % len(owners):
        return None
    k = len(idle) // len(owners)
    reduce_at, finish_at, fwd = [[] for _ in own], [[] for _ in own], {}
    for j, o in enumerate(owners):
        partners = idle[j * k:(j + 1) * k]
        for h in partners:
            fwd[h] = o
        for b, e in own[o]:
            if b % 8 or e % 8:
                return None
            cuts = [b] + [b + ((e - b) * t // (k + 1)) // 64 * 64 for t in range(1, k + 1)] + [e]
            for t, r in enumerate([o] + partners):
                if cuts[t + 1] > cuts[t]:
                    reduce_at[r].append((cuts[t], cuts[t + 1]))
            if e > cuts[1]:
                finish_at[o].append((cuts[1], e))
    if any(len(rs) > max_ranges for rs in reduce_at + finish_at):
        return None
    return reduce_at, finish_at, fwd


def layer_ranges(layer_offsets: list[tuple[int, int, int]], nranks: int) -> list[list[tuple[int, int]]]:
    """``(owner_rank, begin, end)`` per layer -> merged ranges per rank (layer-granular sharding)."""
    out: list[list[tuple[int, int]]] = [[] for _ in range(nranks)]
    for r, b, e in layer_offsets:
        if e <= b:
            continue
        if out[r] and out[r][-1][1] == b:
            out[r][-1] = (out[r][-1][0], e)
        else:
            out[r].append((b, e))
    return out


@dataclass
class OptimizerCfg:
    kind: str = "sgd"
    lr: float = 0.01
    mu: float = 0.0
    b1: float = 0.9
    b2: float = 0.999
    eps: float = 1e-8


def fill_sync(s: "_lib.OnoSync", *, nranks: int, rank: int, n: int, nblocks: int, algo: int,
              g_ptrs: list[int], p_f32_ptrs: list[int | None], p_bf16_ptrs: list[int | None],
              flag_ptrs: list[int], worker_mask: int, member_mask: int, n_workers: int,
              opt: OptimizerCfg, divide: bool = True, timeout_ns: int = 2_000_000_000,
              g_mc: int | None = None, p_mc_f32: int | None = None, p_mc_bf16: int | None = None,
              live_mask: int | None = None) -> None:
    s.nranks, s.rank, s.algo, s.nblocks, s.n = nranks, rank, algo, nblocks, n
    for r in range(nranks):
        s.g[r] = g_ptrs[r]
        s.p_out_f32[r] = p_f32_ptrs[r]
        s.p_out_bf16[r] = p_bf16_ptrs[r]
        s.flags[r] = flag_ptrs[r]
    s.g_mc, s.p_mc_f32, s.p_mc_bf16 = g_mc, p_mc_f32, p_mc_bf16
    s.worker_mask, s.member_mask, s.live_mask = worker_mask, member_mask, live_mask
    s.n_workers = n_workers
    s.kind = OPT_KIND[opt.kind]
    s.lr, s.mu, s.b1, s.b2, s.eps = opt.lr, opt.mu, opt.b1, opt.b2, opt.eps
    s.divide = int(divide)
    s.zero_grad = 0
    s.timeout_ns = timeout_ns


def fill_local(loc: "_lib.OnoSyncLocal", *, p_master: int, m: int | None, v: int | None, state_off: int,
               adam_pows: int | None, epoch: int, ranges: list[tuple[int, int]], sumsq: int | None = None,
               status: int | None = None, fwd: int | None = None) -> None:
    """``fwd``: this rank pre-reduces its ranges for another owner: the f32 sums of the workers' 16-bit slabs go to that
    address (the owner's f32 gradient vector) and nothing else happens on them (ranges must be multiples of 8)."""
    if len(ranges) > _lib.MAX_RANGES:
        raise ValueError(f"at most {_lib.MAX_RANGES} ranges per rank")
    if fwd and any(b % 8 or e % 8 for b, e in ranges):
        raise ValueError("pre-reduced ranges must be multiples of 8 elements")
    loc.p_master, loc.m, loc.v, loc.state_off = p_master, m, v, state_off
    loc.adam_pows, loc.epoch, loc.sumsq, loc.status = adam_pows, epoch, sumsq, status
    loc.fwd = fwd
    loc.n_ranges = len(ranges)
    for i, (b, e) in enumerate(ranges):
        if b % 4:
            raise ValueError("range begins must be multiples of 4 elements")
        loc.ranges[i].begin, loc.ranges[i].end = b, e


def launch_sync(s: "_lib.OnoSync", stream=None, emulated: bool = False) -> None:
    lib = _lib.load()
    fn = lib.ono_sync_step_emulated if emulated else lib.ono_sync_step
    _lib.check(fn(C.byref(s), _lib.stream_ptr(stream)), "ono_sync_step")
