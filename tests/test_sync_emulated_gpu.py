"""Multi-rank logic of the fused reduce-scatter + optimizer + all-gather kernel on ONE GPU.

All ranks run as one cooperative launch (grid.y = rank), each with its own buffers, so block b of
"rank" r really waits on block b of the other ranks through the same flag protocol as on NVLink.
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(nranks, n, owners_fn, kind, workers=None, steps=2, nblocks=4, bf16_out=False):
    from oxidized_neural_orchestra_b200.ops import _lib
    from oxidized_neural_orchestra_b200.parallel import sync as S

    torch.manual_seed(0)
    npad = (n + 3) // 4 * 4
    workers = list(range(nranks)) if workers is None else workers
    g = [torch.zeros(npad, device="cuda") for _ in range(nranks)]
    p = [torch.zeros(npad, device="cuda") for _ in range(nranks)]
    p0 = torch.randn(npad, device="cuda")
    for t in p:
        t.copy_(p0)
    pb = [torch.zeros(npad, device="cuda", dtype=torch.bfloat16) for _ in range(nranks)]
    m = [torch.zeros(npad, device="cuda") for _ in range(nranks)]
    v = [torch.zeros(npad, device="cuda") for _ in range(nranks)]
    flags = [torch.zeros(nblocks * 8, device="cuda", dtype=torch.int32) for _ in range(nranks)]
    epoch = [torch.zeros(nblocks, device="cuda", dtype=torch.int32) for _ in range(nranks)]
    status = [torch.zeros(1, device="cuda", dtype=torch.int32) for _ in range(nranks)]
    sumsq = [torch.zeros(1, device="cuda", dtype=torch.float64) for _ in range(nranks)]
    pows = torch.ones(2, device="cuda")
    ranges = owners_fn(n, nranks)
    opt = S.OptimizerCfg(kind=kind, lr=0.05, mu=0.9)
    s = _lib.OnoSync()
    wmask = sum(1 << w for w in workers)
    S.fill_sync(s, nranks=nranks, rank=0, n=n, nblocks=nblocks, algo=0,
                g_ptrs=[t.data_ptr() for t in g], p_f32_ptrs=[t.data_ptr() for t in p],
                p_bf16_ptrs=[t.data_ptr() if bf16_out else None for t in pb],
                flag_ptrs=[t.data_ptr() for t in flags], worker_mask=wmask, member_mask=(1 << nranks) - 1,
                n_workers=len(workers), opt=opt)
    for r in range(nranks):
        S.fill_local(s.loc[r], p_master=p[r].data_ptr(), m=m[r].data_ptr(), v=v[r].data_ptr(), state_off=0,
                     adam_pows=pows.data_ptr(), epoch=epoch[r].data_ptr(), ranges=ranges[r],
                     sumsq=sumsq[r].data_ptr(), status=status[r].data_ptr())
    ref_p, ref_m, ref_v = p0[:n].double().clone(), torch.zeros(n, device="cuda").double(), torch.zeros(n, device="cuda").double()
    b1t = b2t = 1.0
    total_sq = 0.0
    for step in range(steps):
        gs = [torch.randn(n, device="cuda") for _ in range(nranks)]
        for r in range(nranks):
            g[r][:n] = gs[r]
        if kind == "adam":
            from oxidized_neural_orchestra_b200.ops.elementwise import adam_tick
            adam_tick(pows, 0.9, 0.999)
        S.launch_sync(s, emulated=True)
        avg = sum(gs[w].double() for w in workers) / len(workers)
        total_sq += (avg ** 2).sum().item()
        if kind == "sgd":
            ref_p -= 0.05 * avg
        elif kind == "momentum":
            ref_m = 0.9 * ref_m + avg
            ref_p -= 0.05 * ref_m
        else:
            b1t *= 0.9; b2t *= 0.999
            stepsz = 0.05 * math.sqrt(1 - b2t) / (1 - b1t)
            ref_m = 0.9 * ref_m + 0.1 * avg
            ref_v = 0.999 * ref_v + 0.001 * avg * avg
            ref_p -= stepsz * ref_m / (ref_v.sqrt() + 1e-8)
    torch.cuda.synchronize()
    for r in range(nranks):
        assert status[r].item() == 0
        # Adam divides by sqrt(v): where the averaged gradient nearly cancels, f32 vs f64 summation
        # order shows up in the ratio, hence the wider bound for it.
        tol = 1e-3 if kind == "adam" else 1e-4
        assert (p[r][:n].double() - ref_p).abs().max().item() < tol, f"rank {r}"
        if bf16_out:
            assert (pb[r][:n].float() - p[r][:n]).abs().max().item() <= 2 ** -7 * p[r][:n].abs().max().item()
    return sum(t.item() for t in sumsq), total_sq, ranges


@pytest.mark.parametrize("kind", ["sgd", "momentum", "adam"])
@pytest.mark.parametrize("nranks", [2, 4, 8])
def test_two_shot_all_reduce(kind, nranks):
    from oxidized_neural_orchestra_b200.parallel.sync import even_ranges

    got, want, _ = _run(nranks, 100003, lambda n, N: even_ranges(n, list(range(N)), N), kind, bf16_out=True)
    assert abs(got - want) < 1e-6 * want


def test_parameter_server_ownership_two_servers_six_workers():
    """Ranks 6,7 own everything (servers, no gradients of their own); ranks 0-5 are workers."""
    from oxidized_neural_orchestra_b200.parallel.sync import even_ranges

    _run(8, 50000, lambda n, N: even_ranges(n, [6, 7], N), "adam", workers=[0, 1, 2, 3, 4, 5])


def test_layer_granular_ranges():
    from oxidized_neural_orchestra_b200.parallel.sync import layer_ranges

    offs = [(0, 0, 1000), (1, 1000, 5000), (0, 5000, 5200), (0, 5200, 9000)]
    _run(2, 9000, lambda n, N: layer_ranges(offs, N), "momentum")


@pytest.mark.parametrize("fmt", ["bf16", "f16"])
@pytest.mark.parametrize("kind", ["momentum", "adam"])
@pytest.mark.parametrize("n,align,f32_everywhere", [(70004, 4, True), (70016, 8, True), (70016, 8, False)])
def test_sixteen_bit_gradient_windows(fmt, kind, n, align, f32_everywhere):
    """Four ranks whose gradient windows hold 16-bit values (the wire format of step cadence): the owners sum them in f32
    in rank order, average, apply the optimizer and publish f32 + bf16 parameters. Ranges cut at multiples of 8 take the
    kernel's 16-byte path (eight gradients per load, eight bf16 parameters per store) when only the bf16 parameters travel
    (bf16-tile engines: the owner keeps the only f32 master); the others, and f32 parameters for every rank, its 8-byte path."""
    from oxidized_neural_orchestra_b200.ops import _lib
    from oxidized_neural_orchestra_b200.ops.elementwise import adam_tick, cast16
    from oxidized_neural_orchestra_b200.parallel import sync as S
    from oxidized_neural_orchestra_b200.parallel.sync import even_ranges

    torch.manual_seed(3)
    N, nblocks = 4, 4
    dt = torch.float16 if fmt == "f16" else torch.bfloat16
    g16 = [torch.zeros(n, device="cuda", dtype=dt) for _ in range(N)]
    p0 = torch.randn(n, device="cuda")
    p = [p0.clone() for _ in range(N)]
    pb = [torch.zeros(n, device="cuda", dtype=torch.bfloat16) for _ in range(N)]
    m = [torch.zeros(n, device="cuda") for _ in range(N)]
    v = [torch.zeros(n, device="cuda") for _ in range(N)]
    flags = [torch.zeros(nblocks * 8, device="cuda", dtype=torch.int32) for _ in range(N)]
    epoch = [torch.zeros(nblocks, device="cuda", dtype=torch.int32) for _ in range(N)]
    status = [torch.zeros(1, device="cuda", dtype=torch.int32) for _ in range(N)]
    pows = torch.ones(2, device="cuda")
    ranges = even_ranges(n, list(range(N)), N, align=align)
    s = _lib.OnoSync()
    S.fill_sync(s, nranks=N, rank=0, n=n, nblocks=nblocks, algo=0, g_ptrs=[t.data_ptr() for t in g16],
                p_f32_ptrs=[t.data_ptr() if f32_everywhere else None for t in p], p_bf16_ptrs=[t.data_ptr() for t in pb],
                flag_ptrs=[t.data_ptr() for t in flags], worker_mask=(1 << N) - 1, member_mask=(1 << N) - 1, n_workers=N,
                opt=S.OptimizerCfg(kind=kind, lr=0.05, mu=0.9))
    s.g_dtype = 2 if fmt == "f16" else 1
    for r in range(N):
        S.fill_local(s.loc[r], p_master=p[r].data_ptr(), m=m[r].data_ptr(), v=v[r].data_ptr(), state_off=0,
                     adam_pows=pows.data_ptr(), epoch=epoch[r].data_ptr(), ranges=ranges[r], status=status[r].data_ptr())
    ref_p, ref_m, ref_v = p0.double().clone(), torch.zeros(n, device="cuda").double(), torch.zeros(n, device="cuda").double()
    b1t = b2t = 1.0
    for step in range(2):
        gs = [torch.randn(n, device="cuda") * 0.01 for _ in range(N)]
        for r in range(N):
            cast16(gs[r], g16[r], f16=fmt == "f16")
            assert torch.equal(g16[r], gs[r].to(dt))          # the cast kernel rounds like PyTorch does
        if kind == "adam":
            adam_tick(pows, 0.9, 0.999)
        S.launch_sync(s, emulated=True)
        avg = sum(t.double() for t in g16) / N
        if kind == "momentum":
            ref_m = 0.9 * ref_m + avg
            ref_p -= 0.05 * ref_m
        else:
            b1t *= 0.9; b2t *= 0.999
            ref_m = 0.9 * ref_m + 0.1 * avg
            ref_v = 0.999 * ref_v + 0.001 * avg * avg
            ref_p -= 0.05 * math.sqrt(1 - b2t) / (1 - b1t) * ref_m / (ref_v.sqrt() + 1e-8)
    torch.cuda.synchronize()
    tol = 2e-3 if kind == "adam" else 1e-5
    for r in range(N):
        assert status[r].item() == 0
        if f32_everywhere:
            assert (p[r].double() - ref_p).abs().max().item() < tol, f"rank {r}"
        else:       # only the owner's master moved, over the ranges it owns
            for b, e in ranges[r]:
                assert (p[r][b:e].double() - ref_p[b:e]).abs().max().item() < tol, f"rank {r}"
        assert (pb[r].float().double() - ref_p).abs().max().item() <= 2 ** -7 * ref_p.abs().max().item() + tol


@pytest.mark.parametrize("kind", ["momentum", "adam"])
def test_pre_reduction_by_non_owner_ranks(kind):
    """Two owners, two ranks that own nothing: each owner keeps half of its share and the other half is summed by its
    helper, whose f32 sums land in the owner's f32 gradient vector; a second launch lets the owner finish that half from
    its own memory. The result is that of the one-launch exchange (same summation order, same scale)."""
    from oxidized_neural_orchestra_b200.ops import _lib
    from oxidized_neural_orchestra_b200.ops.elementwise import adam_tick
    from oxidized_neural_orchestra_b200.parallel import sync as S

    torch.manual_seed(11)
    N, n, nblocks = 4, 1 << 16, 4
    q = n // 4
    owned = [[(0, 2 * q)], [(2 * q, n)], [], []]
    first = [[(0, q)], [(2 * q, 3 * q)], [(q, 2 * q)], [(3 * q, n)]]      # who sums which quarter in the first launch
    helper_of = {2: 0, 3: 1}
    z = lambda dt=torch.float32: torch.zeros(n, device="cuda", dtype=dt)
    p0 = torch.randn(n, device="cuda")

    def run(split: bool):
        g16 = [z(torch.bfloat16) for _ in range(N)]
        G = [torch.full((n,), 7.0, device="cuda") for _ in range(N)]       # stale values the helpers must overwrite
        p, pb = [p0.clone() for _ in range(N)], [z(torch.bfloat16) for _ in range(N)]
        m, v = [z() for _ in range(N)], [z() for _ in range(N)]
        flags = [torch.zeros(nblocks * 8, device="cuda", dtype=torch.int32) for _ in range(N)]
        epoch = [torch.zeros(nblocks, device="cuda", dtype=torch.int32) for _ in range(N)]
        status = [torch.zeros(1, device="cuda", dtype=torch.int32) for _ in range(N)]
        pows = torch.ones(2, device="cuda")
        opt = S.OptimizerCfg(kind=kind, lr=0.05, mu=0.9)

        def make(g_ptrs, g_dtype, ranges, members, workers, fwd=None):
            s = _lib.OnoSync()
            S.fill_sync(s, nranks=N, rank=0, n=n, nblocks=nblocks, algo=0, g_ptrs=g_ptrs, p_f32_ptrs=[t.data_ptr() for t in p],
                        p_bf16_ptrs=[t.data_ptr() for t in pb], flag_ptrs=[t.data_ptr() for t in flags], worker_mask=workers,
                        member_mask=members, n_workers=N, opt=opt)
            s.g_dtype = g_dtype
            for r in range(N):
                S.fill_local(s.loc[r], p_master=p[r].data_ptr(), m=m[r].data_ptr(), v=v[r].data_ptr(), state_off=0,
                             adam_pows=pows.data_ptr(), epoch=epoch[r].data_ptr(), ranges=ranges[r], status=status[r].data_ptr(),
                             fwd=(fwd or {}).get(r))
            return s

        every = (1 << N) - 1
        slabs = [t.data_ptr() for t in g16]
        if split:
            launches = [make(slabs, 1, first, every, every, fwd={h: G[o].data_ptr() for h, o in helper_of.items()})]
            for o in (0, 1):        # the owner alone finishes its helper's quarter from its own f32 vector
                rest = [[] for _ in range(N)]
                rest[o] = first[2 + o]
                launches.append(make([t.data_ptr() for t in G], 0, rest, 1 << o, 1 << o))
        else:
            launches = [make(slabs, 1, owned, every, every)]
        gen = torch.Generator(device="cuda").manual_seed(5)
        for step in range(3):
            for r in range(N):
                g16[r].copy_((torch.randn(n, device="cuda", generator=gen) * 0.01).to(torch.bfloat16))
            if kind == "adam":
                adam_tick(pows, 0.9, 0.999)
            for s in launches:
                S.launch_sync(s, emulated=True)
        torch.cuda.synchronize()
        assert all(t.item() == 0 for t in status)
        return p, pb, m

    p_a, pb_a, m_a = run(False)
    p_b, pb_b, m_b = run(True)
    for r in range(N):
        # same summation order and scale in both forms; the two code paths may contract multiply-adds differently
        assert (p_a[r] - p_b[r]).abs().max().item() <= 1e-6, f"rank {r}"
        assert torch.equal(pb_b[r], p_b[r].to(torch.bfloat16)), f"rank {r}"
        assert torch.equal(p_b[r], p_b[0]), f"rank {r}"
    assert (m_a[0] - m_b[0]).abs().max().item() <= 1e-6 and (m_a[1] - m_b[1]).abs().max().item() <= 1e-6
    assert (p_b[0] - p0).abs().max().item() > 1e-4


@pytest.mark.parametrize("kind", ["sgd", "momentum", "adam"])
@pytest.mark.parametrize("nranks", [2, 3, 4, 8])
def test_ring_all_reduce_protocol(kind, nranks):
    """The ring kernel (reduce-scatter + optimizer on the owned chunk + all-gather of fresh parameters, chunked like
    worker/src/middlewares/mod.rs:15-59) with every rank in one cooperative launch: each block pipeline waits on its
    neighbours' step flags exactly as it does over NVLink."""
    import ctypes as C

    from oxidized_neural_orchestra_b200.ops import _lib
    from oxidized_neural_orchestra_b200.ops.elementwise import OPT_KIND, adam_tick

    lib = _lib.load()
    torch.manual_seed(5)
    n, nblocks = 50_000, 3
    npad = (n + 3) // 4 * 4
    z = lambda dt=torch.float32, m=npad: torch.zeros(m, device="cuda", dtype=dt)
    g, acc, p, m, v = ([z() for _ in range(nranks)] for _ in range(5))
    pb = [z(torch.bfloat16) for _ in range(nranks)]
    flags = [z(torch.int32, 2 * nblocks) for _ in range(nranks)]
    epoch = [z(torch.int32, nblocks) for _ in range(nranks)]
    status = torch.zeros(1, device="cuda", dtype=torch.int32)
    pows = torch.ones(2, device="cuda")
    p0 = torch.randn(npad, device="cuda")
    for t in p:
        t.copy_(p0)
    e = _lib.OnoRingEmu()
    e.nranks, e.nblocks, e.n = nranks, nblocks, npad
    for r in range(nranks):
        e.g[r], e.acc[r], e.flags[r], e.epoch[r] = g[r].data_ptr(), acc[r].data_ptr(), flags[r].data_ptr(), epoch[r].data_ptr()
        e.p[r], e.m[r], e.v[r], e.p_bf16[r] = p[r].data_ptr(), m[r].data_ptr(), v[r].data_ptr(), pb[r].data_ptr()
    e.adam_pows, e.kind, e.lr, e.mu, e.b1, e.b2, e.eps = pows.data_ptr(), OPT_KIND[kind], 0.05, 0.9, 0.9, 0.999, 1e-8
    e.status, e.timeout_ns = status.data_ptr(), 2_000_000_000
    ref_p, ref_m, ref_v = p0.double().clone(), torch.zeros(npad, device="cuda").double(), torch.zeros(npad, device="cuda").double()
    b1t = b2t = 1.0
    for step in range(3):       # the flags are epoch-stamped: later calls run on what the earlier ones left
        gs = [torch.randn(npad, device="cuda") for _ in range(nranks)]
        for r in range(nranks):
            g[r].copy_(gs[r])
        if kind == "adam":
            adam_tick(pows, 0.9, 0.999)
        _lib.check(lib.ono_ring_allreduce_emulated(C.byref(e), _lib.stream_ptr()), "ono_ring_allreduce_emulated")
        avg = sum(t.double() for t in gs) / nranks
        if kind == "sgd":
            ref_p -= 0.05 * avg
        elif kind == "momentum":
            ref_m = 0.9 * ref_m + avg
            ref_p -= 0.05 * ref_m
        else:
            b1t *= 0.9; b2t *= 0.999
            ref_m = 0.9 * ref_m + 0.1 * avg
            ref_v = 0.999 * ref_v + 0.001 * avg * avg
            ref_p -= 0.05 * math.sqrt(1 - b2t) / (1 - b1t) * ref_m / (ref_v.sqrt() + 1e-8)
    torch.cuda.synchronize()
    assert status.item() == 0
    for r in range(nranks):
        assert (p[r].double() - ref_p).abs().max().item() < (1e-3 if kind == "adam" else 1e-4), f"rank {r}"
        assert torch.equal(p[r], p[0])                      # every replica ends with the same bits
        assert (pb[r].float() - p[r]).abs().max().item() <= 2 ** -7 * p[r].abs().max().item()
