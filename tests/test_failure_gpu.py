"""Failure detection on the device: a wait that runs out reports a status word and leaves the context usable.

No fault is provoked. The "failed peer" is a flag word that nothing ever sets (all buffers are valid
local allocations), and every wait in the kernels is bounded, so the kernel returns by itself and the
host reads an error status. Host-side failures (a rank that leaves, a dropped message) are covered on
CPU ranks in ``test_strategies_cpu.py`` / ``test_failures_cpu.py``.
"""
import ctypes as C
import time

import pytest
import torch

pytestmark = pytest.mark.gpu

ERR_PEER_FLAG, ERR_BARRIER = 5, 6


def _two_rank_struct(n, nblocks, timeout_ns, live=None):
    from oxidized_neural_orchestra_b200.ops import _lib
    from oxidized_neural_orchestra_b200.parallel import sync as S

    t = dict(
        g=[torch.full((n,), 1.0, device="cuda") for _ in range(2)],
        p=[torch.zeros(n, device="cuda") for _ in range(2)],
        flags=[torch.zeros(nblocks * 8, device="cuda", dtype=torch.int32) for _ in range(2)],
        epoch=torch.zeros(nblocks, device="cuda", dtype=torch.int32),
        status=torch.zeros(1, device="cuda", dtype=torch.int32),
        live=None if live is None else torch.tensor([live], device="cuda", dtype=torch.int32),
    )
    s = _lib.OnoSync()
    S.fill_sync(s, nranks=2, rank=0, n=n, nblocks=nblocks, algo=0, g_ptrs=[x.data_ptr() for x in t["g"]],
                p_f32_ptrs=[x.data_ptr() for x in t["p"]], p_bf16_ptrs=[None, None],
                flag_ptrs=[x.data_ptr() for x in t["flags"]], worker_mask=3, member_mask=3, n_workers=2,
                opt=S.OptimizerCfg(kind="sgd", lr=1.0), timeout_ns=timeout_ns,
                live_mask=None if live is None else t["live"].data_ptr())
    S.fill_local(s.loc[0], p_master=t["p"][0].data_ptr(), m=None, v=None, state_off=0, adam_pows=None,
                 epoch=t["epoch"].data_ptr(), ranges=[(0, n)], status=t["status"].data_ptr())
    return s, t


def test_absent_peer_times_out_with_a_status_and_the_context_survives():
    from oxidized_neural_orchestra_b200.parallel import sync as S

    n, nblocks = 4096, 2
    s, t = _two_rank_struct(n, nblocks, timeout_ns=200_000_000)
    t0 = time.perf_counter()
    S.launch_sync(s)                      # rank 1 never runs: its flag words stay 0
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0
    assert t["status"].item() == ERR_PEER_FLAG
    assert torch.count_nonzero(t["p"][0]).item() == 0      # nothing was applied on a failed barrier
    # the context is intact: ordinary work and a healthy launch still run
    assert torch.ones(8, device="cuda").sum().item() == 8.0
    s1, t1 = _two_rank_struct(n, nblocks, timeout_ns=200_000_000, live=0b01)
    S.launch_sync(s1)
    torch.cuda.synchronize()
    assert t1["status"].item() == 0
    # membership shrunk to rank 0 by the host: only its gradient counts, still divided by the configured
    # worker count (parameter_server/src/storage/blocking/shard.rs:78-83)
    assert torch.allclose(t1["p"][0], torch.full((n,), -0.5, device="cuda"))


def test_async_server_lock_that_is_never_released_gives_up():
    from oxidized_neural_orchestra_b200.ops import _lib

    n, nblocks = 4096, 2
    g = torch.ones(n, device="cuda")
    master = torch.zeros(n, device="cuda")
    locks = torch.ones(nblocks, device="cuda", dtype=torch.int32)     # held by "someone" who never lets go
    status = torch.zeros(1, device="cuda", dtype=torch.int32)
    a = _lib.OnoPsAsync()
    a.nranks, a.rank, a.nblocks = 1, 0, nblocks
    a.g = g.data_ptr()
    a.master[0], a.locks[0], a.state_off[0] = master.data_ptr(), locks.data_ptr(), 0
    a.n_ranges[0] = 1
    a.ranges[0][0].begin, a.ranges[0][0].end = 0, n
    a.n_workers, a.divide, a.kind, a.lr = 1, 1, 0, 1.0
    a.status, a.timeout_ns = status.data_ptr(), 100_000_000
    lib = _lib.load()
    _lib.check(lib.ono_ps_async_step(C.byref(a), _lib.stream_ptr()), "ono_ps_async_step")
    torch.cuda.synchronize()
    assert status.item() == ERR_BARRIER
    assert torch.count_nonzero(master).item() == 0
    locks.zero_()
    status.zero_()
    _lib.check(lib.ono_ps_async_step(C.byref(a), _lib.stream_ptr()), "ono_ps_async_step")
    torch.cuda.synchronize()
    assert status.item() == 0 and torch.allclose(master, torch.full((n,), -1.0, device="cuda"))
    assert locks.sum().item() == 0


def test_gemm_operand_gate_opens_late_or_runs_out_and_the_context_survives():
    """The GEMM's producer waits (bounded) for flag words before its first operand load: the form in which a layer's GEMM is
    queued while its weights are still arriving. Flags already there: it runs. Flags set later from another stream: it runs
    once they are. A flag that nothing sets: the wait runs out, the status word says so, nothing is written, and the next
    launch on the same context works."""
    from oxidized_neural_orchestra_b200.ops.gemm import gemm

    torch.manual_seed(0)
    a = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(192, 128, device="cuda", dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    # the flag words live in pinned host memory here, so that the host itself can open the gate while the kernel waits (on a
    # GPU rank they are words of the rank's window that the owners' signal kernels write)
    flags = torch.zeros(32, dtype=torch.int32).pin_memory()
    target = torch.tensor([3], device="cuda", dtype=torch.int32)
    status = torch.zeros(1, device="cuda", dtype=torch.int32)

    def run(out, timeout_ns, stream=None):
        gemm(a, b, out=out, gate=(flags, target, 4, 0b101), timeout_ns=timeout_ns, status=status, stream=stream)

    flags[0], flags[8] = 3, 7                       # both selected words (index 0 and 2, stride 4) at or past the target
    out = torch.zeros(256, 192, device="cuda")
    run(out, 50_000_000)
    torch.cuda.synchronize()
    assert status.item() == 0 and (out - ref).abs().max().item() <= 2e-3 * ref.abs().max().item()
    # opened late, by the host, while the kernel is already waiting
    flags[8] = 2
    out2 = torch.zeros(256, 192, device="cuda")
    torch.cuda.synchronize()
    run(out2, 5_000_000_000)
    time.sleep(0.05)
    assert not torch.cuda.current_stream().query()          # still waiting at the gate
    flags[8] = 3
    torch.cuda.synchronize()
    assert status.item() == 0 and torch.equal(out2, out)
    # never opened: the wait gives up after its budget
    flags[8] = 1
    out3 = torch.full((256, 192), 9.0, device="cuda")
    run(out3, 30_000_000)
    torch.cuda.synchronize()
    assert status.item() == 5                       # ONO_ERR_TIMEOUT_PEER_FLAG
    assert bool((out3 == 9.0).all())
    status.zero_()
    flags[8] = 3
    run(out3, 30_000_000)
    torch.cuda.synchronize()
    assert status.item() == 0 and torch.equal(out3, out)
