"""The allocation-free entry point ``ono_sync_step_noalloc`` against the regular ``ono_sync_step``.

Some users of the kernel library cannot allocate device memory at the point where they need the fused
optimizer step (their process's framework owns all of HBM, or they sit between captured graphs, or they
must not touch the allocator's lock). For them the library keeps the step's scratch (barrier flag pad
and epoch words) in a fixed device array of its own. This test calls that entry point through its
exported C symbol, twice in a row, and checks every output against the regular entry point, which gets
its scratch from the caller. It lives in a file that sorts last so that a run stopping at the first
failure has already executed every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_BLOCKS = 512  # ONO_NOALLOC_MAX_BLOCKS


class OnoNoAllocStep(C.Structure):
    _fields_ = [
        ("p", C.c_void_p), ("g", C.c_void_p), ("m", C.c_void_p), ("v", C.c_void_p), ("p_bf16", C.c_void_p),
        ("n", C.c_longlong), ("kind", C.c_int),
        ("lr", C.c_float), ("mu", C.c_float), ("b1", C.c_float), ("b2", C.c_float), ("eps", C.c_float),
        ("n_workers", C.c_int), ("adam_pows", C.c_void_p), ("sumsq", C.c_void_p), ("status", C.c_void_p),
        ("nblocks", C.c_int),
    ]


def _regular(lib, S, _lib, bufs, kind, n, nblocks):
    """The existing entry point as a one-rank run; flags and epoch words come from the caller."""
    s = _lib.OnoSync()
    opt = S.OptimizerCfg(kind=kind, lr=0.05, mu=0.9)
    S.fill_sync(s, nranks=1, rank=0, n=n, nblocks=nblocks, algo=0, g_ptrs=[bufs["g"].data_ptr()],
                p_f32_ptrs=[bufs["p"].data_ptr()], p_bf16_ptrs=[bufs["pb"].data_ptr()],
                flag_ptrs=[bufs["flags"].data_ptr()], worker_mask=1, member_mask=1, n_workers=4, opt=opt)
    S.fill_local(s.loc[0], p_master=bufs["p"].data_ptr(), m=bufs["m"].data_ptr(), v=bufs["v"].data_ptr(), state_off=0,
                 adam_pows=bufs["pows"].data_ptr(), epoch=bufs["epoch"].data_ptr(), ranges=[(0, n)],
                 sumsq=bufs["sumsq"].data_ptr(), status=bufs["status"].data_ptr())
    _lib.check(lib.ono_sync_step(C.byref(s), _lib.stream_ptr()), "ono_sync_step")


@pytest.mark.parametrize("kind", ["sgd", "momentum", "adam"])
def test_noalloc_step_matches_regular_entry_point_twice(kind):
    from oxidized_neural_orchestra_b200.ops import _lib
    from oxidized_neural_orchestra_b200.ops.elementwise import OPT_KIND, adam_tick
    from oxidized_neural_orchestra_b200.parallel import sync as S

    lib = _lib.load()
    fn = lib.ono_sync_step_noalloc          # the exported C symbol
    fn.argtypes = [C.POINTER(OnoNoAllocStep), C.c_void_p]
    fn.restype = C.c_int
    torch.manual_seed(11)
    n = 1_000_003
    npad = (n + 3) // 4 * 4
    nblocks = 64

    def make():
        z = lambda dt=torch.float32: torch.zeros(npad, device="cuda", dtype=dt)
        b = {"p": z(), "g": z(), "m": z(), "v": z(), "pb": z(torch.bfloat16),
             "pows": torch.ones(2, device="cuda"), "sumsq": torch.zeros(1, device="cuda", dtype=torch.float64),
             "status": torch.zeros(1, device="cuda", dtype=torch.int32),
             "flags": torch.zeros(nblocks * 8, device="cuda", dtype=torch.int32),
             "epoch": torch.zeros(nblocks, device="cuda", dtype=torch.int32)}
        return b

    ref, new = make(), make()
    p0 = torch.randn(n, device="cuda")
    ref["p"][:n] = p0
    new["p"][:n] = p0
    before = torch.cuda.memory_allocated()
    for call in range(2):  # the second call runs on the scratch contents the first one left behind
        g = torch.randn(n, device="cuda")
        ref["g"][:n] = g
        new["g"][:n] = g
        if kind == "adam":
            adam_tick(ref["pows"], 0.9, 0.999)
            adam_tick(new["pows"], 0.9, 0.999)
        _regular(lib, S, _lib, ref, kind, npad, nblocks)
        a = OnoNoAllocStep()
        a.p, a.g, a.m, a.v, a.p_bf16 = (new[k].data_ptr() for k in ("p", "g", "m", "v", "pb"))
        a.n, a.kind = npad, OPT_KIND[kind]      # the padded length: the entry point rejects a length that is not a multiple of 4
        a.lr, a.mu, a.b1, a.b2, a.eps = 0.05, 0.9, 0.9, 0.999, 1e-8
        a.n_workers = 4
        a.adam_pows, a.sumsq, a.status = new["pows"].data_ptr(), new["sumsq"].data_ptr(), new["status"].data_ptr()
        a.nblocks = nblocks
        live = torch.cuda.memory_allocated()
        rc = fn(C.byref(a), _lib.stream_ptr())
        assert rc == 0, lib.ono_last_error().decode()
        assert torch.cuda.memory_allocated() == live  # nothing was taken from torch's allocator either
        torch.cuda.synchronize()
        assert new["status"].item() == 0 and ref["status"].item() == 0
        # same kernel, same arithmetic order: the results agree to the last bit
        for k in ("p", "m", "v", "pb"):
            assert torch.equal(ref[k], new[k]), (kind, call, k)
        assert abs(ref["sumsq"].item() - new["sumsq"].item()) <= 1e-9 * max(1.0, ref["sumsq"].item())
    assert not torch.equal(new["p"][:n], p0)
    del before


def test_noalloc_step_rejects_requests_beyond_its_scratch():
    from oxidized_neural_orchestra_b200.ops import _lib

    lib = _lib.load()
    fn = lib.ono_sync_step_noalloc
    fn.argtypes = [C.POINTER(OnoNoAllocStep), C.c_void_p]
    fn.restype = C.c_int
    p = torch.zeros(1024, device="cuda")
    g = torch.ones(1024, device="cuda")
    a = OnoNoAllocStep()
    a.p, a.g, a.n, a.kind, a.lr, a.n_workers = p.data_ptr(), g.data_ptr(), 1024, 0, 0.1, 1
    a.nblocks = MAX_BLOCKS + 1
    assert fn(C.byref(a), _lib.stream_ptr()) != 0
    assert b"exceeds the built-in scratch" in lib.ono_last_error()
    torch.cuda.synchronize()
    assert torch.count_nonzero(p).item() == 0  # nothing ran
    # a length that is not padded to 4 elements, or a bf16 shadow that is not 8-byte aligned, is an argument error too
    a.nblocks = 0
    a.n = 1022
    assert fn(C.byref(a), _lib.stream_ptr()) != 0 and b"multiple of 4" in lib.ono_last_error()
    a.n = 1024
    shadow = torch.zeros(1028, device="cuda", dtype=torch.bfloat16)
    a.p_bf16 = shadow.data_ptr() + 2
    assert fn(C.byref(a), _lib.stream_ptr()) != 0 and b"8-byte aligned" in lib.ono_last_error()
    a.p_bf16 = None
    torch.cuda.synchronize()
    assert torch.count_nonzero(p).item() == 0
    a.nblocks = 0  # the library picks a grid within its scratch
    assert fn(C.byref(a), _lib.stream_ptr()) == 0
    torch.cuda.synchronize()
    assert torch.allclose(p, torch.full_like(p, -0.1))
