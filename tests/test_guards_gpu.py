"""Memory-safety and determinism checks that stand in for a device sanitizer: every output sits inside a larger
allocation whose guard bands must come back untouched, over all tile-edge residues of the GEMM (M, N in
{1, tile-1, tile, tile+1}) and over vector lengths of the fused optimizer kernel that no vector width or block count
divides; and the kernels whose reduction order is fixed must give the same bits twice."""
import pytest
import torch

pytestmark = pytest.mark.gpu

SENTINEL = -7.25e11     # nothing a test computes comes near it (compared after the same rounding to f32 / bf16)


def _guarded(rows, cols, dtype=torch.float32, band=8, col_band=16):
    """A [rows, cols] view in the middle of a sentinel-filled allocation; returns (view, whole, mask of the guard)."""
    ld = (cols + 15) // 16 * 16 + col_band
    whole = torch.full((rows + 2 * band, ld), SENTINEL, device="cuda", dtype=dtype)
    view = whole[band:band + rows, :cols]
    guard = torch.ones_like(whole, dtype=torch.bool)
    guard[band:band + rows, :cols] = False
    return view, whole, guard


def _intact(whole, guard):
    return bool((whole[guard] == torch.tensor(SENTINEL, dtype=whole.dtype, device="cuda")).all().item())


EDGES = [1, 31, 32, 33, 127, 128, 129, 255, 256, 257]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("pair", [-1, 1])
def test_gemm_writes_nothing_outside_its_outputs_at_every_tile_edge(dtype, pair):
    from oxidized_neural_orchestra_b200.ops.gemm import gemm

    torch.manual_seed(0)
    K = 72
    for M in EDGES:
        for N in (1, 31, 33, 127, 129, 257):
            if pair == 1 and M <= 128:
                continue
            a = torch.randn(M, 80, device="cuda", dtype=dtype)[:, :K]
            b = torch.randn(N, 80, device="cuda", dtype=dtype)[:, :K]
            out, out_w, out_g = _guarded(M, N)
            out_t, outt_w, outt_g = _guarded(N, M)
            ob, ob_w, ob_g = _guarded(M, N, torch.bfloat16)
            status = torch.zeros(1, dtype=torch.int32, device="cuda")
            gemm(a, b, out=out, out_t=out_t, out_bf16=ob, pair=pair, status=status)
            torch.cuda.synchronize()
            assert status.item() == 0
            ref = a.double() @ b.double().t()
            tol = 4e-3 * max(1.0, ref.abs().max().item())
            assert (out.double() - ref).abs().max().item() <= tol, (M, N)
            assert (out_t.double() - ref.t()).abs().max().item() <= tol, (M, N)
            assert _intact(out_w, out_g) and _intact(outt_w, outt_g) and _intact(ob_w, ob_g), (M, N)


def _sync_once(n, g0, opt="adam", iters=2):
    from oxidized_neural_orchestra_b200.ops import _lib
    from oxidized_neural_orchestra_b200.parallel import sync as S

    band = 64
    bufs = {k: torch.full((n + 2 * band,), SENTINEL, device="cuda") for k in "pgmv"}
    for k in "pmv":
        bufs[k][band:band + n] = 0
    bufs["g"][band:band + n] = g0
    p, g, m, v = (bufs[k][band:band + n] for k in "pgmv")
    nblocks = min(2 * _lib.load().ono_num_sms(), max(1, n // 4 // 1024))
    flags = torch.zeros(8192, device="cuda", dtype=torch.int32)
    epoch = torch.zeros(1024, device="cuda", dtype=torch.int32)
    pows = torch.full((2,), 0.5, device="cuda")
    s = _lib.OnoSync()
    S.fill_sync(s, nranks=1, rank=0, n=n, nblocks=nblocks, algo=0, g_ptrs=[g.data_ptr()], p_f32_ptrs=[p.data_ptr()],
                p_bf16_ptrs=[None], flag_ptrs=[flags.data_ptr()], worker_mask=1, member_mask=1, n_workers=1,
                opt=S.OptimizerCfg(kind=opt, lr=0.01, mu=0.9))
    S.fill_local(s.loc[0], p_master=p.data_ptr(), m=m.data_ptr(), v=v.data_ptr(), state_off=0, adam_pows=pows.data_ptr(),
                 epoch=epoch.data_ptr(), ranges=[(0, n)])
    for _ in range(iters):
        g.copy_(g0)
        S.launch_sync(s)
    torch.cuda.synchronize()
    for k in "pgmv":
        t = bufs[k]
        assert bool((t[:band] == SENTINEL).all()) and bool((t[band + n:] == SENTINEL).all()), (k, n)
    return p.clone(), m.clone(), v.clone()


@pytest.mark.parametrize("n", [4, 4 * 1021, 4 * 4099, 4 * 65537 + 4])
def test_fused_optimizer_kernel_stays_inside_its_vectors_and_repeats_bit_for_bit(n):
    torch.manual_seed(1)
    g0 = torch.randn(n, device="cuda") * 1e-2
    first = _sync_once(n, g0)
    second = _sync_once(n, g0)
    assert all(torch.equal(a, b) for a, b in zip(first, second))
    assert first[0].abs().max().item() > 0


def test_emulated_four_rank_reduce_scatter_repeats_bit_for_bit():
    """The multi-rank kernel sums the ranks' shards in rank order, whatever order the blocks run in."""
    import json
    import subprocess
    import sys
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    outs = []
    for _ in range(2):
        r = subprocess.run([sys.executable, os.path.join(root, "bench", "kernels.py"), "sync", "--emulate-ranks", "4",
                            "--elems", str(1 << 20), "--iters", "2", "--checksum"], capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        outs.append(json.loads(r.stdout.strip().splitlines()[-1])["checksum"])
    assert outs[0] == outs[1]


def test_column_sums_and_gemm_repeat_bit_for_bit():
    from oxidized_neural_orchestra_b200.ops.gemm import gemm

    torch.manual_seed(2)
    a = torch.randn(512, 1024, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(768, 1024, device="cuda", dtype=torch.bfloat16)
    outs = []
    for _ in range(2):
        out = torch.empty(512, 768, device="cuda")
        gemm(a, b, out=out)
        outs.append(out)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1])
    from oxidized_neural_orchestra_b200.ops.elementwise import colsum

    d = torch.randn(4096, 1000, device="cuda")
    sums = []
    for _ in range(2):
        o = torch.empty(1000, device="cuda")
        colsum(d, o)
        sums.append(o)
    torch.cuda.synchronize()
    assert torch.equal(sums[0], sums[1])
    assert torch.allclose(sums[0].double(), d.double().sum(0), atol=1e-3)


@pytest.mark.parametrize("shape", [(256, 516), (260, 1000), (4096, 784), (64, 1024)])
@pytest.mark.parametrize("which", ["both", "copy", "transpose"])
def test_vector_copy_and_transpose_match_and_stay_inside(shape, which):
    from oxidized_neural_orchestra_b200.ops.elementwise import rows

    R, W = shape
    torch.manual_seed(4)
    src = torch.randn(R, W + 12, device="cuda")[:, :W]
    dst, dst_w, dst_g = _guarded(R, W)
    dt, dt_w, dt_g = _guarded(W, R)
    rows(src, dst=dst if which != "transpose" else None, dst_t=dt if which != "copy" else None)
    torch.cuda.synchronize()
    if which != "transpose":
        assert torch.equal(dst, src)
    if which != "copy":
        assert torch.equal(dt, src.t())
    assert _intact(dst_w, dst_g | (which == "transpose")) and _intact(dt_w, dt_g | (which == "copy"))
