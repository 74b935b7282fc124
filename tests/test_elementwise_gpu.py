"""Elementwise CUDA kernels against plain PyTorch fp32 references."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind", ["sgd", "momentum", "adam"])
def test_optimizers_match_reference_formulas(kind):
    from oxidized_neural_orchestra_b200.ops import elementwise as ew

    torch.manual_seed(0)
    n = 10007  # exercises the scalar tail
    p = torch.randn(n + 1, device="cuda")[:n].clone()
    buf = lambda: torch.zeros(((n + 3) // 4) * 4, device="cuda")[:n]
    p0 = buf(); p0.copy_(p)
    m, v = buf(), buf()
    pows = torch.ones(2, device="cuda")
    pb = torch.zeros(((n + 3) // 4) * 4, device="cuda", dtype=torch.bfloat16)[:n]
    rp, rm, rv = p0.clone().double(), torch.zeros(n, device="cuda").double(), torch.zeros(n, device="cuda").double()
    lr, mu, b1, b2, eps = 0.01, 0.9, 0.9, 0.999, 1e-8
    b1t = b2t = 1.0
    for t in range(3):
        g = buf(); g.copy_(torch.randn(n, device="cuda"))
        if kind == "adam":
            ew.adam_tick(pows, b1, b2)
        ew.optim_step(p0, g, kind=kind, lr=lr, mu=mu, b1=b1, b2=b2, eps=eps, m=m, v=v, adam_pows=pows,
                      grad_scale=0.5, p_bf16=pb)
        gd = g.double() * 0.5
        if kind == "sgd":
            rp -= lr * gd
        elif kind == "momentum":
            rm = mu * rm + gd
            rp -= lr * rm
        else:
            b1t *= b1; b2t *= b2
            step = lr * math.sqrt(1 - b2t) / (1 - b1t)
            rm = b1 * rm + (1 - b1) * gd
            rv = b2 * rv + (1 - b2) * gd * gd
            rp -= step * rm / (rv.sqrt() + eps)
    torch.cuda.synchronize()
    assert (p0.double() - rp).abs().max().item() < 1e-5
    assert (pb.float() - p0).abs().max().item() <= 2 ** -8 * p0.abs().max().item() + 1e-6


def test_loss_kernel_composed_softmax_ce_and_mse():
    from oxidized_neural_orchestra_b200.ops import elementwise as ew

    torch.manual_seed(1)
    B, C = 37, 1000
    z = torch.randn(B, 1008, device="cuda")[:, :C] * 3
    y = torch.nn.functional.one_hot(torch.randint(0, C, (B,), device="cuda"), C).float()
    for kind in ("cross_entropy", "mse"):
        # Composition of the reference's Softmax layer and loss in fp64 (softmax.rs:44-64,
        # cross_entropy.rs:35-47, mse.rs:35-47): the clamp only guards the division.
        pd = torch.softmax(z.double(), 1)
        n = B * C
        if kind == "cross_entropy":
            ps = pd.clamp_min(1.1920929e-07)
            L = -(y * torch.log(ps)).sum() / n
            g = -(y / ps) / n
        else:
            L = ((pd - y) ** 2).sum() / n
            g = 2 * (pd - y) / n
        ref = (pd * (g - (pd * g).sum(1, keepdim=True))).float()
        d = torch.zeros(B, C, device="cuda")
        dt = torch.zeros(C, 48, device="cuda")[:, :B]
        db = torch.zeros(B, C, device="cuda", dtype=torch.bfloat16)
        ls = torch.zeros(1, device="cuda", dtype=torch.float64)
        cor = torch.zeros(1, device="cuda", dtype=torch.int32)
        ew.loss_backward(z, y, kind=kind, softmax=True, loss_sum=ls, d=d, d_t=dt, d_bf16=db, correct=cor)
        torch.cuda.synchronize()
        assert abs(ls.item() - L.item()) < 1e-5 * max(1.0, abs(L.item()))
        scale = ref.abs().max().item()
        assert (d - ref).abs().max().item() < 1e-4 * scale
        assert (dt.t() - ref).abs().max().item() < 1e-4 * scale
        assert (db.float() - ref).abs().max().item() < 1e-2 * scale
        assert cor.item() == (z.argmax(1) == y.argmax(1)).sum().item()


def test_rows_gather_cast_transpose_and_colsum():
    from oxidized_neural_orchestra_b200.ops import elementwise as ew

    torch.manual_seed(2)
    src = torch.randn(300, 77, device="cuda")
    idx = torch.randperm(300, device="cuda")[:100].int()
    dst = torch.zeros(100, 80, device="cuda")
    dst_t = torch.zeros(77, 112, device="cuda")
    db = torch.zeros(100, 80, device="cuda", dtype=torch.bfloat16)
    dtb = torch.zeros(77, 112, device="cuda", dtype=torch.bfloat16)
    ew.rows(src, idx=idx, dst=dst, dst_t=dst_t, dst_bf16=db, dst_t_bf16=dtb)
    ref = src[idx.long()]
    assert torch.equal(dst[:, :77], ref)
    assert torch.equal(dst_t[:, :100], ref.t())
    assert torch.equal(db[:, :77], ref.to(torch.bfloat16))
    assert torch.equal(dtb[:, :100], ref.t().to(torch.bfloat16))
    out = torch.ones(77, device="cuda")
    ew.colsum(ref.contiguous(), out, beta=2.0)
    assert (out - (ref.sum(0) + 2.0)).abs().max().item() < 1e-4
    ss = torch.zeros(1, device="cuda", dtype=torch.float64)
    ew.sumsq(src.view(-1), ss)
    assert abs(ss.item() - (src.double() ** 2).sum().item()) < 1e-6 * ss.item()


@pytest.mark.parametrize("width", [784, 10, 8192])
def test_rows_gather_from_pinned_host_memory(width):
    """The batch feeder's path: the kernel reads the selected rows straight out of pinned host memory (a few blocks with
    16-byte loads when the rows allow it, the generic kernel otherwise)."""
    from oxidized_neural_orchestra_b200.ops import elementwise as ew

    torch.manual_seed(1)
    src = torch.randn(300, width).pin_memory()
    idx = torch.randperm(300)[:77].to(torch.int32).cuda()
    dst = torch.full((80, width), -7.0, device="cuda")
    ew.rows(src, idx=idx, n_rows=77, dst=dst)
    torch.cuda.synchronize()
    assert torch.equal(dst[:77].cpu(), src[idx.cpu().long()])
    assert torch.all(dst[77:] == -7.0)


def test_philox_init_is_shard_independent_and_distributed_right():
    from oxidized_neural_orchestra_b200.ops import elementwise as ew

    n = 1 << 18
    full = torch.empty(n, device="cuda")
    ew.philox_init(full, seed=42, index_offset=0, kind="normal", a=0.5, b=2.0)
    part = torch.empty(1000, device="cuda")
    ew.philox_init(part, seed=42, index_offset=5000, kind="normal", a=0.5, b=2.0)
    assert torch.equal(part, full[5000:6000])
    assert abs(full.mean().item() - 0.5) < 0.02 and abs(full.std().item() - 2.0) < 0.02
    u = torch.empty(n, device="cuda")
    ew.philox_init(u, seed=7, index_offset=0, kind="uniform", a=-0.25, b=0.75)
    assert u.min().item() >= -0.25 and u.max().item() < 0.75
    assert abs(u.mean().item() - 0.25) < 0.01
    other = torch.empty(n, device="cuda")
    ew.philox_init(other, seed=8, index_offset=0, kind="uniform", a=-0.25, b=0.75)
    assert not torch.equal(u, other)
