"""Numerics of the tcgen05 GEMM against a plain PyTorch fp32 reference of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    A = a.float().t() if a_mn else a.float()
    B = b.float() if b_mn else b.float().t()
    return A.double() @ B.double()


def _tol(dtype, K):
    # tf32 keeps 10 mantissa bits (truncated), bf16 inputs are exact products accumulated in f32.
    return (4e-3 if dtype == torch.float32 else 2e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(128, 128, 64), (32, 10, 784), (300, 200, 136), (512, 1024, 512),
                                   (1024, 4096, 784), (129, 257, 72)])
def test_gemm_k_major(dtype, shape):
    from oxidized_neural_orchestra_b200.ops.gemm import gemm

    M, N, K = shape
    torch.manual_seed(0)
    ld = lambda n: (n + 15) // 16 * 16
    a = torch.randn(M, ld(K), device="cuda", dtype=dtype)[:, :K]
    b = torch.randn(N, ld(K), device="cuda", dtype=dtype)[:, :K]
    out = torch.zeros(M, ld(N), device="cuda")[:, :N]
    out_t = torch.zeros(N, ld(M), device="cuda")[:, :M]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    gemm(a, b, out=out, out_t=out_t, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    ref = _ref(a, b, False, False)
    scale = ref.abs().max().item()
    assert (out.double() - ref).abs().max().item() <= _tol(dtype, K) * scale
    assert (out_t.double() - ref.t()).abs().max().item() <= _tol(dtype, K) * scale


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, False), (True, True)])
@pytest.mark.parametrize("shape", [(128, 128, 64), (256, 320, 200), (512, 1024, 512)])
def test_gemm_bf16_mn_major(a_mn, b_mn, shape):
    from oxidized_neural_orchestra_b200.ops.gemm import gemm

    M, N, K = shape
    torch.manual_seed(1)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(M, N, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn, out=out, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    ref = _ref(a, b, a_mn, b_mn)
    assert (out.double() - ref).abs().max().item() <= 2e-3 * ref.abs().max().item()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm_epilogue(dtype):
    """bias + activation forward, then derivative-through-activation backward, bf16 copies, beta."""
    from oxidized_neural_orchestra_b200.ops.gemm import gemm

    torch.manual_seed(2)
    M, N, K = 200, 272, 96
    a = torch.randn(M, K, device="cuda", dtype=dtype)
    b = torch.randn(N, K, device="cuda", dtype=dtype) * 0.1
    bias = torch.randn(N, device="cuda")
    for act, param, fn in [("relu", 0.0, torch.relu), ("sigmoid", 1.5, lambda z: 1.5 * torch.sigmoid(z)),
                           ("tanh", 2.0, lambda z: 2.0 * torch.tanh(z)),
                           ("gelu", 0.0, torch.nn.functional.gelu)]:
        out = torch.empty(M, N, device="cuda")
        pre = torch.empty(M, N, device="cuda")
        ob = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        otb = torch.empty(N, 208, device="cuda", dtype=torch.bfloat16)[:, :M]
        gemm(a, b, out=out, pre=pre, out_bf16=ob, out_t_bf16=otb, bias=bias, act=act, act_param=param)
        z = (a.float() @ b.float().t()) + bias
        ref = fn(z)
        tol = 3e-2
        assert (pre - z).abs().max().item() < tol
        assert (out - ref).abs().max().item() < tol
        assert (ob.float() - ref).abs().max().item() < tol + 2e-2 * ref.abs().max().item()
        assert (otb.float().t() - ref).abs().max().item() < tol + 2e-2 * ref.abs().max().item()
        # backward: v = (a @ b^T) * act'(stored), with the derivative evaluated on the stored tensor
        # exactly as the kernel does (the reference differentiates through the stored activation).
        stored = (pre if act == "gelu" else out).clone()
        if act == "relu":
            deriv = (stored > 0).float()
        elif act == "sigmoid":
            deriv = stored * (1 - stored / param)
        elif act == "tanh":
            deriv = param - stored * stored / param
        else:
            zz = stored.clone().requires_grad_(True)
            fn(zz).backward(torch.ones_like(zz))
            deriv = zz.grad
        dref = (a.float() @ b.float().t()) * deriv
        base = torch.ones(M, N, device="cuda")
        dout = base.clone()
        gemm(a, b, out=dout, aux=stored, dact=act, dact_param=param, beta=2.0)
        assert (dout - (dref + 2.0)).abs().max().item() < 5e-2 * max(1.0, dref.abs().max().item())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape,bn", [((256, 256, 128), 256), ((512, 1024, 512), 256), ((300, 200, 136), 128),
                                      ((1024, 4096, 784), 256), ((129, 257, 72), 128), ((2048, 512, 4096), 0)])
def test_gemm_cta_pairs_k_major(dtype, shape, bn):
    """256-row tiles on CTA pairs (cta_group::2) give the same numbers as the fp32 reference."""
    from oxidized_neural_orchestra_b200.ops.gemm import gemm

    M, N, K = shape
    torch.manual_seed(3)
    ld = lambda n: (n + 15) // 16 * 16
    a = torch.randn(M, ld(K), device="cuda", dtype=dtype)[:, :K]
    b = torch.randn(N, ld(K), device="cuda", dtype=dtype)[:, :K]
    bias = torch.randn(N, device="cuda")
    out = torch.zeros(M, ld(N), device="cuda")[:, :N]
    ob = torch.zeros(M, ld(N), device="cuda", dtype=torch.bfloat16)[:, :N]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    gemm(a, b, out=out, out_bf16=ob, bias=bias, bn=bn, pair=1, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    ref = _ref(a, b, False, False) + bias.double()
    scale = ref.abs().max().item()
    assert (out.double() - ref).abs().max().item() <= _tol(dtype, K) * scale
    assert (ob.double() - ref).abs().max().item() <= 1e-2 * scale


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, False), (True, True)])
def test_gemm_cta_pairs_mn_major_and_split_k(a_mn, b_mn):
    from oxidized_neural_orchestra_b200.ops.gemm import gemm

    M, N, K = 512, 768, 1024
    torch.manual_seed(4)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=torch.bfloat16)
    ref = _ref(a, b, a_mn, b_mn)
    for split in (0, 4):
        out = torch.zeros(M, N, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn, out=out, split_k=split, pair=1, status=status)
        torch.cuda.synchronize()
        assert status.item() == 0
        assert (out.double() - ref).abs().max().item() <= 2e-3 * ref.abs().max().item()


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, False), (True, True)])
@pytest.mark.parametrize("shape", [(128, 128, 64), (256, 320, 200), (512, 1024, 512), (1000, 4096, 1024)])
def test_gemm_tf32_mn_major(a_mn, b_mn, shape):
    """f32 storage with the M / N dimension contiguous (tf32 tiles, 128-byte swizzle on 32-byte units)."""
    from oxidized_neural_orchestra_b200.ops.gemm import gemm

    M, N, K = shape
    torch.manual_seed(5)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda")
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda")
    out = torch.zeros(M, N, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn, out=out, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    ref = _ref(a, b, a_mn, b_mn)
    assert (out.double() - ref).abs().max().item() <= 4e-3 * ref.abs().max().item()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm_reduce_add_output_and_push_add(dtype):
    """The output tile is added into the destination by TMA reductions (the form the weight gradient takes
    when it is pushed into its owner's accumulator)."""
    from oxidized_neural_orchestra_b200.ops.elementwise import push_add
    from oxidized_neural_orchestra_b200.ops.gemm import gemm

    torch.manual_seed(6)
    M, N, K = 384, 520, 200
    a = torch.randn(M, 208, device="cuda", dtype=dtype)[:, :K]
    b = torch.randn(N, 208, device="cuda", dtype=dtype)[:, :K]
    acc = torch.full((M, 528), 1.0, device="cuda")[:, :N]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(3):
        gemm(a, b, out=acc, reduce_out=True, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    ref = 3.0 * _ref(a, b, False, False) + 1.0
    assert (acc.double() - ref).abs().max().item() <= 3 * _tol(dtype, K) * ref.abs().max().item()
    x, y = torch.arange(1000, device="cuda", dtype=torch.float32), torch.ones(1000, device="cuda")
    push_add(x, y)
    assert torch.equal(y, x + 1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(342, 128, 3136), (100, 10, 4096), (1024, 10, 4096), (342, 130, 3140)])
def test_gemm_few_tiles_long_reduction_takes_the_two_pass_split(dtype, shape):
    """Three tiles and 98 k-blocks: the reduction is split over the SMs and a finishing pass applies the whole epilogue."""
    from oxidized_neural_orchestra_b200.ops.gemm import gemm

    M, N, K = shape
    torch.manual_seed(5)
    ld = lambda n: (n + 15) // 16 * 16
    a = (torch.randn(M, ld(K), device="cuda") / 8).to(dtype)[:, :K]
    b = (torch.randn(N, ld(K), device="cuda") / 8).to(dtype)[:, :K]
    bias = torch.randn(N, device="cuda")
    out = torch.full((M, ld(N)), 9.0, device="cuda")[:, :N]
    pre = torch.full((M, ld(N)), 9.0, device="cuda")[:, :N]
    out_t = torch.full((N, ld(M)), 9.0, device="cuda")[:, :M]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(2):      # the scratch accumulator is cleared by every call
        gemm(a, b, out=out, out_t=out_t, pre=pre, bias=bias, act="relu", pair=-1, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    z = a.double() @ b.double().t() + bias.double()
    tol = (4e-3 if dtype == torch.float32 else 2e-3) * z.abs().max().item()
    assert (pre.double() - z).abs().max().item() <= tol
    assert (out.double() - z.clamp_min(0)).abs().max().item() <= tol
    assert (out_t.double() - z.clamp_min(0).t()).abs().max().item() <= tol
    assert bool((out._base[:, N:] == 9.0).all()) and bool((out_t._base[:, M:] == 9.0).all())


def _opt_ref(kind, p, g, m, v, lr, mu, b1, b2, eps, gs, pows):
    g = g * gs
    if kind == "sgd":
        return p - lr * g, m, v
    if kind == "momentum":
        m = mu * m + g
        return p - lr * m, m, v
    m = b1 * m + (1 - b1) * g
    v = b2 * v + (1 - b2) * g * g
    step = lr * (1 - pows[1]) ** 0.5 / (1 - pows[0])
    return p - step * m / (v.sqrt() + eps), m, v


@pytest.mark.parametrize("kind", ["sgd", "momentum", "adam"])
@pytest.mark.parametrize("dtype,pair,bn", [(torch.bfloat16, 1, 0), (torch.bfloat16, 1, 256), (torch.bfloat16, -1, 0), (torch.float32, -1, 0)])
@pytest.mark.parametrize("shape", [(512, 768, 256), (300, 260, 96), (1024, 1000, 512)])
def test_gemm_epilogue_applies_the_optimizer_to_its_own_tile(kind, dtype, pair, bn, shape):
    """Weight-gradient form dW = A^T d with the optimizer in the epilogue: master, state and bf16 shadow are updated in place,
    nothing else is written (the matrices are views into wider buffers whose other columns must stay untouched). bf16 CTA
    pairs with 256-column tiles take the form that moves the master / state / shadow tiles with TMA, the rest the form that
    reads and writes them from registers."""
    from oxidized_neural_orchestra_b200.ops.gemm import gemm

    M, N, K = shape
    torch.manual_seed(7)
    ld = (N + 15) // 16 * 16 + 16
    up = lambda n: (n + 15) // 16 * 16
    a = (torch.randn(K, up(M), device="cuda") / 4).to(dtype)[:, :M]       # MN-major operands, as the engines pass them
    d = (torch.randn(K, up(N), device="cuda") / 4).to(dtype)[:, :N]
    wide = lambda dt=torch.float32: torch.full((M, ld), 3.0, device="cuda", dtype=dt)
    pw, mw, vw, sw = wide(), wide(), wide(), wide(torch.bfloat16)
    p, m, v, sh = pw[:, :N], mw[:, :N], vw[:, :N], sw[:, :N]
    p.copy_(torch.randn(M, N, device="cuda"))
    m.copy_(torch.randn(M, N, device="cuda") * 0.1)
    v.copy_(torch.rand(M, N, device="cuda") * 0.1)
    pows = torch.tensor([0.9 ** 3, 0.999 ** 3], device="cuda")
    p0, m0, v0 = p.double().clone(), m.double().clone(), v.double().clone()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    gemm(a, d, a_mn_major=True, b_mn_major=True, pair=pair, bn=bn, status=status,
         apply=dict(p=p, m=m, v=v, p_bf16=sh, kind=kind, lr=0.05, mu=0.9, b1=0.9, b2=0.999, eps=1e-8, grad_scale=0.25,
                    adam_pows=pows))
    torch.cuda.synchronize()
    assert status.item() == 0
    g = a.double().t() @ d.double()
    rp, rm, rv = _opt_ref(kind, p0, g, m0, v0, 0.05, 0.9, 0.9, 0.999, 1e-8, 0.25, pows.double().tolist())
    gtol = (4e-3 if dtype == torch.float32 else 2e-3) * g.abs().max().item()
    # Adam normalises the step: an error of gtol in g moves p by at most ~lr * gtol / sqrt(v)
    ptol = 0.05 * gtol * (40 if kind == "adam" else 1.5) + 1e-6
    assert (p.double() - rp).abs().max().item() <= ptol
    if kind != "sgd":
        assert (m.double() - rm).abs().max().item() <= gtol
    else:
        assert torch.equal(m.double(), m0)
    if kind == "adam":
        assert (v.double() - rv).abs().max().item() <= 2 * gtol * g.abs().max().item()
    else:
        assert torch.equal(v.double(), v0)
    assert (sh.float() - p).abs().max().item() <= 2 ** -8 * p.abs().max().item()
    for w in (pw, mw, vw):
        assert bool((w[:, N:] == 3.0).all())
    assert bool((sw[:, N:] == 3.0).all())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("fmt", ["bf16", "f16"])
@pytest.mark.parametrize("shape", [(256, 512, 128), (384, 264, 200), (130, 72, 64)])
def test_gemm_sixteen_bit_wire_output(dtype, fmt, shape):
    """The 16-bit output in both wire formats, through TMA stores (aligned rows) and thread stores (the rest)."""
    from oxidized_neural_orchestra_b200.ops.gemm import gemm

    M, N, K = shape
    torch.manual_seed(8)
    up = lambda n: (n + 15) // 16 * 16
    a = (torch.randn(K, up(M), device="cuda") / 4).to(dtype)[:, :M]
    b = (torch.randn(K, up(N), device="cuda") / 4).to(dtype)[:, :N]
    odt = torch.float16 if fmt == "f16" else torch.bfloat16
    wide = torch.full((M, N + 24), 5.0, device="cuda", dtype=odt)
    out = wide[:, :N]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    gemm(a, b, a_mn_major=True, b_mn_major=True, status=status, **{"out_f16" if fmt == "f16" else "out_bf16": out})
    torch.cuda.synchronize()
    assert status.item() == 0
    ref = a.double().t() @ b.double()
    tol = (2 ** -10 if fmt == "f16" else 2 ** -7) * ref.abs().max().item() + 4e-3 * ref.abs().max().item()
    assert (out.double() - ref).abs().max().item() <= tol
    assert bool((wide[:, N:] == 5.0).all())


@pytest.mark.parametrize("shape,split,pair", [((64, 576, 8192), 37, -1), ((342, 128, 3136), 0, -1), ((512, 768, 2048), 4, 1)])
def test_split_k_repeats_bit_for_bit_and_is_safe_on_two_streams(shape, split, pair):
    """Every split writes its own slab and the finishing pass adds the slabs in order: two runs give the same bits, and two
    such GEMMs on two streams (each with its own workspace) do not disturb one another."""
    from oxidized_neural_orchestra_b200.ops.gemm import gemm

    M, N, K = shape
    torch.manual_seed(9)
    up = lambda n: (n + 15) // 16 * 16
    a = torch.randn(K, up(M), device="cuda", dtype=torch.bfloat16)[:, :M]
    b = torch.randn(K, up(N), device="cuda", dtype=torch.bfloat16)[:, :N]
    a2 = torch.randn(K, up(M), device="cuda", dtype=torch.bfloat16)[:, :M]
    ref, ref2 = a.double().t() @ b.double(), a2.double().t() @ b.double()
    outs = []
    for _ in range(3):
        out = torch.full((M, N), 7.0, device="cuda")
        gemm(a, b, a_mn_major=True, b_mn_major=True, out=out, split_k=split, pair=pair)
        outs.append(out)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    assert (outs[0].double() - ref).abs().max().item() <= 2e-3 * ref.abs().max().item()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    o1 = [torch.empty(M, N, device="cuda") for _ in range(8)]
    o2 = [torch.empty(M, N, device="cuda") for _ in range(8)]
    for i in range(8):
        with torch.cuda.stream(s1):
            gemm(a, b, a_mn_major=True, b_mn_major=True, out=o1[i], split_k=split, pair=pair, stream=s1)
        with torch.cuda.stream(s2):
            gemm(a2, b, a_mn_major=True, b_mn_major=True, out=o2[i], split_k=split, pair=pair, stream=s2)
    torch.cuda.synchronize()
    for i in range(8):
        assert torch.equal(o1[i], outs[0])
        assert (o2[i].double() - ref2).abs().max().item() <= 2e-3 * ref2.abs().max().item()
        assert torch.equal(o2[i], o2[0])
