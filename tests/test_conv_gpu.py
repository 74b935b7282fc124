"""Convolution / pooling on the GPU engine against PyTorch autograd (NCHW, fp32) and the CPU oracle."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

LAYERS = [
    dict(kind="conv", input_dim=[1, 12, 12], kernel_dim=[8, 1, 3], stride=1, padding=1, act=("relu", 0.0)),
    dict(kind="pool", input_dim=[8, 12, 12], filter_size=2, stride=2, padding=0, act=None),
    dict(kind="conv", input_dim=[8, 6, 6], kernel_dim=[16, 8, 3], stride=2, padding=1, act=("tanh", 1.0)),
    dict(kind="dense", **{"in": 16 * 3 * 3, "out": 32}, act=("sigmoid", 1.0)),
    dict(kind="dense", **{"in": 32, "out": 10}, act=("softmax", 0.0)),
]


def _torch_ref(params, x, y):
    off = 0
    ps = []

    def take(shape):
        nonlocal off
        n = int(np.prod(shape))
        t = params[off:off + n].view(*shape).clone().requires_grad_(True)
        off += n
        ps.append(t)
        return t

    B = x.shape[0]
    a = x.view(B, 1, 12, 12)
    k1, b1 = take((8, 1, 3, 3)), take((8,))
    a = torch.relu(F.conv2d(a, k1, b1, stride=1, padding=1))
    a = F.max_pool2d(a, 2, 2)
    k2, b2 = take((16, 8, 3, 3)), take((16,))
    a = torch.tanh(F.conv2d(a, k2, b2, stride=2, padding=1))
    a = a.reshape(B, -1)                      # NCHW flatten, the reference's order
    w3, b3 = take((144, 32)), take((32,))
    a = torch.sigmoid(a @ w3 + b3)
    w4, b4 = take((32, 10)), take((10,))
    p = torch.softmax(a @ w4 + b4, 1)
    L = -(y * torch.log(p.clamp_min(1.1920929e-07))).sum() / p.numel()
    L.backward()
    return L.item(), torch.cat([t.grad.reshape(-1) for t in ps])


@pytest.mark.parametrize("tile", ["tf32", "bf16"])
def test_conv_engine_grads_match_autograd(tile):
    from oxidized_neural_orchestra_b200.models.conv_engine import ConvNetEngine

    torch.manual_seed(0)
    n = 8 * 9 + 8 + 16 * 72 + 16 + 145 * 32 + 33 * 10
    npad = (n + 15) // 16 * 16
    params = torch.zeros(npad, device="cuda")
    params[:n] = torch.randn(n, device="cuda") * 0.2
    grads = torch.zeros(npad, device="cuda")
    pb = params.to(torch.bfloat16) if tile == "bf16" else None
    B = 24
    eng = ConvNetEngine(LAYERS, batch_size=B, tile_dtype=tile, loss="cross_entropy", params=params, grads=grads,
                        params_bf16=pb)
    eng.refresh()
    x = torch.rand(B, 144, device="cuda") + 0.05   # positive inputs: zero padding never wins the max
    y = F.one_hot(torch.randint(0, 10, (B,), device="cuda"), 10).float()
    eng.step(x, y, B)
    torch.cuda.synchronize()
    assert eng.status.item() == 0
    pref = pb.float() if tile == "bf16" else params
    xr = x.to(torch.bfloat16).float() if tile == "bf16" else x
    ref_loss, ref_g = _torch_ref(pref[:n], xr, y)
    tol = 6e-2 if tile == "bf16" else 2e-2
    assert abs(eng.loss_sum.item() - ref_loss) <= tol * abs(ref_loss)
    err = (grads[:n] - ref_g).abs().max().item()
    assert err <= tol * ref_g.abs().max().item(), (err, ref_g.abs().max().item())
    # ragged batch + accumulation into the same gradient buffer
    if tile == "tf32":
        grads.zero_()
        eng.step(x[:10].contiguous(), y[:10].contiguous(), 10)
        eng.step(x[10:].contiguous(), y[10:].contiguous(), 14, accumulate=True)
        torch.cuda.synchronize()
        _, g1 = _torch_ref(params[:n], x[:10], y[:10])
        _, g2 = _torch_ref(params[:n], x[10:], y[10:])
        assert (grads[:n] - (g1 + g2)).abs().max().item() <= tol * (g1 + g2).abs().max().item()


def test_cnn_through_the_api_tracks_the_oracle():
    import orchestra
    from orchestra import Sequential, orchestrate
    from orchestra.activations import ReLU, Softmax
    from orchestra.arch import Conv2d, Dense, MaxPooling
    from orchestra.datasets import InlineDataset
    from orchestra.initialization import Kaiming
    from orchestra.loss_fns import CrossEntropy
    from orchestra.optimizers import GradientDescentWithMomentum

    rng = np.random.default_rng(0)
    xs = rng.random((32, 64), dtype=np.float32) + 0.05
    ys = np.eye(4, dtype=np.float32)[rng.integers(0, 4, 32)]
    model = Sequential([Conv2d((1, 8, 8), (6, 1, 3), 1, 1, Kaiming(), ReLU(0.0)), MaxPooling((6, 8, 8), 2, 2, 0),
                        Conv2d((6, 4, 4), (8, 6, 3), 1, 0, Kaiming(), ReLU(0.0)), Dense(4, Kaiming(), Softmax())])
    out = {}
    for dev in ("cpu", "gpu"):
        tr = orchestra.all_reduce([f"{dev}:0"], InlineDataset(xs, ys, 64, 4), GradientDescentWithMomentum(0.2, 0.9),
                                  CrossEntropy(), max_epochs=10, batch_size=32, seed=3)
        m = orchestrate(model, tr).wait(quiet=True)
        out[dev] = (np.array(m.loss_history()), m.weights_array())
    (lc, wc), (lg, wg) = out["cpu"], out["gpu"]
    assert lg[-1] < lg[0]
    assert np.allclose(lc, lg, rtol=5e-2, atol=1e-5)
    assert np.abs(wc - wg).max() < 5e-2 * max(1.0, np.abs(wc).max())


def test_single_channel_first_layer_uses_direct_kernels_and_tracks_the_oracle():
    """LeNet-style front: 5x5 convolution on one input channel (direct CUDA-core kernels), pooling, dense."""
    import orchestra
    from orchestra import Sequential, orchestrate
    from orchestra.activations import Softmax, Tanh
    from orchestra.arch import Conv2d, Dense, MaxPooling
    from orchestra.datasets import InlineDataset
    from orchestra.initialization import Xavier
    from orchestra.loss_fns import CrossEntropy
    from orchestra.optimizers import GradientDescent

    rng = np.random.default_rng(1)
    xs = rng.random((48, 144), dtype=np.float32)
    ys = np.eye(5, dtype=np.float32)[rng.integers(0, 5, 48)]
    model = Sequential([Conv2d((1, 12, 12), (6, 1, 5), 1, 2, Xavier(), Tanh()), MaxPooling((6, 12, 12), 2, 2, 0),
                        Dense(5, Xavier(), Softmax())])
    out = {}
    for dev in ("cpu", "gpu"):
        tr = orchestra.all_reduce([f"{dev}:0"], InlineDataset(xs, ys, 144, 5), GradientDescent(0.5), CrossEntropy(),
                                  max_epochs=8, batch_size=16, seed=5)
        m = orchestrate(model, tr).wait(quiet=True)
        out[dev] = (np.array(m.loss_history()), m.weights_array())
    (lc, wc), (lg, wg) = out["cpu"], out["gpu"]
    assert lg[-1] < lg[0]
    assert np.allclose(lc, lg, rtol=5e-2, atol=1e-5)
    assert np.abs(wc - wg).max() < 5e-2 * max(1.0, np.abs(wc).max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(5, 28, 28, 3, 1, 1, 32), (7, 28, 28, 3, 2, 1, 40), (3, 28, 28, 5, 1, 0, 6),
                                   (4, 12, 17, 5, 2, 2, 33), (3, 9, 9, 2, 1, 0, 8), (2, 120, 120, 3, 1, 1, 16)])
def test_direct_single_channel_kernels_match_conv2d(dtype, shape):
    """Image-tiled kernels (k = 3, 5; image fits shared memory) and the generic ones (k = 2; 120 x 120) against PyTorch."""
    from oxidized_neural_orchestra_b200.ops import conv as CV

    B, H, W, K, S, P, Fo = shape
    torch.manual_seed(3)
    g = CV.geom(B, 1, H, W, K, S, P)
    x = torch.randn(B * H * W, 4, device="cuda").to(dtype)[:, :1]          # pixel-major, one channel, padded rows
    kp = torch.randn(Fo, K, K, device="cuda") * 0.3
    bias = torch.randn(Fo, device="cuda")
    rows = B * g.OH * g.OW
    y = torch.full((rows, Fo + 8), 7.0, device="cuda", dtype=dtype)[:, :Fo]
    CV.conv1_fwd(g, Fo, x, kp, bias, y, act="tanh", act_param=1.0)
    xi = x.double().reshape(B, 1, H, W)       # float64 reference: cuDNN's fp32 convolutions may run on tf32
    ref = torch.tanh(F.conv2d(xi, kp.double().view(Fo, 1, K, K), bias.double(), stride=S, padding=P))
    ref_rows = ref.permute(0, 2, 3, 1).reshape(rows, Fo)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    assert (y.float() - ref_rows).abs().max().item() <= tol
    assert bool((y._base[:, Fo:] == 7.0).all())
    dy = (torch.randn(rows, Fo + 8, device="cuda") * 0.1).to(dtype)[:, :Fo]
    gk, gb = torch.full((Fo, K, K), 3.0, device="cuda"), torch.full((Fo,), 3.0, device="cuda")
    CV.conv1_wgrad(g, Fo, x, dy, gk, gb, beta=0.0)
    again_k, again_b = torch.empty_like(gk), torch.empty_like(gb)
    CV.conv1_wgrad(g, Fo, x, dy, again_k, again_b, beta=0.0)
    kr = kp.double().view(Fo, 1, K, K).requires_grad_(True)
    br = bias.double().requires_grad_(True)
    out = F.conv2d(xi, kr, br, stride=S, padding=P)
    out.backward(dy.double().reshape(B, g.OH, g.OW, Fo).permute(0, 3, 1, 2))
    scale = max(1.0, kr.grad.abs().max().item())
    wtol = (3e-2 if dtype == torch.bfloat16 else 2e-4) * scale
    assert (gk - kr.grad.view(Fo, K, K)).abs().max().item() <= wtol
    assert (gb - br.grad).abs().max().item() <= wtol * 4
    assert torch.equal(gk, again_k) and torch.equal(gb, again_b)      # fixed summation order
    CV.conv1_wgrad(g, Fo, x, dy, gk, gb, beta=1.0)                     # accumulate
    assert (gk - 2 * kr.grad.view(Fo, K, K)).abs().max().item() <= 2 * wtol


STAGED = [
    dict(kind="dense", **{"in": 40, "out": 2 * 6 * 6}, act=("tanh", 1.0)),
    dict(kind="conv", input_dim=[2, 6, 6], kernel_dim=[4, 2, 3], stride=1, padding=1, act=("relu", 0.0)),
    dict(kind="pool", input_dim=[4, 6, 6], filter_size=2, stride=2, padding=0, act=None),
    dict(kind="dense", **{"in": 4 * 3 * 3, "out": 18}, act=("sigmoid", 1.0)),
    dict(kind="pool", input_dim=[2, 3, 3], filter_size=3, stride=1, padding=1, act=None),
    dict(kind="conv", input_dim=[2, 3, 3], kernel_dim=[3, 2, 2], stride=1, padding=0, act=("tanh", 1.0)),
    dict(kind="dense", **{"in": 3 * 2 * 2, "out": 5}, act=("softmax", 0.0)),
]


def _staged_ref(params, x, y):
    off, ps = 0, []

    def take(shape):
        nonlocal off
        n = int(np.prod(shape))
        t = params[off:off + n].view(*shape).clone().requires_grad_(True)
        off += n
        ps.append(t)
        return t

    B = x.shape[0]
    w, b = take((40, 72)), take((72,))
    a = torch.tanh(x @ w + b).view(B, 2, 6, 6)
    k, b = take((4, 2, 3, 3)), take((4,))
    a = F.max_pool2d(torch.relu(F.conv2d(a, k, b, padding=1)), 2, 2).reshape(B, -1)
    w, b = take((36, 18)), take((18,))
    a = torch.sigmoid(a @ w + b).view(B, 2, 3, 3)
    a = F.max_pool2d(F.pad(a, (1, 1, 1, 1)), 3, 1)          # zero padding takes part in the max (max_pooling.rs:47-157)
    k, b = take((3, 2, 2, 2)), take((3,))
    a = torch.tanh(F.conv2d(a, k, b)).reshape(B, -1)
    w, b = take((12, 5)), take((5,))
    p = torch.softmax(a @ w + b, 1)
    L = -(y * torch.log(p.clamp_min(1.1920929e-07))).sum() / p.numel()
    L.backward()
    return L.item(), torch.cat([t.grad.reshape(-1) for t in ps])


@pytest.mark.parametrize("tile", ["tf32", "bf16"])
def test_layer_kinds_in_any_order_dense_before_conv_and_several_alternations(tile):
    """dense -> conv -> pool -> dense -> pool -> conv -> dense: the chained-unit engine against autograd."""
    from oxidized_neural_orchestra_b200.models.conv_engine import StagedEngine, make_engine

    torch.manual_seed(1)
    n = 41 * 72 + (4 * 18 + 4) + 37 * 18 + (3 * 8 + 3) + 13 * 5
    npad = (n + 15) // 16 * 16
    params = torch.zeros(npad, device="cuda")
    params[:n] = torch.randn(n, device="cuda") * 0.3
    grads = torch.zeros(npad, device="cuda")
    pb = params.to(torch.bfloat16) if tile == "bf16" else None
    B = 20
    eng = make_engine(STAGED, batch_size=B, tile_dtype=tile, loss="cross_entropy", params=params, grads=grads, params_bf16=pb)
    assert isinstance(eng, StagedEngine) and eng.n_params == n
    eng.refresh()
    x = torch.rand(B, 40, device="cuda")
    y = F.one_hot(torch.randint(0, 5, (B,), device="cuda"), 5).float()
    eng.step(x, y, B)
    torch.cuda.synchronize()
    assert eng.status.item() == 0
    pref = pb.float() if tile == "bf16" else params
    ref_loss, ref_g = _staged_ref(pref[:n], x.to(torch.bfloat16).float() if tile == "bf16" else x, y)
    tol = 8e-2 if tile == "bf16" else 2e-2
    assert abs(eng.loss_sum.item() - ref_loss) <= tol * abs(ref_loss)
    err = (grads[:n] - ref_g).abs().max().item()
    assert err <= tol * ref_g.abs().max().item(), (err, ref_g.abs().max().item())
