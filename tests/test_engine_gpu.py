"""The GPU engine's loss and flat gradients against PyTorch autograd (fp32) on the same network."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _torch_ref(layers, params, x, y, loss):
    """Reference forward/backward with the reference's conventions (loss normalised by B*C)."""
    off = 0
    ws = []
    a = x
    for sp in layers:
        i, o = sp["in"], sp["out"]
        W = params[off:off + i * o].view(i, o).clone().requires_grad_(True)
        b = params[off + i * o:off + (i + 1) * o].clone().requires_grad_(True)
        off += (i + 1) * o
        ws += [W, b]
        z = a @ W + b
        act = sp.get("act")
        if act is None:
            a = z
        elif act[0] == "relu":
            a = torch.where(z > 0, z, act[1] * z)
        elif act[0] == "sigmoid":
            a = act[1] * torch.sigmoid(z)
        elif act[0] == "tanh":
            a = act[1] * torch.tanh(z)
        elif act[0] == "gelu":
            a = torch.nn.functional.gelu(z)
        elif act[0] == "softmax":
            a = torch.softmax(z, dim=1)
    n = a.numel()
    if loss == "cross_entropy":
        L = -(y * torch.log(a.clamp_min(1.1920929e-07))).sum() / n
    else:
        L = ((a - y) ** 2).sum() / n
    L.backward()
    return L.item(), torch.cat([w.grad.reshape(-1) for w in ws])


CASES = [
    ([dict(kind="dense", **{"in": 784, "out": 128}, act=("relu", 0.0)),
      dict(kind="dense", **{"in": 128, "out": 10}, act=("softmax", 0.0))], "cross_entropy", 32),
    ([dict(kind="dense", **{"in": 100, "out": 72}, act=("tanh", 1.7)),
      dict(kind="dense", **{"in": 72, "out": 40}, act=("sigmoid", 1.0)),
      dict(kind="dense", **{"in": 40, "out": 6}, act=("sigmoid", 1.0))], "mse", 50),
    ([dict(kind="dense", **{"in": 256, "out": 512}, act=("gelu", 0.0)),
      dict(kind="dense", **{"in": 512, "out": 256}, act=("relu", 0.1)),
      dict(kind="dense", **{"in": 256, "out": 16}, act=("softmax", 0.0))], "cross_entropy", 200),
    # softmax as an inner layer's activation (arch/layers/softmax.rs:24-64 allows it anywhere), first and middle layer
    ([dict(kind="dense", **{"in": 64, "out": 48}, act=("softmax", 0.0)),
      dict(kind="dense", **{"in": 48, "out": 40}, act=("tanh", 1.0)),
      dict(kind="dense", **{"in": 40, "out": 24}, act=("softmax", 0.0)),
      dict(kind="dense", **{"in": 24, "out": 8}, act=("softmax", 0.0))], "cross_entropy", 96),
    ([dict(kind="dense", **{"in": 30, "out": 20}, act=("relu", 0.0)),
      dict(kind="dense", **{"in": 20, "out": 12}, act=("softmax", 0.0)),
      dict(kind="dense", **{"in": 12, "out": 5}, act=None)], "mse", 40),
]


@pytest.mark.parametrize("tile", ["tf32", "bf16"])
@pytest.mark.parametrize("case", range(len(CASES)))
def test_engine_grads_match_autograd(tile, case):
    from oxidized_neural_orchestra_b200.models.engine import GpuEngine

    layers, loss, B = CASES[case]
    torch.manual_seed(case)
    n = sum((sp["in"] + 1) * sp["out"] for sp in layers)
    n_pad = (n + 15) // 16 * 16
    params = torch.zeros(n_pad, device="cuda")
    params[:n] = torch.randn(n, device="cuda") * 0.1
    grads = torch.zeros(n_pad, device="cuda")
    pb = params.to(torch.bfloat16) if tile == "bf16" else None
    eng = GpuEngine(layers, batch_size=B, tile_dtype=tile, loss=loss, params=params, grads=grads, params_bf16=pb)
    eng.refresh()
    x = torch.rand(B, layers[0]["in"], device="cuda")
    C = layers[-1]["out"]
    y = torch.nn.functional.one_hot(torch.randint(0, C, (B,), device="cuda"), C).float()
    eng.step(x, y, B)
    torch.cuda.synchronize()
    assert eng.status.item() == 0
    pref = pb.float() if tile == "bf16" else params
    ref_loss, ref_g = _torch_ref(layers, pref[:n], x.to(torch.bfloat16).float() if tile == "bf16" else x, y, loss)
    tol = 3e-2 if tile == "bf16" else 2e-2  # tf32 truncates to 10 mantissa bits per operand, chained over layers
    assert abs(eng.loss_sum.item() - ref_loss) <= tol * max(1e-3, abs(ref_loss))
    g = grads[:n]
    err = (g - ref_g).abs().max().item()
    assert err <= tol * ref_g.abs().max().item(), (err, ref_g.abs().max().item())


def test_engine_ragged_batch_and_accumulate():
    from oxidized_neural_orchestra_b200.models.engine import GpuEngine

    layers, loss, B = CASES[0]
    torch.manual_seed(7)
    n = sum((sp["in"] + 1) * sp["out"] for sp in layers)
    params = torch.randn((n + 15) // 16 * 16, device="cuda") * 0.1
    grads = torch.zeros_like(params)
    eng = GpuEngine(layers, batch_size=B, tile_dtype="tf32", loss=loss, params=params, grads=grads)
    eng.refresh()
    x = torch.rand(B, 784, device="cuda")
    y = torch.nn.functional.one_hot(torch.randint(0, 10, (B,), device="cuda"), 10).float()
    eng.step(x, y, 20)                       # ragged: 20 of 32 rows
    eng.step(x[20:].contiguous(), y[20:].contiguous(), 12, accumulate=True)
    torch.cuda.synchronize()
    _, g1 = _torch_ref(layers, params[:n], x[:20], y[:20], loss)
    _, g2 = _torch_ref(layers, params[:n], x[20:], y[20:], loss)
    ref = g1 + g2
    assert (grads[:n] - ref).abs().max().item() <= 5e-3 * ref.abs().max().item()
