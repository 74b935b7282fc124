"""The CPU oracle engine against PyTorch (CPU autograd) and the reference's documented quirks.

Layer cases mirror machine_learning/src/arch/layers/{dense.rs:121-198, conv/test_conv2d.rs,
max_pooling.rs:160-392}; convergence cases mirror machine_learning/src/test/test_sequential_*.rs.
"""
import json
import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from orchestra import _orchestra as core


def _spec(kind, **kw):
    return {kind: kw}


def _run(layers, x_size, params, x, d_out):
    seq = core.Sequential(json.dumps(layers), x_size)
    B = x.shape[0]
    y = seq.forward(params, x.reshape(-1), B)
    g = seq.backward(params, d_out.reshape(-1), B)
    return y.reshape(B, -1), g


def test_dense_forward_backward_hand_computed():
    # W[in,out] row-major then b (dense.rs:75-91)
    params = np.array([1, 2, 3, 4, 5, 6, 0.5, -0.5], dtype=np.float32)  # W = [[1,2],[3,4],[5,6]], b = [.5,-.5]
    x = np.array([[1, 0, -1], [2, 1, 0]], dtype=np.float32)
    d = np.array([[1, 0], [0.5, 2]], dtype=np.float32)
    y, g = _run([_spec("dense", dim=[3, 2], act_fn=None)], 3, params, x, d)
    assert y.tolist() == [[-3.5, -4.5], [5.5, 7.5]]
    dW = x.T @ d
    assert g[:6].reshape(3, 2).tolist() == dW.tolist() and g[6:].tolist() == [1.5, 2.0]


@pytest.mark.parametrize("cfg", [
    dict(c=1, h=5, w=5, f=2, k=3, s=1, p=0), dict(c=2, h=6, w=7, f=3, k=3, s=2, p=1),
    dict(c=3, h=8, w=8, f=4, k=2, s=3, p=0),  # stride that drops the trailing rows/cols (test_conv2d.rs:300-352)
    dict(c=1, h=28, w=28, f=4, k=5, s=1, p=2),
])
def test_conv2d_matches_torch(cfg):
    c, h, w, f, k, s, p = (cfg[n] for n in "chwfksp")
    rng = np.random.default_rng(1)
    B = 3
    K = rng.standard_normal((f, c, k, k)).astype(np.float32)
    b = rng.standard_normal(f).astype(np.float32)
    x = rng.standard_normal((B, c, h, w)).astype(np.float32)
    layers = [_spec("conv", input_dim=[c, h, w], kernel_dim=[f, c, k], stride=s, padding=p, act_fn={"tanh": {"amp": 1.5}})]
    xt = torch.tensor(x, requires_grad=True)
    Kt, bt = torch.tensor(K, requires_grad=True), torch.tensor(b, requires_grad=True)
    yt = 1.5 * torch.tanh(F.conv2d(xt, Kt, bt, stride=s, padding=p))
    d = rng.standard_normal(tuple(yt.shape)).astype(np.float32)
    yt.backward(torch.tensor(d))
    y, g = _run(layers, c * h * w, np.concatenate([K.reshape(-1), b]), x.reshape(B, -1), d.reshape(B, -1))
    assert np.allclose(y, yt.detach().numpy().reshape(B, -1), atol=1e-4)
    assert np.allclose(g[:K.size], Kt.grad.numpy().reshape(-1), atol=1e-3)
    assert np.allclose(g[K.size:], bt.grad.numpy(), atol=1e-3)


def test_max_pool_zero_padding_competes_and_routes_gradient():
    # all-negative input: the zero padding wins the max and the gradient there is dropped
    x = -np.ones((1, 1, 2, 2), dtype=np.float32)
    layers = [_spec("max_pooling", input_dim=[1, 2, 2], filter_size=2, stride=2, padding=1, act_fn=None)]
    seq = core.Sequential(json.dumps(layers), 4)
    y = seq.forward(np.zeros(0, dtype=np.float32), x.reshape(-1), 1)
    assert y.tolist() == [0.0, 0.0, 0.0, 0.0]  # max_pooling.rs:68-82
    # positive input: matches torch (which pads with -inf) and routes d to the arg-max
    rng = np.random.default_rng(2)
    x = rng.random((2, 3, 6, 6)).astype(np.float32) + 0.1
    layers = [_spec("max_pooling", input_dim=[3, 6, 6], filter_size=3, stride=2, padding=1, act_fn=None)]
    seq = core.Sequential(json.dumps(layers), 108)
    y = seq.forward(np.zeros(0, dtype=np.float32), x.reshape(-1), 2)
    xt = torch.tensor(x, requires_grad=True)
    yt = F.max_pool2d(xt, 3, 2, 1)
    assert np.allclose(y.reshape(yt.shape), yt.detach().numpy())


def test_softmax_cross_entropy_composition_and_loss_scale():
    rng = np.random.default_rng(3)
    B, C = 5, 7
    z = rng.standard_normal((B, C)).astype(np.float32)
    yl = np.eye(C, dtype=np.float32)[rng.integers(0, C, B)]
    p = torch.softmax(torch.tensor(z), 1).numpy()
    loss, delta = core.loss_prime("cross_entropy", p.reshape(-1), yl.reshape(-1))
    # n = B*C normalises loss and gradient (cross_entropy.rs:35-47): 1/C of the textbook mean
    assert loss == pytest.approx(float(F.cross_entropy(torch.tensor(z), torch.tensor(yl.argmax(1))) / C), rel=1e-5)
    layers = [_spec("dense", dim=[C, C], act_fn="softmax")]
    params = np.concatenate([np.eye(C, dtype=np.float32).reshape(-1), np.zeros(C, dtype=np.float32)])
    seq = core.Sequential(json.dumps(layers), C)
    out = seq.forward(params, z.reshape(-1), B)
    assert np.allclose(out.reshape(B, C), p, atol=1e-6)
    g = seq.backward(params, delta, B)
    # dz = (p - y)/n for one-hot labels; db = column sums
    assert np.allclose(g[C * C:], ((p - yl) / (B * C)).sum(0), atol=1e-6)
    loss, delta = core.loss_prime("mse", p.reshape(-1), yl.reshape(-1))
    assert loss == pytest.approx(float(((p - yl) ** 2).mean()), rel=1e-5)
    assert np.allclose(delta.reshape(B, C), 2 * (p - yl) / (B * C), atol=1e-7)


def test_leaky_relu_backward_quirk_and_exact():
    layers = [_spec("dense", dim=[1, 1], act_fn={"relu": {"slope": 0.1}})]
    params = np.array([1.0, 0.0], dtype=np.float32)
    x = np.array([[-2.0]], dtype=np.float32)
    d = np.array([[3.0]], dtype=np.float32)
    exact = core.Sequential(json.dumps(layers), 1, True)
    exact.forward(params, x.reshape(-1), 1)
    assert exact.backward(params, d.reshape(-1), 1)[1] == pytest.approx(0.3)      # slope * d
    quirk = core.Sequential(json.dumps(layers), 1, False)
    a = quirk.forward(params, x.reshape(-1), 1)
    assert quirk.backward(params, d.reshape(-1), 1)[1] == pytest.approx(0.1 * a[0])  # relu.rs:41-45: slope * a


def test_adam_formula_eps_outside_bias_correction():
    spec = json.dumps({"adam": {"learning_rate": 0.1, "beta1": 0.9, "beta2": 0.999, "epsilon": 1e-8}})
    opt = core.Optimizer(spec, 2)
    p = np.array([1.0, -1.0], dtype=np.float32)
    g = np.array([0.5, -2.0], dtype=np.float32)
    m = v = np.zeros(2)
    b1t = b2t = 1.0
    ref = p.astype(np.float64)
    for _ in range(3):
        p = opt.step(p, g)
        b1t *= 0.9
        b2t *= 0.999
        m = 0.9 * m + 0.1 * g
        v = 0.999 * v + 0.001 * g * g
        ref = ref - 0.1 * math.sqrt(1 - b2t) / (1 - b1t) * m / (np.sqrt(v) + 1e-8)  # adam.rs:75-91
    assert np.allclose(p, ref, atol=1e-6)


def test_param_gen_is_seeded_shard_independent_and_scaled():
    spec = {"rand": {"distribution": {"xavier_uniform": {"fan_in": 784, "fan_out": 128}}, "limit": 100480, "index_offset": 0}}
    a = core.param_gen_fill(json.dumps(spec), 0)
    lim = math.sqrt(6.0 / (784 + 128))
    assert a.shape == (100480,) and np.abs(a).max() <= lim and a.std() == pytest.approx(lim / math.sqrt(3), rel=0.02)
    part = dict(spec)
    part["rand"] = dict(spec["rand"], limit=50, index_offset=1000)
    assert np.array_equal(core.param_gen_fill(json.dumps(part), 0), a[1000:1050])
    assert not np.array_equal(core.param_gen_fill(json.dumps(spec), 1), a)
    k = core.param_gen_fill(json.dumps({"rand": {"distribution": {"kaiming": {"fan_in": 50}}, "limit": 200000, "index_offset": 0}}), 3)
    assert k.std() == pytest.approx(math.sqrt(2 / 50), rel=0.02) and abs(k.mean()) < 0.01
    chained = {"chained": {"specs": [{"const": {"value": 2.0, "limit": 3}}, {"inline": {"params": [1.0, 5.0]}}]}}
    assert core.param_gen_fill(json.dumps(chained), 0).tolist() == [2.0, 2.0, 2.0, 1.0, 5.0]


def _trainer_spec(layers, x, y, loss, opt, batch, epochs, offline=0):
    return {"layers": layers, "optimizer": opt, "dataset": {"x_size": x, "y_size": y}, "loss_fn": loss,
            "offline_epochs": offline, "max_epochs": epochs, "batch_size": batch, "seed": 5}


def test_round_trainer_semantics_and_xor_convergence():
    xs = np.array([0, 0, 0, 1, 1, 0, 1, 1], dtype=np.float32)
    ys = np.array([0, 1, 1, 0], dtype=np.float32)
    layers = [_spec("dense", dim=[2, 8], act_fn={"tanh": {"amp": 1.0}}), _spec("dense", dim=[8, 1], act_fn={"sigmoid": {"amp": 1.0}})]
    spec = _trainer_spec(layers, 2, 1, "mse", {"gradient_descent": {"learning_rate": 0.5}}, 3, 5, offline=1)
    tr = core.RoundTrainer(json.dumps(spec), xs, ys)
    rng = np.random.default_rng(0)
    p0 = rng.standard_normal(tr.n_params).astype(np.float32) * 0.5
    p, r, losses, last = tr.train(p0, np.zeros_like(p0))
    # a round = offline_epochs + 1 epochs, 2 batches each (3 + ragged 1); local SGD: p = p0 - lr * residual
    assert len(losses) == 2 and not last and tr.epochs_done == 2
    assert np.allclose(p, p0 - 0.5 * r, atol=1e-5)
    p, r, losses, last = tr.train(p, r)
    p, r, losses, last = tr.train(p, r)
    assert len(losses) == 1 and last and tr.epochs_done == 5  # min(remaining, offline + 1)
    # convergence (test_sequential_dense.rs: loss < 0.01)
    spec = _trainer_spec(layers, 2, 1, "mse", {"gradient_descent": {"learning_rate": 1.0}}, 4, 4000)
    tr = core.RoundTrainer(json.dumps(spec), xs, ys)
    p, r = p0, np.zeros_like(p0)
    loss = 1.0
    for _ in range(4000):
        p, r, losses, last = tr.train(p, r)
        loss = losses[-1]
        if loss < 0.01:
            break
    assert loss < 0.01


def test_conv_pool_dense_network_learns_symbols():
    # 3x3 symbol classification with conv + max-pool + dense + softmax (test_sequential_conv_dense.rs)
    syms = np.array([[1, 0, 1, 0, 1, 0, 1, 0, 1], [0, 1, 0, 1, 1, 1, 0, 1, 0], [1, 1, 1, 1, 0, 1, 1, 1, 1]], dtype=np.float32)
    xs = np.tile(syms, (4, 1)).reshape(-1)
    ys = np.tile(np.eye(3, dtype=np.float32), (4, 1)).reshape(-1)
    layers = [_spec("conv", input_dim=[1, 3, 3], kernel_dim=[4, 1, 2], stride=1, padding=1, act_fn={"relu": {"slope": 0.0}}),
              _spec("max_pooling", input_dim=[4, 4, 4], filter_size=2, stride=2, padding=0, act_fn=None),
              _spec("dense", dim=[16, 3], act_fn="softmax")]
    spec = _trainer_spec(layers, 9, 3, "cross_entropy", {"gradient_descent": {"learning_rate": 0.5}}, 6, 3000)
    tr = core.RoundTrainer(json.dumps(spec), xs, ys)
    rng = np.random.default_rng(4)
    p = rng.standard_normal(tr.n_params).astype(np.float32) * 0.3
    r = np.zeros_like(p)
    for _ in range(3000):
        p, r, losses, last = tr.train(p, r)
        if losses[-1] < 0.01:
            break
    assert losses[-1] < 0.01
    loss, acc = tr.evaluate(p, syms.reshape(-1), np.eye(3, dtype=np.float32).reshape(-1))
    assert acc == 1.0


@pytest.mark.parametrize("kind", ["tanh", "sigmoid"])
def test_vectorised_activations_stay_within_a_few_ulp_of_libm(kind):
    """tanh and sigmoid are branch-free polynomial code (vectorised per instruction-set level); their values must stay
    within a few float ulp of the exact function over the whole useful range, including the switch-over at |x| = 0.625,
    large arguments and zero."""
    n = 4096
    x = np.concatenate([np.linspace(-30, 30, n - 9), [0.0, -0.0, 0.625, -0.625, 0.6249999, 1e-6, -1e-6, 88.0, -88.0]]).astype(np.float32)
    n = x.size
    params = np.concatenate([np.eye(n, dtype=np.float32).reshape(-1), np.zeros(n, np.float32)])   # identity weights, no bias
    y, _ = _run([_spec("dense", dim=[n, n], act_fn={kind: {"amp": 1.0}})], n, params, x.reshape(1, n), np.zeros((1, n), np.float32))
    exact = np.tanh(x.astype(np.float64)) if kind == "tanh" else 1.0 / (1.0 + np.exp(-x.astype(np.float64)))
    err = np.abs(y.reshape(-1).astype(np.float64) - exact)
    assert err.max() <= 4 * np.finfo(np.float32).eps, (err.max(), x[err.argmax()])
    assert y.reshape(-1)[n - 9] == (0.0 if kind == "tanh" else 0.5)


def _gate(bits, fn):
    xs = np.array([[(i >> (bits - 1 - b)) & 1 for b in range(bits)] for i in range(1 << bits)], dtype=np.float32)
    ys = np.array([fn(r) for r in xs.astype(int)], dtype=np.float32)
    return xs.reshape(-1), ys


_SIG = {"sigmoid": {"amp": 1.0}}
_SMALL_NETS = {
    # test_sequential_dense.rs:21-69 (y = x + 1 with one 1 -> 1 dense layer, lr 0.1, 100 epochs, batch 4)
    "linear": (np.array([0, 1, 2, 3], np.float32), np.array([1, 2, 3, 4], np.float32), 1, [(1, 1, None)], 0.1, 4, 100, 1e-3),
    # :71-124 (AND of two inputs, 2 -> 1 sigmoid)
    "and2": (*_gate(2, lambda r: float(r.all())), 2, [(2, 1, _SIG)], 1.0, 4, 6000, 0.01),
    # :126-188 (AND of three inputs, 3 -> 2 -> 1 sigmoid)
    "and3": (*_gate(3, lambda r: float(r.all())), 3, [(3, 2, _SIG), (2, 1, _SIG)], 1.0, 8, 8000, 0.01),
    # :250-323 (parity of four inputs, 4 -> 8 -> 3 -> 1 sigmoid)
    "xor4": (*_gate(4, lambda r: float(r.sum() % 2)), 4, [(4, 8, _SIG), (8, 3, _SIG), (3, 1, _SIG)], 1.0, 16, 20000, 0.02),
}


@pytest.mark.parametrize("name", sorted(_SMALL_NETS))
def test_small_networks_of_the_reference_converge(name):
    """The reference's dense convergence topologies (machine_learning/src/test/test_sequential_dense.rs), which there run
    without an assertion: here the full-batch MSE must fall below a bound within the epoch budget."""
    xs, ys, x_size, dims, lr, batch, epochs, bound = _SMALL_NETS[name]
    layers = [_spec("dense", dim=[i, o], act_fn=a) for i, o, a in dims]
    spec = _trainer_spec(layers, x_size, 1, "mse", {"gradient_descent": {"learning_rate": lr}}, batch, epochs)
    tr = core.RoundTrainer(json.dumps(spec), xs, ys)
    rng = np.random.default_rng(3)
    p, r = (rng.standard_normal(tr.n_params) * 0.7).astype(np.float32), np.zeros(tr.n_params, np.float32)
    loss = float("inf")
    for _ in range(epochs):
        p, r, losses, last = tr.train(p, r)
        loss = losses[-1]
        if loss < bound or last:
            break
    assert loss < bound, (name, loss)
