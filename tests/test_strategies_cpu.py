"""Distributed semantics on CPU ranks through the public API: the three strategies, the wire formats,
the switch, early stopping, stop requests and the divergence guard.

The reference shipped without an all-reduce or switch test and was bitten by sum-vs-mean, layer-order
and shard-order bugs (docs/report/riesgos.md:26); the first tests below pin exactly those.
"""
import json

import numpy as np
import pytest

import orchestra
from orchestra import Sequential, _orchestra as core, orchestrate
from orchestra.activations import ReLU, Sigmoid, Softmax, Tanh
from orchestra.arch import Conv2d, Dense, MaxPooling
from orchestra.datasets import InlineDataset, LocalDataset
from orchestra.initialization import Const, Kaiming, XavierUniform
from orchestra.loss_fns import CrossEntropy, Mse
from orchestra.optimizers import Adam, GradientDescent, GradientDescentWithMomentum
from orchestra.serializer import BaseSerializer, SparseSerializer
from orchestra.store import BlockingStore, WildStore
from orchestra.sync import BarrierSync, NonBlockingSync


def _data(n=24, x=6, y=3, seed=0):
    rng = np.random.default_rng(seed)
    xs = rng.random((n, x)).astype(np.float32)
    ys = np.eye(y, dtype=np.float32)[rng.integers(0, y, n)]
    return xs, ys


def _model():
    return Sequential([Dense(5, XavierUniform(), Tanh()), Dense(4, XavierUniform(), ReLU(0.0)), Dense(3, XavierUniform(), Softmax())])


def _expected_one_round(model, training, xs, ys, nworkers, lr):
    """p0 - lr * mean over workers of the gradient of their whole partition at p0 (one batch each)."""
    plan = json.loads(core.adapt_configs(model.to_json(), training.to_json(with_data=False)))
    p0 = np.concatenate([core.param_gen_fill(json.dumps(l["param_gen"]), 3) for l in plan["layers"] if l["param_gen"]])
    specs = json.dumps([l["spec"] for l in plan["layers"]])
    grads = []
    for (b, e) in core.dataset_partitions(len(xs), nworkers):
        seq = core.Sequential(specs, xs.shape[1])
        out = seq.forward(p0, xs[b:e].reshape(-1), e - b)
        _, delta = core.loss_prime("cross_entropy", out, ys[b:e].reshape(-1))
        grads.append(seq.backward(p0, delta, e - b))
    return p0 - lr * np.mean(grads, axis=0), p0


def test_all_reduce_averages_and_keeps_layer_order():
    xs, ys = _data()
    tr = orchestra.all_reduce([f"cpu:{i}" for i in range(3)], InlineDataset(xs, ys, 6, 3), GradientDescent(0.1),
                              CrossEntropy(), max_epochs=1, batch_size=8, seed=3)
    m = orchestrate(_model(), tr).wait()
    want, p0 = _expected_one_round(_model(), tr, xs, ys, 3, 0.1)
    got = m.weights_array()
    assert got.shape == want.shape and np.allclose(got, want, atol=1e-6)
    assert not np.allclose(got, p0)
    assert len(m.loss_history()) == 1 and m.stop_reason == "max_epochs"


@pytest.mark.parametrize("nservers,sharding", [(1, "layer"), (2, "layer"), (2, "even")])
def test_parameter_server_matches_all_reduce_for_plain_sgd(nservers, sharding):
    xs, ys = _data()
    n = 3 + nservers
    tr = orchestra.parameter_server([f"cpu:{i}" for i in range(n)], nservers, InlineDataset(xs, ys, 6, 3),
                                    GradientDescent(0.1), CrossEntropy(), BarrierSync(), BlockingStore(), max_epochs=1,
                                    batch_size=8, seed=3, b200={"sharding": sharding})
    m = orchestrate(_model(), tr).wait()
    want, _ = _expected_one_round(_model(), tr, xs, ys, 3, 0.1)
    assert np.allclose(m.weights_array(), want, atol=1e-6)  # shard order / layer order / mean over workers


def test_f16_wire_and_sparse_serializer_are_lossy_but_train():
    xs, ys = _data(n=60)
    base = dict(dataset=InlineDataset(xs, ys, 6, 3), optimizer=GradientDescent(0.5), loss_fn=CrossEntropy(),
                max_epochs=60, batch_size=10, seed=3)
    addrs = [f"cpu:{i}" for i in range(3)]
    exact = orchestrate(_model(), orchestra.all_reduce(addrs, **base)).wait()
    f16 = orchestrate(_model(), orchestra.all_reduce(addrs, b200={"wire_dtype": "f16"}, **base)).wait()
    d = np.abs(exact.weights_array() - f16.weights_array()).max()
    assert 0 < d < 5e-2  # re-quantised at every hop (compressor.rs:106-118), close but not equal
    sp = orchestrate(_model(), orchestra.parameter_server(addrs + ["cpu:3"], 1, sync=BarrierSync(), store=BlockingStore(),
                                                          serializer=SparseSerializer(0.5), **base)).wait()
    for m in (exact, f16, sp):
        h = m.loss_history()
        assert len(h) == 60 and h[-1] < h[0]


def test_async_and_wild_stores_terminate_and_learn():
    xs, ys = _data(n=60)
    for sync, store in ((NonBlockingSync(), BlockingStore()), (NonBlockingSync(), WildStore()), (BarrierSync(), WildStore())):
        tr = orchestra.parameter_server([f"cpu:{i}" for i in range(5)], 2, InlineDataset(xs, ys, 6, 3), GradientDescent(0.3),
                                        CrossEntropy(), sync, store, max_epochs=40, batch_size=10, seed=3, offline_epochs=1)
        h = orchestrate(_model(), tr).wait().loss_history()
        assert len(h) == 40 and h[-1] < h[0]


def test_strategy_switch_promotes_servers_and_keeps_training():
    xs, ys = _data(n=60)
    tr = orchestra.strategy_switch([f"cpu:{i}" for i in range(4)], 1, InlineDataset(xs, ys, 6, 3), Adam(0.01),
                                   CrossEntropy(), BarrierSync(), BlockingStore(), max_epochs=30, batch_size=5, seed=3,
                                   b200={"switch_window": 2, "switch_threshold": 10.0})
    s = orchestrate(_model(), tr)
    kinds = []
    for ev in s.events():
        kinds.append(ev["kind"])
    assert "switch" in kinds and kinds.count("upgraded") == 1 and kinds[-1] == "complete"
    assert kinds.index("switch") < kinds.index("upgraded")
    m = s.wait()
    assert m.metrics()["switched"] is True
    # progress is carried across the switch by default (switch_resets_progress = false)
    s2 = orchestrate(_model(), tr)
    m2 = s2.wait()
    assert len(m2.loss_history()) == 30 and m2.loss_history()[-1] < m2.loss_history()[0]


def test_early_stopping_and_stop_request():
    xs, ys = _data()
    tr = orchestra.all_reduce(["cpu:0", "cpu:1"], InlineDataset(xs, ys, 6, 3), GradientDescent(0.01), CrossEntropy(),
                              max_epochs=500, batch_size=4, seed=3, early_stopping_tolerance=10.0)
    m = orchestrate(_model(), tr).wait()
    assert m.stop_reason == "early_stopping" and len(m.loss_history()) == 3  # 3 rounds within tolerance
    tr = orchestra.parameter_server(["cpu:0", "cpu:1", "cpu:2"], 1, InlineDataset(xs, ys, 6, 3), GradientDescent(0.01),
                                    CrossEntropy(), BarrierSync(), BlockingStore(), max_epochs=1_000_000, batch_size=4, seed=3)
    s = orchestrate(_model(), tr)
    s.stop()
    m = s.wait()
    assert m.stop_reason == "stopped" and len(m.loss_history()) < 1_000_000


def test_non_finite_loss_aborts_the_run():
    xs, ys = _data()
    model = Sequential([Dense(4, Const(50.0)), Dense(3, Const(50.0))])
    tr = orchestra.all_reduce(["cpu:0", "cpu:1"], InlineDataset(xs * 1e18, ys, 6, 3), GradientDescent(1e18), Mse(),
                              max_epochs=20, batch_size=4, seed=1)
    with pytest.raises(RuntimeError, match="non-finite"):
        orchestrate(model, tr).wait()


def test_cnn_through_the_api_and_safetensors(tmp_path):
    rng = np.random.default_rng(0)
    xs = rng.random((16, 36)).astype(np.float32)
    ys = np.eye(2, dtype=np.float32)[(xs[:, :18].sum(1) > xs[:, 18:].sum(1)).astype(int)]
    sp, lp = tmp_path / "x.bin", tmp_path / "y.bin"
    xs.tofile(sp)
    ys.tofile(lp)
    model = Sequential([Conv2d((1, 6, 6), (3, 1, 3), 1, 1, Kaiming(), ReLU(0.0)), MaxPooling((3, 6, 6), 2, 2, 0),
                        Dense(2, Kaiming(), Softmax())])
    tr = orchestra.parameter_server(["cpu:0", "cpu:1", "cpu:2"], 1, LocalDataset(str(sp), str(lp), 36, 2),
                                    GradientDescentWithMomentum(0.2, 0.9), CrossEntropy(), BarrierSync(), BlockingStore(),
                                    max_epochs=30, batch_size=4, seed=2)
    m = orchestrate(model, tr).wait()
    assert m.loss_history()[-1] < m.loss_history()[0]
    out = tmp_path / "m.safetensors"
    m.save_safetensors(out)
    names = [t[0] for t in core.load_safetensors(str(out))]
    assert sorted(names) == sorted([f"layer_{i}.{k}" for i in range(3) for k in ("weight", "bias")])
    assert len(m.weights()) == 3 * 9 + 3 + (27 + 1) * 2


def test_api_argument_errors_match_the_reference_types():
    with pytest.raises(ValueError):
        Dense(0, Kaiming())
    with pytest.raises(TypeError):
        Dense(3, "kaiming")
    with pytest.raises(TypeError):
        Dense(3, Kaiming(), act_fn="relu")
    with pytest.raises(ValueError):
        Sequential([])
    with pytest.raises(ValueError):
        Conv2d((1, 0, 3), (1, 1, 1), 1, 0, Kaiming())
    with pytest.raises(ValueError):
        LocalDataset("/nonexistent/x.bin", "/nonexistent/y.bin", 1, 1)
    xs, ys = _data()
    ds = InlineDataset(xs, ys, 6, 3)
    with pytest.raises(ValueError):
        orchestra.all_reduce(["cpu:0"], ds, GradientDescent(0.1), Mse(), 1, 1, early_stopping_tolerance=0.0)
    with pytest.raises(TypeError):
        orchestra.all_reduce(["cpu:0"], ds, "sgd", Mse(), 1, 1)
    with pytest.raises(ValueError):  # validated by the C++ core at orchestrate()
        orchestrate(_model(), orchestra.parameter_server(["cpu:0"], 1, ds, GradientDescent(0.1), CrossEntropy(),
                                                         BarrierSync(), BlockingStore(), 1, 1))
    with pytest.raises(ValueError):
        orchestrate(_model(), orchestra.all_reduce(["cpu:0"], ds, GradientDescent(-1.0), CrossEntropy(), 1, 1))
    # a single worker is a valid ring of one
    m = orchestrate(_model(), orchestra.all_reduce(["cpu:0"], ds, GradientDescent(0.1), CrossEntropy(), 2, 4, seed=1)).wait()
    assert len(m.loss_history()) == 2


def test_warm_start_from_a_saved_checkpoint(tmp_path):
    """b200.init_from replaces the initialisers by a safetensors checkpoint (weights resume where a run stopped)."""
    import numpy as np

    import orchestra
    from orchestra import Sequential, orchestrate
    from orchestra.activations import Softmax, Tanh
    from orchestra.arch import Dense
    from orchestra.datasets import InlineDataset
    from orchestra.initialization import XavierUniform
    from orchestra.loss_fns import CrossEntropy
    from orchestra.optimizers import GradientDescent

    rng = np.random.default_rng(0)
    xs = rng.random((40, 6), dtype=np.float32)
    ys = np.eye(3, dtype=np.float32)[rng.integers(0, 3, 40)]
    model = Sequential([Dense(5, XavierUniform(), Tanh()), Dense(3, XavierUniform(), Softmax())])
    addrs = ["cpu:0", "cpu:1"]
    first = orchestrate(model, orchestra.all_reduce(addrs, InlineDataset(xs, ys, 6, 3), GradientDescent(0.5), CrossEntropy(), 5, 5,
                                                    seed=1)).wait(quiet=True)
    ckpt = tmp_path / "first.safetensors"
    first.save_safetensors(ckpt)
    # a step size of ~0 leaves the loaded weights where they are, and the first reported loss is the saved model's
    again = orchestrate(model, orchestra.all_reduce(addrs, InlineDataset(xs, ys, 6, 3), GradientDescent(1e-12), CrossEntropy(), 1, 5,
                                                    seed=1, b200={"init_from": str(ckpt)})).wait(quiet=True)
    assert np.allclose(again.weights_array(), first.weights_array(), atol=1e-7)
    assert again.loss_history()[0] < first.loss_history()[0]
    with pytest.raises(ValueError):
        bad = Sequential([Dense(7, XavierUniform(), Tanh()), Dense(3, XavierUniform(), Softmax())])
        orchestrate(bad, orchestra.all_reduce(addrs, InlineDataset(xs, ys, 6, 3), GradientDescent(0.1), CrossEntropy(), 1, 5,
                                              b200={"init_from": str(ckpt)}))


@pytest.mark.parametrize("strategy", ["all_reduce", "parameter_server"])
@pytest.mark.parametrize("opt_name", ["momentum", "adam"])
def test_cpu_ranks_resume_with_optimizer_state(tmp_path, strategy, opt_name):
    """Weights + optimizer state + shuffle position on CPU ranks: 3 + 3 epochs give what 6 epochs give, and without the
    state they do not. The sidecar is the file GPU ranks write and read (utils/state.py)."""
    from oxidized_neural_orchestra_b200.utils.state import load_state

    xs, ys = _data(n=48, x=6, y=3, seed=5)
    model = _model()
    opt = (lambda: GradientDescentWithMomentum(0.2, 0.9)) if opt_name == "momentum" else (lambda: Adam(0.01))
    addrs = ["cpu:0", "cpu:1"]

    def run(epochs, **b200):
        ds = InlineDataset(xs, ys, 6, 3)
        if strategy == "all_reduce":
            tr = orchestra.all_reduce(addrs, ds, opt(), CrossEntropy(), epochs, 8, seed=4, b200=b200 or None)
        else:
            tr = orchestra.parameter_server(addrs, 2, ds, opt(), CrossEntropy(), BarrierSync(), BlockingStore(), epochs, 8, seed=4,
                                            b200={"colocate": True, **b200})
        return orchestrate(model, tr).wait(quiet=True)

    whole = run(6)
    ckpt, state = tmp_path / "m.safetensors", tmp_path / "m.state.safetensors"
    half = run(3, state_path=str(state))
    half.save_safetensors(ckpt)
    st = load_state(str(state), len(half.weights_array()))
    assert st["meta"]["epochs"] == "3" and np.abs(st["m"]).max() > 0
    assert (st["v"].max() > 0) == (opt_name == "adam")
    resumed = run(3, init_from=str(ckpt), init_state_from=str(state))
    cold = run(3, init_from=str(ckpt), start_epoch=3)
    err_resumed = np.abs(resumed.weights_array() - whole.weights_array()).max()
    err_cold = np.abs(cold.weights_array() - whole.weights_array()).max()
    assert err_resumed < 1e-6, err_resumed
    assert err_cold > 20 * max(err_resumed, 1e-7), (err_cold, err_resumed)
    assert np.allclose(resumed.loss_history(), whole.loss_history()[3:], rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("strategy", ["all_reduce", "parameter_server"])
def test_cpu_ranks_write_periodic_checkpoints_that_continue_the_run(tmp_path, strategy):
    """`checkpoint_path` / `checkpoint_every` on CPU ranks: weights + state files every two epochs, and a run resumed
    from the middle one ends where the uninterrupted run ends."""
    xs, ys = _data(n=48, x=6, y=3, seed=5)
    model = _model()
    addrs = ["cpu:0", "cpu:1"]

    def run(epochs, **b200):
        ds = InlineDataset(xs, ys, 6, 3)
        if strategy == "all_reduce":
            tr = orchestra.all_reduce(addrs, ds, Adam(0.01), CrossEntropy(), epochs, 8, seed=4, b200=b200 or None)
        else:
            tr = orchestra.parameter_server(addrs, 2, ds, Adam(0.01), CrossEntropy(), BarrierSync(), BlockingStore(), epochs, 8, seed=4,
                                            b200={"colocate": True, **b200})
        return orchestrate(model, tr).wait(quiet=True)

    pat = str(tmp_path / "ck_{epoch}.safetensors")
    whole = run(6, checkpoint_path=pat, checkpoint_every=2)
    files = sorted(p.name for p in tmp_path.iterdir())
    assert files == ["ck_2.safetensors", "ck_2.state.safetensors", "ck_4.safetensors", "ck_4.state.safetensors",
                     "ck_6.safetensors", "ck_6.state.safetensors"]
    last = np.concatenate([np.asarray(t[2]).reshape(-1) for t in sorted(
        core.load_safetensors(str(tmp_path / "ck_6.safetensors")), key=lambda t: (int(t[0].split("_")[1].split(".")[0]), t[0].endswith("bias")))])
    assert np.allclose(last, whole.weights_array(), atol=1e-7)
    resumed = run(2, init_from=str(tmp_path / "ck_4.safetensors"), init_state_from=str(tmp_path / "ck_4.state.safetensors"))
    assert np.abs(resumed.weights_array() - whole.weights_array()).max() < 1e-6
