"""End-to-end runs on one GPU through the public API, checked against the CPU oracle run of the same
configuration (same Philox initial parameters; one batch per epoch so the batch order cannot differ)."""
import numpy as np
import pytest

import orchestra
from orchestra import Sequential, orchestrate
from orchestra.activations import GELU, ReLU, Sigmoid, Softmax
from orchestra.arch import Dense
from orchestra.datasets import InlineDataset
from orchestra.initialization import XavierUniform
from orchestra.loss_fns import CrossEntropy, Mse
from orchestra.optimizers import Adam, GradientDescent, GradientDescentWithMomentum
from orchestra.store import BlockingStore
from orchestra.sync import BarrierSync

pytestmark = pytest.mark.gpu


def _data(n=64, x=784, y=10, seed=0):
    rng = np.random.default_rng(seed)
    xs = rng.random((n, x), dtype=np.float32)
    ys = np.eye(y, dtype=np.float32)[rng.integers(0, y, n)]
    return xs, ys


def _mlp():
    return Sequential([Dense(128, XavierUniform(), ReLU(0.0)), Dense(10, XavierUniform(), Softmax())])


@pytest.mark.parametrize("cadence", ["round", "step"])
@pytest.mark.parametrize("opt", [GradientDescent(0.5), Adam(0.01), GradientDescentWithMomentum(0.2, 0.9)])
def test_single_gpu_all_reduce_tracks_the_cpu_oracle(cadence, opt):
    xs, ys = _data()
    hist = {}
    for dev in ("cpu", "gpu"):
        tr = orchestra.all_reduce([f"{dev}:0"], InlineDataset(xs, ys, 784, 10), opt, CrossEntropy(), max_epochs=12,
                                  batch_size=64, seed=5, b200={"sync_every": cadence})
        m = orchestrate(_mlp(), tr).wait(quiet=True)
        hist[dev] = (np.array(m.loss_history()), m.weights_array())
    (lc, wc), (lg, wg) = hist["cpu"], hist["gpu"]
    assert lc.shape == lg.shape == (12,)
    assert lg[-1] < lg[0]
    # tf32 tiles against the f32 oracle over 12 chained optimizer steps: the curves track each other
    assert np.allclose(lc, lg, rtol=1e-1, atol=1e-4)
    assert np.abs(wc - wg).max() < 1e-1 * max(1.0, np.abs(wc).max())


def test_single_gpu_parameter_server_bf16_gelu_and_metrics():
    xs, ys = _data(n=256, x=256, y=16)
    model = Sequential([Dense(512, XavierUniform(), GELU()), Dense(256, XavierUniform(), Sigmoid()),
                        Dense(16, XavierUniform(), Softmax())])
    tr = orchestra.parameter_server(["gpu:0"], 1, InlineDataset(xs, ys, 256, 16), GradientDescentWithMomentum(0.1, 0.9),
                                    CrossEntropy(), BarrierSync(), BlockingStore(), max_epochs=6, batch_size=64, seed=1,
                                    b200={"sync_every": "step", "tile_dtype": "bf16", "colocate": True, "sharding": "even"})
    m = orchestrate(model, tr).wait(quiet=True)
    h = m.loss_history()
    assert len(h) == 6 and h[-1] < h[0]
    met = m.metrics()
    assert met["steps"] == 24 and met["launches_per_step"] > 5
    assert met["h2d_bytes_per_step"] == 64 * (256 + 16) * 4 and met["d2h_bytes_per_step"] == 8


def test_single_gpu_mse_regression_and_ragged_batches():
    rng = np.random.default_rng(3)
    xs = rng.random((50, 8), dtype=np.float32)
    ys = (xs @ rng.random((8, 2), dtype=np.float32)).astype(np.float32)
    model = Sequential([Dense(32, XavierUniform(), Sigmoid()), Dense(2, XavierUniform())])
    tr = orchestra.all_reduce(["gpu:0"], InlineDataset(xs, ys, 8, 2), Adam(0.02), Mse(), max_epochs=40, batch_size=16,
                              seed=2)
    h = orchestrate(model, tr).wait(quiet=True).loss_history()
    assert len(h) == 40 and h[-1] < 0.5 * h[0]


def test_compressed_gradient_wire_on_the_gpu_trains_and_reports_what_it_sent():
    """f16 wire and the sparse serializer in the reference's round cadence (compressor.rs:71-118)."""
    import numpy as np

    import orchestra
    from orchestra import Sequential, orchestrate
    from orchestra.activations import Softmax, Tanh
    from orchestra.arch import Dense
    from orchestra.datasets import InlineDataset
    from orchestra.initialization import XavierUniform
    from orchestra.loss_fns import CrossEntropy
    from orchestra.optimizers import GradientDescent
    from orchestra.serializer import SparseSerializer

    rng = np.random.default_rng(0)
    xs = rng.random((256, 32), dtype=np.float32)
    ys = np.eye(4, dtype=np.float32)[(xs[:, :4].argmax(1))]
    model = Sequential([Dense(64, XavierUniform(), Tanh()), Dense(4, XavierUniform(), Softmax())])

    def run(**kw):
        tr = orchestra.all_reduce(["gpu:0"], InlineDataset(xs, ys, 32, 4), GradientDescent(0.5), CrossEntropy(), 30, 64, seed=2, **kw)
        return orchestrate(model, tr).wait(quiet=True)

    plain = run()
    f16 = run(b200={"wire_dtype": "f16"})
    sparse = run(serializer=SparseSerializer(0.25))
    assert f16.metrics()["wire"] == "f16" and f16.metrics()["wire_sent_fraction"] == pytest.approx(1.0, abs=0.02)
    assert sparse.metrics()["wire"] == "f16+sparse" and 0.1 < sparse.metrics()["wire_sent_fraction"] < 0.45
    lp, lf, ls = (np.array(m.loss_history()) for m in (plain, f16, sparse))
    assert np.allclose(lp, lf, rtol=2e-2)                      # f16 rounding barely moves the trajectory
    assert ls[-1] < ls[0] and ls[-1] < 1.5 * lp[-1] + 0.05     # dropped entries arrive later through the residual


def test_trace_and_metrics_files_of_a_gpu_run(tmp_path):
    import json

    rng = np.random.default_rng(0)
    xs = rng.random((128, 16), dtype=np.float32)
    ys = np.eye(4, dtype=np.float32)[rng.integers(0, 4, 128)]
    model = Sequential([Dense(32, XavierUniform(), ReLU(0.0)), Dense(4, XavierUniform(), Softmax())])
    tp, mp = tmp_path / "trace.json", tmp_path / "metrics.jsonl"
    tr = orchestra.all_reduce(["gpu:0"], InlineDataset(xs, ys, 16, 4), GradientDescent(0.1), CrossEntropy(), 3, 32, seed=1,
                              b200={"sync_every": "step", "trace_path": str(tp), "metrics_path": str(mp)})
    orchestrate(model, tr).wait(quiet=True)
    doc = json.load(open(tp))
    names = [e["name"] for e in doc["traceEvents"]]
    assert names.count("epoch") == 3 and "step" in names and "report_and_decide" in names
    steps = [e for e in doc["traceEvents"] if e["name"] == "step"]
    assert all(e["tid"] == 1 and e["dur"] > 0 for e in steps)          # device spans from CUDA events
    recs = [json.loads(l) for l in open(mp)]
    assert len(recs) == 3 and all(r["steps"] >= 1 and r["device_ms"] > 0 and r["samples_per_sec"] > 0 for r in recs)


def test_phase_timing_reports_compute_exchange_and_refresh_per_step(tmp_path):
    import json

    rng = np.random.default_rng(0)
    xs = rng.random((128, 16), dtype=np.float32)
    ys = np.eye(4, dtype=np.float32)[rng.integers(0, 4, 128)]
    model = Sequential([Dense(32, XavierUniform(), ReLU(0.0)), Dense(4, XavierUniform(), Softmax())])
    tp, mp = tmp_path / "trace.json", tmp_path / "metrics.jsonl"
    tr = orchestra.all_reduce(["gpu:0"], InlineDataset(xs, ys, 16, 4), GradientDescent(0.1), CrossEntropy(), 2, 32, seed=1,
                              b200={"sync_every": "step", "phase_timing": True, "trace_path": str(tp), "metrics_path": str(mp)})
    m = orchestrate(model, tr).wait(quiet=True)
    recs = [json.loads(l) for l in open(mp)]
    assert len(recs) == 2
    for r in recs:
        assert set(r["phase_ms"]) == {"compute", "exchange", "refresh"} and all(v > 0 for v in r["phase_ms"].values())
    # the first epoch's very first step carries one-time costs (kernel images loaded on first use, attribute calls), which the
    # phase means of that epoch include but the step-to-step maximum does not; the second epoch is steady state
    assert sum(recs[1]["phase_ms"].values()) <= recs[1]["max_step_ms"] * 1.5
    names = [e["name"] for e in json.load(open(tp))["traceEvents"]]
    assert names.count("compute") == 8 and names.count("exchange") == 8      # 4 steps per epoch, device rows
    assert set(m.metrics()["phase_ms"]) == {"compute", "exchange", "refresh"}


@pytest.mark.parametrize("tile", ["tf32", "bf16"])
def test_gradient_push_through_the_gemm_epilogue_matches_the_plain_path(tile, monkeypatch):
    """Weight-gradient tiles added into the owner's accumulator by TMA reductions (here the owner is this GPU)."""
    monkeypatch.setenv("ONO_PUSH_SINGLE", "1")
    xs, ys = _data(n=192, x=256, y=12)
    model = Sequential([Dense(384, XavierUniform(), ReLU(0.0)), Dense(256, XavierUniform(), Sigmoid()),
                        Dense(12, XavierUniform(), Softmax())])
    out = {}
    for push in ("off", "on"):
        tr = orchestra.parameter_server(["gpu:0"], 1, InlineDataset(xs, ys, 256, 12), GradientDescentWithMomentum(0.2, 0.9),
                                        CrossEntropy(), BarrierSync(), BlockingStore(), max_epochs=8, batch_size=64, seed=3,
                                        b200={"sync_every": "step", "tile_dtype": tile, "colocate": True, "sharding": "even",
                                              "grad_push": push})
        m = orchestrate(model, tr).wait(quiet=True)
        out[push] = (np.array(m.loss_history()), m.weights_array(), m.metrics())
    assert out["on"][2]["grad_push"] is True and out["off"][2]["grad_push"] is False
    assert out["on"][0][-1] < out["on"][0][0]
    # same products, added by reductions instead of stores: equal up to the order of f32 additions
    assert np.allclose(out["on"][0], out["off"][0], rtol=1e-4, atol=1e-6)
    assert np.abs(out["on"][1] - out["off"][1]).max() < 1e-4


def test_warm_start_on_the_gpu_loads_the_checkpoint(tmp_path):
    xs, ys = _data(n=64, x=32, y=12)
    model = Sequential([Dense(16, XavierUniform(), ReLU(0.0)), Dense(12, XavierUniform(), Softmax())])
    first = orchestrate(model, orchestra.all_reduce(["gpu:0"], InlineDataset(xs, ys, 32, 12), GradientDescent(0.5), CrossEntropy(),
                                                    4, 32, seed=1)).wait(quiet=True)
    ckpt = tmp_path / "m.safetensors"
    first.save_safetensors(ckpt)
    again = orchestrate(model, orchestra.all_reduce(["gpu:0"], InlineDataset(xs, ys, 32, 12), GradientDescent(1e-12), CrossEntropy(),
                                                    1, 32, seed=1, b200={"init_from": str(ckpt)})).wait(quiet=True)
    assert np.allclose(again.weights_array(), first.weights_array(), atol=1e-6)


def test_resume_with_optimizer_state_continues_the_uninterrupted_run(tmp_path):
    """Weights + optimizer state + shuffle position: 3 + 3 epochs give what 6 epochs give; without the state they do not."""
    from orchestra.optimizers import Adam

    xs, ys = _data(n=128, x=32, y=12)
    model = Sequential([Dense(24, XavierUniform(), ReLU(0.0)), Dense(12, XavierUniform(), Softmax())])

    def run(epochs, **b200):
        tr = orchestra.all_reduce(["gpu:0"], InlineDataset(xs, ys, 32, 12), Adam(0.01), CrossEntropy(), epochs, 32, seed=4,
                                  b200={"sync_every": "step", **b200})
        return orchestrate(model, tr).wait(quiet=True)

    whole = run(6)
    ckpt, state = tmp_path / "m.safetensors", tmp_path / "m.state.safetensors"
    half = run(3, state_path=str(state))
    half.save_safetensors(ckpt)
    from oxidized_neural_orchestra_b200.utils.state import load_state

    st = load_state(str(state), len(half.weights_array()))
    assert st["meta"]["epochs"] == "3" and st["meta"]["optimizer"] == "adam" and np.abs(st["m"]).max() > 0 and st["v"].min() >= 0
    resumed = run(3, init_from=str(ckpt), init_state_from=str(state))
    cold = run(3, init_from=str(ckpt), start_epoch=3)
    err_resumed = np.abs(resumed.weights_array() - whole.weights_array()).max()
    err_cold = np.abs(cold.weights_array() - whole.weights_array()).max()
    assert err_resumed < 1e-5, err_resumed
    assert err_cold > 20 * max(err_resumed, 1e-7), (err_cold, err_resumed)
    assert np.allclose(resumed.loss_history(), whole.loss_history()[3:], rtol=1e-4, atol=1e-6)


def test_state_sidecar_moves_between_gpu_and_cpu_ranks(tmp_path):
    """The optimizer-state file is the same for both kinds of rank: three epochs on a GPU rank, then three more on a CPU rank
    from its weights + state land where six epochs on the GPU rank land (up to tf32 tiles against f32 loops), and clearly
    closer than a continuation that drops the state."""
    from orchestra.optimizers import GradientDescentWithMomentum

    xs, ys = _data(n=128, x=32, y=12)
    model = Sequential([Dense(24, XavierUniform(), ReLU(0.0)), Dense(12, XavierUniform(), Softmax())])

    def run(addr, epochs, **b200):
        if addr.startswith("gpu"):
            b200 = {"sync_every": "step", **b200}
        tr = orchestra.all_reduce([addr], InlineDataset(xs, ys, 32, 12), GradientDescentWithMomentum(0.5, 0.9), CrossEntropy(), epochs, 128, seed=4, b200=b200 or None)
        return orchestrate(model, tr).wait(quiet=True)

    # one batch per epoch (batch = the whole set): the step and the round cadence coincide and the batch order cannot differ
    whole = run("gpu:0", 6)
    ckpt, state = tmp_path / "m.safetensors", tmp_path / "m.state.safetensors"
    half = run("gpu:0", 3, state_path=str(state))
    half.save_safetensors(ckpt)
    resumed = run("cpu:0", 3, init_from=str(ckpt), init_state_from=str(state))
    cold = run("cpu:0", 3, init_from=str(ckpt), start_epoch=3)
    err_resumed = np.abs(resumed.weights_array() - whole.weights_array()).max()
    err_cold = np.abs(cold.weights_array() - whole.weights_array()).max()
    assert err_resumed < 2e-3, err_resumed
    assert err_cold > 5 * err_resumed, (err_cold, err_resumed)
    # and back: the CPU rank's state continues on the GPU rank
    state2, ckpt2 = tmp_path / "c.state.safetensors", tmp_path / "c.safetensors"
    chalf = run("cpu:0", 3, state_path=str(state2))
    chalf.save_safetensors(ckpt2)
    back = run("gpu:0", 3, init_from=str(ckpt2), init_state_from=str(state2))
    assert np.abs(back.weights_array() - whole.weights_array()).max() < 2e-3


def test_switch_that_would_leave_no_worker_is_declined():
    """A strategy switch on one GPU would promote the only rank to a server and leave nobody to train (the reference's
    planner needs more workers than servers): the run says so in its metrics and keeps training in all-reduce."""
    from orchestra.optimizers import Adam
    from orchestra.store import BlockingStore
    from orchestra.sync import BarrierSync

    xs, ys = _data(n=96, x=32, y=12)
    model = Sequential([Dense(24, XavierUniform(), ReLU(0.0)), Dense(12, XavierUniform(), Softmax())])
    tr = orchestra.strategy_switch(["gpu:0"], 1, InlineDataset(xs, ys, 32, 12), Adam(0.01), CrossEntropy(), BarrierSync(), BlockingStore(),
                                   6, 32, seed=4, b200={"sync_every": "step", "colocate": True, "switch_metric": "grad_norm", "switch_window": 2,
                                                        "switch_threshold": 10.0, "switch_check_every": 2})
    m = orchestrate(model, tr).wait(quiet=True)
    met = m.metrics()
    assert met["switch_declined"] is True and not met["switched"] and met["switched_at_step"] is None
    hist = m.loss_history()
    assert len(hist) == 6 and hist[-1] < hist[0]


def test_periodic_checkpoints_load_back_and_continue_the_run(tmp_path):
    from orchestra.optimizers import Adam

    xs, ys = _data(n=128, x=32, y=12)
    model = Sequential([Dense(24, XavierUniform(), ReLU(0.0)), Dense(12, XavierUniform(), Softmax())])

    def run(epochs, **b200):
        tr = orchestra.all_reduce(["gpu:0"], InlineDataset(xs, ys, 32, 12), Adam(0.01), CrossEntropy(), epochs, 32, seed=4,
                                  b200={"sync_every": "step", **b200})
        return orchestrate(model, tr).wait(quiet=True)

    pat = str(tmp_path / "ck_{epoch}.safetensors")
    whole = run(4, checkpoint_path=pat, checkpoint_every=2)
    files = sorted(p.name for p in tmp_path.iterdir())
    assert files == ["ck_2.safetensors", "ck_2.state.safetensors", "ck_4.safetensors", "ck_4.state.safetensors"]
    from orchestra import _orchestra as core

    last = np.concatenate([np.asarray(t[2]).reshape(-1) for t in sorted(core.load_safetensors(str(tmp_path / "ck_4.safetensors")),
                                                                       key=lambda t: (int(t[0].split("_")[1].split(".")[0]), t[0].endswith("bias")))])
    assert np.allclose(last, whole.weights_array(), atol=1e-7)
    resumed = run(2, init_from=str(tmp_path / "ck_2.safetensors"), init_state_from=str(tmp_path / "ck_2.state.safetensors"))
    assert np.abs(resumed.weights_array() - whole.weights_array()).max() < 1e-5


@pytest.mark.parametrize("tile", ["bf16", "tf32"])
@pytest.mark.parametrize("opt", [GradientDescentWithMomentum(0.1, 0.9), Adam(0.005), GradientDescent(0.2)])
def test_optimizer_in_the_weight_gradient_epilogue_matches_the_separate_pass(tile, opt, monkeypatch):
    """On one GPU the weight-gradient GEMMs update master, state and shadow in their epilogues; the run must follow the
    run whose optimizer is the separate fused pass (same arithmetic per element, only the GEMM's f32 result is not
    rounded through memory in between: the two are equal to rounding). The runtime only chooses this for layers large
    enough for the TMA form; here it is forced onto a small model so that both epilogue forms are exercised."""
    monkeypatch.setenv("ONO_WGRAD_APPLY", "force")
    xs, ys = _data(n=256, x=512, y=16, seed=4)
    model = Sequential([Dense(1024, XavierUniform(), GELU()), Dense(512, XavierUniform(), ReLU(0.0)),
                        Dense(16, XavierUniform(), Softmax())])
    got = {}
    for mode in ("auto", "off"):
        tr = orchestra.parameter_server(["gpu:0"], 1, InlineDataset(xs, ys, 512, 16), opt, CrossEntropy(), BarrierSync(),
                                        BlockingStore(), max_epochs=5, batch_size=64, seed=3,
                                        b200={"sync_every": "step", "tile_dtype": tile, "colocate": True, "sharding": "even",
                                              "wgrad_apply": mode})
        m = orchestrate(model, tr).wait(quiet=True)
        assert m.metrics()["wgrad_apply"] == (mode == "auto")
        got[mode] = (np.array(m.loss_history()), m.weights_array())
    (la, wa), (lo, wo) = got["auto"], got["off"]
    assert la[-1] < la[0]
    if isinstance(opt, Adam):
        # Adam normalises every element's step to about lr: where a gradient is at rounding level, one differently
        # contracted multiply-add flips the direction of a whole step, so single weights drift apart by a few lr while
        # the loss and the bulk of the weights stay together
        assert np.allclose(la, lo, rtol=2e-2, atol=1e-6)
        assert np.abs(wa - wo).mean() < 1e-3 and np.abs(wa - wo).max() < 0.05
    else:
        assert np.allclose(la, lo, rtol=2e-3, atol=1e-6)
        assert np.abs(wa - wo).max() < 2e-3 * max(1.0, np.abs(wo).max())
