"""The optimizer-state sidecar is a plain safetensors file: round trip, layout, rejections."""
import json
import struct

import numpy as np
import pytest

from oxidized_neural_orchestra_b200.utils.state import load_state, save_state


def test_round_trip_and_container_layout(tmp_path):
    rng = np.random.default_rng(0)
    m, v, pows = rng.standard_normal(53).astype(np.float32), rng.random(53).astype(np.float32), np.array([0.5, 0.25], np.float32)
    path = tmp_path / "x.state.safetensors"
    save_state(str(path), m, v, pows, optimizer="adam", epochs=7)
    raw = path.read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    assert hlen % 8 == 0 and header["optimizer.m"] == {"dtype": "F32", "shape": [53], "data_offsets": [0, 212]}
    assert header["optimizer.v"]["data_offsets"] == [212, 424] and header["optimizer.adam_pows"]["shape"] == [2]
    assert len(raw) == 8 + hlen + 4 * (53 + 53 + 2)
    st = load_state(str(path), 53)
    assert np.array_equal(st["m"], m) and np.array_equal(st["v"], v) and np.array_equal(st["adam_pows"], pows)
    assert st["meta"] == {"optimizer": "adam", "epochs": "7"}
    # the same container loads with the checkpoint reader of the core library
    from orchestra import _orchestra as core

    names = sorted(t[0] for t in core.load_safetensors(str(path)))
    assert names == ["optimizer.adam_pows", "optimizer.m", "optimizer.v"]


def test_state_of_another_model_is_rejected(tmp_path):
    path = tmp_path / "x.state.safetensors"
    save_state(str(path), np.zeros(10, np.float32), np.zeros(10, np.float32), np.ones(2, np.float32))
    with pytest.raises(ValueError, match="does not fit"):
        load_state(str(path), 11)


def test_weight_checkpoint_writer_matches_the_core_writer(tmp_path):
    """The Python writer used for periodic checkpoints produces what the core library's exporter produces."""
    import json

    from orchestra import _orchestra as core
    from oxidized_neural_orchestra_b200.utils.state import save_tensors, weight_tensors

    model = {"layers": [{"conv": {"input_dim": [1, 8, 8], "kernel_dim": [4, 1, 3], "stride": 1, "padding": 1, "init": "xavier", "act_fn": {"tanh": {"amp": 1.0}}}},
                        {"max_pooling": {"input_dim": [4, 8, 8], "filter_size": 2, "stride": 2, "padding": 0}},
                        {"dense": {"output_size": 5, "init": "xavier_uniform", "act_fn": "softmax"}}]}
    n = 4 * 9 + 4 + 64 * 5 + 5
    params = np.arange(n, dtype=np.float32) / 7
    a, b = tmp_path / "core.safetensors", tmp_path / "py.safetensors"
    try:
        core.save_safetensors(str(a), json.dumps(model), 64, params)
    except Exception as exc:      # the model document above must be valid for the core: fail loudly if the schema moved
        pytest.fail(f"core writer rejected the model: {exc}")
    layers = [{"kind": "conv", "kernel_dim": [4, 1, 3]}, {"kind": "pool"}, {"kind": "dense", "in": 64, "out": 5}]
    save_tensors(str(b), weight_tensors(layers, params))
    ta = {t[0]: (list(t[1]), np.asarray(t[2])) for t in core.load_safetensors(str(a))}
    tb = {t[0]: (list(t[1]), np.asarray(t[2])) for t in core.load_safetensors(str(b))}
    assert sorted(ta) == sorted(tb) == sorted(f"layer_{i}.{k}" for i in range(3) for k in ("weight", "bias"))
    assert a.read_bytes() == b.read_bytes()        # same entry order (by name) and layout: equal byte for byte
    for k in ta:
        assert ta[k][0] == tb[k][0] and np.array_equal(ta[k][1], tb[k][1]), k
    with pytest.raises(ValueError, match="covers"):
        weight_tensors(layers, params[:-1])
