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
