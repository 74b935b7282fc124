"""Device gradient compression against the host codec (the C++ restatement of comms/src/sparse/protocol.rs)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,r", [(5000, 0.1), (16384, 0.5), (200_003, 0.01), (1_000_000, 0.25)])
def test_threshold_equals_the_host_codec(n, r):
    from orchestra import _orchestra as core
    from oxidized_neural_orchestra_b200.ops import compress as cp

    torch.manual_seed(n)
    x = torch.randn(n, device="cuda") * 1e-2
    thr = cp.sparse_threshold(x, r, seed=77)
    ref = core.sparse_threshold(x.cpu().numpy(), r, 77)
    assert thr.item() == pytest.approx(ref, rel=0, abs=0)


def test_mask_splits_wire_and_residual_like_the_reference():
    from oxidized_neural_orchestra_b200.ops import compress as cp

    torch.manual_seed(0)
    n = 100_000
    x = torch.randn(n, device="cuda") * 1e-2
    x0 = x.clone()
    thr = cp.sparse_threshold(x, 0.05, seed=3)
    wire = torch.empty_like(x)
    sent = torch.zeros(1, device="cuda", dtype=torch.int64)
    cp.wire_mask(x, wire, thr, sent)
    sel = x0.abs() >= thr
    assert sent.item() == int(sel.sum().item()) and 0.02 * n < sent.item() < 0.1 * n
    assert torch.equal(wire, torch.where(sel, x0.half().float(), torch.zeros_like(x0)))
    assert torch.equal(x, torch.where(sel, torch.zeros_like(x0), x0))          # the unsent part stays as residual
    # plain f16 wire: everything is sent, nothing stays
    y = x0.clone()
    cp.wire_mask(y, wire, None)
    assert torch.equal(wire, x0.half().float()) and torch.count_nonzero(y).item() == 0


def test_compact_and_lift_round_trip_matches_the_host_decoder():
    from orchestra import _orchestra as core
    from oxidized_neural_orchestra_b200.ops import compress as cp

    torch.manual_seed(1)
    n = 300_000
    x = torch.randn(n, device="cuda") * 1e-2
    x0 = x.clone()
    thr = cp.sparse_threshold(x, 0.02, seed=9)
    idx, val, count = cp.sparse_compact(x, thr, capacity=n // 8)
    c = count.item()
    sel = (x0.abs() >= thr).nonzero().flatten()
    assert c == sel.numel()
    assert torch.equal(idx[:c].long(), sel)                                      # ascending index order
    assert torch.equal(val[:c], x0[sel].half())
    assert torch.count_nonzero(x[sel]).item() == 0                              # sent entries leave the residual
    acc = torch.zeros(n, device="cuda")
    cp.sparse_lift(acc, idx, val, count)
    # the host codec encodes the same selection as runs and decodes it to the same dense vector
    enc = core.sparse_drop(x0.cpu().numpy(), float(thr.item()))
    host = np.asarray(core.sparse_lift(enc, np.zeros(n, dtype=np.float32)))
    assert np.array_equal(acc.cpu().numpy(), host)
    # an undersized buffer reports the true count so that the caller can fall back to the dense wire
    idx2, val2, count2 = cp.sparse_compact(x0.clone(), thr, capacity=16)
    assert count2.item() == c
