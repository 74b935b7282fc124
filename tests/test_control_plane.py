"""Control-plane logic of the C++ core against the reference's own golden cases.

Goldens come from orchestrator/src/calculator/tsp.rs:121-180, bipartite.rs:141-227,
orchestrator/src/configs/adapter.rs:1204-1332, comms/src/sparse/protocol.rs:146-224 and the documents
in docs/config-schema.md.
"""
import json
import math
import os

import numpy as np
import pytest

from orchestra import _orchestra as core


# ---- calculators --------------------------------------------------------------------------------
def test_tsp_goldens():
    assert core.tsp_cycle(10, []) == []
    assert core.tsp_cycle(3, [(0, 1, 1), (0, 2, 2), (1, 2, 3)]) == [0, 1, 2]
    assert core.tsp_cycle(4, [(0, 1, 1), (0, 2, 1000), (0, 3, 1), (1, 2, 1), (1, 3, 1000), (2, 3, 1)]) == [0, 1, 2, 3]
    edges = [(0, 1, 1000), (0, 2, 1), (0, 3, 1), (0, 4, 1000), (1, 2, 1000), (1, 3, 1), (1, 4, 1), (2, 3, 1000),
             (2, 4, 1), (3, 4, 1000)]
    assert core.tsp_cycle(5, edges) == [0, 2, 4, 1, 3]
    assert core.tsp_cycle(1, []) == [0]  # a ring of one rank


def test_central_vertices_goldens():
    assert core.central_vertices(0, [], 1) == []
    assert core.central_vertices(3, [(0, 1, 1), (0, 2, 1), (1, 2, 1)], 0) == []
    assert core.central_vertices(3, [(0, 1, 5), (0, 2, 2), (1, 2, 2)], 2) == [0, 1]
    assert core.central_vertices(4, [(0, 1, 1), (0, 2, 1), (0, 3, 1), (1, 2, 1000), (1, 3, 1000), (2, 3, 1000)], 3) == [1, 2, 3]
    edges = [(0, 1, 1000), (0, 2, 1), (0, 3, 1000), (0, 4, 1), (1, 2, 1), (1, 3, 1000), (1, 4, 1), (2, 3, 1), (2, 4, 1),
             (3, 4, 1)]
    assert core.central_vertices(5, edges, 3) == [0, 1, 3]
    assert core.central_vertices(3, [(0, 1, 1)], 7) == [0, 1, 2]


# ---- adapter ------------------------------------------------------------------------------------
def test_dataset_partitions_and_lpt():
    assert core.dataset_partitions(3, 3) == [(0, 1), (1, 2), (2, 3)]
    assert core.dataset_partitions(4, 3) == [(0, 2), (2, 3), (3, 4)]  # the first `rem` get one more row
    assert core.dataset_partitions(10, 4) == [(0, 3), (3, 6), (6, 8), (8, 10)]
    # largest first into the least loaded bin, ties to the lowest bin
    assert core.balanced_partitions([401536, 57034], 2) == [[0], [1]]
    assert core.balanced_partitions([5, 4, 3, 3, 2], 2) == [[0, 3], [1, 2, 4]]


MODEL = {"layers": [
    {"conv": {"input_dim": [1, 28, 28], "kernel_dim": [32, 1, 3], "stride": 1, "padding": 1, "init": "kaiming",
              "act_fn": {"relu": {"slope": 0.0}}}},
    {"max_pooling": {"input_dim": [32, 28, 28], "filter_size": 2, "stride": 2, "padding": 0}},
    {"dense": {"output_size": 128, "init": "xavier_uniform", "act_fn": {"re_l_u": {"slope": 0.0}}}},
    {"dense": {"output_size": 10, "init": {"normal": {"mean": 0.0, "std_dev": 0.1}}, "act_fn": "softmax"}},
]}


def _training(algorithm, n=4, **extra):
    t = {"addrs": [f"cpu:{i}" for i in range(n)], "algorithm": algorithm,
         "dataset": {"src": {"inline": {"samples": [], "labels": [], "rows": 103}}, "x_size": 784, "y_size": 10},
         "optimizer": {"adam": {"lr": 0.001, "b1": 0.9, "b2": 0.999, "eps": 1e-8}}, "loss_fn": "cross_entropy",
         "batch_size": 8, "max_epochs": 2, "offline_epochs": 0, "seed": 7}
    t.update(extra)
    return t


def test_model_config_round_trip_accepts_both_relu_spellings():
    out = json.loads(core.normalize_model_config(json.dumps(MODEL)))
    assert out["layers"][2]["dense"]["act_fn"] == {"relu": {"slope": 0.0}}
    assert out["layers"][1]["max_pooling"]["act_fn"] is None
    assert core.model_param_count(json.dumps(MODEL), 784) == 32 * 9 + 32 + (6272 + 1) * 128 + 129 * 10


def test_plan_parameter_server_layer_sharding():
    plan = json.loads(core.adapt_configs(json.dumps(MODEL), json.dumps(_training(
        {"parameter_server": {"nservers": 2, "synchronizer": "barrier", "store": "blocking"}}))))
    assert plan["algorithm"] == "parameter_server"
    assert len(plan["servers"]) == 2 and len(plan["workers"]) == 2
    # LPT: the big dense layer alone on server 0; conv + last dense on server 1, in model order
    sizes = plan["server_sizes"]
    assert sizes == [(6272 + 1) * 128, 32 * 9 + 32 + 1290]
    assert plan["server_ordering"] == [1, 0, 1]
    lo = plan["layer_offsets"]
    assert lo[0] == [1, 0, 320] and lo[2] == [0, 0, sizes[0]] and lo[3] == [1, 320, 320 + 1290]
    assert plan["server_ranges"][1] == [[0, 320], [320 + sizes[0], 320 + sizes[0] + 1290]]
    # the worker's optimizer is plain gradient descent, the server keeps Adam (adapter.rs:737-758)
    w = plan["workers"][0]["spec"]
    assert "gradient_descent" in w["trainer"]["optimizer"]
    assert "adam" in plan["servers"][0]["spec"]["optimizer"]
    assert plan["servers"][0]["spec"]["synchronizer"] == {"barrier": {"barrier_size": 2}}
    # partitions over the workers only
    assert [w["partition"] for w in plan["workers"]] == [[0, 52], [52, 103]]
    # fan_in / fan_out are the flattened layer sizes, also for conv (adapter.rs:1116-1133)
    dist = plan["layers"][0]["param_gen"]["rand"]
    assert dist["distribution"] == {"kaiming": {"fan_in": 784}} and dist["limit"] == 320


def test_plan_all_reduce_and_switch():
    plan = json.loads(core.adapt_configs(json.dumps(MODEL), json.dumps(_training("all_reduce", n=3))))
    assert [w["rank"] for w in plan["workers"]] == [0, 1, 2] and plan["servers"] == []
    assert plan["workers"][1]["spec"]["algorithm"]["all_reduce"]["pos"] == 1
    assert plan["workers"][0]["spec"]["algorithm"]["all_reduce"]["amount_of_layers"] == 3
    plan = json.loads(core.adapt_configs(json.dumps(MODEL), json.dumps(_training(
        {"strategy_switch": {"nservers": 1, "synchronizer": "non_blocking", "store": "wild"}}, n=3,
        early_stopping={"tolerance": 1e-4}))))
    acts = plan["switch"]["post_actions"]
    assert [a["action"] for a in acts] == ["upgrade", "switch", "switch"]
    assert acts[0]["ranges"] == [[0, plan["n_params"]]]
    assert plan["switch"]["window"] == 6 and plan["switch"]["threshold"] == 0.01
    assert plan["early_stopping"] == {"window": 3, "tolerance": 1e-4}
    # strategy switch partitions the data over every address (adapter.rs:142-143)
    assert [w["partition"] for w in plan["workers"]] == [[0, 35], [35, 69], [69, 103]]


def test_even_sharding_and_global_batch():
    t = _training({"parameter_server": {"nservers": 2, "synchronizer": "barrier", "store": "blocking"}}, n=8,
                  b200={"sharding": "even", "global_batch": 20, "colocate": True, "sync_every": "step"})
    plan = json.loads(core.adapt_configs(json.dumps(MODEL), json.dumps(t)))
    P = plan["n_params"]
    r0, r1 = plan["server_ranges"]
    assert r0[0][0] == 0 and r0[0][1] == r1[0][0] and r1[0][1] == P and r0[0][1] % 4 == 0
    assert len(plan["workers"]) == 8
    assert [w["spec"]["trainer"]["batch_size"] for w in plan["workers"]] == [3, 3, 3, 3, 2, 2, 2, 2]


@pytest.mark.parametrize("mutate,msg", [
    (lambda m, t: m.update(layers=[]), "at least one layer"),
    (lambda m, t: t.update(addrs=[]), "at least one network address"),
    (lambda m, t: t.update(algorithm={"parameter_server": {"nservers": 4, "synchronizer": "barrier", "store": "blocking"}}),
     "amount of workers"),
    (lambda m, t: t.update(batch_size=1000), "exceeds dataset size"),
    (lambda m, t: t["dataset"].update(y_size=11), "must match the dataset's y_size"),
    (lambda m, t: t["dataset"].update(x_size=100), "layer expects an input"),
    (lambda m, t: t.update(optimizer={"adam": {"lr": -1.0, "b1": 0.9, "b2": 0.999, "eps": 1e-8}}), "positive"),
    (lambda m, t: t.update(serializer={"sparse_capable": {"r": 1.5}}), "[0, 1]"),
])
def test_validator_rejections(mutate, msg):
    m, t = json.loads(json.dumps(MODEL)), _training("all_reduce")
    mutate(m, t)
    with pytest.raises(ValueError) as e:
        core.adapt_configs(json.dumps(m), json.dumps(t))
    assert msg in str(e.value)


# ---- codecs -------------------------------------------------------------------------------------
def test_sparse_codec_goldens():
    golden = bytes([4, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 2, 0, 0, 0, 0, 60, 0, 188, 1, 0, 0, 0, 1, 0, 0, 0, 0, 64])
    grad = np.array([1.0, -1.0, 0.0, 2.0], dtype=np.float32)
    assert core.sparse_drop(grad, 1.0) == golden
    assert core.sparse_lift(golden, np.zeros(4, dtype=np.float32)).tolist() == [1.0, -1.0, 0.0, 2.0]
    short = bytes([3, 0, 0, 0, 0, 0, 0, 0, 1, 0, 0, 0, 2, 0, 0, 0, 0, 60, 0, 188])
    assert core.sparse_lift(short).tolist() == [0.0, 1.0, -1.0]
    with pytest.raises(RuntimeError):
        core.sparse_lift(golden[:-1], np.zeros(4, dtype=np.float32))
    with pytest.raises(RuntimeError):
        core.sparse_lift(bytes([1, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 2, 0, 0, 0, 0, 60, 0, 60]))


def test_f16_matches_numpy_and_threshold_quantile():
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(5000).astype(np.float32) * s for s in (1e-6, 1e-3, 1.0, 300.0, 1e5)])
    with np.errstate(over="ignore"):
        assert np.array_equal(core.f16_round_trip(x), x.astype(np.float16).astype(np.float32))
    g = rng.standard_normal(100000).astype(np.float32)
    thr = core.sparse_threshold(g, 0.9, 3)
    kept = float((np.abs(g) >= thr).mean())
    assert 0.85 < kept < 0.95  # k = floor(n (1 - r)): the threshold is the (1-r)-quantile
    assert core.sparse_threshold(np.zeros(10, dtype=np.float32), 0.5, 0) == pytest.approx(6.103515625e-05)
    sparse, _, payload = core.compress_gradient(g, True, 0.01, 1)
    assert sparse and len(payload) < 2 * g.size
    sparse, _, payload = core.compress_gradient(g, True, 1.0, 1)  # everything kept: dense is smaller
    assert not sparse and len(payload) == 2 * g.size


# ---- trackers -----------------------------------------------------------------------------------
def test_trackers_follow_reference_rules():
    c = core.ConvergenceTracker(3, 0.1)
    for v, want in [(1.0, False), (0.95, False), (0.9, True)]:
        c.record(v)
        assert c.converged() is want
    c.record(0.5)
    assert not c.converged()
    s = core.SwitchTracker(3, 0.01)
    for v in (1.0, 0.999, 0.9985):
        s.record(v)
    assert s.should_switch()
    s.record(0.5)
    assert not s.should_switch()
    r = core.LossRecorder()
    r.record(0, 1.0)
    assert r.max(2) is None
    r.record(1, float("nan"))
    assert r.max(2) is None  # non-normal losses are ignored
    r.record(1, 3.0)
    assert r.max(2) == 3.0 and r.mean(2) == 2.0
    p = core.SessionPolicy(2)
    p.enable_early_stopping(3, 1e-3)
    seen = []
    for k in range(3):
        seen.append(p.on_losses(0, [0.5]))
        seen.append(p.on_losses(1, [0.4]))
    assert seen == [0, 0, 0, 0, 0, 1] and p.stopped()


# ---- files --------------------------------------------------------------------------------------
def test_safetensors_layout_and_reload(tmp_path):
    n = core.model_param_count(json.dumps(MODEL), 784)
    params = np.arange(n, dtype=np.float32)
    path = str(tmp_path / "m.safetensors")
    core.save_safetensors(path, json.dumps(MODEL), 784, params)
    tensors = {name: (shape, data) for name, shape, data in core.load_safetensors(path)}
    assert tensors["layer_0.weight"][0] == [32, 1, 3, 3] and tensors["layer_0.bias"][0] == [32]
    assert tensors["layer_1.weight"][0] == [0] and tensors["layer_1.bias"][0] == [0]  # max-pool (trained_model.rs:81-113)
    assert tensors["layer_2.weight"][0] == [6272, 128] and tensors["layer_3.bias"][0] == [10]
    assert np.array_equal(tensors["layer_2.weight"][1], params[320:320 + 6272 * 128])
    assert np.array_equal(tensors["layer_3.bias"][1], params[-10:])
    st = pytest.importorskip("safetensors.numpy")
    loaded = st.load_file(path)
    assert loaded["layer_3.weight"].shape == (128, 10)
    assert np.array_equal(loaded["layer_3.weight"].reshape(-1), params[-1290:-10])


def test_csv_conversion_skips_header_and_caches(tmp_path):
    p = tmp_path / "d.csv"
    p.write_text("a,b,c\n1,2,3\n\n4.5, 5 ,6\n")
    out = core.ensure_binary_dataset(str(p))
    assert out.endswith("d.bin")
    assert core.read_f32_file(out).tolist() == [1.0, 2.0, 3.0, 4.5, 5.0, 6.0]
    p.write_text("9,9,9\n")
    assert core.read_f32_file(core.ensure_binary_dataset(str(p))).tolist()[:3] == [1.0, 2.0, 3.0]  # cached
    t = tmp_path / "t.tsv"
    t.write_text("1\t2\n3\t4\n")
    assert core.read_f32_file(core.ensure_binary_dataset(str(t)), 1, 2).tolist() == [2.0, 3.0]
    assert core.ensure_binary_dataset(str(tmp_path / "x.bin")) == str(tmp_path / "x.bin")


def test_ownership_boundaries_snap_to_row_blocks_for_pushed_gradients():
    """Even flat shards moved to 128-row blocks of the weight matrices (biases never split), still a partition."""
    from oxidized_neural_orchestra_b200.parallel.sync import even_ranges
    from oxidized_neural_orchestra_b200.runtime.gpu_rank import snap_to_row_blocks

    dims = [(512, 1024), (1024, 1024), (1024, 12)]
    plan_layers, eng_layers, off = [], [], 0
    for i, o in dims:
        plan_layers.append({"offset": off})
        eng_layers.append({"kind": "dense", "in": i, "out": o})
        off += i * o + o
    n, n_pad = off, (off + 15) // 16 * 16
    for owners in (2, 3, 4):
        ranges = even_ranges(n_pad, list(range(owners)), 4)
        snapped = snap_to_row_blocks(ranges, plan_layers, eng_layers, n, n_pad)
        flat = sorted(r for rs in snapped for r in rs)
        assert flat[0][0] == 0 and flat[-1][1] == n_pad
        assert all(a[1] == b[0] for a, b in zip(flat, flat[1:]))                 # contiguous, no overlap
        starts = {pl["offset"]: (i, o) for pl, (i, o) in zip(plan_layers, dims)}
        for b, _ in flat[1:]:
            # every interior boundary is a layer start, a bias start, or a multiple of 128 rows inside a weight block
            ok = False
            for w0, (i, o) in starts.items():
                if b == w0 or b == w0 + i * o or (w0 < b < w0 + i * o and (b - w0) % (128 * o) == 0):
                    ok = True
            assert ok, (owners, b)


def test_pre_reduce_plan_splits_every_owned_range_among_owner_and_idle_partners():
    """Four owners on eight ranks: every owned range is cut in two at a multiple of 64, the owner sums the first part and its
    idle partner the second; together the parts tile the owned ranges exactly. Layouts that do not allow it return None."""
    from oxidized_neural_orchestra_b200.parallel.sync import pre_reduce_plan

    layers = [(0, 8192 * 64 + 64), (8192 * 64 + 64, 8192 * 64 + 64 + 1000 * 64 + 1000)]
    own = [[] for _ in range(8)]
    for b, e in layers:                       # striped: a quarter of every layer per owner (ranks 0..3)
        cuts = [b + (e - b) * j // 4 // 64 * 64 for j in range(4)] + [e]
        for o in range(4):
            own[o].append((cuts[o], cuts[o + 1]))
    reduce_at, finish_at, fwd = pre_reduce_plan(own, 16)
    assert fwd == {4: 0, 5: 1, 6: 2, 7: 3}
    for o in range(4):
        parts = sorted(reduce_at[o] + reduce_at[o + 4])
        assert [p[0] for p in parts[::2]] == [b for b, _ in own[o]] and [p[1] for p in parts[1::2]] == [e for _, e in own[o]]
        assert all(parts[i][1] == parts[i + 1][0] for i in range(0, len(parts), 2))      # the two parts of a range meet
        assert finish_at[o] == reduce_at[o + 4] and all(b % 64 == 0 for b, _ in finish_at[o])
        mine, theirs = sum(e - b for b, e in reduce_at[o]), sum(e - b for b, e in reduce_at[o + 4])
        assert abs(mine - theirs) <= 64 * len(own[o])
    # one owner, three idle ranks: four parts per range
    reduce_at, finish_at, fwd = pre_reduce_plan([[(0, 4096)], [], [], []], 16)
    assert reduce_at == [[(0, 1024)], [(1024, 2048)], [(2048, 3072)], [(3072, 4096)]] and finish_at[0] == [(1024, 4096)]
    assert fwd == {1: 0, 2: 0, 3: 0}
    assert pre_reduce_plan([[(0, 512)], [(512, 1024)]], 16) is None                  # nobody idle
    assert pre_reduce_plan([[(0, 512)], [(512, 1024)], []], 16) is None              # idle ranks do not divide among the owners
    assert pre_reduce_plan([[(0, 1004)], []], 16) is None                            # a range end that is not a multiple of 8
    assert pre_reduce_plan([[(i * 64, i * 64 + 64) for i in range(0, 40, 2)], []], 16) is None   # range table too long
