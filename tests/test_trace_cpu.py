"""Run tracing (Chrome trace JSON) and the metrics JSONL sink, without a GPU."""
import json

from oxidized_neural_orchestra_b200.utils.trace import MetricsSink, Tracer


def test_tracer_writes_a_loadable_chrome_trace(tmp_path):
    t = Tracer(str(tmp_path / "trace_{rank}.json"), rank=3)
    with t.span("epoch", epoch=0):
        with t.span("report_and_decide"):
            pass
    t.instant("switch", to="parameter_server")
    path = t.write()
    assert path.endswith("trace_3.json")
    doc = json.load(open(path))
    names = [e["name"] for e in doc["traceEvents"]]
    assert {"process_name", "epoch", "report_and_decide", "switch"} <= set(names)
    spans = [e for e in doc["traceEvents"] if e.get("ph") == "X"]
    assert all(e["pid"] == 3 and e["dur"] >= 0 for e in spans)
    outer = next(e for e in spans if e["name"] == "epoch")
    inner = next(e for e in spans if e["name"] == "report_and_decide")
    assert outer["ts"] <= inner["ts"] and inner["ts"] + inner["dur"] <= outer["ts"] + outer["dur"] + 1.0


def test_tracer_and_sink_are_inert_without_a_path(tmp_path):
    t = Tracer(None)
    with t.span("x"):
        pass
    assert t.write() is None and not t.on
    s = MetricsSink(None)
    s.write(a=1)
    assert not s.on


def test_metrics_sink_appends_one_json_record_per_line(tmp_path):
    s = MetricsSink(str(tmp_path / "m.jsonl"), rank=1)
    s.write(epoch=1, loss=0.5, samples_per_sec=1000.0)
    s.write(epoch=2, loss=0.4, samples_per_sec=1100.0)
    assert s.path.endswith("m.jsonl.rank1")
    recs = [json.loads(l) for l in open(s.path)]
    assert [r["epoch"] for r in recs] == [1, 2] and all(r["rank"] == 1 and "time" in r for r in recs)
