"""The span tracer, its Chrome-trace export and breakdown, and stamped benchmark records."""
import json

from dew_b200.telemetry.records import Records, compare, stamp
from dew_b200.telemetry.trace import Span, Tracer, breakdown, merge


def test_tracer_spans_export_and_breakdown(tmp_path):
    ticks = iter(range(0, 1000, 1))
    clock = lambda: next(ticks) * 1e-3                                      # one millisecond per reading
    idle = Tracer(enabled=False, clock=clock)
    with idle.span("nothing") as s:
        assert s is None
    assert idle.spans == []
    t = Tracer(enabled=True, device_time=False, rank=3, clock=clock)
    with t.span("step", index=7):
        with t.span("forward"):
            pass
        with t.span("all_reduce"):
            pass
    with t.span("all_gather"):
        pass
    names = [(s.name, s.depth) for s in t.spans]
    assert names == [("forward", 1), ("all_reduce", 1), ("step", 0), ("all_gather", 0)]
    summary = t.summary()
    assert summary["step"]["count"] == 1 and summary["step"]["host_us"] > summary["forward"]["host_us"] > 0
    path = t.export(str(tmp_path / "rank3.json"))
    events = json.load(open(path))["traceEvents"]
    xs = [e for e in events if e["ph"] == "X"]
    assert len(xs) == 4 and all(e["pid"] == 3 and e["tid"] == 0 for e in xs) and xs[2]["args"] == {"index": 7}
    other = Tracer(enabled=True, device_time=False, rank=4, clock=clock)
    with other.span("step"):
        pass
    merged = merge([path, other.export(str(tmp_path / "rank4.json"))], str(tmp_path / "all.json"))
    assert {e["pid"] for e in json.load(open(merged))["traceEvents"]} == {3, 4}
    b = breakdown(t.spans)
    step = next(s for s in t.spans if s.name == "step")
    gather = next(s for s in t.spans if s.name == "all_gather")
    assert b["collective_us"] == gather.host_us and b["compute_us"] == step.host_us            # only top-level spans are counted
    spans = [Span("matmul", 0, 10, 8.0), Span("all_reduce", 10, 5, 4.0)]
    assert breakdown(spans, wall_us=20.0) == {"compute_us": 8.0, "collective_us": 4.0, "idle_us": 8.0, "wall_us": 20.0}
    t.clear()
    assert t.spans == []


def test_records_are_stamped_appended_and_compared(tmp_path):
    s = stamp()
    assert {"time", "host", "torch", "device"} <= set(s)
    rec = Records(str(tmp_path / "bench" / "records.jsonl"), stamp_fn=lambda: {"device": "B200", "commit": "abc"})
    rec.append({"kernel": "gemm", "shape": "4096", "ms": 0.10})
    rec.append({"kernel": "gemm", "shape": "8192", "ms": 0.80})
    rec.append({"kernel": "gemm", "shape": "4096", "ms": 0.09})
    rows = rec.read()
    assert len(rows) == 3 and rows[0]["device"] == "B200" and rec.latest(kernel="gemm", shape="4096")["ms"] == 0.09 and rec.latest(kernel="conv") is None
    after = [{"kernel": "gemm", "shape": "4096", "ms": 0.06}, {"kernel": "gemm", "shape": "16384", "ms": 5.0}]
    diff = compare(rows, after, ("kernel", "shape"), "ms")
    assert len(diff) == 1 and diff[0]["before"] == 0.09 and abs(diff[0]["ratio"] - 0.06 / 0.09) < 1e-12


def test_trainer_steps_appear_in_the_process_tracer():
    import torch
    import dew_b200 as dew
    from dew_b200.models import CausalTransformer
    from dew_b200.objectives.lm import LMObjective
    from dew_b200.telemetry.trace import TRACER
    m = CausalTransformer(vocab_size=16, emb_features=16, num_layers=1, num_heads=2, head_dim=8, mlp_features=32, max_seq_len=8, qk_norm=False)
    tr = dew.Trainer(LMObjective(m, 7), dew.OptimConfig(learning_rate=1e-3), tracker=dew.MemoryTracker())
    batch = {"tokens": torch.randint(0, 16, (4, 8))}
    TRACER.clear()
    tr.fit([batch] * 2, steps=2, log_every=10)
    assert TRACER.spans == []                                              # idle by default
    TRACER.enabled = True
    try:
        tr.fit([batch] * 3, steps=3, log_every=10)
    finally:
        TRACER.enabled = False
    steps = [s for s in TRACER.spans if s.name == "train_step"]
    assert len(steps) == 3 and [s.args["step"] for s in steps] == [0, 1, 2] and all(s.host_us > 0 for s in steps)
    TRACER.clear()
