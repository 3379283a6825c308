"""Interval books, token clock and the fit search."""
import math

import pytest
import torch

from dew_b200.training import interval as I
from dew_b200.training.planning import FitSearch, NoPlanFits, Plan, ladder


def test_book_sums_and_nonfinite_streak():
    it = I.Interval({"log": 2, "checkpoint": 4})
    it.add(torch.tensor(6.0), torch.tensor(3.0), examples=2, tokens=10, flops=100.0)
    it.add(torch.tensor(float("nan")), torch.tensor(3.0), examples=2, tokens=10, committed=False)
    assert it.due(2) == ["log"] and it.due(4) == ["log", "checkpoint"] and it.due(3) == []
    row = it.take("log")
    assert row["loss"] == pytest.approx(2.0) and row["steps"] == 2 and row["nonfinite_steps"] == 1
    assert it.clock.consumed_tokens == 20 and it.clock.committed_tokens == 10
    assert I.streak_of(it.books["log"]).current == 1            # the streak survives the restart of the sums
    for _ in range(4):
        it.add(torch.tensor(float("inf")), torch.tensor(1.0))
    with pytest.raises(I.NonFiniteLoss):
        I.checked_finite(I.streak_of(it.books["log"]), 6, skips=True)
    it.add(torch.tensor(1.0), torch.tensor(1.0))
    assert I.streak_of(it.books["log"]).current == 0
    both = it.take("checkpoint")
    assert both["steps"] == 7 and math.isfinite(both["loss"])


def test_token_clock_control_round_trip_and_crossing():
    c = I.TokenClock()
    c.dispatched(4, 100)
    c.update_boundary()
    before = c.committed_tokens
    c.dispatched(4, 100)
    c.update_boundary()
    assert c.crossed(before, 150) and not c.crossed(before, 250)
    again = I.TokenClock.from_control(c.control())
    assert again.committed_tokens == 200 and again.consumed_examples == 8


def test_fit_search_walks_the_ladder():
    assert ladder(8)[:4] == [Plan(8, False), Plan(8, True), Plan(4, False), Plan(4, True)]
    # memory model: 10 GiB of state + 3 GiB per row, a third of the activations with rematerialisation
    gib = 1 << 30
    cost = lambda p: 10 * gib + p.microbatch * 3 * gib // (3 if p.remat else 1)
    s = FitSearch(8, capacity_bytes=24 * gib, limit_fraction=0.9, measure=cost)
    assert s.run() == Plan(8, True)                      # 18 GiB fits 21.6; 34 GiB without remat does not
    assert [t.fits for t in s.trials] == [False, True] and "remat" in s.report()
    with pytest.raises(NoPlanFits):
        FitSearch(2, capacity_bytes=8 * gib, measure=cost).run()


def test_fit_search_starts_where_an_earlier_run_settled(tmp_path):
    import torch
    from dew_b200.training.planning import PlanRecords, step_key
    gib = 1 << 30
    cost = lambda p: 10 * gib + p.microbatch * 3 * gib // (3 if p.remat else 1)
    records = PlanRecords(str(tmp_path / "cache" / "plans.json"))
    model = torch.nn.Linear(4, 4)
    key = step_key(model, (8, 128), device="B200")
    assert key == step_key(torch.nn.Linear(4, 4), (8, 128), device="B200") != step_key(model, (8, 256), device="B200") != step_key(torch.nn.Linear(4, 5), (8, 128), device="B200")
    first = FitSearch(8, capacity_bytes=16 * gib, limit_fraction=0.9, measure=cost)
    assert first.run(remembered=records, key=key) == Plan(4, True) and len(first.trials) == 4
    later = FitSearch(8, capacity_bytes=16 * gib, limit_fraction=0.9, measure=cost)
    assert later.run(remembered=records, key=key) == Plan(4, True) and len(later.trials) == 1          # no rung above it is tried again
    assert records.get("other") is None and records.get(key) == Plan(4, True)
    # a remembered plan that no longer fits (a smaller device) walks on down from there
    small = FitSearch(8, capacity_bytes=13 * gib, limit_fraction=0.9, measure=cost)
    assert small.run(remembered=records, key=key) == Plan(1, True) and small.trials[0].plan == Plan(4, True)


def test_pause_ends_the_run_at_a_fraction_and_a_resume_goes_on(tmp_path):
    import dew_b200 as dew
    from dew_b200.models import CausalTransformer
    from dew_b200.objectives.lm import LMObjective
    with pytest.raises(ValueError):
        dew.Pause(1.0)
    assert dew.Pause(0.5).at(10) == 5
    with pytest.raises(ValueError):
        dew.Pause(0.01).at(10)

    def trainer():
        torch.manual_seed(0)
        m = CausalTransformer(vocab_size=32, emb_features=16, num_layers=1, num_heads=2, num_kv_heads=2, head_dim=8, mlp_features=24, max_seq_len=8)
        return dew.Trainer(LMObjective(m, 8, ema_decay=None), dew.OptimConfig(learning_rate=1e-2), key=0, checkpoints=dew.Checkpoints(str(tmp_path / "run")))
    g = torch.Generator().manual_seed(0)
    data = [{"tokens": torch.randint(0, 32, (2, 9), generator=g)} for _ in range(8)]
    state = trainer().fit(list(data), steps=8, pause=dew.Pause(0.5), log_every=1000)
    assert state.step == 4
    state = trainer().fit(list(data), steps=8, log_every=1000)               # resumes from the pause's checkpoint
    assert state.step == 8


def test_checkpoint_integrity_passes_over_a_damaged_step(tmp_path):
    import warnings
    import dew_b200 as dew
    from dew_b200.checkpoints import CorruptCheckpoint
    from dew_b200.models import CausalTransformer
    from dew_b200.objectives.lm import LMObjective

    def trainer():
        torch.manual_seed(0)
        m = CausalTransformer(vocab_size=32, emb_features=16, num_layers=1, num_heads=2, num_kv_heads=2, head_dim=8, mlp_features=24, max_seq_len=8)
        return dew.Trainer(LMObjective(m, 8, ema_decay=None), dew.OptimConfig(learning_rate=1e-2), key=0,
                           checkpoints=dew.Checkpoints(str(tmp_path / "run"), keep=3))
    g = torch.Generator().manual_seed(0)
    data = [{"tokens": torch.randint(0, 32, (2, 9), generator=g)} for _ in range(6)]
    t = trainer()
    t.fit(list(data), steps=6, checkpoint_every=2, log_every=1000)
    ck = t.checkpoints
    ck.wait()
    assert ck.steps() == [2, 4, 6] and all(ck.verify(6).values()) and ck.resumed() == 6
    # damage the newest step's model file: flip a byte in the middle
    victim = next((tmp_path / "run" / "6").glob("*/tree.safetensors"))
    raw = bytearray(victim.read_bytes())
    raw[len(raw) // 2] ^= 0xFF
    victim.write_bytes(bytes(raw))
    assert not all(ck.verify(6).values())
    with pytest.raises(CorruptCheckpoint):
        ck.restore(None, 6)
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        assert ck.resumed() == 4
    assert any("integrity" in str(w.message) for w in caught)
    state = trainer().fit(list(data), steps=6, log_every=1000)        # resumes from step 4, not the damaged 6
    assert state.step == 6


def test_console_tracker_lines():
    import io
    import dew_b200 as dew
    ticks = iter([0.0, 2.0, 4.0])
    out = io.StringIO()
    t = dew.ConsoleTracker(steps=30, stream=out, clock=lambda: next(ticks))
    t.log(10, {"loss": torch.tensor(2.5), "tokens": 1000, "learning_rate": 3e-4})
    t.log(20, {"loss": 2.25, "tokens": 1000, "learning_rate": 3e-4})
    t.log(30, {"loss": 2.0, "tokens": 1000})
    lines = out.getvalue().splitlines()
    assert lines[0].startswith("step 10/30 | loss 2.5000 | learning_rate 3.000e-04")
    assert "5,000 tokens/s" in lines[1] and "0.200 s/step" in lines[1] and "eta 0:00:02" in lines[1]
    assert lines[2].startswith("step 30/30") and "eta 0:00:00" in lines[2]
    dew.Trackers(t, dew.MemoryTracker()).artifact(30, "grid", object())
    assert "artifact grid" in out.getvalue()


@pytest.mark.parametrize("kind", ["m3", "muon", "normuon", "lion", "adamw"])
def test_optimizer_state_of_every_kind_round_trips_through_a_checkpoint(tmp_path, kind):
    """Every tensor tree of the optimizer state (M3's slow / chunk / slow_direction beside mu / nu) is stored as tensors
    and comes back as tensors, so that the step after a resume equals the step of the run that was never stopped."""
    import dew_b200 as dew
    from dew_b200.models import CausalTransformer
    from dew_b200.objectives.lm import LMObjective

    def trainer(directory):
        torch.manual_seed(0)
        m = CausalTransformer(vocab_size=32, emb_features=16, num_layers=1, num_heads=2, num_kv_heads=2, head_dim=8, mlp_features=24, max_seq_len=8)
        opts = {"frequency": 2} if kind == "m3" else {}
        return dew.Trainer(LMObjective(m, 8, ema_decay=None), dew.OptimConfig(optimizer=kind, learning_rate=1e-3, optimizer_opts=opts), key=0,
                           checkpoints=dew.Checkpoints(str(directory), keep=4))
    g = torch.Generator().manual_seed(0)
    data = [{"tokens": torch.randint(0, 32, (2, 9), generator=g)} for _ in range(5)]
    whole = trainer(tmp_path / "whole").fit(list(data), steps=5, log_every=1000)
    first = trainer(tmp_path / "cut")
    first.fit(list(data), steps=3, log_every=1000)
    first.checkpoints.wait()
    restored = first.checkpoints.restore(None)
    from dew_b200.utils.trees import flatten
    for name, tree in restored.opt_state.items():
        if isinstance(tree, dict):
            assert all(isinstance(v, torch.Tensor) for v in flatten(tree).values()), name
    resumed = trainer(tmp_path / "cut").fit(list(data[3:]), steps=5, log_every=1000)      # a list has no position: hand it the rest
    a, b = flatten(whole.variables["params"]), flatten(resumed.variables["params"])
    assert a.keys() == b.keys()
    for k in a:
        assert torch.equal(a[k], b[k]), (kind, k)


def test_json_records_refuse_values_they_cannot_express(tmp_path):
    from dew_b200.utils.files import atomic_write_json, read_json
    atomic_write_json(tmp_path / "ok.json", {"a": torch.tensor(3), "b": (1, 2), "c": tmp_path})
    assert read_json(tmp_path / "ok.json")["a"] == 3
    with pytest.raises(TypeError):
        atomic_write_json(tmp_path / "bad.json", {"a": torch.zeros(3)})


def test_step_flops_are_counted_and_scale_with_the_batch():
    from dew_b200.models import CausalTransformer
    from dew_b200.objectives.lm import LMObjective
    from dew_b200.telemetry.instrumentation import model_flops_utilization, step_flops
    torch.manual_seed(0)
    m = CausalTransformer(vocab_size=64, emb_features=32, num_layers=2, num_heads=2, num_kv_heads=2, head_dim=16, mlp_features=64, max_seq_len=16, tie_embeddings=False)
    obj = LMObjective(m, 16, ema_decay=None)
    batch = {"tokens": torch.randint(0, 64, (4, 17))}
    f = step_flops(obj, batch)
    analytic = m.model_flops(4 * 16, 16) * 3
    assert 0.7 < f.total / analytic < 1.4, (f.total, analytic)            # counted FLOPs agree with 6 N D + attention
    assert 1.7 < f.backward / f.forward < 2.3
    half = step_flops(obj, batch, rows=2)
    assert abs(half.total - f.total) / f.total < 0.05                     # counted on two rows and scaled
    assert abs(model_flops_utilization(2.25e15, 1000.0) - 1.0) < 1e-9


def test_benchmark_step_smoke_and_perf_gate(tmp_path):
    import json
    from dew_b200.telemetry import benchmark_step, perf_gate
    rows = benchmark_step.run("cpu-smoke", ["causal_transformer"])
    assert rows and rows[0]["ms_p50"] > 0 and rows[0]["gflop_per_step"] > 0
    rec = tmp_path / "records.jsonl"
    rec.write_text("\n".join(json.dumps(r) for r in rows) + "\n" + json.dumps({"metric": "tok/s", "n_gpus": 1, "value": 100.0, "e2e": {"value": 98.0}}))
    gate = tmp_path / "gate.json"
    gate.write_text(json.dumps({"gates": [{"match": {"metric": "tok/s", "n_gpus": 1}, "field": "value", "min": 102, "tolerance": 0.03},
                                          {"match": {"metric": "tok/s"}, "field": "e2e.value", "min": 90},
                                          {"match": {"model": "causal_transformer"}, "field": "ms_p50", "max": 1e6}]}))
    assert perf_gate.main(["--records", str(rec), "--gate", str(gate)]) == 0       # 100 >= 102 * 0.97
    gate.write_text(json.dumps({"gates": [{"match": {"metric": "tok/s"}, "field": "value", "min": 120}, {"match": {"metric": "absent"}, "field": "value", "min": 1}]}))
    assert perf_gate.main(["--records", str(rec), "--gate", str(gate)]) == 1
