"""Decision models: typed questions laid out with a state, answered from one forward pass, trained with proper scoring rules,
calibrated, served in the JSON wire form."""
import json
import math

import numpy as np
import pytest
import torch

import dew_b200 as dew
from dew_b200.decision import (AURC, ECE, Abstention, Accuracy, BidirectionalBackbone, Binning, Brier, Budget, Calibration, Choice, Decide,
                               DecisionHead, DecisionInputs, DecisionModel, DecisionObjective, Decisions, EntropyConfidence, Example,
                               Finalists, Group, GroupedExamples, JevConfidence, JointSchemaHead, Knockout, LabelReadout, Layout, LogLoss,
                               MacroF1, Noul, Question, RankedProbability, Refused, Score, Scored, SlotReadout, Spherical, Temperatures,
                               TopProbability, bucket, collate, decisions, first_fit, measure, mixture, usage_of)
from dew_b200.decision.task import knocked_out, near_equal
from dew_b200.eval.metrics import expected_calibration_error
from dew_b200.models import CausalTransformer
from dew_b200.objectives.base import Step


# ------------------------------------------------------------------------------------------------ questions
def test_questions_options_answers_and_wire_round_trip():
    n = Noul("is it spam?", {"true": "unsolicited"})
    c = Choice("which colour", {"red": "warm", "blue": None})
    s = Score("how urgent", ["not", "somewhat", "very"])
    assert n.options == ("false", "true") and c.options == ("red", "blue") and s.options == ("0", "1", "2")
    assert n.answer([0.25, 0.75]).noul == 0.75
    assert c.answer([0.2, 0.8]).choice == "blue"
    assert abs(s.answer([0.0, 0.5, 0.5]).score - 1.5) < 1e-12
    for q in (n, c, s):
        assert Question.from_wire(json.loads(json.dumps(q.wire()))) == q
    assert c.index("blue") == 1 and c.index(0) == 0 and n.index(True) == 1
    with pytest.raises(ValueError):
        c.index("green")
    with pytest.raises(ValueError):
        Choice("x", ["a", "a"])
    with pytest.raises(ValueError):
        Score("x", ["only"])
    with pytest.raises(ValueError):
        Question.from_wire({"type": "rank", "instructions": "x"})
    with pytest.raises(ValueError):
        c.answer([0.5, 0.6])


def test_confidences():
    c = Choice("q", ["a", "b", "c", "d"])
    jev = JevConfidence()
    assert abs(jev(c, [0.7, 0.1, 0.1, 0.1]) - (0.7 - 0.25) / 0.75) < 1e-12
    assert jev(c, [0.25] * 4) == 0.0 and jev(Choice("q", ["only"]), [1.0]) == 1.0
    s = Score("q", ["a", "b", "c"])
    assert jev(s, [0, 1, 0]) == 1.0 and jev(s, [0.5, 0, 0.5]) == 0.0
    assert TopProbability()(c, [0.7, 0.1, 0.1, 0.1]) == 0.7
    assert abs(EntropyConfidence()(c, [0.25] * 4)) < 1e-12 and EntropyConfidence()(c, [1, 0, 0, 0]) == 1.0


# ------------------------------------------------------------------------------------------------ scoring rules
def test_scoring_rules_are_zero_when_right_and_proper():
    opts = torch.tensor([[True, True, True, False]])
    sure = torch.tensor([[50.0, 0.0, 0.0, 99.0]])           # the value past the options must not matter
    t = torch.tensor([[1.0, 0, 0, 0]])
    ordinal = torch.tensor([True])
    for rule in (LogLoss(), Brier(), Spherical(), RankedProbability()):
        assert float(rule.charge(sure, t, opts, ordinal)) < 1e-6
    # proper: the expected charge under a true distribution is least at that distribution
    true = torch.tensor([0.6, 0.3, 0.1, 0.0])
    def expected(rule, forecast):
        lg = torch.log(forecast.clamp_min(1e-9))[None].repeat(3, 1)
        return float((rule.charge(lg, torch.eye(4)[:3], opts.repeat(3, 1), ordinal.repeat(3)) * true[:3]).sum())
    for rule in (LogLoss(), Brier(), Spherical(), RankedProbability(), LogLoss() + 0.5 * Brier()):
        honest = expected(rule, true)
        for other in (torch.tensor([0.8, 0.15, 0.05, 0]), torch.tensor([0.4, 0.4, 0.2, 0]), torch.tensor([1 / 3, 1 / 3, 1 / 3, 0])):
            assert honest <= expected(rule, other) + 1e-6, rule.name
    assert float(RankedProbability().charge(sure * 0, t, opts, torch.tensor([False]))) == 0.0
    assert (LogLoss() + 0.5 * Brier()).name == "log_loss+0.5*brier"
    with pytest.raises(ValueError):
        LogLoss() * -1.0
    # rps: a forecast one level off costs less than one two levels off
    far = RankedProbability().charge(torch.tensor([[0.0, 0.0, 50.0, 0.0]]), t, opts, ordinal)
    near = RankedProbability().charge(torch.tensor([[0.0, 50.0, 0.0, 0.0]]), t, opts, ordinal)
    assert float(near) < float(far)


# ------------------------------------------------------------------------------------------------ layout
QS = {"parity": Choice("is the number even or odd", ["even", "odd"]), "big": Noul("is the number at least 500"),
      "size": Score("how large is the number", ["small", "medium", "large"])}


@pytest.mark.parametrize("shape", ["marker", "state_first", "joint"])
def test_layout_places_markers_spans_and_counts_cuts(shape):
    lay = Layout(shape=shape, max_len=320, head_max_len=280)
    rows = lay.rows("the number is 123", QS)
    assert len(rows) == (1 if shape == "joint" else 3)
    sp = lay.specials
    for r in rows:
        assert len(r.tokens) == len(r.token_kind) <= 320 and r.cut == {} and r.state_kept == r.state_tokens
        for qi, name in enumerate(r.names):
            assert len(r.markers[qi]) == len(QS[name].options) == r.counts[qi]
            for m, (a, b) in zip(r.markers[qi], r.spans[qi]):
                assert r.tokens[m] == sp.marker
                assert (m == a - 1) if shape == "marker" else (m == b)            # marker before / after its option
                assert sp.marker not in r.tokens[a:b]
            first = lay.tokenizer.decode(r.tokens[r.spans[qi][0][0]:r.spans[qi][0][1]])
            assert first.startswith(QS[name].options[0])
            assert QS[name].kind in lay.tokenizer.decode(r.tokens[r.asked[qi][0]:r.asked[qi][1]])
    # a long state keeps its first tokens and the cut is counted
    long = lay.rows("x" * 1000, {"parity": QS["parity"]})[0]
    assert len(long) == 320 and long.state_tokens == 1000 and long.cut["state"] == 1000 - long.state_kept
    usage = usage_of([long])
    assert usage.truncated and usage.cut["state"] == (1, 1000 - long.state_kept)
    # options that read alike are refused
    with pytest.raises(Refused) as e:
        Layout(shape=shape, max_len=64, head_max_len=8).rows("s", {"q": Choice("pick", {"aaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaa1": None,
                                                                                          "aaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaaa2": None})})
    assert e.value.reason == "options_alike"


def test_head_budget_cuts_longest_options_first():
    lay = Layout(shape="state_first", max_len=256, head_max_len=60)
    q = Choice("pick", {"a": "short", "b": "a very long description " * 5})
    r = lay.rows("state", {"q": q})[0]
    (a0, a1), (b0, b1) = r.spans[0]
    assert r.cut["options"] > 0 and (a1 - a0) == len(lay.piece("a: short"))          # the short option is whole
    assert lay.labels is False and r.label_ids is None


def test_first_fit_packing_and_collation():
    lay = Layout(shape="state_first", max_len=128, head_max_len=96)
    rows = []
    for i in range(6):
        rows += lay.rows("n" * (3 + 5 * i), {"parity": QS["parity"]})
    windows, left = first_fit(rows, 256)
    assert not left and sorted(i for w in windows for i in w) == list(range(6))
    assert all(sum(len(rows[i]) for i in w) <= 256 for w in windows) and len(windows) < 6
    inputs, where = collate(rows, windows, 256, max(len(w) for w in windows), 2)
    for i, r in enumerate(rows):
        (b, q), = where[i]
        seg = int(inputs.segment_of[b, q])
        span = (inputs.segment_ids[b] == seg).nonzero().flatten()
        assert len(span) == len(r) and inputs.tokens[b, span].tolist() == r.tokens
        assert inputs.positions[b, span].tolist() == list(range(len(r)))
        assert inputs.tokens[b, inputs.markers[b, q]].tolist() == [lay.specials.marker] * 2
        assert int(inputs.row_end[b, q]) == int(span[-1])
    with pytest.raises(ValueError):
        first_fit(rows, 16)
    _, left = first_fit(rows, 128, max_windows=1)
    assert left


# ------------------------------------------------------------------------------------------------ heads
@pytest.mark.parametrize("shape,head", [("marker", "decision"), ("state_first", "decision"), ("joint", "joint"), ("state_first", "labels"),
                                        ("state_first", "slots")])
def test_heads_score_only_real_options_and_ignore_other_rows(shape, head):
    torch.manual_seed(0)
    lay = Layout(shape=shape, max_len=200, head_max_len=150, labels=head in ("labels", "slots"))
    bb = BidirectionalBackbone(260, 64, 1, max_len=256)
    h = {"decision": lambda: DecisionHead(64, 1), "joint": lambda: JointSchemaHead(64), "labels": lambda: LabelReadout(),
         "slots": lambda: SlotReadout(64, slots=8, head_dim=16)}[head]()
    model = DecisionModel(bb, h).eval()
    rows_a = lay.rows("the number is 12", QS)
    rows_b = lay.rows("a quite different state, 977", QS)
    Q = len(rows_a[0].names)
    alone, _ = collate(rows_a, [[i] for i in range(len(rows_a))], 200, Q, 4)
    both, where = collate(rows_a + rows_b, [[i, i + len(rows_a)] for i in range(len(rows_a))], 400, 2 * Q, 4)
    with torch.no_grad():
        la, lb = model(alone), model(both)
    assert la.shape == (len(rows_a), Q, 4)
    assert torch.isinf(la[~alone.options]).all() and torch.isfinite(la[alone.options]).all()
    # a row's logits do not depend on what else shares its window
    for i in range(len(rows_a)):
        for qi, (b, q) in enumerate(where[i]):
            k = rows_a[i].counts[qi]
            assert torch.allclose(la[i, qi, :k], lb[b, q, :k], atol=1e-4), (shape, head)


# ------------------------------------------------------------------------------------------------ training + calibration + serving
def _number_examples(n, seed):
    g = np.random.default_rng(seed)
    out = []
    for v in g.integers(0, 1000, n):
        out.append(Example(f"{int(v):03d}", QS, {"parity": int(v % 2), "big": bool(v >= 500), "size": int(min(2, v // 334))}))
    return out


def test_decision_objective_trains_a_causal_backbone_and_the_task_serves_it(tmp_path):
    torch.manual_seed(0)
    lay = Layout(shape="joint", max_len=192, head_max_len=170)
    backbone = CausalTransformer(vocab_size=260, emb_features=64, num_layers=2, num_heads=2, num_kv_heads=2, head_dim=32, mlp_features=128,
                                 max_seq_len=256)
    model = DecisionModel(backbone, JointSchemaHead(64, layers=1))
    obj = DecisionObjective(model, lay, rule=LogLoss() + 0.5 * Brier(), length=192)
    train = _number_examples(256, 0)
    batches = [obj.batch(train[i:i + 32]) for i in range(0, 256, 32)]
    assert batches[0]["tokens"].shape[1] == 192 and batches[0]["targets"].shape[1:] == (3, 3)
    tr = dew.Trainer(obj, dew.OptimConfig(learning_rate=3e-3, weight_decay=0.0), tracker=(t := dew.MemoryTracker()))
    tr.fit(batches * 40, steps=280, log_every=70)
    assert t.rows[-1]["loss"] < 0.5 * t.rows[0]["loss"] and t.rows[-1]["accuracy"] > 0.8
    held = _number_examples(128, 1)
    report = measure([obj.decisions(obj.batch(held[i:i + 32])) for i in range(0, 128, 32)])
    assert report["scored_questions"] == 384 and report["accuracy"] > 0.6 and 0 <= report["ece"] <= 1 and 0 <= report["aurc"] <= 1
    assert report["brier"] < 2 / 3 + 0.05
    task = Decide(model, lay, budget=Budget(tokens=2048, lengths=(192, 384)))
    fitted = task.calibrated(held, bins=5, target_error=0.2, least=10)
    assert set(fitted.calibration.temperatures.by_kind) == {"choice", "noul", "score"}
    answers = fitted.decide([{"state": "124", "questions": QS}, {"state": "901", "questions": {"big": QS["big"]}}])
    assert list(answers[0]) == list(QS) and list(answers[1]) == ["big"]
    assert abs(answers[0]["size"].probabilities.sum() - 1) < 1e-6
    assert 0 < fitted.real_token_share() <= 1
    # the wire form, refusals kept per body
    out = fitted.systemone([{"state": "124", "questions": {n: q.wire() for n, q in QS.items()}}, {"questions": {}},
                            {"state": "1", "questions": {"q": {"type": "choice", "instructions": "x", "criteria": ["a", "b"]}}, "extra": 1}],
                           details=True)
    assert isinstance(out[1], ValueError) and isinstance(out[2], ValueError)
    a = out[0]["answers"]
    assert a["parity"]["type"] == "choice" and set(a["parity"]["probabilities"]) == {"even", "odd"} and "abstained" in a["parity"]
    assert 0 <= a["big"]["noul"] <= 1 and a["size"]["legend"] == ["small", "medium", "large"]
    assert out[0]["usage"]["input_tokens"] > 0 and out[0]["usage"]["truncated"] is False
    with pytest.raises(Refused):
        fitted.systemone({"state": "9" * 500, "questions": {"big": QS["big"].wire()}}, whole=True)
    with pytest.raises(ValueError):
        fitted.systemone({"state": "1", "questions": {"big": QS["big"].wire()}}, details=True, strict=True)
    # save and read back: same answers
    fitted.save(str(tmp_path))
    model2 = DecisionModel(CausalTransformer(vocab_size=260, emb_features=64, num_layers=2, num_heads=2, num_kv_heads=2, head_dim=32,
                                             mlp_features=128, max_seq_len=256), JointSchemaHead(64, layers=1))
    again = Decide.load(str(tmp_path), model2)
    b = again.decide("124", QS)
    for n in QS:
        assert np.allclose(b[n].probabilities, answers[0][n].probabilities, atol=1e-5)
    assert again.calibration.record() == fitted.calibration.record()


def test_consistency_term_pulls_grouped_questions_together():
    torch.manual_seed(0)
    lay = Layout(shape="state_first", max_len=160, head_max_len=120)
    model = DecisionModel(BidirectionalBackbone(260, 32, 1, max_len=160), DecisionHead(32, 1))
    q1 = Choice("is it even or odd", ["even", "odd"])
    q2 = Choice("odd or even?", ["odd", "even"])
    group = Group("parity", {"a": {"even": "E", "odd": "O"}, "b": {"odd": "O", "even": "E"}})
    ex = [Example(f"{v:03d}", {"a": q1, "b": q2}, groups=[group]) for v in range(16)]            # no answers: only consistency trains
    obj = DecisionObjective(model, lay, consistency=1.0, length=160)
    batch = obj.batch(ex)
    assert int(batch["group_id"].max()) == 16 and not bool(batch["scored"].any())
    first = float(obj.loss(None, batch, Step(train=True))[1].metrics["consistency"].value())
    tr = dew.Trainer(obj, dew.OptimConfig(learning_rate=3e-3, weight_decay=0.0), tracker=(t := dew.MemoryTracker()))
    tr.fit([batch] * 60, steps=60, log_every=20)
    assert t.rows[-1]["consistency"] < 0.5 * first
    with pytest.raises(ValueError):
        Example("s", {"a": q1, "b": q2}, groups=[Group("g", {"a": {"even": "E", "odd": "O"}})])
    with pytest.raises(ValueError):
        Example("s", {"a": q1, "b": q2}, groups=[Group("g", {"a": {"even": "E", "odd": "O"}, "b": {"odd": "X", "even": "E"}})])
    GroupedExamples([Example("s", {"a": q1}), Example("t", {"b": q2})], [Group("g", {"0.a": {"even": "E", "odd": "O"}, "1.b": {"odd": "O", "even": "E"}})])


# ------------------------------------------------------------------------------------------------ metrics and calibration
def test_metrics_merge_over_batches_and_match_direct_formulas():
    g = torch.Generator().manual_seed(0)
    p = torch.softmax(torch.randn(200, 4, generator=g) * 2, -1)
    y = torch.randint(0, 4, (200,), generator=g)
    d = Decisions(p, torch.nn.functional.one_hot(y, 4).float(), torch.ones(200, 4, dtype=torch.bool), torch.ones(200, dtype=torch.bool),
                  torch.zeros(200, dtype=torch.bool), torch.zeros(200, dtype=torch.int64))
    parts = [Decisions(*(getattr(d, f)[i:i + 50] for f in ("probabilities", "targets", "options", "scored", "ordinal", "classes"))) for i in range(0, 200, 50)]
    whole, split = measure([d]), measure(parts)
    for k in whole:
        assert abs(whole[k] - split[k]) < 1e-9, k
    assert abs(whole["accuracy"] - float((p.argmax(-1) == y).double().mean())) < 1e-9
    from sklearn.metrics import f1_score
    assert abs(whole["macro_f1"] - f1_score(y.numpy(), p.argmax(-1).numpy(), average="macro")) < 1e-9
    assert abs(whole["log_loss"] - float(torch.nn.functional.nll_loss(p.double().log(), y))) < 1e-6
    assert abs(whole["ece"] - expected_calibration_error(p, y, bins=15)) < 1e-6
    # a confidence that ranks right answers first has a smaller risk-coverage area than one that ranks them last
    right = torch.tensor([1, 1, 1, 0, 0, 0])
    def aurc(conf):
        pp = torch.stack([torch.tensor(conf), 1 - torch.tensor(conf)], 1)
        tgt = torch.stack([right.float(), 1 - right.float()], 1)
        dd = Decisions(pp, tgt, torch.ones(6, 2, dtype=torch.bool), torch.ones(6, dtype=torch.bool), torch.zeros(6, dtype=torch.bool), torch.zeros(6, dtype=torch.int64))
        return measure([dd], [AURC()])["aurc"]
    assert aurc([0.9, 0.85, 0.8, 0.7, 0.65, 0.6]) > 0                   # every top option is class 0: three wrong
    assert AURC.finalize(([(0.9, True), (0.8, True), (0.7, False)],)) < AURC.finalize(([(0.9, False), (0.8, True), (0.7, True)],))
    assert AURC.finalize(([(0.5, True), (0.5, False)],)) == AURC.finalize(([(0.5, False), (0.5, True)],))


def test_calibration_recovers_a_temperature_and_gates_by_target_error():
    g = np.random.default_rng(0)
    q = Choice("q", ["a", "b", "c"])
    scored = []
    for _ in range(600):
        z = g.normal(size=3) * 2
        p = np.exp(z) / np.exp(z).sum()
        y = g.choice(3, p=p)
        scored.append(Scored.of(q, z * 3.0, np.eye(3)[y]))              # the model is three times too sharp
    t = Temperatures.fit(scored)
    assert abs(t.of("choice", 3) - 3.0) < 0.5 and bucket(q) == "choice:3-5"
    assert Temperatures.fit(scored[:5]).by_bucket == {} and "choice" in Temperatures.fit(scored[:5]).by_kind
    sharp = [Scored.of(q, s.logits / 30, s.gold) for s in scored]
    assert abs(Temperatures.fit(sharp).of("choice", 3) - 0.5) < 1e-6               # never sharpens past 0.5
    cal = Calibration.fit(scored, bins=10, target_error=0.1)
    thr = cal.abstention.of("choice:3-5")
    kept = [s for s in scored if cal.apply(q, s.logits)[1] >= thr]
    err = np.mean([np.argmax(s.logits) != np.argmax(s.gold) for s in kept])
    assert 0 < len(kept) < len(scored) and err <= 0.1 + 1e-9
    p, reported, abstained = cal.apply(q, np.array([1.2, 0.0, 0.0]))
    assert abstained and abs(p.sum() - 1) < 1e-9
    assert Calibration.from_record(json.loads(json.dumps(cal.record()))).record() == cal.record()
    assert isinstance(cal.binning, Binning) and isinstance(cal.abstention, Abstention)


# ------------------------------------------------------------------------------------------------ tournaments and data
def test_tournament_groups_and_combination():
    assert [len(g) for g in near_equal(list("abcdefghij"), 4)] == [4, 3, 3]
    out = knocked_out({"a": 0.7, "b": 0.3}, {"a": 0.5, "b": 0.3, "c": 0.15, "d": 0.05}, 0.01)
    assert abs(sum(out.values()) - 1) < 1e-12 and abs(out["a"] / out["b"] - 7 / 3) < 1e-9 and abs(out["c"] / out["d"] - 3) < 1e-9
    assert abs(out["c"] + out["d"] - 0.01) < 1e-9
    torch.manual_seed(0)
    lay = Layout(shape="state_first", max_len=256, head_max_len=200)
    model = DecisionModel(BidirectionalBackbone(260, 32, 1, max_len=256), DecisionHead(32, 1))
    wide = Choice("which letter", [f"option {i}" for i in range(23)])
    ko = Decide(model, lay, tournament=Knockout(group=5)).decide("state", {"w": wide, "n": Noul("yes?")})
    assert len(ko["w"].options) <= 5 and set(ko["w"].options) <= set(wide.options) and list(ko) == ["w", "n"]
    fin = Decide(model, lay, tournament=Finalists(group=6, keep=2, final=8, residual=0.01)).decide("state", {"w": wide})
    assert fin["w"].options == wide.options and abs(fin["w"].probabilities.sum() - 1) < 1e-9
    with pytest.raises(ValueError):
        Knockout(group=1)


def test_tables_and_mixtures_become_examples():
    rows = [{"text": "good film", "label": "pos"}, {"text": "bad film", "label": "neg"}, {"text": "meh", "label": None}]
    ex = decisions(rows, instructions="sentiment?")
    assert ex[0].questions["label"].options == ("neg", "pos") and ex[0].answers == {"label": "pos"} and ex[2].answers == {}
    assert ex[1].distribution("label").tolist() == [1.0, 0.0] and ex[2].distribution("label") is None
    ints = decisions([{"text": "a", "label": 1}, {"text": "b", "label": 0}], options=["no", "yes"])
    assert ints[0].distribution("label").tolist() == [0.0, 1.0]
    soft = Example("s", {"q": Choice("q", ["a", "b"])}, targets={"q": {"a": 3, "b": 1}})
    assert soft.distribution("q").tolist() == [0.75, 0.25]
    with pytest.raises(ValueError):
        Example("s", {"q": Choice("q", ["a", "b"])}, answers={"other": "a"})
    wired = decisions([{"state": {"k": 1}, "questions": {"q": {"type": "noul", "instructions": "ok?"}}, "answers": {"q": True}}])
    assert wired[0].distribution("q").tolist() == [0.0, 1.0]
    a, b = mixture({"x": ex[:2], "y": ints}, {"x": 3, "y": 1}, 40, seed=1), mixture({"x": ex[:2], "y": ints}, {"x": 3, "y": 1}, 40, seed=1)
    la, lb = list(a), list(b)
    assert [e.state for e in la] == [e.state for e in lb] and 20 < sum(e.state in ("good film", "bad film") for e in la) < 40
