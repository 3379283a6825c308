"""Decision models: typed questions answered from one forward pass, trained with a proper scoring rule, calibrated."""
import torch

import dew_b200 as dew
from dew_b200.decision import Abstention, Choice, Decide, DecisionObjective, Score, Temperatures, binning, layout_row
from dew_b200.models import CausalTransformer


def test_layout_and_score_buckets():
    q = [Choice("colour", ("red", "green")), Score("risk", 0, 10, buckets=5)]
    row, pos = layout_row([5, 6, 7], q, marker_id=99, max_len=8)
    assert row.tolist() == [5, 6, 7, 99, 99, 0, 0, 0] and pos.tolist() == [3, 4]
    assert q[1].bucket(9.9) == 4 and q[1].bucket(-1) == 0 and len(q[1].options) == 5
    assert abs(q[1].expectation([0, 0, 1, 0, 0]) - 5.0) < 1e-6


def test_decide_learns_answers_and_calibrates():
    torch.manual_seed(0)
    qs = [Choice("parity", ("even", "odd")), Choice("big", ("no", "yes"))]
    backbone = CausalTransformer(vocab_size=40, emb_features=32, num_layers=1, num_heads=2, num_kv_heads=2, head_dim=16, mlp_features=64, max_seq_len=16)
    task = Decide(backbone, qs, marker_id=39, max_len=8, width=16)
    g = torch.Generator().manual_seed(1)
    states = [[int(torch.randint(1, 30, (1,), generator=g))] * 3 for _ in range(64)]
    tokens, pos = task.encode(states)
    answers = torch.tensor([[s[0] % 2, int(s[0] >= 15)] for s in states])
    obj = DecisionObjective(task, rule="log")
    tr = dew.Trainer(obj, dew.OptimConfig(learning_rate=5e-3, weight_decay=0.0), tracker=(t := dew.MemoryTracker()))
    batch = {"tokens": tokens, "positions": pos, "answers": answers}
    tr.fit(dew.Loader(lambda part: iter([batch] * 200), batch=64), steps=150, log_every=50)
    assert t.rows[-1]["accuracy"] > 0.9 and t.rows[-1]["loss"] < t.rows[0]["loss"]
    ans = task.answer(states[:2])
    assert set(ans[0]) == {"parity", "big"} and abs(sum(ans[0]["parity"].values()) - 1) < 1e-5
    logits = [l.detach() for l in task.logits(tokens, pos)]
    temps = Temperatures.fit(logits, answers)
    assert temps.value.shape == (2,) and bool((temps.value > 0).all())
    probs = torch.softmax(logits[0], -1)
    rows, ece = binning(probs.max(-1).values, probs.argmax(-1) == answers[:, 0])
    assert 0 <= ece <= 1 and sum(r[0] for r in rows) == 64
    cov, acc = Abstention(0.8).coverage_accuracy(probs, answers[:, 0])
    assert 0 <= cov <= 1 and acc >= 0.9
