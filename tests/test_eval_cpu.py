"""General calibration arithmetic and continual-learning summaries."""
import numpy as np
import pytest
import torch

from dew_b200.eval import calibration as C
from dew_b200.eval.continual import AccuracyMatrix, continual_run, label_accuracy, label_scores


def test_calibration_arithmetic():
    g = np.random.default_rng(0)
    z = g.normal(size=(2000, 4)) * 2
    p = C.softmax(z)
    y = np.array([g.choice(4, p=row) for row in p])
    assert C.fit_temperature(z * 2.5, np.eye(4)[y]) == pytest.approx(2.5, rel=0.1)
    real = np.ones((2000, 4), bool); real[:, 3] = False
    p3 = C.softmax(np.where(real, z, -np.inf))
    assert np.allclose(p3[:, 3], 0) and np.allclose(p3.sum(-1), 1)
    y3 = np.array([g.choice(4, p=row) for row in p3])
    assert C.fit_temperature(np.where(real, z * 0.5, 7.0), np.eye(4)[y3], real) == pytest.approx(0.5, rel=0.1)     # values past the options do not matter
    tops, right = p.max(-1), p.argmax(-1) == y
    table = C.reliability_bins(tops, right, 15)
    assert table.shape == (3, 15) and table[0].sum() == 2000 and C.expected_calibration_error(table) < 0.05
    halves = C.reliability_bins(tops[:1000], right[:1000]) + C.reliability_bins(tops[1000:], right[1000:])
    assert np.allclose(halves, table)                                        # additive over passes
    over = C.softmax(z * 3)
    assert C.expected_calibration_error(C.reliability_bins(over.max(-1), over.argmax(-1) == y)) > 0.1
    assert C.maximum_calibration_error(table) >= C.expected_calibration_error(table)
    hm = C.histogram_map(over.max(-1), over.argmax(-1) == y, 10)
    mapped = C.histogram_mapped(over.max(-1), hm)
    assert C.expected_calibration_error(C.reliability_bins(mapped, over.argmax(-1) == y)) < 0.03           # the map repairs the over-confidence
    assert C.tied_prefixes([0.9, 0.5, 0.9, 0.2], [True, False, False, True]) == [(0.9, 2, 1), (0.5, 3, 1), (0.2, 4, 2)]
    assert C.abstention_threshold([0.9, 0.8, 0.7, 0.6], [True, True, False, True], 0.0) == 0.8
    assert C.abstention_threshold([0.9, 0.8, 0.7, 0.6], [True, True, False, True], 0.3) == 0.6
    assert C.abstention_threshold([0.9, 0.8], [False, False], 0.1) == C.REJECT_ALL
    assert C.abstention_threshold([0.9, 0.8, 0.7, 0.6], [True, True, True, True], 0.2, conservative=True) == 0.6     # (0 + 1) / (4 + 1) = 0.2
    assert C.risk_coverage_area([0.9, 0.8, 0.7], [True, True, False]) == pytest.approx((0 + 0 + 1 / 3) / 3)
    assert C.risk_coverage_area([0.5, 0.5], [True, False]) == C.risk_coverage_area([0.5, 0.5], [False, True]) == 0.5
    assert C.brier_score(np.eye(3), [0, 1, 2]) == 0.0 and C.brier_score(np.full((2, 2), 0.5), [0, 1]) == 0.5


def test_continual_summaries_and_label_scoring():
    a = AccuracyMatrix(np.array([[0.9, 0.1, 0.2], [0.7, 0.8, 0.3], [0.5, 0.6, 0.9]]))
    assert a.average_accuracy == pytest.approx(2.0 / 3) and a.forgetting.tolist() == pytest.approx([0.4, 0.2])
    assert a.backward_transfer == pytest.approx(((0.5 - 0.9) + (0.6 - 0.8)) / 2) and a.forward_transfer([0.1, 0.1, 0.1]) == pytest.approx((0.0 + 0.2) / 2)
    assert set(a.summary()) == {"average_accuracy", "average_forgetting", "backward_transfer"}
    with pytest.raises(ValueError):
        AccuracyMatrix(np.zeros((2, 3)))
    # a learner that remembers only its last task: it forgets everything before
    known = set()

    def fit(i, task):
        known.clear(); known.add(task)
    run = continual_run(["a", "b", "c"], fit, lambda i, j: 1.0 if ["a", "b", "c"][j] in known else 0.0)
    assert run.values.tolist() == [[1, 0, 0], [0, 1, 0], [0, 0, 1]] and run.average_forgetting == 1.0 and run.backward_transfer == -1.0

    class Bigram(torch.nn.Module):
        """Predicts token t + 1 = token t + 1 (mod 8) with high confidence."""
        def __init__(self):
            super().__init__(); self.p = torch.nn.Parameter(torch.zeros(1))
        def forward(self, tokens):
            return torch.nn.functional.one_hot((tokens + 1) % 8, 8).float() * 10.0
    m = Bigram()
    prompts, labels = [[1, 2, 3], [5, 6]], [[4], [7], [0]]
    s = label_scores(m, prompts, labels)
    assert s.shape == (2, 3) and s.argmax(-1).tolist() == [0, 1]
    assert label_accuracy(m, prompts, labels, [0, 1]) == 1.0 and label_accuracy(m, prompts, labels, [0, 1], allowed=[1, 2]) == 0.5
