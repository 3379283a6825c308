"""Frozen-encoder probes separate a representation that holds the label from one that does not."""
import torch

from dew_b200.objectives.jepa_probes import ProbeReport, features, knn_probe, ridge_probe


def _data(n, seed):
    g = torch.Generator().manual_seed(seed)
    y = torch.randint(0, 3, (n,), generator=g)
    centres = torch.tensor([[2.0, 0.0, 0.0, 0.0], [0.0, 2.0, 0.0, 0.0], [0.0, 0.0, 2.0, 0.0]])
    x = centres[y] + 0.4 * torch.randn(n, 4, generator=g)
    return [{"image": x[i:i + 32], "label": y[i:i + 32]} for i in range(0, n, 32)]


def test_probes():
    train, val = _data(256, 0), _data(128, 1)
    torch.manual_seed(0)
    lift = torch.nn.Linear(4, 16)
    good = lambda x: torch.tanh(lift(x))[:, None, :].expand(-1, 5, -1)          # tokens that all carry the label
    blind = lambda x: torch.randn(x.shape[0], 5, 16)                            # tokens that carry nothing
    fx, fy = features(good, train)
    assert fx.shape == (256, 16) and fy.shape == (256,) and not fx.requires_grad
    report = ProbeReport(train, val)
    seen, unseen = report(good), report(blind)
    assert seen["probe/ridge_accuracy"] > 0.95 and seen["probe/knn_accuracy"] > 0.95
    assert unseen["probe/ridge_accuracy"] < 0.6 and unseen["probe/knn_accuracy"] < 0.6
    tx, ty = features(good, train, pool="first")
    vx, vy = features(good, val, pool="first")
    assert ridge_probe(tx, ty, vx, vy)["accuracy"] == seen["probe/ridge_accuracy"]
    assert knn_probe(tx, ty, tx, ty, k=1)["accuracy"] == 1.0
