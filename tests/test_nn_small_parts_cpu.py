"""Scan orders of patch grids and the activation watch."""
import pytest
import torch

from dew_b200.nn.inspection import ActivationWatch, activation_statistics, outliers
from dew_b200.nn.scan_orders import hilbert, inverse, order, raster, reorder, sincos_2d, zigzag


@pytest.mark.parametrize("hw", [(4, 4), (8, 8), (6, 10), (5, 7), (1, 9), (16, 3), (12, 12)])
def test_orders_are_permutations_of_neighbouring_steps(hw):
    h, w = hw
    for name in ("raster", "zigzag", "hilbert"):
        p = order(name, h, w)
        assert sorted(p.tolist()) == list(range(h * w))
        assert torch.equal(inverse(p)[p], torch.arange(h * w))
    for p, reach in ((zigzag(h, w), 1), (hilbert(h, w), 2)):
        ys, xs = p // w, p % w
        step = (ys[1:] - ys[:-1]).abs() + (xs[1:] - xs[:-1]).abs()
        assert int(step.max()) <= reach if h * w > 1 else True
    if h % 2 == 0 and w % 2 == 0:                                  # even grids: the Hilbert curve never jumps
        p = hilbert(h, w)
        assert int(((p[1:] // w - p[:-1] // w).abs() + (p[1:] % w - p[:-1] % w).abs()).max()) == 1


def test_hilbert_keeps_neighbourhoods_together_and_reorder_round_trips():
    p = hilbert(16, 16)
    ys, xs = (p // 16).float(), (p % 16).float()
    # tokens 16 apart in the sequence stay close on the grid (a raster order puts them a full row apart, but 15 columns away one step earlier)
    d = ((ys[16:] - ys[:-16]) ** 2 + (xs[16:] - xs[:-16]) ** 2).sqrt()
    assert float(d.mean()) < 6.0
    r = raster(16, 16)
    dr = (((r // 16)[1:] - (r // 16)[:-1]).abs() + ((r % 16)[1:] - (r % 16)[:-1]).abs()).max()
    assert int(dr) == 16
    x = torch.randn(2, 256, 5)
    assert torch.equal(reorder(reorder(x, p), inverse(p)), x)
    with pytest.raises(KeyError, match="scan order"):
        order("spiral", 4, 4)


def test_sincos_2d():
    e = sincos_2d(3, 5, 16)
    assert e.shape == (15, 16)
    assert torch.allclose(e[0], torch.tensor([0.0] * 4 + [1.0] * 4 + [0.0] * 4 + [1.0] * 4))
    assert torch.allclose(e[5 * 1 + 2, :8], e[5 * 1 + 4, :8]) and not torch.allclose(e[5 * 1 + 2, 8:], e[5 * 1 + 4, 8:])     # same row, other column
    with pytest.raises(ValueError):
        sincos_2d(2, 2, 6)


def test_activation_watch_reports_and_flags_outlier_channels():
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.ReLU(), torch.nn.Linear(16, 4))
    with torch.no_grad():
        model[2].weight[1] *= 200.0                                # one output channel far above the rest
    x = torch.randn(64, 8)
    with ActivationWatch(model, ["0", "1", "2"]) as watch:
        model(x)
        model(x)
        stats = watch.collect()
    assert stats["0/calls"] == 2.0 and abs(stats["1/zeros"] - float((model[0](x) <= 0).float().mean())) < 1e-6
    want = activation_statistics(model(x))
    assert abs(stats["2/rms"] - float(want["rms"])) < 1e-4 and stats["2/top_channel"] == 1.0
    assert outliers(stats, kurtosis=1e9, ratio=1.5) == ["2"]
    assert watch.collect() == {}
    model(x)                                                      # hooks are gone after the block
    assert watch.collect() == {}
    g = torch.randn(10000, 4)
    assert abs(float(activation_statistics(g)["kurtosis"])) < 0.2
