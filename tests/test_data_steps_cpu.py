"""Row-count-changing stages, token steps, streamed orders, the ordered pool and the wrapped sources."""
import threading
import time

import numpy as np
import pytest
import torch

from dew_b200.data.concurrent import OrderedPool
from dew_b200.data.dataset import Memory
from dew_b200.data.ordering import WindowShuffle, locality_order, skipping
from dew_b200.data.sources import Concatenate, HFDataset, IteratorSource, TorchDataset
from dew_b200.data.steps import causal_windows, formatted, over_length, rename, require_length, select, target_count, where


def _memory(rows):
    return Memory(rows) if not isinstance(rows, dict) else Memory(rows)


def test_filter_and_flat_map_with_exact_resume():
    rows = [{"id": i, "tokens": list(range(i + 1))} for i in range(12)]
    ds = Memory(rows).filter(lambda r: r["id"] % 3 != 0).flat_map(over_length(4, "split")).map(lambda r: {"id": r["id"], "n": len(r["tokens"])})
    got = list(ds)
    want = []
    for r in rows:
        if r["id"] % 3:
            n = r["id"] + 1
            want += [{"id": r["id"], "n": min(4, n - lo)} for lo in range(0, n, 4)]
    assert got == want
    again = Memory(rows).filter(lambda r: r["id"] % 3 != 0).flat_map(over_length(4, "split")).map(lambda r: {"id": r["id"], "n": len(r["tokens"])})
    it = iter(again)
    head = [next(it) for _ in range(5)]
    pos = again.position()
    fresh = Memory(rows).filter(lambda r: r["id"] % 3 != 0).flat_map(over_length(4, "split")).map(lambda r: {"id": r["id"], "n": len(r["tokens"])})
    fresh.restore(pos)
    assert head + list(fresh) == want


def test_generic_and_length_steps():
    row = {"question": "2+2", "answer": "4", "label": 1, "tokens": list(range(10)), "mask": [0] * 4 + [1] * 6}
    assert select("label", "answer")(row) == {"label": 1, "answer": "4"}
    with pytest.raises(KeyError, match="holds no"):
        select("nope")(row)
    assert rename(text="question")(row)["text"] == "2+2" and "question" not in rename(text="question")(row)
    assert formatted("Q: {question} A: {answer}")(row)["text"] == "Q: 2+2 A: 4"
    assert where(label={1, 2})(row) and not where(label=0)(row)
    assert [r["tokens"] for r in over_length(4, "split")(row)] == [[0, 1, 2, 3], [4, 5, 6, 7], [8, 9]]
    assert [r["mask"] for r in over_length(4, "split")(row)] == [[0, 0, 0, 0], [1, 1, 1, 1], [1, 1]]
    assert next(over_length(4, "truncate_left")(row))["tokens"] == [6, 7, 8, 9]
    assert list(over_length(4, "drop")(row)) == [] and list(over_length(10, "raise")(row)) == [row]
    with pytest.raises(ValueError, match="holds 10 tokens"):
        list(over_length(4, "raise")(row))
    with pytest.raises(ValueError, match="policy"):
        over_length(4, "wrap")
    assert target_count(row) == 6 and target_count({"tokens": [1, 2, 3]}) == 2
    with pytest.raises(ValueError, match="promised"):
        require_length(8)(row)


@pytest.mark.parametrize("n,window,stride", [(23, 8, None), (17, 8, 4), (9, 8, None), (8, 8, None), (40, 6, 3)])
def test_causal_windows_train_every_target_once(n, window, stride):
    doc = {"tokens": np.arange(100, 100 + n)}
    trained = np.zeros(n, dtype=int)
    for w in causal_windows(window, stride=stride)(doc):
        assert len(w["tokens"]) <= window + 1 and w["mask"][0] == 0
        assert np.array_equal(w["tokens"], doc["tokens"][w["offset"]:w["offset"] + len(w["tokens"])])
        trained[w["offset"] + np.nonzero(w["mask"])[0]] += 1
    assert trained[0] == 0 and (trained[1:] == 1).all()


def test_locality_order_and_window_shuffle():
    sizes = [5, 0, 7, 3, 9, 4]
    pairs = list(locality_order(sizes, seed=1, epoch=0, open_shards=2))
    assert sorted(pairs) == sorted((s, i) for s, n in enumerate(sizes) for i in range(n))
    for s in range(len(sizes)):                                  # every shard is read front to back
        assert [i for t, i in pairs if t == s] == list(range(sizes[s]))
    open_now, most = set(), 0
    done = {s: 0 for s in range(len(sizes))}
    for s, i in pairs:
        open_now.add(s)
        done[s] += 1
        most = max(most, len(open_now))
        if done[s] == sizes[s]:
            open_now.discard(s)
    assert most <= 2
    assert pairs != list(locality_order(sizes, seed=1, epoch=1, open_shards=2)) and pairs == list(locality_order(sizes, seed=1, epoch=0, open_shards=2))
    sh = WindowShuffle(8, seed=3)
    out = list(sh(range(30)))
    assert sorted(out) == list(range(30)) and out != list(range(30)) and sh.position == 30
    for w in range(4):
        assert sorted(out[8 * w:8 * w + 8]) == list(range(8 * w, min(30, 8 * w + 8)))
    for cut in (0, 5, 8, 13, 29):
        again = WindowShuffle(8, seed=3)
        again.restore(cut)
        assert list(again(range(30))) == out[cut:]
    assert list(skipping(range(6), {1, 4})) == [0, 2, 3, 5]


def test_ordered_pool_keeps_order_bounds_flight_and_restores():
    active, peak, lock = [0], [0], threading.Lock()

    def slow(x):
        with lock:
            active[0] += 1
            peak[0] = max(peak[0], active[0])
        time.sleep(0.002 * (5 - x % 5))
        with lock:
            active[0] -= 1
        return x * x
    pool = OrderedPool(slow, workers=4, depth=6)
    assert list(pool(range(25))) == [x * x for x in range(25)] and pool.position == 25 and 1 < peak[0] <= 4
    ran = []
    again = OrderedPool(lambda x: ran.append(x) or x, workers=2)
    again.restore(20)
    assert list(again(range(25))) == [20, 21, 22, 23, 24] and sorted(ran) == [20, 21, 22, 23, 24] and again.position == 25

    def bad(x):
        if x == 3:
            raise RuntimeError("record 3")
        return x
    got = []
    with pytest.raises(RuntimeError, match="record 3"):
        for y in OrderedPool(bad, workers=2)(range(10)):
            got.append(y)
    assert got == [0, 1, 2]


def test_wrapped_sources():
    a, b = Memory([{"x": i} for i in range(3)]), Memory([{"x": 10 + i} for i in range(2)])
    cat = Concatenate([a, b])
    assert len(cat) == 5 and [r["x"] for r in cat] == [0, 1, 2, 10, 11]
    batches = list(Concatenate([a, b]).batched(2))
    assert [bt["x"].tolist() for bt in batches] == [[0, 1], [2, 10]]

    class Pairs(torch.utils.data.Dataset):
        def __len__(self):
            return 4

        def __getitem__(self, i):
            return torch.full((2,), float(i)), i % 2
    ds = TorchDataset(Pairs(), fields=("image", "label")).batched(2)
    first = next(iter(ds))
    assert first["image"].shape == (2, 2) and first["label"].tolist() == [0, 1]
    with pytest.raises(TypeError, match="field names"):
        next(iter(TorchDataset(Pairs())))

    class Table:                                               # the two calls of a datasets.Dataset this wrapper uses
        rows = [{"text": "a", "n": 1, "extra": 0}, {"text": "b", "n": 2, "extra": 0}]

        def __len__(self):
            return len(self.rows)

        def __getitem__(self, i):
            return self.rows[i]
    assert list(HFDataset(Table(), columns=("text", "n"))) == [{"text": "a", "n": 1}, {"text": "b", "n": 2}]
    src = IteratorSource(lambda: ({"v": i} for i in range(7))).filter(lambda r: r["v"] != 2)
    assert [r["v"] for r in src] == [0, 1, 3, 4, 5, 6]
    part = IteratorSource(lambda: ({"v": i} for i in range(7)))
    it = iter(part)
    head = [next(it)["v"] for _ in range(3)]
    resumed = IteratorSource(lambda: ({"v": i} for i in range(7)))
    resumed.restore(part.position())
    assert head + [r["v"] for r in resumed] == list(range(7))
