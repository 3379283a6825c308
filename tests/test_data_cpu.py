"""Data layer: packing (whole documents, streaming), the on-disk cache, and the file-backed sources."""
import json

import numpy as np
import pytest
import torch

from dew_b200.data import Cached, Hub, JsonLines, Packer, Parquet, pack_whole


def _docs(n=40, seed=0):
    rng = np.random.default_rng(seed)
    return [list(rng.integers(1, 100, size=int(rng.integers(3, 30)))) for _ in range(n)]


def test_pack_whole_keeps_documents_intact_and_orders_segments():
    docs = _docs()
    out = pack_whole(docs, seq_len=63, pad_id=0)
    tokens, segs, pos = out["tokens"], out["segments"], out["positions"]
    assert tokens.shape[1] == 64 and out["fill"] > 0.85
    found = []
    for r in range(tokens.shape[0]):
        live = segs[r] > 0
        assert np.all(np.diff(segs[r][live]) >= 0)                      # non-decreasing ids, padding (0) only at the end
        assert not live[np.argmin(live):].any() if not live.all() else True
        for s in range(1, segs[r].max() + 1):
            m = segs[r] == s
            found.append(list(tokens[r][m]))
            assert list(pos[r][m]) == list(range(m.sum()))              # positions restart at every document
    assert sorted(map(tuple, found)) == sorted(map(tuple, docs))       # every document appears once, whole


def test_streaming_packer_emits_every_token_once():
    docs = _docs(200, seed=1)
    rows = list(Packer(seq_len=63, open_rows=4).pack(docs))
    got = sorted(tuple(r["tokens"][r["segments"] == s]) for r in rows for s in range(1, r["segments"].max() + 1))
    assert got == sorted(map(tuple, docs))
    fill = sum((r["segments"] > 0).sum() for r in rows) / (len(rows) * 64)
    assert fill > 0.8


def test_packed_rows_train_through_the_lm_objective():
    import dew_b200 as dew
    from dew_b200.models import CausalTransformer
    from dew_b200.objectives.lm import LMObjective
    out = pack_whole(_docs(30, seed=2), seq_len=32, pad_id=0)
    torch.manual_seed(0)
    m = CausalTransformer(vocab_size=100, emb_features=16, num_layers=1, num_heads=2, num_kv_heads=2, head_dim=8, mlp_features=24, max_seq_len=32)
    t = dew.Trainer(LMObjective(m, 32, ema_decay=None), dew.OptimConfig(learning_rate=1e-2), key=0)
    batch = {"tokens": torch.from_numpy(out["tokens"][:4]), "segments": torch.from_numpy(out["segments"][:4])}
    state = t.fit([batch] * 3, steps=3, log_every=1)
    assert state.step == 3 and t.history[-1]["loss"] < t.history[0]["loss"]


def test_cache_builds_once_and_rebuilds_after_an_interrupted_write(tmp_path):
    calls = []

    def build():
        calls.append(1)
        return pack_whole(_docs(20, seed=3), seq_len=31)
    c = Cached(build, tmp_path, key=("lm", "bytes", 31))
    a = c.dataset()
    b = Cached(build, tmp_path, key=("lm", "bytes", 31)).dataset()
    assert len(calls) == 1 and len(a) == len(b) and torch.equal(a._get(0)["tokens"], b._get(0)["tokens"])
    (c.path / "COMPLETE").unlink()                       # a run cut short leaves no marker
    Cached(build, tmp_path, key=("lm", "bytes", 31)).dataset()
    assert len(calls) == 2
    Cached(build, tmp_path, key=("lm", "bytes", 63)).dataset()      # another key is another entry
    assert len(calls) == 3


def test_jsonl_parquet_and_local_hub_snapshots(tmp_path):
    rows = [{"text": f"row {i}", "n": i} for i in range(7)]
    p = tmp_path / "train.jsonl"
    p.write_text("\n".join(json.dumps(r) for r in rows))
    assert [r["n"] for r in JsonLines(p)] == list(range(7))
    import pyarrow as pa
    import pyarrow.parquet as pq
    snap = tmp_path / "hub" / "datasets--acme--toy" / "snapshots" / "abc123" / "data"
    snap.mkdir(parents=True)
    pq.write_table(pa.Table.from_pylist(rows), snap / "train-00000.parquet")
    assert len(Parquet(snap / "train-00000.parquet", columns=["n"])) == 7
    ds = Hub("acme/toy", cache_dir=tmp_path)
    assert [r["text"] for r in ds][:2] == ["row 0", "row 1"]
    with pytest.raises(FileNotFoundError, match="no network"):
        Hub("acme/missing", cache_dir=tmp_path)
