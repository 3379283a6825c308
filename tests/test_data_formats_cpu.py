"""Data formats and corpus tools: images and augmentation, hash-keyed holdouts, tar shards, corpus analysis, video clips."""
import io
import json
import os

import numpy as np
import pytest

from dew_b200.data import Augment, Clips, DataPartition, Holdout, ImageFolder, Memory, TarShards, write_shards
from dew_b200.data import analysis as AN
from dew_b200.data.holdout import stratified_counts, unit_hash
from dew_b200.data.images import bucketed, buckets, caption_dropout, center_crop, decode, random_crop, resize_shorter, row_key
from dew_b200.data.shards import read_shard
from dew_b200.data.video import clip_starts, clips


def _png(h, w, colour):
    from PIL import Image
    buf = io.BytesIO()
    Image.fromarray(np.full((h, w, 3), colour, dtype=np.uint8)).save(buf, format="PNG")
    return buf.getvalue()


def test_images_decode_resize_crop_and_augment_by_key(tmp_path):
    arr = decode(_png(40, 60, (255, 0, 127)))
    assert arr.shape == (40, 60, 3) and arr.dtype == np.float32 and abs(arr[0, 0, 0] - 1.0) < 1e-6 and abs(arr[0, 0, 1] + 1.0) < 1e-6
    small = resize_shorter(arr, 20)
    assert small.shape == (20, 30, 3) and np.allclose(small[..., 0], 1.0, atol=1e-3)
    assert center_crop(small, 20).shape == (20, 20, 3)
    a, origin_a = random_crop(small, 16, 16, key=5)
    b, origin_b = random_crop(small, 16, 16, key=5)
    assert origin_a == origin_b and a.shape == (16, 16, 3)
    table = buckets(256)
    assert (256, 256) in table and all(h % 64 == 0 and w % 64 == 0 and max(h / w, w / h) <= 2.0 for h, w in table)
    wide, bucket = bucketed(np.zeros((100, 190, 3), np.float32), table)
    assert bucket[1] > bucket[0] and wide.shape[:2] == bucket
    drops = [caption_dropout("a cat", k, 0.3) for k in range(2000)]
    assert 0.25 < drops.count("") / 2000 < 0.35 and caption_dropout("a cat", 7, 0.3) == caption_dropout("a cat", 7, 0.3)
    # a folder with sidecar captions and a captions file
    for i, colour in enumerate([(255, 0, 0), (0, 255, 0), (0, 0, 255)]):
        (tmp_path / f"img{i}.png").write_bytes(_png(48 + 8 * i, 64, colour))
    (tmp_path / "img0.txt").write_text("red square\n")
    (tmp_path / "captions.jsonl").write_text(json.dumps({"file": "img1.png", "caption": "green square"}) + "\n")
    folder = ImageFolder(str(tmp_path))
    assert len(folder) == 3 and [folder._get(i)["caption"] for i in range(3)] == ["red square", "green square", ""]
    aug = Augment(size=32, crop="random", flip=True, drop_caption=0.0)
    rows = list(folder.map(aug))
    again = list(folder.map(aug))
    assert rows[0]["sample"].shape == (32, 32, 3) and rows[0]["original_size"].tolist() == [48, 64]
    assert all(np.array_equal(r["sample"], s["sample"]) and r["flipped"] == s["flipped"] for r, s in zip(rows, again))
    assert row_key({"path": "x"}) == row_key({"path": "x"}) != row_key({"path": "y"})
    batch = next(iter(folder.map(Augment(size=32)).batched(2)))
    assert batch["sample"].shape == (2, 32, 32, 3)
    with pytest.raises(ValueError):
        Augment(crop="stretch")


def test_holdout_is_stable_under_order_and_growth():
    rows = [{"id": f"doc{i}", "text": f"t{i}", "label": i % 3} for i in range(2000)]
    h = Holdout(0.1, salt="v1")
    train, held = h.split(Memory(rows))
    assert len(train) + len(held) == 2000 and 150 < len(held) < 250
    held_ids = {held._get(i)["id"] for i in range(len(held))}
    # the same rows are held out of a shuffled, grown copy
    rng = np.random.default_rng(0)
    grown = [rows[i] for i in rng.permutation(2000)] + [{"id": f"new{i}", "text": "", "label": 0} for i in range(500)]
    _, held2 = h.split(Memory(grown))
    ids2 = {held2._get(i)["id"] for i in range(len(held2))}
    assert held_ids == {i for i in ids2 if i.startswith("doc")}
    assert {held._get(i)["id"] for i in range(len(held))} != {r["id"] for r in rows if Holdout(0.1, salt="v2").is_held(r["id"])}
    counts = stratified_counts(held, "label")
    assert set(counts) == {0, 1, 2} and min(counts.values()) > 30
    assert 0 <= unit_hash("a") < 1 and unit_hash("a") == unit_hash("a") != unit_hash("b")
    grouped = Holdout(0.5, key="group")
    assert grouped.is_held(grouped.key_of({"group": "g1", "id": 1})) == grouped.is_held(grouped.key_of({"group": "g1", "id": 2}))
    with pytest.raises(ValueError):
        Holdout(1.5)


def test_tar_shards_partition_and_resume(tmp_path):
    samples = [{"__key__": f"s{i:04d}", "txt": f"caption {i}", "json": {"i": i}, "npy": np.full((2, 2), i, np.float32), "cls": str(i % 4)} for i in range(25)]
    index = write_shards(samples, str(tmp_path), samples_per_shard=10)
    assert [s["samples"] for s in index["shards"]] == [10, 10, 5] and index["samples"] == 25
    first = list(read_shard(str(tmp_path / "shard-00000.tar")))
    assert first[3]["txt"] == "caption 3" and first[3]["json"] == {"i": 3} and first[3]["cls"] == 3 and float(first[3]["npy"][0, 0]) == 3.0
    ds = TarShards(str(tmp_path))
    assert len(ds) == 25 and [s["json"]["i"] for s in ds] == list(range(25))
    # two ranks read disjoint shards that together cover everything
    a = [s["json"]["i"] for s in TarShards(str(tmp_path)).partition(DataPartition(0, 2))]
    b = [s["json"]["i"] for s in TarShards(str(tmp_path)).partition(DataPartition(1, 2))]
    assert sorted(a + b) == list(range(25)) and not set(a) & set(b)
    # resume mid-shard: the position names the shard and the sample inside it
    reader = TarShards(str(tmp_path))
    it = iter(reader)
    seen = [next(it)["json"]["i"] for _ in range(13)]
    position = reader.position()
    assert position["shard"] == 1 and position["sample"] == 3
    resumed = TarShards(str(tmp_path))
    resumed.restore(position)
    assert seen + [s["json"]["i"] for s in resumed] == list(range(25))
    shuffled = [s["json"]["i"] for s in TarShards(str(tmp_path), buffer=8).shuffle(3)]
    assert sorted(shuffled) == list(range(25)) and shuffled != list(range(25))
    batches = list(TarShards(str(tmp_path)).map(lambda s: {"i": s["json"]["i"], "x": s["npy"]}).batched(10, drop_last=False))
    assert [len(b["i"]) for b in batches] == [10, 10, 5] and batches[0]["x"].shape == (10, 2, 2)


def test_corpus_analysis_reports():
    lengths = [10, 20, 30, 200, 5, 5, 50]
    rep = AN.length_report(lengths, seq_len=64)
    assert rep["documents"] == 7 and rep["max"] == 200 and rep["cut_documents"] == pytest.approx(1 / 7) and rep["cut_tokens"] == pytest.approx(136 / 320)
    pack = AN.packing_report(lengths, 64)
    # first-fit decreasing: [64], [50, 10], [30, 20, 5, 5] -> three windows
    assert pack["windows"] == 3 and pack["real_token_share"] == pytest.approx(184 / 192) and pack["padded_real_token_share"] == pytest.approx(184 / 448)
    vocab = AN.vocabulary_report([[1, 1, 2], [3, 1]], vocab_size=8)
    assert vocab["used"] == 3 and vocab["coverage"] == pytest.approx(3 / 8) and vocab["top"][0] == (1, 0.6)
    with pytest.raises(ValueError):
        AN.vocabulary_report([[9]], 8)
    base = "the quick brown fox jumps over the lazy dog near the river bank at dawn"
    texts = [base, base + "  ", base.replace("dawn", "dusk"), "an entirely different sentence about compilers and kernels", base]
    d = AN.duplicates(texts, threshold=0.6)
    assert d["exact_groups"] == [[0, 1, 4]] and d["exact_duplicate_share"] == pytest.approx(2 / 5) and (0, 2) in d["near_pairs"]
    assert not any(3 in p for p in d["near_pairs"])

    class Tok:
        vocab_size = 256

        def encode(self, t):
            return list(t.encode())
    report = AN.analyse([{"text": t} for t in texts], Tok(), seq_len=32)
    assert report["sampled"] == 5 and report["packing"]["windows"] >= 5 and report["duplicates"]["near_pairs"] >= 1 and report["vocabulary"]["used"] > 10


def test_video_clips_stride_padding_and_keys():
    video = np.arange(20)[:, None, None, None] * np.ones((1, 2, 2, 3))
    assert clip_starts(20, 4, 2).tolist() == [0, 7]                         # span 7: non-overlapping starts
    c = clips(video, length=4, stride=2, count=None, fps=30.0)
    assert c["clip"].shape == (2, 4, 2, 2, 3) and c["clip"][1, :, 0, 0, 0].tolist() == [7, 9, 11, 13] and c["fps"].tolist() == [15.0, 15.0]
    short = clips(video[:5], length=4, stride=2)
    assert short["frames_mask"].tolist() == [[True, True, True, False]] and short["clip"][0, :, 0, 0, 0].tolist() == [0, 2, 4, 4]
    stage = Clips(length=4, stride=1, count=1)
    a, b = stage({"video": video, "id": "v1"}), stage({"video": video, "id": "v1"})
    assert a["clip"].shape == (4, 2, 2, 3) and int(a["first_frame"]) == int(b["first_frame"])
    many = {int(Clips(length=4)({"video": video, "id": f"v{i}"})["first_frame"]) for i in range(40)}
    assert len(many) > 5


def test_rl_prompts_and_synthesised_training_rows(tmp_path):
    import json
    from dew_b200.data.prompts import Prompts, decode_column
    from dew_b200.data.synthesis import Sample, best_of_n, dpo_rows, preference_pairs, scored_samples, sft_rows, write_records
    from dew_b200.data import ByteTokenizer
    tok = ByteTokenizer()
    rows = [{"prompt": "2+2=", "data_source": "math", "reward_model": {"ground_truth": "4"}, "extra_info": {"split": "train"}},
            {"prompt": [5, 6, 7], "ground_truth": "x"},
            {"prompt": "a very long prompt " * 10}]
    ds = Prompts(rows, tok, max_prompt_len=16, column_width=32)
    first = ds._get(0)
    n = int(first["prompt_length"])
    assert first["prompt"].shape == (16,) and first["prompt"][-n:].tolist() == list(tok.encode("2+2=")) and np.all(first["prompt"][:-n] == 0)
    assert decode_column(first["ground_truth"]) == "4" and decode_column(first["data_source"]) == "math" and json.loads(decode_column(first["extra_info"])) == {"split": "train"}
    assert ds._get(1)["prompt"][-3:].tolist() == [5, 6, 7] and decode_column(ds._get(1)["ground_truth"]) == "x" and decode_column(ds._get(1)["data_source"]) == ""
    long = ds._get(2)
    assert int(long["prompt_length"]) == 16 and long["prompt"].tolist() == list(tok.encode("a very long prompt " * 10))[-16:]          # keeps its tail
    batch = next(iter(ds.batched(2)))
    assert batch["prompt"].shape == (2, 16) and batch["ground_truth"].shape == (2, 32)
    path = tmp_path / "p.jsonl"
    path.write_text("\n".join(json.dumps(r) for r in rows))
    assert len(Prompts(str(path), tok, max_prompt_len=8)) == 3
    # samples -> best-of-n rows and preference pairs
    gen = lambda prompts, k: [[[p[0], d] for d in range(k)] for p in prompts]
    reward = lambda p, c: float(c[1] == p[0] % 3) + 0.1 * (c[1] == 0)
    samples = scored_samples(gen, [[3], [4], [8]], 3, reward)
    assert len(samples) == 9 and samples[4].index == 1 and samples[4].draw == 1
    best = best_of_n(samples, minimum=1.0)
    assert [(s.index, s.completion[1]) for s in best] == [(0, 0), (1, 1), (2, 2)]
    pairs = preference_pairs(samples, margin=0.5)
    assert len(pairs) == 3 and all(a.reward - b.reward > 0.5 and a.index == b.index for a, b in pairs)
    more = preference_pairs(samples, margin=0.05, per_prompt=2)
    assert len(more) >= 3 and all(len({a.draw for a, b in more if a.index == i}) == len([1 for a, b in more if a.index == i]) for i in range(3))
    sft = sft_rows(best, seq_len=5)
    assert sft["tokens"].shape == (3, 6) and sft["loss_mask"][0].tolist() == [0, 1, 1, 0, 0, 0]
    dpo = dpo_rows(pairs, seq_len=5)
    assert dpo["chosen"].shape == dpo["rejected"].shape == (3, 6) and np.array_equal(dpo["chosen"][:, 0], dpo["rejected"][:, 0])
    assert write_records(str(tmp_path / "out" / "pairs.jsonl"), pairs, {"generator": "toy", "n": 3}) == 3
    lines = (tmp_path / "out" / "pairs.jsonl").read_text().splitlines()
    assert json.loads(lines[0]) == {"provenance": {"generator": "toy", "n": 3}} and set(json.loads(lines[1])) >= {"prompt", "chosen", "rejected", "chosen_reward"}
    assert best_of_n([Sample((1,), (2, 3), 1.0, 0, 0), Sample((1,), (2,), 1.0, 0, 1)])[0].draw == 1          # a tie goes to the shorter completion
