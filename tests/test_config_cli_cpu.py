"""Configuration overrides, sweeps, the CLI's train / inspect commands, and pipeline(dir) from a run record."""
import json

import pytest
import torch

from dew_b200.cli import main as cli
from dew_b200.config import RunConfig, apply_overrides, set_path, sweep


def _recipe(tmp_path, **trainer):
    cfg = RunConfig()
    cfg.model.fields = dict(vocab_size=259, emb_features=32, num_layers=1, num_heads=4, mlp_features=64, max_seq_len=64)
    cfg.data.seq_len, cfg.data.batch = 16, 4
    cfg.tokenizer = "byte"
    for k, v in trainer.items():
        setattr(cfg.trainer, k, v)
    p = tmp_path / "recipe.json"
    cfg.save(p)
    return p


def test_overrides_and_unknown_paths():
    cfg = apply_overrides(RunConfig(), ["trainer.mesh.fsdp=8", "optimizer.learning_rate=1e-3", "model.fields.num_layers=3", "trainer.resume=never"])
    assert cfg.trainer.mesh.fsdp == 8 and cfg.optimizer.learning_rate == 1e-3 and cfg.model.fields["num_layers"] == 3
    with pytest.raises(KeyError):
        set_path(cfg, "trainer.no_such_field", 1)
    again = RunConfig.from_record(cfg.to_record())
    assert again.trainer.mesh.fsdp == 8 and not cfg.changes(again)
    again.model.fields["num_layers"] = 5
    assert cfg.changes(again) == {"fields.num_layers": (3, 5)}
    points = list(sweep(RunConfig(), {"optimizer.learning_rate": [1e-3, 3e-4], "trainer.key": [0, 1]}))
    assert len(points) == 4 and len({p.trainer.name for p in points}) == 4


def test_cli_train_writes_checkpoint_and_pipeline_reads_it(tmp_path, capsys):
    recipe = _recipe(tmp_path, steps=4, log_every=2, checkpoint_dir=str(tmp_path / "run"))
    assert cli.main(["train", str(recipe), "--cpu", "--set", "optimizer.learning_rate=1e-3"]) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["step"] == 4
    from dew_b200.inference import pipeline
    task = pipeline(tmp_path / "run")
    gen = task(["hello"], max_new_tokens=3)
    assert int(gen.lengths[0]) == 8 and isinstance(gen.text[0], str)
    assert cli.main(["export", str(tmp_path / "run"), str(tmp_path / "hf")]) == 0
    assert (tmp_path / "hf" / "model.safetensors").exists()


def test_cli_inspect_reports_placement(tmp_path, capsys):
    recipe = _recipe(tmp_path)
    assert cli.main(["inspect", str(recipe), "--devices", "8", "--set", "trainer.mesh.fsdp=8"]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["mesh"]["fsdp"] == 8 and rep["fits"]
    assert cli.main(["launch", "--dry-run", "--processes-per-host", "2", "--", "python", "x.py"]) == 0


@pytest.mark.parametrize("recipe,shrink", [
    ("lm/train.py", ["model.fields.emb_features=32", "model.fields.num_layers=1", "model.fields.num_heads=2", "model.fields.num_kv_heads=2",
                     "model.fields.mlp_features=48", "model.fields.vocab_size=64", "model.fields.max_seq_len=16", "data.seq_len=16", "data.batch=2"]),
    ("lm/moe.py", ["model.fields.emb_features=32", "model.fields.num_layers=1", "model.fields.num_heads=2", "model.fields.num_kv_heads=2",
                   "model.fields.mlp_features=48", "model.fields.vocab_size=64", "model.fields.max_seq_len=16", "data.seq_len=16", "data.batch=2",
                   "model.fields.mixture.experts=4", "model.fields.mixture.top_k=2", "model.fields.mixture.expert_features=16",
                   "model.fields.mixture.shared_features=16"]),
    ("diffusion/train.py", ["model.fields.emb_features=32", "model.fields.num_layers=1", "model.fields.num_heads=2", "data.image_shape=[16,16,3]", "data.batch=2"]),
])
def test_shipped_recipes_train_through_the_cli(recipe, shrink, tmp_path, capsys):
    import os
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "recipes", recipe)
    args = ["train", path, "--cpu", "--set", "trainer.steps=3", "--set", f"trainer.checkpoint_dir={tmp_path / 'run'}", "--set", "trainer.log_every=1"]
    for s in shrink:
        args += ["--set", s]
    assert cli.main(args) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["step"] == 3


def test_cli_sweep_trains_every_point(tmp_path, capsys):
    recipe = _recipe(tmp_path, steps=3, log_every=1, checkpoint_dir=str(tmp_path / "sweep"))
    assert cli.main(["sweep", str(recipe), "--cpu", "--grid", "optimizer.learning_rate=1e-3,3e-3", "--grid", "trainer.key=0,1"]) == 0
    lines = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    assert len(lines) == 5 and lines[-1]["points"] == 4 and lines[-1]["best"] in {l["name"] for l in lines[:4]}
    assert all(l["step"] == 3 for l in lines[:4]) and len({l["name"] for l in lines[:4]}) == 4
    assert len(list((tmp_path / "sweep").iterdir())) == 4


def test_records_rebuild_objects_and_refuse_unknown_names_and_fields():
    """A record names a class by import path (or alias) and its fields; rebuilding converts fields by annotation, and unknown
    aliases, unknown fields and untrusted packages raise (src/dew/registry.py)."""
    import pytest
    import torch
    from dew_b200.models.causal_transformer import Mixture, TransformerConfig
    from dew_b200.optim import OptimConfig
    from dew_b200.utils import registry as R
    cfg = TransformerConfig(vocab_size=64, emb_features=32, num_layers=2, num_heads=2, layer_types=("gdn", "attention"),
                            mixture=Mixture(experts=4, top_k=2))
    rec = R.to_record(cfg)
    assert rec["class"] == "dew_b200.models.causal_transformer:TransformerConfig" and rec["fields"]["mixture"]["fields"]["experts"] == 4
    import json
    back = R.from_record(json.loads(json.dumps(rec)))
    assert back == cfg and isinstance(back.layer_types, tuple) and isinstance(back.mixture, Mixture)
    opt = R.from_record({"class": "optim", "fields": {"learning_rate": 1, "optimizer": "lion"}}, kind="optimizer")
    assert isinstance(opt, OptimConfig) and isinstance(opt.learning_rate, (int, float)) and opt.optimizer == "lion"
    model = R.from_record({"class": "causal_transformer", "fields": {"vocab_size": 32, "emb_features": 16, "num_layers": 1, "num_heads": 2}}, kind="model")
    assert sum(p.numel() for p in model.parameters()) > 0
    assert R.from_record(R.to_record(torch.bfloat16)) is torch.bfloat16
    assert R.from_record({"function": "dew_b200.utils.registry:lookup"}) is R.lookup
    with pytest.raises(KeyError, match="known"):
        R.from_record({"class": "no_such_model"}, kind="model")
    with pytest.raises(TypeError, match="has no field"):
        R.from_record({"class": "optim", "fields": {"learning_rat": 1}}, kind="optimizer")
    with pytest.raises(PermissionError, match="trusted"):
        R.from_record({"class": "subprocess:Popen", "fields": {"args": ["true"]}})
    with pytest.raises(R.Unrecordable):
        R.to_record(torch.zeros(2))

    @R.register("toy_model", "model")
    class Toy(torch.nn.Module):
        def __init__(self, width: int = 4):
            super().__init__()
            self.width = width
    assert "toy_model" in R.registry("model") and R.lookup("toy_model") is Toy
    with pytest.raises(ValueError, match="already"):
        R.register("toy_model", "model")(object)


def test_cli_plan_and_data_tools(tmp_path, capsys):
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    assert cli.main(["plan", os.path.join(root, "recipes", "lm", "train.py"), "--devices", "8", "--set", "trainer.mesh.fsdp=8"]) == 0
    plan = json.loads(capsys.readouterr().out)
    assert plan["fits"] and plan["tokens_per_s"] > 0 and 0.2e9 < plan["parameters"] < 0.6e9 and set(plan["by_family"]) >= {"gemm", "attention", "head", "update"}
    rows = tmp_path / "rows.jsonl"
    rows.write_text("\n".join(json.dumps({"id": f"r{i}", "text": f"sample text number {i % 3}", "label": i % 2}) for i in range(12)) + "\n")
    assert cli.main(["data", "analyse", str(rows), "--seq-len", "32"]) == 0
    report = json.loads(capsys.readouterr().out)
    assert report["sampled"] == 12 and report["duplicates"]["exact_duplicate_share"] == 0.75 and report["packing"]["windows"] >= 6
    assert cli.main(["data", "shards", str(rows), str(tmp_path / "shards"), "--samples-per-shard", "5"]) == 0
    assert json.loads(capsys.readouterr().out) == {"shards": 3, "samples": 12, "directory": str(tmp_path / "shards")}
    from dew_b200.data import TarShards
    got = list(TarShards(str(tmp_path / "shards")))
    assert got[4]["__key__"] == "r4" and got[4]["txt"] == "sample text number 1" and got[4]["json"] == {"label": 0}
    assert cli.main(["data", "analyse", str(tmp_path / "shards"), "--text-key", "txt", "--seq-len", "32"]) == 0
    assert json.loads(capsys.readouterr().out)["sampled"] == 12


def test_cli_serve_answers_completions_from_a_run(tmp_path, capsys):
    import threading
    import time
    import urllib.request
    recipe = _recipe(tmp_path, steps=2, log_every=2, checkpoint_dir=str(tmp_path / "run"))
    assert cli.main(["train", str(recipe), "--cpu"]) == 0
    capsys.readouterr()
    result = {}
    t = threading.Thread(target=lambda: result.setdefault("code", cli.main(["serve", str(tmp_path / "run"), "--cpu", "--port", "0", "--slots", "2",
                                                                               "--capacity", "16", "--page-size", "4", "--max-seconds", "6"])))
    t.start()
    address = None
    for _ in range(100):
        time.sleep(0.1)
        out = capsys.readouterr().out
        if "serving" in out:
            address = json.loads(out.strip().splitlines()[-1])["serving"]
            break
    assert address is not None
    req = urllib.request.Request(address + "/v1/completions", data=json.dumps({"prompt": "hi", "max_tokens": 3, "temperature": 0}).encode(), method="POST")
    with urllib.request.urlopen(req, timeout=30) as r:
        body = json.loads(r.read())
    assert body["usage"]["completion_tokens"] == 3 and body["model"] == "run"
    t.join(timeout=30)
    assert result.get("code") == 0
