"""``dewb`` command line: ``train``, ``sweep``, ``profile``, ``inspect``, ``plan``, ``serve``, ``export``, ``data export | analyse | shards``, ``launch``.

Parity: src/dew/_cli/main.py (subcommands Train with ``--set path=value``, Profile, Inspect, Export, DataExport),
src/dew/_cli/launch.py.  Importing this module imports no CUDA library.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import sys
from pathlib import Path
from typing import Optional, Sequence


def _load_recipe(path: str):
    """A recipe is a Python file defining ``config() -> RunConfig`` or a JSON record."""
    from ..config import RunConfig
    p = Path(path)
    if p.suffix == ".json":
        return RunConfig.from_record(json.loads(p.read_text()))
    spec = importlib.util.spec_from_file_location("dewb_recipe", p)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.config()


def cmd_train(args) -> int:
    import torch

    from ..config import apply_overrides, build
    cfg = apply_overrides(_load_recipe(args.recipe), args.set or [])
    device = "cuda" if torch.cuda.is_available() and not args.cpu else "cpu"
    trainer, dataset = build(cfg, device=device)
    tc = cfg.trainer
    state = trainer.fit(dataset, steps=tc.steps, epochs=tc.epochs, tokens=tc.tokens, examples=tc.examples, log_every=tc.log_every,
                        checkpoint_every=tc.checkpoint_every, checkpoint_final=tc.checkpoint_final, resume=tc.resume)
    last = trainer.history[-1] if trainer.history else {}
    print(json.dumps({"step": state.step, **{k: v for k, v in last.items() if isinstance(v, (int, float))}}))
    return 0


def cmd_inspect(args) -> int:
    from ..config import apply_overrides
    from ..parallel.layout import Layout, placement_report
    from ..parallel.mesh import MeshSpec
    from ..utils.registry import lookup
    from ..models import causal_transformer, dit  # noqa: F401
    cfg = apply_overrides(_load_recipe(args.recipe), args.set or [])
    model = lookup(cfg.model.name, "model")(device="meta", **cfg.model.fields)
    m = cfg.trainer.mesh
    rep = placement_report(model, MeshSpec(fsdp=m.fsdp, tensor=m.tensor, expert=m.expert, stage=m.stage), Layout(), devices=args.devices,
                           memory_bytes=args.memory_gb * 1e9, state_dtype=cfg.optimizer.state_dtype)
    rep.pop("leaves")
    print(json.dumps(rep, indent=1, default=str))
    return 0 if rep["fits"] and not rep["refusals"] else 1


def cmd_export(args) -> int:
    from ..inference import pipeline
    from ..interop.hf import Pretrained
    task = pipeline(args.checkpoint)
    from ..utils.trees import variables_for_call
    import torch
    named = variables_for_call(task.model, task.variables)
    with torch.no_grad():
        for n, p in task.model.named_parameters():
            if n in named:
                p.copy_(named[n].to(p.dtype))
    Pretrained.save(task.model, args.out)
    print(f"wrote {args.out}")
    return 0


def cmd_sweep(args) -> int:
    """Train every point of a grid (``--grid path=v1,v2``, repeated; the Cartesian product) one after another, each in its
    own directory under the recipe's checkpoint directory, and print one JSON line per point plus the best one."""
    import torch

    from ..config import _parse, apply_overrides, build, sweep
    base = apply_overrides(_load_recipe(args.recipe), args.set or [])
    grid = {}
    for item in args.grid or []:
        path, _, values = item.partition("=")
        if not values:
            raise SystemExit(f"--grid takes path=v1,v2,..., got {item!r}")
        grid[path] = [_parse(v) for v in values.split(",")]
    device = "cuda" if torch.cuda.is_available() and not args.cpu else "cpu"
    results = []
    for cfg in sweep(base, grid):
        if cfg.trainer.checkpoint_dir:
            cfg.trainer.checkpoint_dir = str(Path(cfg.trainer.checkpoint_dir) / cfg.trainer.name)
        trainer, dataset = build(cfg, device=device)
        tc = cfg.trainer
        state = trainer.fit(dataset, steps=tc.steps, epochs=tc.epochs, tokens=tc.tokens, examples=tc.examples, log_every=tc.log_every,
                            checkpoint_every=tc.checkpoint_every, checkpoint_final=tc.checkpoint_final, resume=tc.resume)
        last = next((h for h in reversed(trainer.history) if "loss" in h), {})
        row = {"name": tc.name, "step": state.step, "loss": last.get("loss")}
        results.append(row)
        print(json.dumps(row))
    scored = [r for r in results if isinstance(r["loss"], (int, float))]
    if scored:
        print(json.dumps({"best": min(scored, key=lambda r: r["loss"])["name"], "points": len(results)}))
    return 0


def cmd_profile(args) -> int:
    from ..telemetry import kernel_bench
    kernel_bench.main(["--only", args.only] + (["--out", args.out] if args.out else []))
    return 0


def cmd_data_export(args) -> int:
    """Tokenise a text file into a flat uint16 token file readable by ``TokenFiles``."""
    import numpy as np

    from ..data import ByteTokenizer
    tok = ByteTokenizer()
    ids = []
    for line in Path(args.text).read_text().splitlines():
        ids.extend(tok.encode(line, eos=True))
    np.asarray(ids, dtype=np.uint16).tofile(args.out)
    print(f"{len(ids)} tokens -> {args.out}")
    return 0


def cmd_plan(args) -> int:
    """Predict a recipe's training step on B200s before running it: per-family milliseconds, tokens / s, MFU and the memory the
    layout needs (``ops.step_cost``), for the recipe's model, batch and mesh."""
    from ..config import apply_overrides
    from ..ops.step_cost import Transformer, transformer_step
    cfg = apply_overrides(_load_recipe(args.recipe), args.set or [])
    f = cfg.model.fields
    if cfg.model.name != "causal_transformer":
        raise SystemExit(f"the step model covers decoder-only transformers, not {cfg.model.name!r}")
    heads = f["num_heads"]
    mix = f.get("mixture") or {}
    model = Transformer(features=f["emb_features"], layers=f["num_layers"], heads=heads, kv_heads=f.get("num_kv_heads") or heads,
                        head_dim=f.get("head_dim") or f["emb_features"] // heads, mlp=f.get("mlp_features") or 4 * f["emb_features"],
                        vocab=f["vocab_size"], experts=mix.get("experts", 0), top_k=mix.get("top_k", 0),
                        expert_mlp=mix.get("expert_features", 0), shared_experts=1 if mix.get("shared_features") else 0,
                        tied=bool(f.get("tie_embeddings", True)))
    m = cfg.trainer.mesh
    world = args.devices
    micro = max(1, cfg.data.batch // max(1, cfg.trainer.microbatches or 1))
    out = transformer_step(model, sequences=cfg.data.batch, seq_len=cfg.data.seq_len, microbatch=micro, world=world, tensor=max(1, m.tensor),
                           expert=max(1, m.expert), remat=bool(f.get("remat")), mx_experts=bool(mix))
    out["parameters"] = model.params
    print(json.dumps(out, indent=1, default=float))
    return 0 if out["fits"] else 1


def _rows_of(path: str):
    from ..data import JsonLines, TarShards
    p = Path(path)
    if p.is_dir():
        return TarShards(str(p))
    if p.suffix in (".jsonl", ".json"):
        return JsonLines(str(p))
    return ({"text": line} for line in p.read_text().splitlines() if line.strip())


def cmd_data_analyse(args) -> int:
    """Length, packing, vocabulary and duplicate statistics of a corpus (a text file, a JSON-lines file or a shard directory)."""
    from ..data import ByteTokenizer
    from ..data.analysis import analyse
    report = analyse(_rows_of(args.source), ByteTokenizer(), seq_len=args.seq_len, text_key=args.text_key, sample=args.sample)
    print(json.dumps(report, indent=1))
    return 0


def cmd_data_shards(args) -> int:
    """Write a JSON-lines file as tar shards: each record's fields become a sample's members (strings as .txt-like text, the rest as
    .json), keyed by the record's ``id`` / ``key`` where it has one."""
    from ..data.shards import write_shards

    def samples():
        for i, row in enumerate(_rows_of(args.source)):
            out = {"__key__": str(row.get("id", row.get("key", f"{i:09d}")))}
            rest = {}
            for k, v in row.items():
                if k in ("id", "key"):
                    continue
                if isinstance(v, str) and k in ("text", "caption", "txt"):
                    out["txt"] = v
                else:
                    rest[k] = v
            if rest:
                out["json"] = rest
            yield out
    index = write_shards(samples(), args.out, samples_per_shard=args.samples_per_shard)
    print(json.dumps({"shards": len(index["shards"]), "samples": index["samples"], "directory": args.out}))
    return 0


def cmd_serve(args) -> int:
    """Serve a run's language model over HTTP (``/v1/completions``, ``/v1/chat/completions``, ``/metrics``)."""
    import time

    import torch

    from ..inference import Server, pipeline
    from ..inference.http import CompletionService
    from ..nn.kv_cache import KVCache
    task = pipeline(args.checkpoint)
    if torch.cuda.is_available() and not args.cpu:
        task.model.cuda()
    server = Server.from_task(task, slots=args.slots, capacity=args.capacity, kv_cache=KVCache(page_size=args.page_size), host_pages=args.host_pages,
                              cuda_graph=torch.cuda.is_available() and not args.cpu)
    with CompletionService(server, name=args.name or Path(args.checkpoint).name, host=args.host, port=args.port) as service:
        print(json.dumps({"serving": f"http://{service.address[0]}:{service.address[1]}", "model": service.name}), flush=True)
        began = time.monotonic()
        try:
            while args.max_seconds is None or time.monotonic() - began < args.max_seconds:
                time.sleep(0.2)
        except KeyboardInterrupt:
            pass
    return 0


def main(argv: Optional[Sequence[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "launch":
        from . import launch
        return launch.main(argv[1:])
    ap = argparse.ArgumentParser(prog="dewb")
    sub = ap.add_subparsers(dest="command", required=True)
    t = sub.add_parser("train"); t.add_argument("recipe"); t.add_argument("--set", action="append"); t.add_argument("--cpu", action="store_true")
    t.set_defaults(fn=cmd_train)
    w = sub.add_parser("sweep"); w.add_argument("recipe"); w.add_argument("--set", action="append"); w.add_argument("--grid", action="append")
    w.add_argument("--cpu", action="store_true"); w.set_defaults(fn=cmd_sweep)
    i = sub.add_parser("inspect"); i.add_argument("recipe"); i.add_argument("--set", action="append")
    i.add_argument("--devices", type=int, default=8); i.add_argument("--memory-gb", type=float, default=180.0); i.set_defaults(fn=cmd_inspect)
    e = sub.add_parser("export"); e.add_argument("checkpoint"); e.add_argument("out"); e.set_defaults(fn=cmd_export)
    p = sub.add_parser("profile"); p.add_argument("--only", default="gemm,rows,attention"); p.add_argument("--out", default=None); p.set_defaults(fn=cmd_profile)
    d = sub.add_parser("data"); ds = d.add_subparsers(dest="data_command", required=True)
    de = ds.add_parser("export"); de.add_argument("text"); de.add_argument("out"); de.set_defaults(fn=cmd_data_export)
    da = ds.add_parser("analyse"); da.add_argument("source"); da.add_argument("--seq-len", type=int, default=2048)
    da.add_argument("--text-key", default="text"); da.add_argument("--sample", type=int, default=10000); da.set_defaults(fn=cmd_data_analyse)
    dh = ds.add_parser("shards"); dh.add_argument("source"); dh.add_argument("out"); dh.add_argument("--samples-per-shard", type=int, default=1000)
    dh.set_defaults(fn=cmd_data_shards)
    sv = sub.add_parser("serve"); sv.add_argument("checkpoint"); sv.add_argument("--host", default="127.0.0.1"); sv.add_argument("--port", type=int, default=8000)
    sv.add_argument("--slots", type=int, default=64); sv.add_argument("--capacity", type=int, default=2048); sv.add_argument("--page-size", type=int, default=16)
    sv.add_argument("--host-pages", type=int, default=0); sv.add_argument("--name", default=None); sv.add_argument("--cpu", action="store_true")
    sv.add_argument("--max-seconds", type=float, default=None); sv.set_defaults(fn=cmd_serve)
    pl = sub.add_parser("plan"); pl.add_argument("recipe"); pl.add_argument("--set", action="append"); pl.add_argument("--devices", type=int, default=8)
    pl.set_defaults(fn=cmd_plan)
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
