"""``dewb`` command line: ``train``, ``sweep``, ``profile``, ``inspect``, ``export``, ``data export``, ``launch``.

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
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
