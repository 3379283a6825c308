"""Step benchmark of the built-in backbones: ``python -m dew_b200.telemetry.benchmark_step --preset small [--models a,b]``.

Per model: ms / step (p10 / p50 / p90 over the timed steps, after warm-up), FLOPs per step (counted, see
``telemetry.instrumentation``), model-FLOP utilisation against the datasheet and the measured peak, peak memory, and set-up
seconds.  ``--preset cpu-smoke`` runs tiny shapes on the CPU (what the tests run); ``small`` is the reference's bf16,
batch-16 preset on one GPU.  Reference: tools/benchmark_step.py (presets ``cpu-smoke`` / ``small``, docs/benchmarks.md:26-39).
"""
from __future__ import annotations

import argparse
import json
import statistics
import time
from typing import Any, Callable, Dict, List

import torch

PRESETS = {
    "cpu-smoke": dict(device="cpu", dtype=torch.float32, batch=2, image=16, width=32, layers=1, heads=2, steps=3, warmup=1, seq=32, vocab=128),
    "small": dict(device="cuda", dtype=torch.bfloat16, batch=16, image=64, width=384, layers=6, heads=6, steps=20, warmup=5, seq=512, vocab=32000),
}


def _builders(p: Dict[str, Any]) -> Dict[str, Callable[[], Any]]:
    import dew_b200 as dew
    from dew_b200 import models as M

    def diffusion(make_model):
        def build():
            model = make_model()
            obj = dew.DiffusionObjective(model, dew.presets.EDM(), ema_decay=None) if hasattr(dew, "DiffusionObjective") else None
            g = torch.Generator().manual_seed(0)
            batch = {"sample": torch.rand(p["batch"], 3, p["image"], p["image"], generator=g) * 2 - 1}
            return obj, batch
        return build

    def lm():
        from dew_b200.objectives.lm import LMObjective
        model = M.CausalTransformer(vocab_size=p["vocab"], emb_features=p["width"], num_layers=p["layers"], num_heads=p["heads"],
                                    num_kv_heads=p["heads"], head_dim=p["width"] // p["heads"], mlp_features=4 * p["width"], max_seq_len=p["seq"])
        g = torch.Generator().manual_seed(0)
        return LMObjective(model, p["seq"], ema_decay=None), {"tokens": torch.randint(0, p["vocab"], (p["batch"], p["seq"] + 1), generator=g)}
    out: Dict[str, Callable[[], Any]] = {"causal_transformer": lm}
    if hasattr(M, "SimpleDiT"):
        out["simple_dit"] = diffusion(lambda: M.SimpleDiT(image_size=p["image"], patch_size=4 if p["image"] >= 16 else 2, emb_features=p["width"],
                                                          num_layers=p["layers"], num_heads=p["heads"]))
    return out


def run(preset: str, models: List[str] = ()) -> List[Dict[str, Any]]:
    import dew_b200 as dew
    from .instrumentation import model_flops_utilization, step_flops
    from .benchmark import measured_peaks
    p = PRESETS[preset]
    rows = []
    for name, build in _builders(p).items():
        if models and name not in models:
            continue
        t0 = time.perf_counter()
        try:
            obj, batch = build()
        except Exception as e:  # a backbone this build does not have is reported, not fatal
            rows.append({"model": name, "error": f"{type(e).__name__}: {str(e)[:120]}"})
            continue
        dev = torch.device(p["device"])
        obj.model.to(dev)
        trainer = dew.Trainer(obj, dew.OptimConfig(learning_rate=1e-4), key=0, param_dtype=p["dtype"] if dev.type == "cuda" else None)
        state = trainer._fresh_state()
        batch = {k: v.to(dev) for k, v in batch.items()}
        eng = trainer.engine()
        for _ in range(p["warmup"]):
            state, _ = eng.step(state, batch)
        setup_s = time.perf_counter() - t0
        times = []
        for _ in range(p["steps"]):
            if dev.type == "cuda":
                torch.cuda.synchronize()
            t1 = time.perf_counter()
            state, _ = eng.step(state, batch)
            if dev.type == "cuda":
                torch.cuda.synchronize()
            times.append((time.perf_counter() - t1) * 1e3)
        times.sort()
        flops = step_flops(obj, batch, rows=min(2, p["batch"]))
        p50 = statistics.median(times)
        peaks = measured_peaks()
        rows.append({"model": name, "preset": preset, "ms_p10": times[max(0, len(times) // 10)], "ms_p50": p50, "ms_p90": times[min(len(times) - 1, len(times) * 9 // 10)],
                     "gflop_per_step": flops.total / 1e9, "mfu_datasheet": model_flops_utilization(flops.total, p50),
                     "mfu_of_measured": model_flops_utilization(flops.total, p50, peak_tflops=peaks["bf16_tflops"]),
                     "samples_per_s": p["batch"] / (p50 * 1e-3), "peak_gib": (torch.cuda.max_memory_allocated() / 2 ** 30) if dev.type == "cuda" else None,
                     "setup_s": setup_s})
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="small", choices=sorted(PRESETS))
    ap.add_argument("--models", default="")
    args = ap.parse_args(argv)
    for row in run(args.preset, [m for m in args.models.split(",") if m]):
        print(json.dumps(row))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
