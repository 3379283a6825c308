"""``python -m dew_b200.eval --model DIR --tasks hellaswag,arc_easy``: score a released checkpoint (a directory ``Pretrained.load`` reads) on
evaluation-harness tasks through ``HarnessModel``.  The harness (``lm_eval``) is an optional dependency: without it the command says so
and exits 2; ``--perplexity FILE`` needs nothing else and reports the rolling log-likelihood of a text file, which is also what a smoke
test of a converted checkpoint wants.

Reference: src/dew/eval/__main__.py (the harness command line with this library registered as a model).
"""
from __future__ import annotations

import argparse
import json
import math
import sys
from typing import List, Optional


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="python -m dew_b200.eval", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="a release directory (config.json + safetensors)")
    ap.add_argument("--tokenizer", default=None, help="a tokenizer directory (default: the model's); 'bytes' for the byte tokenizer")
    ap.add_argument("--tasks", default="", help="comma-separated harness task names")
    ap.add_argument("--perplexity", default=None, help="a text file: report its rolling log-likelihood per token and per byte")
    ap.add_argument("--limit", type=int, default=None, help="examples per task")
    ap.add_argument("--batch-size", type=int, default=16)
    ap.add_argument("--max-length", type=int, default=2048)
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--device", default=None)
    args = ap.parse_args(argv)
    if not args.tasks and not args.perplexity:
        ap.error("nothing to do: give --tasks or --perplexity")

    import torch
    from ..interop.hf import Pretrained
    from .harness import HarnessModel
    device = args.device or ("cuda" if torch.cuda.is_available() else "cpu")
    model = Pretrained.load(args.model, dtype=getattr(torch, args.dtype), device=device).eval()
    if args.tokenizer == "bytes":
        from ..data.tokenizer import ByteTokenizer
        tokenizer = ByteTokenizer()
    else:
        import transformers
        tokenizer = transformers.AutoTokenizer.from_pretrained(args.tokenizer or args.model)
    lm = HarnessModel(model, tokenizer, max_length=args.max_length, batch_size=args.batch_size)
    report = {"model": args.model, "family": getattr(model, "family", None)}
    if args.perplexity:
        text = open(args.perplexity, encoding="utf-8").read()
        total = float(lm.loglikelihood_rolling([(text,)])[0])
        tokens = max(1, len(lm._encode(text)))
        report["perplexity"] = {"log_likelihood": total, "tokens": tokens, "per_token_perplexity": math.exp(-total / tokens),
                                "bits_per_byte": -total / math.log(2) / max(1, len(text.encode("utf-8")))}
    if args.tasks:
        try:
            import lm_eval
        except ImportError:
            print("the evaluation harness (lm_eval) is not installed: --tasks needs it; --perplexity does not", file=sys.stderr)
            return 2
        results = lm_eval.simple_evaluate(model=lm, tasks=[t for t in args.tasks.split(",") if t], limit=args.limit)
        report["tasks"] = results.get("results", results)
    print(json.dumps(report, indent=2, default=str))
    return 0


if __name__ == "__main__":
    sys.exit(main())
