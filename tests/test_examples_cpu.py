"""The example scripts run end to end at a few steps on CPU."""
import importlib.util
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "examples", f"{name}.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("kind", ["dense", "moe", "hybrid", "mamba2"])
def test_train_lm_example(kind):
    losses = _load("train_lm").main(["--kind", kind, "--steps", "20", "--device", "cpu"])
    assert losses[-1] < losses[0]


@pytest.mark.parametrize("process", ["edm", "flow"])
def test_train_diffusion_example(process):
    losses = _load("train_diffusion").main(["--process", process, "--steps", "12", "--device", "cpu"])
    assert len(losses) >= 2


def test_train_masked_lm_example():
    losses = _load("train_masked_lm").main(["--steps", "30", "--device", "cpu"])
    assert losses[-1] < losses[0]


def test_evaluate_and_serve_example():
    assert _load("evaluate_and_serve").main(["--device", "cpu"])


def test_train_jepa_example():
    losses, acc = _load("train_jepa").main(["--steps", "40", "--device", "cpu"])
    assert losses[-1] < losses[0] and acc >= 0.5


def test_train_rlvr_example():
    history = _load("train_rlvr").main(["--rounds", "6", "--pretrain", "60", "--device", "cpu"])
    assert len(history) == 6 and all(0.0 <= h <= 1.0 for h in history)


def test_moe_mesh_example_on_two_cpu_ranks():
    import json
    import subprocess
    import sys
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29571", os.path.join(ROOT, "examples", "moe_mesh.py"), "--steps", "12", "--backend", "gloo"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert out.returncode == 0, out.stdout[-1500:] + out.stderr[-3000:]
    r = json.loads(next(l for l in out.stdout.splitlines() if l.startswith("RESULT "))[len("RESULT "):])
    assert r["world"] == 2 and r["last"] < r["first"]


def test_sample_text_to_image_example():
    hits, total = _load("sample_text_to_image").main(["--steps", "150", "--device", "cpu"])
    assert total == 6 and hits >= 3


def test_train_supervised_example():
    assert _load("train_supervised").main(["--steps", "300", "--device", "cpu"]) > 0.7


def test_pinn_burgers_example_and_gauss_newton_on_a_linear_system():
    import torch
    from dew_b200.optim.gauss_newton import LevenbergMarquardt, gauss_newton_direction
    # on a linear least-squares problem one undamped step lands on the solution, primal and dual alike
    torch.manual_seed(0)
    A, b = torch.randn(12, 4, dtype=torch.float64), torch.randn(12, dtype=torch.float64)
    x = torch.zeros(4, dtype=torch.float64)
    step = gauss_newton_direction(A @ x - b, A, 1e-12)
    assert torch.allclose(x - step, torch.linalg.lstsq(A, b[:, None]).solution[:, 0], atol=1e-8)
    wide = torch.randn(3, 7, dtype=torch.float64)
    d = gauss_newton_direction(wide @ torch.zeros(7, dtype=torch.float64) - b[:3], wide, 1e-12)
    assert torch.allclose(wide @ (-d), b[:3], atol=1e-8)                     # the dual solve satisfies every residual
    history = _load("pinn_burgers").main(["--steps", "12"])
    assert history[-1] < 0.05 * history[0]


def test_route_decisions_example():
    report = _load("route_decisions").main(["--steps", "200"])
    assert report["accuracy"] > 0.8 and report["scored_questions"] == 768 and report["brier"] < 0.4
    assert 0.3 < report["answered"] <= 1.0 and report["answered_accuracy"] >= report["accuracy"] - 0.02


def test_sft_chat_example():
    losses, right, answers = _load("sft_chat").main(["--steps", "150", "--device", "cpu"])
    assert losses[-1] < 0.5 * losses[0] and right >= 3 and set(answers) == {"red", "green", "blue", "pink", "grey", "gold"}


def test_serve_decisions_example_answers_over_http():
    one, many, metrics = _load("serve_decisions").main(["--steps", "60"])
    assert set(one["answers"]) == {"parity", "half", "size"} and "abstained" in one["answers"]["parity"] and one["usage"]["input_tokens"] > 0
    assert len(many) == 4 and all("answers" in m for m in many[:3]) and many[3]["reason"] == "malformed"
    assert "dew_decide_requests" in metrics and "dew_decide_passes" in metrics


def test_forward_only_lm_example():
    results = _load("forward_only_lm").main(["--steps", "60", "--draws", "4"])
    assert results["forward_only"][-1] < results["forward_only"][0] - 0.15 and results["backprop"][-1] < results["forward_only"][-1]
