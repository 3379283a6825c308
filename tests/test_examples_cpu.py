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
