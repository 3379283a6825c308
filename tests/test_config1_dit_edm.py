"""BASELINE config 1 on CPU: SimpleDiT (patch 4, emb 128, 4 layers, 4 heads) trained with the EDM pixel-space
denoising objective on 64x64x3 images uniform in [-1, 1] from seed 0, batch 16, AdamW 2e-4, 20 steps, with EMA
weights and a checkpoint save / restore round trip."""
import torch

import dew_b200 as dew
from dew_b200.diffusion import EDM
from dew_b200.models import SimpleDiT
from dew_b200.objectives.diffusion import DiffusionObjective
from dew_b200.utils.trees import flatten


def _data(batch=16, n=64):
    g = torch.Generator().manual_seed(0)
    images = torch.rand(n, 64, 64, 3, generator=g) * 2 - 1
    return dew.Memory({"sample": images}).repeat().batched(batch)


def _objective():
    model = SimpleDiT(patch_size=4, emb_features=128, num_layers=4, num_heads=4)
    return DiffusionObjective(model, EDM(regime="pixel"), dew.InputSpec(dew.Field("sample", (64, 64, 3))), ema_decay=0.999)


def test_config1_trains_with_ema_and_checkpoint_roundtrip(tmp_path):
    torch.manual_seed(0)
    ckpt = dew.Checkpoints(tmp_path / "run", keep=2)
    tracker = dew.MemoryTracker()
    trainer = dew.Trainer(_objective(), dew.OptimConfig(learning_rate=2e-4, weight_decay=0.0), key=0,
                          checkpoints=ckpt, tracker=tracker)
    state = trainer.fit(_data(), steps=20, log_every=5, checkpoint_every=10)
    assert state.step == 20 and state.updates == 20
    losses = [r["loss"] for r in tracker.rows]
    assert all(torch.isfinite(torch.tensor(l)) for l in losses)
    assert losses[-1] < losses[0], losses          # the denoiser learns
    live, ema = flatten(state.variables["params"]), flatten(state.ema["params"])
    assert any(not torch.equal(live[k], ema[k]) for k in live)      # EMA lags the live weights
    assert ckpt.steps() == [10, 20]

    # bit-exact round trip into a fresh trainer, then resume two more steps
    ckpt2 = dew.Checkpoints(tmp_path / "run", keep=2)
    trainer2 = dew.Trainer(_objective(), dew.OptimConfig(learning_rate=2e-4, weight_decay=0.0), key=0, checkpoints=ckpt2)
    fresh = trainer2._fresh_state()
    restored = trainer2.engine().adopt(ckpt2.restore(fresh))
    assert restored.step == 20
    r_live, r_ema = flatten(restored.variables["params"]), flatten(restored.ema["params"])
    for k in live:
        assert torch.equal(live[k], r_live[k]), k
        assert torch.equal(ema[k], r_ema[k]), k
    mu, r_mu = flatten(state.opt_state["mu"]), flatten(restored.opt_state["mu"])
    for k in mu:
        assert torch.equal(mu[k], r_mu[k]), k
    state2 = trainer2.fit(_data(), steps=22, log_every=1)
    assert state2.step == 22


def test_edm_sampling_runs():
    obj = _objective()
    variables = obj.init(0)
    out = obj.generate(variables, (2, 64, 64, 3), key=1, steps=4, solver=dew.Heun())
    assert out.shape == (2, 64, 64, 3) and torch.isfinite(out).all()
