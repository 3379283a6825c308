"""Representation alignment (REPA / iREPA) and guidance distillation on a tiny DiT."""
import pytest
import torch

import dew_b200 as dew
from dew_b200.diffusion import presets
from dew_b200.inputs import Condition, Field, InputSpec
from dew_b200.models.dit import SimpleDiT
from dew_b200.objectives import Step
from dew_b200.objectives.diffusion_extras import (AlignedDiffusionObjective, Alignment, GuidanceDistillationObjective,
                                                  Projector, guide, spatial_zscore)


def _dit(**kw):
    return SimpleDiT(patch_size=4, emb_features=32, num_layers=3, num_heads=2, **kw)


def _patch_means(px):
    """A fixed 'encoder': 4 x 4 patch means of the normalised pixels and their squares -> [B, 16, 6]."""
    B = px.shape[0]
    p = px.reshape(B, 4, 4, 4, 4, 3).mean((2, 4))
    return torch.cat([p, p * p], -1).reshape(B, 16, 6)


def test_projectors_and_zscore():
    tok = torch.randn(2, 16, 8)
    assert Projector("mlp", 8, 5, width=12)(tok).shape == (2, 16, 5)
    assert Projector("conv", 8, 5)(tok).shape == (2, 16, 5)
    with pytest.raises(ValueError):
        Projector("conv", 8, 5)(torch.randn(2, 15, 8))
    f = torch.randn(2, 16, 4)
    z = spatial_zscore(f, 1.0)
    assert torch.allclose(z.mean(1), torch.zeros(2, 4), atol=1e-5) and torch.allclose(z.std(1), torch.ones(2, 4), atol=1e-3)
    half = spatial_zscore(f, 0.5)
    assert torch.allclose(half * (f.std(1, keepdim=True) + 1e-6), f - 0.5 * f.mean(1, keepdim=True), atol=1e-5)


@pytest.mark.parametrize("kind,norm", [("mlp", None), ("conv", 0.6)])
def test_alignment_term_trains_the_projector_and_the_backbone(kind, norm):
    torch.manual_seed(0)
    model = _dit()
    al = Alignment(layer="blocks.1", encoder=_patch_means, weight=0.5, projector=kind, width=16, spatial_norm=norm, resolution=None)
    obj = AlignedDiffusionObjective(model, presets.EDM(regime="pixel"), InputSpec(Field("sample", (16, 16, 3))), alignment=al,
                                    hidden_features=32, encoder_features=6, ema_decay=None)
    variables = obj.init(0)
    assert any("alignment_projector" in "/".join(map(str, k)) or "alignment_projector" in str(k) for k in _flat(variables["params"]))
    batch = {"sample": torch.rand(4, 16, 16, 3) * 2 - 1}
    stat, aux = obj.loss(variables, batch, Step(key=1, train=True))
    base = AlignedDiffusionObjective.__mro__[1].loss(obj, variables, batch, Step(key=1, train=True))[0]
    align = aux.metrics["alignment"]
    assert -1.0 <= float(align.value()) <= 1.0
    assert torch.allclose(stat.total, base.total + 0.25 * align.total, atol=1e-5)
    (stat.total / stat.mass).backward()
    grads = {n: p.grad for n, p in obj.model.named_parameters() if p.grad is not None and float(p.grad.abs().sum()) > 0}
    assert any(n.startswith("alignment_projector") for n in grads) and any(n.startswith("backbone.blocks.0") for n in grads)
    # a layer that yields another token count is refused
    bad = Alignment(layer="blocks.1", encoder=lambda px: torch.zeros(px.shape[0], 9, 6), resolution=None)
    obj2 = AlignedDiffusionObjective(_dit(), presets.EDM(regime="pixel"), InputSpec(Field("sample", (16, 16, 3))), alignment=bad,
                                     hidden_features=32, encoder_features=6, ema_decay=None)
    with pytest.raises(ValueError):
        obj2.loss(obj2.init(0), batch, Step(key=1, train=True))


def _flat(tree, prefix=()):
    for k, v in tree.items():
        if isinstance(v, dict):
            yield from _flat(v, prefix + (k,))
        else:
            yield prefix + (k,)


def test_aligned_objective_trains_through_the_trainer():
    torch.manual_seed(0)
    al = Alignment(layer="blocks.1", encoder=_patch_means, projector="mlp", width=16, resolution=None)
    obj = AlignedDiffusionObjective(_dit(), presets.EDM(regime="pixel"), InputSpec(Field("sample", (16, 16, 3))), alignment=al,
                                    hidden_features=32, encoder_features=6, ema_decay=None)
    trainer = dew.Trainer(obj, dew.OptimConfig(learning_rate=2e-3), key=0)
    g = torch.Generator().manual_seed(0)
    data = [{"sample": torch.rand(4, 16, 16, 3, generator=g) * 2 - 1} for _ in range(12)]
    before = {n: p.detach().clone() for n, p in obj.model.named_parameters()}
    trainer.fit(iter(data), steps=12)
    moved = [n for n, p in obj.model.named_parameters() if not torch.equal(p, before[n])]
    assert any(n.startswith("alignment_projector") for n in moved) and any(n.startswith("backbone") for n in moved)


def test_guidance_distillation_matches_the_guided_teacher():
    torch.manual_seed(0)
    inputs = InputSpec(Field("sample", (16, 16, 3)), {"label": Condition(Field("label", ()), null=4)})
    teacher = _dit(num_classes=4)
    with torch.no_grad():                       # give the teacher a non-zero head so its two branches differ
        for p in teacher.parameters():
            p.add_(0.05 * torch.randn_like(p))
    student = _dit(num_classes=4, guidance_embed=True)
    obj = GuidanceDistillationObjective(student, presets.Flow(), inputs, teacher=teacher, scales=(1.0, 8.0), ema_decay=None)
    variables = obj.init(0)
    batch = {"sample": torch.rand(4, 16, 16, 3) * 2 - 1, "label": torch.tensor([0, 1, 2, 3])}
    stat, aux = obj.loss(variables, batch, Step(key=3, train=True))
    scale = float(aux.metrics["guidance_scale"].value())
    assert 1.0 <= scale <= 8.0 and float(stat.total.detach()) > 0
    (stat.total / stat.mass).backward()
    assert any(p.grad is not None and float(p.grad.abs().sum()) > 0 for p in student.parameters())
    assert all(p.grad is None for p in teacher.parameters())
    # a student that already equals the guided teacher has zero loss: scales (1, 1) make the target the conditional branch
    same = GuidanceDistillationObjective(teacher, presets.Flow(), inputs, scales=(1.0, 1.0), ema_decay=None)
    s2, _ = same.loss(None, batch, Step(key=3, train=False))
    assert float(s2.total) < 1e-10
    c, u = torch.randn(3, 2), torch.randn(3, 2)
    assert torch.allclose(guide(c, u, torch.tensor([1.0, 0.0, 2.0])), torch.stack([c[0], u[1], u[2] + 2 * (c[2] - u[2])]))
    with pytest.raises(ValueError):
        GuidanceDistillationObjective(_dit(), presets.Flow(), InputSpec(Field("sample", (16, 16, 3))))


def test_end_to_end_objective_routes_each_gradient_to_its_part():
    from dew_b200.models.autoencoders import KLAutoEncoder
    from dew_b200.objectives.end_to_end import EndToEndObjective
    torch.manual_seed(0)
    vae = KLAutoEncoder(channels=3, latent_channels=4, features=8, downsample=1, scale=1.0)
    dit = SimpleDiT(patch_size=2, emb_features=32, num_layers=2, num_heads=2, input_channels=4, output_channels=4)
    al = Alignment(layer="blocks.0", encoder=lambda px: _patch_means(px), projector="mlp", width=16, resolution=None)
    obj = EndToEndObjective(dit, vae, presets.Flow(), InputSpec(Field("sample", (8, 8, 4))), alignment=al, hidden_features=32, encoder_features=6,
                            vae_align=1.5, kl_weight=1e-4, ema_decay=None)
    batch = {"sample": torch.rand(4, 16, 16, 3) * 2 - 1}
    v = obj.init(0)
    stat, aux = obj.loss(v, batch, Step(key=2, train=True))
    assert {"denoising", "reconstruction", "alignment", "latent_alignment", "latent_std"} <= set(aux.metrics)
    (stat.total / stat.mass).backward()
    named = dict(obj.model.named_parameters())
    g = lambda prefix: sum(float(p.grad.abs().sum()) for n, p in named.items() if n.startswith(prefix) and p.grad is not None)
    assert g("autoencoder.encoder") > 0 and g("autoencoder.decoder") > 0 and g("denoiser.backbone") > 0 and g("denoiser.alignment_projector") > 0
    # the denoising loss does not reach the encoder: with the latent's alignment term off and the reconstruction term
    # cancelled, the encoder's gradient is exactly zero although the diffusion model still trains
    obj.model.zero_grad()
    cancel = lambda recon, images: -(recon - images).abs().reshape(images.shape[0], -1).mean(1)
    obj2 = EndToEndObjective(dit, vae, presets.Flow(), InputSpec(Field("sample", (8, 8, 4))), alignment=al, hidden_features=32, encoder_features=6,
                             vae_align=0.0, kl_weight=0.0, extra_vae_loss=cancel, ema_decay=None)
    s2, _ = obj2.loss(None, batch, Step(key=2, train=True))
    (s2.total / s2.mass).backward()
    named2 = dict(obj2.model.named_parameters())
    assert all(p.grad is None or float(p.grad.abs().sum()) < 1e-10 for n, p in named2.items() if n.startswith("autoencoder.encoder"))
    assert any(p.grad is not None and float(p.grad.abs().sum()) > 0 for n, p in named2.items() if n.startswith("denoiser.backbone"))
    obj2.model.zero_grad()
    # a few steps train all parts
    trainer = dew.Trainer(obj, dew.OptimConfig(learning_rate=1e-3), key=0)
    before = {n: p.detach().clone() for n, p in obj.model.named_parameters()}
    trainer.fit([batch] * 4, steps=4)
    moved = {n.split(".")[0] + "." + n.split(".")[1] for n, p in obj.model.named_parameters() if not torch.equal(p, before[n])}
    assert {"autoencoder.encoder", "autoencoder.decoder", "denoiser.backbone", "denoiser.alignment_projector"} <= moved
    x = obj.generate(None, (2, 8, 8, 4), key=1, steps=3)
    assert x.shape == (2, 16, 16, 3)
