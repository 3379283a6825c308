"""Adversarial diffusion distillation: each loss reaches only its own parameters; a few trainer steps run."""
import torch

import dew_b200 as dew
from dew_b200.diffusion import presets
from dew_b200.inputs import Field, InputSpec
from dew_b200.models.dit import SimpleDiT
from dew_b200.objectives import Step
from dew_b200.objectives.adversarial import (AdversarialDistillationObjective, Head, hinge_discriminator, hinge_generator)


def _dit():
    return SimpleDiT(patch_size=4, emb_features=32, num_layers=3, num_heads=2)


def _objective(**kw):
    torch.manual_seed(0)
    teacher = _dit()
    with torch.no_grad():
        for p in teacher.parameters():
            p.add_(0.05 * torch.randn_like(p))
    return AdversarialDistillationObjective(_dit(), presets.Flow(), InputSpec(Field("sample", (16, 16, 3))), teacher=teacher,
                                            layers=("blocks.0", "blocks.2"), width=32, head_channels=16, ema_decay=None, **kw)


def test_hinge_forms_and_head_shape():
    r, f = [torch.tensor([2.0, 0.0])], [torch.tensor([-2.0, 0.5])]
    assert float(hinge_discriminator(r, f)) == 0.5 + 0.75
    assert float(hinge_generator(f)) == 0.75
    assert Head(32, 16, 16)(torch.randn(2, 16, 32), torch.randn(2, 16)).shape == (2, 16)


def test_each_term_reaches_only_its_own_parameters():
    obj = _objective(r1_gamma=1e-2)
    v = obj.init(0)
    batch = {"sample": torch.rand(4, 16, 16, 3) * 2 - 1}
    stat, aux = obj.loss(v, batch, Step(key=1, train=True))
    assert {"generator", "discriminator", "distillation", "r1", "real_score", "fake_score"} <= set(aux.metrics)
    # generator + distillation alone: no gradient on the heads; discriminator alone: none on the student
    names = dict(obj.model.named_parameters())
    (stat.total / stat.mass).backward()
    assert all(p.grad is None for p in obj.teacher.parameters())
    assert any(n.startswith("backbone") and p.grad is not None and float(p.grad.abs().sum()) > 0 for n, p in names.items())
    assert any(n.startswith("discriminator") and p.grad is not None and float(p.grad.abs().sum()) > 0 for n, p in names.items())
    # the generator term alone leaves the heads without a gradient (it reads them through detached weights)
    obj.model.zero_grad()
    obj3 = _objective(r1_gamma=0.0, distill_weight=0.0)
    s3, a3 = obj3.loss(obj3.init(0), batch, Step(key=1, train=True))
    heads = [p for n, p in obj3.model.named_parameters() if n.startswith("discriminator")]
    student = [p for n, p in obj3.model.named_parameters() if n.startswith("backbone")]
    # total = generator + discriminator; the discriminator part has no path to the student
    gs = torch.autograd.grad(s3.total, student, retain_graph=True, allow_unused=True)
    gh = torch.autograd.grad(s3.total, heads, allow_unused=True)
    assert any(g is not None and float(g.abs().sum()) > 0 for g in gs) and any(g is not None and float(g.abs().sum()) > 0 for g in gh)


def test_trains_and_samples():
    obj = _objective()
    trainer = dew.Trainer(obj, dew.OptimConfig(learning_rate=1e-3), key=0)
    g = torch.Generator().manual_seed(0)
    data = [{"sample": torch.rand(4, 16, 16, 3, generator=g) * 2 - 1} for _ in range(6)]
    before = {n: p.detach().clone() for n, p in obj.model.named_parameters()}
    trainer.fit(iter(data), steps=6)
    moved = [n for n, p in obj.model.named_parameters() if not torch.equal(p, before[n])]
    assert any(n.startswith("backbone") for n in moved) and any(n.startswith("discriminator") for n in moved)
    x = obj.generate(None, (2, 16, 16, 3), key=3)
    assert x.shape == (2, 16, 16, 3) and bool(torch.isfinite(x).all())
