"""The released text-to-image / video transformer families as architectures: shapes, zero-initialised outputs, gradients reaching
every parameter, the properties their designs promise (rotary positions relative, magnitudes preserved), the registry names, and
one training step through the diffusion objective."""
import math

import pytest
import torch

from dew_b200.models import latent_backbones as LB
from dew_b200.utils.registry import lookup


def _ctx(B, T=5, dt=64, dp=32):
    g = torch.Generator().manual_seed(1)
    return {"text": torch.randn(B, T, dt, generator=g), "pooled": torch.randn(B, dp, generator=g), "guidance": torch.full((B,), 3.5)}


@pytest.mark.parametrize("name,kw", [("flux", dict(guidance_embed=True)), ("flux2", {}), ("qwen_image", dict(double_layers=2)),
                                      ("z_image", dict(single_layers=3)), ("sd3", dict(qk_norm=True)), ("wan", {})])
def test_family_shapes_zero_init_and_gradients(name, kw):
    torch.manual_seed(0)
    model = lookup(name, "model")(emb_features=64, num_heads=4, input_channels=4, **kw)
    x = torch.randn(2, 8, 8, 4)
    t = torch.rand(2)
    out = model(x, t, _ctx(2))
    assert out.shape == x.shape and torch.count_nonzero(out) == 0          # the output projection starts at zero
    for p in model.parameters():                                            # away from the zero initialisation
        if p.requires_grad and torch.count_nonzero(p) == 0:
            torch.nn.init.normal_(p, std=0.02)
    out = model(x, t, _ctx(2))
    out.pow(2).mean().backward()
    dead = [n for n, p in model.named_parameters() if p.requires_grad and (p.grad is None or torch.count_nonzero(p.grad) == 0)]
    # (the last block of a model without single-stream blocks only reads the text's keys and values: the gain on its text queries is idle)
    dead = [n for n in dead if not n.endswith(("txt_qknorm.q.weight", "txt_qk.q.weight"))]
    assert dead == [], dead
    # the text changes the prediction, and so does the time
    other = _ctx(2)
    other["text"] = other["text"] + 1.0
    with torch.no_grad():
        assert not torch.allclose(model(x, t, other), model(x, t, _ctx(2)))
        assert not torch.allclose(model(x, t * 0.5, _ctx(2)), model(x, t, _ctx(2)))


def test_wan_takes_video_and_images():
    torch.manual_seed(0)
    m = LB.WanTransformer(emb_features=64, num_heads=4, input_channels=4, num_layers=2)
    for p in m.parameters():
        if torch.count_nonzero(p) == 0:
            torch.nn.init.normal_(p, std=0.02)
    v = torch.randn(1, 3, 8, 8, 4)
    assert m(v, torch.rand(1), _ctx(1)).shape == v.shape
    assert m(v[:, 0], torch.rand(1), _ctx(1)).shape == v[:, 0].shape


def test_axis_rope_depends_on_relative_positions_only():
    torch.manual_seed(0)
    q, k = torch.randn(1, 6, 2, 16), torch.randn(1, 6, 2, 16)
    ids = LB.grid_ids(1, 1, 2, 3, "cpu")
    dims = (4, 6, 6)
    c0, s0 = LB.axis_rope(ids, dims)
    c1, s1 = LB.axis_rope(ids + torch.tensor([5, 7, 11]), dims)              # every token shifted by the same offset on every axis
    a0 = torch.einsum("bihd,bjhd->bhij", LB.apply_axis_rope(q, c0, s0), LB.apply_axis_rope(k, c0, s0))
    a1 = torch.einsum("bihd,bjhd->bhij", LB.apply_axis_rope(q, c1, s1), LB.apply_axis_rope(k, c1, s1))
    assert torch.allclose(a0, a1, atol=1e-4)
    with pytest.raises(ValueError, match="rotary axes"):
        LB.RectifiedFlowTransformer(emb_features=64, num_heads=4, axes_dims=(4, 4, 4))


def test_edm2_preserves_magnitudes_and_keeps_weights_normalised():
    torch.manual_seed(0)
    net = LB.EDM2UNet(input_channels=4, features=32, multipliers=(1, 2), blocks_per_level=1, attention_levels=(1,), num_classes=10)
    x = torch.randn(4, 16, 16, 4)
    t = torch.randn(4)
    ctx = {"label": torch.tensor([1, 2, 3, 4])}
    assert torch.count_nonzero(net(x, t, ctx)) == 0                          # the output gain starts at zero
    with torch.no_grad():
        net.out_gain.fill_(1.0)
        for blk in list(net.enc) + list(net.dec):
            if hasattr(blk, "emb_gain"):
                blk.emb_gain.fill_(0.5)
    net.train()
    out = net(x, t, ctx)
    # unit-variance input -> an output of order one, although no layer has a bias or a norm with learned gain
    assert 0.3 < float(out.detach().std()) < 3.0, float(out.detach().std())
    # forced weight normalisation: after a training forward every weight has unit norm per output channel
    for name, m in net.named_modules():
        if isinstance(m, LB.MPConv) and name != "logvar_linear":            # (the log-variance head runs only when asked)
            n = torch.linalg.vector_norm(m.weight.float().flatten(1), dim=1) / math.sqrt(m.weight[0].numel())
            assert torch.allclose(n, torch.ones_like(n), atol=1e-3)
    u = net.log_variance(t)
    assert u.shape == (4,)
    (out.pow(2).mean() + u.sum()).backward()
    assert all(p.grad is not None for p in net.parameters() if p.requires_grad)
    # the magnitude-preserving primitives themselves
    a, b = torch.randn(10000), torch.randn(10000)
    assert abs(float(LB.mp_sum(a, b, 0.3).std()) - 1.0) < 0.05
    assert abs(float(LB.mp_silu(a).pow(2).mean().sqrt()) - 1.0) < 0.05
    assert abs(float(LB.mp_cat(a[None], b[None, :5000], 1).pow(2).mean().sqrt()) - 1.0) < 0.05


def test_flux_trains_through_the_diffusion_objective():
    import dew_b200 as dew
    torch.manual_seed(0)
    model = LB.RectifiedFlowTransformer(emb_features=64, num_heads=4, input_channels=3, text_features=16, pooled_features=None, double_layers=1,
                                        single_layers=1)
    from dew_b200.diffusion import Flow
    from dew_b200.objectives.diffusion import DiffusionObjective
    obj = DiffusionObjective(model, Flow(), dew.InputSpec(dew.Field("sample", (8, 8, 3))), ema_decay=None)
    trainer = dew.Trainer(obj, dew.OptimConfig(learning_rate=1e-3), key=0)
    eng = trainer.engine()
    state = eng.fresh_state(trainer.key)
    batch = {"sample": torch.rand(4, 8, 8, 3) * 2 - 1}
    losses = []
    for _ in range(3):
        state, metrics = eng.step(state, batch)
        losses.append(float(metrics["loss"].value()))
    assert all(math.isfinite(v) for v in losses) and state.step == 3
