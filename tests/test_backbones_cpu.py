"""Every diffusion backbone runs forward / backward behind the same call and trains under a flow-matching objective;
the latent path goes through the autoencoder."""
import pytest
import torch

import dew_b200 as dew
from dew_b200.diffusion import Flow
from dew_b200.models import HybridDiT, KLAutoEncoder, SimpleDiT, SimpleMMDiT, SimpleUDiT, UNet, UViT, VideoDiT, ViT
from dew_b200.objectives.diffusion import DiffusionObjective


@pytest.mark.parametrize("make", [
    lambda: UNet(features=(16, 32), attention_levels=(1,), blocks_per_level=1),
    lambda: UViT(patch_size=4, emb_features=32, num_layers=4, num_heads=2),
    lambda: SimpleUDiT(patch_size=4, emb_features=32, num_layers=4, num_heads=2),
    lambda: SimpleMMDiT(patch_size=4, emb_features=32, num_layers=2, num_heads=2, text_features=8),
    lambda: HybridDiT(patch_size=4, emb_features=32, num_layers=2, num_heads=2, state_dim=8),
    lambda: SimpleDiT(patch_size=4, emb_features=32, num_layers=2, num_heads=2, routes=((0.5, 0, 1),)),
])
def test_backbone_forward_backward(make):
    torch.manual_seed(0)
    m = make()
    x = torch.randn(2, 16, 16, 3)
    ctx = {"text": torch.randn(2, 5, 8)} if isinstance(m, SimpleMMDiT) else None
    y = m(x, torch.rand(2), ctx, train=True)
    assert y.shape == x.shape
    for p in m.parameters():                     # zero-initialised heads block gradients at init: open them
        if p.dim() >= 1 and float(p.abs().sum()) == 0:
            torch.nn.init.normal_(p, std=0.02)
    m(x, torch.rand(2), ctx, train=True).pow(2).mean().backward()
    assert any(p.grad is not None and float(p.grad.abs().sum()) > 0 for p in m.parameters())


def test_video_dit_and_vit():
    v = VideoDiT(patch_size=4, emb_features=32, num_layers=1, num_heads=2)
    assert v(torch.randn(2, 3, 8, 8, 3), torch.rand(2)).shape == (2, 3, 8, 8, 3)
    assert ViT(patch_size=4, features=32, num_layers=2, num_heads=2)(torch.randn(2, 8, 8, 3)).shape == (2, 4, 32)


def test_flow_matching_in_latent_space():
    torch.manual_seed(0)
    ae = KLAutoEncoder(features=8, downsample=1)
    z = ae.encode(torch.randn(2, 16, 16, 3))
    assert z.shape == (2, 8, 8, 4) and ae.decode(z).shape == (2, 16, 16, 3)
    model = SimpleDiT(patch_size=2, emb_features=16, num_layers=1, num_heads=2, input_channels=4, output_channels=4)
    obj = DiffusionObjective(model, Flow(), dew.InputSpec(dew.Field("sample", (16, 16, 3))), autoencoder=ae, ema_decay=None)
    tr = dew.Trainer(obj, dew.OptimConfig(learning_rate=1e-3), tracker=(t := dew.MemoryTracker()))
    data = dew.Memory({"sample": torch.rand(8, 16, 16, 3) * 2 - 1}).repeat().batched(4)
    st = tr.fit(data, steps=3, log_every=1)
    assert st.step == 3 and all(r["loss"] == r["loss"] for r in t.rows)
    img = obj.generate(st.variables, (2, 8, 8, 4), key=0, steps=3, solver=dew.Euler())
    assert img.shape == (2, 16, 16, 3)


def test_hyper_connections_and_altup_reduce_to_the_residual_stack_and_train():
    """With one effective stream both connection kinds reproduce the ordinary residual stack; with several they train."""
    import torch
    from dew_b200.models import CausalTransformer
    from dew_b200.nn.streams import AltUp, HyperConnections
    kw = dict(vocab_size=40, emb_features=32, num_layers=3, num_heads=4, head_dim=8, mlp_features=64, max_seq_len=32)
    torch.manual_seed(0)
    plain = CausalTransformer(**kw)
    tokens = torch.randint(0, 40, (2, 12))
    for field in ("hyper_connections", "altup"):
        torch.manual_seed(0)
        multi = CausalTransformer(**kw, **{field: 2})
        multi.load_state_dict(plain.state_dict(), strict=False)
        out = multi(tokens)
        assert out.shape == (2, 12, 40)
        out.float().pow(2).mean().backward()
        grads = [p.grad for n, p in multi.named_parameters() if "streams" in n and p.grad is not None]
        assert grads and any(float(g.abs().sum()) > 0 for g in grads)
    # one stream: H' = H + f(norm(H)) exactly
    hc = HyperConnections(8, 1, 0, dynamic=False)
    H = torch.randn(2, 5, 1, 8)
    x, ctx = hc.read(H)
    assert torch.allclose(x, H[:, :, 0]) and torch.allclose(hc.write(H, torch.ones(2, 5, 8), ctx), H + 1)
    au = AltUp(1, 0)
    x, pred = au.read(H)
    assert torch.allclose(au.write(H, torch.ones(2, 5, 8), pred), H + 1)


def test_more_backbone_families_forward_and_backward():
    import torch
    from dew_b200.models.diffusion_backbones import HierarchicalMMDiT, JepaEncoder, JepaVideoEncoder, SSMDiT, UNet3D
    from dew_b200.utils.registry import lookup
    torch.manual_seed(0)
    t = torch.rand(2)
    vid = torch.randn(2, 3, 16, 16, 3)
    net = UNet3D(features=(16, 32), heads=2)
    for p in net.out[-1].parameters():
        torch.nn.init.normal_(p, std=0.02)
    y = net(vid, t)
    assert y.shape == vid.shape
    y.pow(2).mean().backward()
    assert all(p.grad is not None for n, p in net.named_parameters() if "gate" not in n or True)
    # temporal mixing: with open gates a change in one frame reaches the others
    with torch.no_grad():
        for m in net.modules():
            if hasattr(m, "gate"):
                m.gate.fill_(1.0)
        other = vid.clone(); other[:, 0] += 1.0
        assert float((net(other, t)[:, 2] - net(vid, t)[:, 2]).abs().max()) > 0
    img = torch.randn(2, 16, 16, 3)
    h = HierarchicalMMDiT(emb_features=32, num_heads=2, text_features=8)
    for p in h.output.out.parameters():
        torch.nn.init.normal_(p, std=0.02)
    out = h(img, t, {"text": torch.randn(2, 5, 8)})
    assert out.shape == img.shape
    out.pow(2).mean().backward()
    assert h.merge.weight.grad is not None and float(h.merge.weight.grad.abs().sum()) > 0
    s = SSMDiT(emb_features=64, num_layers=2, num_heads=2, state_dim=16)
    assert s.kinds == ["mamba2", "mamba2"] and s(img, t).shape == img.shape
    enc = JepaEncoder(emb_features=32, num_layers=2, num_heads=2)
    full = enc(img)
    keep = torch.zeros(16, dtype=torch.bool); keep[:6] = True
    assert full.shape == (2, 16, 32) and enc(img, keep).shape == (2, 6, 32)
    venc = JepaVideoEncoder(frames=3, emb_features=32, num_layers=1, num_heads=2)
    assert venc(vid).shape == (2, 3 * 16, 32)
    for name in ("unet_3d", "hierarchical_mmdit", "ssm_dit", "jepa_encoder", "jepa_video_encoder"):
        assert lookup(name) is not None
