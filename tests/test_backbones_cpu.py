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
