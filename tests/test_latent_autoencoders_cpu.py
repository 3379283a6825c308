"""Latent autoencoders: the KL VAE's published layout, deep-compression and causal video autoencoders, latent normalisation, tiling."""
import pytest
import torch

from dew_b200.models.latent_autoencoders import (DCAE, AutoencoderKL, CausalConv3d, CausalVideoVAE, LatentNormalization, _channel_to_space,
                                                 _space_to_channel, _tiled)


def _small_kl(**kw):
    return AutoencoderKL(block_out_channels=(32, 64, 64), layers_per_block=1, norm_groups=8, **kw)


def test_kl_autoencoder_shapes_names_and_normalisation():
    torch.manual_seed(0)
    ae = _small_kl(latent_channels=4)
    x = torch.rand(2, 32, 48, 3) * 2 - 1
    z = ae.encode(x)
    assert z.shape == (2, 8, 12, 4) and ae.decode(z).shape == x.shape and ae.downsample == 4
    mean, _ = ae.moments(x)
    assert torch.allclose(z, mean.permute(0, 2, 3, 1) * 0.18215, atol=1e-6)
    a = ae.encode(x, sample=True, generator=torch.Generator().manual_seed(1))
    b = ae.encode(x, sample=True, generator=torch.Generator().manual_seed(1))
    assert torch.equal(a, b) and not torch.equal(a, z)
    keys = set(ae.state_dict())
    # the published checkpoints' key layout: their state dicts load without a name map
    for k in ("encoder.conv_in.weight", "encoder.down_blocks.0.resnets.0.norm1.weight", "encoder.down_blocks.0.downsamplers.0.conv.weight",
              "encoder.down_blocks.1.resnets.0.conv_shortcut.weight", "encoder.mid_block.attentions.0.to_q.weight",
              "encoder.mid_block.attentions.0.to_out.0.bias", "encoder.mid_block.resnets.1.conv2.bias", "encoder.conv_norm_out.weight",
              "decoder.up_blocks.0.resnets.1.conv1.weight", "decoder.up_blocks.0.upsamplers.0.conv.weight", "decoder.up_blocks.2.resnets.1.norm2.bias",
              "decoder.conv_out.bias", "quant_conv.weight", "post_quant_conv.bias"):
        assert k in keys, k
    assert "encoder.down_blocks.2.downsamplers.0.conv.weight" not in keys and "decoder.up_blocks.2.upsamplers.0.conv.weight" not in keys
    assert len(ae.decoder.up_blocks[0].resnets) == len(ae.encoder.down_blocks[0].resnets) + 1
    flux = AutoencoderKL.flux(block_out_channels=(32, 64), layers_per_block=1, norm_groups=8)
    assert flux.latent_channels == 16 and flux.quant_conv is None and flux.normalization.shift == 0.1159
    zf = flux.encode(x)
    mf, _ = flux.moments(x)
    assert torch.allclose(zf, (mf.permute(0, 2, 3, 1) - 0.1159) * 0.3611, atol=1e-6)
    n = LatentNormalization(shift=[0.1, -0.2], factor=[2.0, 4.0], divides=True)
    t = torch.randn(3, 5, 5, 2)
    assert torch.allclose(n.restore(n.normalize(t)), t, atol=1e-6) and torch.allclose(n.normalize(t)[..., 1], (t[..., 1] + 0.2) / 4.0)


def test_kl_autoencoder_learns_to_reconstruct_and_tiles():
    torch.manual_seed(0)
    ae = _small_kl(latent_channels=4)
    yy, xx = torch.meshgrid(torch.linspace(-1, 1, 32), torch.linspace(-1, 1, 32), indexing="ij")
    x = torch.stack([torch.stack([torch.sin(3 * xx + p), torch.cos(2 * yy - p), xx * yy], -1) for p in (0.0, 1.0, 2.0, 3.0)])
    opt = torch.optim.Adam(ae.parameters(), lr=2e-3)
    first = None
    for _ in range(60):
        loss = ae.loss(x)
        first = first if first is not None else float(loss)
        opt.zero_grad(); loss.backward(); opt.step()
    assert float(loss) < 0.35 * first
    # tiling: a function without spatial context (a pointwise map) is reproduced exactly, whatever the tiles
    img = torch.randn(1, 3, 40, 56)
    up = lambda t: torch.nn.functional.interpolate(t * 2 + 1, scale_factor=2.0, mode="nearest")
    assert torch.allclose(_tiled(up, img, 16, 4, 2.0), up(img), atol=1e-5)
    big = torch.rand(1, 64, 96, 3) * 2 - 1
    with torch.no_grad():
        z_t, z = ae.encode(big, tile=32), ae.encode(big)
        assert z_t.shape == z.shape and torch.isfinite(z_t).all()
        x_t = ae.decode(z, tile=32)
        assert x_t.shape == big.shape and torch.isfinite(x_t).all()
        assert float((x_t - ae.decode(z)).abs().mean()) < 0.5 * float(ae.decode(z).abs().mean()) + 0.1


def test_deep_compression_autoencoder_shortcuts():
    x = torch.arange(2 * 4 * 4 * 4, dtype=torch.float32).reshape(2, 4, 4, 4)
    down = _space_to_channel(x, 8)
    assert down.shape == (2, 8, 2, 2)
    assert torch.allclose(down[0, 0, 0, 0], (x[0, 0, 0, 0] + x[0, 0, 0, 1]) / 2)            # pixel-unshuffled neighbours averaged in pairs
    up = _channel_to_space(down, 4)
    assert up.shape == (2, 4, 4, 4)
    with pytest.raises(ValueError):
        _space_to_channel(x, 7)
    torch.manual_seed(0)
    ae = DCAE(latent_channels=8, widths=(16, 32, 32, 64), depths=(1, 1, 1, 1))
    img = torch.rand(2, 32, 32, 3) * 2 - 1
    z = ae.encode(img)
    assert z.shape == (2, 4, 4, 8) and ae.downsample == 8 and ae.decode(z).shape == img.shape
    loss0 = float(ae.loss(img))
    opt = torch.optim.Adam(ae.parameters(), lr=2e-3)
    for _ in range(40):
        loss = ae.loss(img)
        opt.zero_grad(); loss.backward(); opt.step()
    assert float(loss) < 0.7 * loss0


def test_causal_video_autoencoder_is_causal_and_compresses_time():
    torch.manual_seed(0)
    conv = CausalConv3d(2, 3)
    v = torch.randn(1, 2, 5, 6, 6)
    later = v.clone()
    later[:, :, 3:] += 1.0
    assert torch.allclose(conv(v)[:, :, :3], conv(later)[:, :, :3]) and not torch.allclose(conv(v)[:, :, 3:], conv(later)[:, :, 3:])
    vae = CausalVideoVAE(latent_channels=4, widths=(8, 16, 16, 16), layers=1, groups=4, shift=[0.0, 0.1, 0.2, 0.3], factor=[1.0, 2.0, 1.0, 0.5])
    clip = torch.rand(1, 9, 32, 32, 3) * 2 - 1
    z = vae.encode(clip)
    assert z.shape == (1, 3, 4, 4, 4) and vae.frames_to_latents(9) == 3 and vae.decode(z).shape == clip.shape
    # the first latent frame depends on the first frame alone: an image encodes to the same latent as a clip's first frame
    z_img = vae.encode(clip[:, 0])
    assert z_img.shape == (1, 1, 4, 4, 4) and torch.allclose(z_img[:, 0], z[:, 0], atol=1e-5)
    changed = clip.clone()
    changed[:, 5:] = 0.0
    z2 = vae.encode(changed)
    assert torch.allclose(z2[:, :2], z[:, :2], atol=1e-5) and not torch.allclose(z2[:, 2], z[:, 2])
    with pytest.raises(ValueError):
        vae.encode(clip[:, :8])
    assert torch.isfinite(vae.loss(clip))
