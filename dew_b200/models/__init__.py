from .dit import SimpleDiT

__all__ = ["SimpleDiT", "CausalTransformer", "Mixture"]


def __getattr__(name):
    if name in ("CausalTransformer", "Mixture", "TransformerConfig"):
        from . import causal_transformer as m
        return getattr(m, name)
    if name in ("UNet", "UViT", "SimpleUDiT", "SimpleMMDiT", "VideoDiT", "HybridDiT"):
        from . import diffusion_backbones as m
        return getattr(m, name)
    if name in ("KLAutoEncoder", "ViT"):
        from . import autoencoders as m
        return getattr(m, name)
    if name in ("AutoencoderKL", "DCAE", "CausalVideoVAE", "LatentNormalization"):
        from . import latent_autoencoders as m
        return getattr(m, name)
    if name in ("VisionLanguageModel", "AudioEncoder", "Projector", "log_mel"):
        from . import multimodal as m
        return getattr(m, name)
    if name in ("ClassicDecoder", "ClassicConfig"):
        from . import classic_decoder as m
        return getattr(m, name)
    raise AttributeError(name)
