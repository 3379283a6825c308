"""What a generative objective is fed: the sample field and its conditions (``spec``), the condition encoders (``encoders``) and image
conditions for latent diffusion (``diffusion``).  The encoders that bind released towers live in ``dew_b200.interop``."""
from .spec import Condition, Field, InputSpec, unit_range

__all__ = ["Condition", "Field", "InputSpec", "unit_range", "CharTable", "ConditionEncoder", "TowerEncoder", "encode_conditions",
           "CLIPImageTransform", "latent_image_conditions"]


def __getattr__(name):
    if name in ("CharTable", "ConditionEncoder", "TowerEncoder", "encode_conditions", "char_codes"):
        from . import encoders
        return getattr(encoders, name)
    if name in ("CLIPImageTransform", "latent_image_conditions", "blend_known"):
        from . import diffusion
        return getattr(diffusion, name)
    raise AttributeError(name)
