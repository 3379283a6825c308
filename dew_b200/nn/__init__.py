from .attention import SelfAttention
from .layers import Embedding, LayerNorm, Linear, RMSNorm, declare, reset_all, sinusoidal
from .mlp import GeluMLP, SwiGLU

__all__ = ["SelfAttention", "Embedding", "LayerNorm", "Linear", "RMSNorm", "declare", "reset_all", "sinusoidal",
           "GeluMLP", "SwiGLU"]
