from . import averaging, schedules
from .averaging import ema_update, power_decay
from .config import OptimConfig, Optimizer, newton_schulz
from .schedules import WSD, Constant, Cosine, Exponential, Linear, OneCycle, Power

__all__ = ["OptimConfig", "Optimizer", "newton_schulz", "ema_update", "power_decay", "Cosine", "Power", "Linear", "WSD",
           "OneCycle", "Exponential", "Constant", "averaging", "schedules"]
