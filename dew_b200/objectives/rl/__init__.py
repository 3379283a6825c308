from .preference import DPO
from .policy import GRPO, PPO

__all__ = ["DPO", "GRPO", "PPO"]
