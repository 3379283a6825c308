from .preference import DPO
from .policy import GRPO, PPO

__all__ = ["DPO", "GRPO", "PPO"]
from .dreamer import DreamerModel, DreamerPolicy, DreamerRollout, DreamerV3  # noqa: E402,F401
