from .preference import DPO
from .policy import GRPO, PPO

__all__ = ["DPO", "GRPO", "PPO"]
from .dreamer import DreamerModel, DreamerPolicy, DreamerRollout, DreamerV3  # noqa: E402,F401
from .control import ActorCritic, ControlPPO, episode_gae  # noqa: E402,F401
from .nft import DiffusionNFT  # noqa: E402,F401
from .tssm import TSSM, TSSMCache  # noqa: E402,F401
