from .state import CHECKPOINTED, MODEL_STATE, TrainState
from .tracker import ConsoleTracker, LocalTracker, MemoryTracker, MLflowTracker, TensorBoardTracker, Tracker, Trackers, Wandb, WandbTracker
from .trainer import Best, Cooldown, Evaluation, Pause, Plateau, Preempted, ProfileWindow, Trainer

__all__ = ["Cooldown", "Trainer", "TrainState", "Best", "Plateau", "Pause", "Evaluation", "ProfileWindow", "Preempted", "Tracker",
           "LocalTracker", "ConsoleTracker", "MemoryTracker", "WandbTracker", "Wandb", "MLflowTracker", "TensorBoardTracker", "Trackers",
           "CHECKPOINTED", "MODEL_STATE"]
