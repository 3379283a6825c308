"""Pixel-space diffusion recipe: SimpleDiT under the EDM process (``--set objective.options.process=flow`` for rectified flow)."""
from dew_b200.config import RunConfig


def config() -> RunConfig:
    cfg = RunConfig()
    cfg.model.name = "simple_dit"
    cfg.model.fields = dict(patch_size=4, emb_features=384, num_layers=12, num_heads=6)
    cfg.objective.name = "diffusion"
    cfg.objective.options = dict(process="edm", ema_decay=0.999)
    cfg.optimizer.learning_rate, cfg.optimizer.weight_decay = 2e-4, 0.0
    cfg.data.source, cfg.data.image_shape, cfg.data.batch = "synthetic_images", (64, 64, 3), 16
    cfg.trainer.steps, cfg.trainer.log_every = 10_000, 50
    cfg.trainer.checkpoint_dir, cfg.trainer.name = "runs/dit", "dit"
    return cfg
