"""Decoder-only LM pre-training recipe.  ``python -m dew_b200.cli.main train recipes/lm/train.py --set trainer.steps=1000
--set data.source=token_files --set data.path='data/*.bin'``; every field below can be overridden with ``--set path=value``."""
from dew_b200.config import RunConfig


def config() -> RunConfig:
    cfg = RunConfig()
    cfg.model.name = "causal_transformer"
    cfg.model.fields = dict(vocab_size=32000, emb_features=1024, num_layers=12, num_heads=16, num_kv_heads=4, mlp_features=2816,
                            max_seq_len=2048, qk_norm=False, tie_embeddings=False)
    cfg.objective.name = "lm"
    cfg.optimizer.learning_rate, cfg.optimizer.schedule, cfg.optimizer.warmup = 3e-4, "cosine", 200
    cfg.optimizer.weight_decay, cfg.optimizer.clip_grads, cfg.optimizer.b2 = 0.1, 1.0, 0.95
    cfg.data.seq_len, cfg.data.batch = 2048, 8
    cfg.trainer.steps, cfg.trainer.log_every, cfg.trainer.checkpoint_every = 10_000, 50, 1000
    cfg.trainer.checkpoint_dir, cfg.trainer.name = "runs/lm", "lm"
    return cfg
