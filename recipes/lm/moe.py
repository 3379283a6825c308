"""Mixture-of-experts LM recipe: 64 experts, top 6, one shared expert, aux-loss-free balancing bias."""
from dew_b200.config import RunConfig


def config() -> RunConfig:
    cfg = RunConfig()
    cfg.model.fields = dict(vocab_size=32000, emb_features=1024, num_layers=12, num_heads=16, num_kv_heads=4, mlp_features=2816,
                            max_seq_len=2048, qk_norm=False, tie_embeddings=False,
                            mixture=dict(experts=64, top_k=6, expert_features=512, shared_features=512, bias=True, score_function="sigmoid"))
    cfg.objective.options = dict(balance=0.001)
    cfg.optimizer.learning_rate, cfg.optimizer.schedule, cfg.optimizer.warmup = 3e-4, "wsd", 200
    cfg.optimizer.weight_decay, cfg.optimizer.clip_grads, cfg.optimizer.b2 = 0.1, 1.0, 0.95
    cfg.data.seq_len, cfg.data.batch = 2048, 8
    cfg.trainer.steps, cfg.trainer.log_every = 10_000, 50
    cfg.trainer.checkpoint_dir, cfg.trainer.name = "runs/moe", "moe"
    return cfg
