"""Hybrid stacks: gated-delta-net and Mamba-2 layers interleaved with attention train, and decode step by step to the
same outputs as a full forward pass."""
import torch

import dew_b200 as dew
from dew_b200.models import CausalTransformer
from dew_b200.nn.linear_attention import RecurrentCache
from dew_b200.objectives.lm import LMObjective
from dew_b200.sampling.text import make_cache


def _hybrid(kind, seed=0):
    torch.manual_seed(seed)
    opts = dict(num_k_heads=2, num_v_heads=4, head_k_dim=8, head_v_dim=8) if kind == "gdn" else dict(state_dim=8, head_dim=8, expand=2)
    return CausalTransformer(vocab_size=61, emb_features=32, num_layers=4, num_heads=4, num_kv_heads=2, mlp_features=64, max_seq_len=64,
                             layer_types=(kind, kind, kind, "attention"), mixer_options=opts)


def test_hybrid_models_train():
    for kind in ("gdn", "mamba2"):
        m = _hybrid(kind)
        tokens = torch.randint(0, 61, (4, 33), generator=torch.Generator().manual_seed(1))
        tr = dew.Trainer(LMObjective(m, 32), dew.OptimConfig(learning_rate=5e-3, weight_decay=0.0), tracker=(t := dew.MemoryTracker()))
        tr.fit(dew.Loader(lambda part: iter([{"tokens": tokens}] * 20), batch=4), steps=12, log_every=4)
        assert t.rows[-1]["loss"] < t.rows[0]["loss"], kind


def test_hybrid_decode_matches_full_forward():
    for kind in ("gdn", "mamba2"):
        m = _hybrid(kind, 2).eval()
        tokens = torch.randint(0, 61, (2, 12), generator=torch.Generator().manual_seed(3))
        with torch.no_grad():
            full = m(tokens)
            cache = RecurrentCache(make_cache(m, 2, 32))
            pos = torch.arange(8)[None].expand(2, 8)
            out = [m(tokens[:, :8], positions=pos, cache=cache)]
            for t in range(8, 12):
                out.append(m(tokens[:, t:t + 1], positions=torch.full((2, 1), t), cache=cache))
        got = torch.cat(out, 1)
        assert torch.allclose(got, full, atol=2e-4), (kind, float((got - full).abs().max()))
