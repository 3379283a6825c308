"""Optimizer state in host memory, streamed through two slots: the same trajectory as the resident engine."""
import pytest
import torch

import dew_b200 as dew
from dew_b200.models import CausalTransformer
from dew_b200.objectives.lm import LMObjective
from dew_b200.training.offload import HostOffloadEngine


def _trainer(offload, **kw):
    torch.manual_seed(0)
    model = CausalTransformer(vocab_size=64, emb_features=32, num_layers=2, num_heads=2, num_kv_heads=1, head_dim=16, mlp_features=64,
                              max_seq_len=16, qk_norm=False, tie_embeddings=False)
    opt = dew.OptimConfig(learning_rate=1e-2, weight_decay=0.1, clip_grads=kw.pop("clip", None), optimizer_opts={"b2": 0.95})
    return dew.Trainer(LMObjective(model, 16, ema_decay=None), opt, key=3, microbatches=2, offload=offload, **kw)


@pytest.mark.parametrize("clip", [None, 0.05])
def test_streamed_update_matches_resident_update(clip):
    batches = [{"tokens": torch.randint(0, 64, (4, 17), generator=torch.Generator().manual_seed(i))} for i in range(4)]
    a, b = _trainer(None, clip=clip), _trainer("optimizer", clip=clip)
    ea, eb = a.engine(), b.engine()
    assert isinstance(eb, HostOffloadEngine)
    eb.bucket_elems = 1000                                  # parameters are cut across buckets and slots are reused many times
    sa, sb = ea.fresh_state(a.key), eb.fresh_state(b.key)
    for batch in batches:
        sa, ma = ea.step(sa, batch)
        sb, mb = eb.step(sb, batch)
        assert abs(float(ma["loss"].value()) - float(mb["loss"].value())) < 1e-6
        assert abs(float(ma["grad_norm"]) - float(mb["grad_norm"])) < 1e-5 * max(1.0, float(ma["grad_norm"]))
    from dew_b200.utils.trees import flatten
    pa, pb = flatten(sa.variables["params"]), flatten(sb.variables["params"])
    assert set(pa) == set(pb)
    for k in pa:
        assert torch.allclose(pa[k], pb[k], atol=1e-6), k
    assert int(sb.opt_state["count"]) == 4 and sb.updates == 4
    report = eb.device_bytes()
    assert report["host_state"] == 12 * sum(p.numel() for p in pb.values()) and report["slots"] == 2 * 3 * 1000 * 4


def test_offload_refuses_what_it_does_not_do():
    torch.manual_seed(0)
    model = CausalTransformer(vocab_size=64, emb_features=32, num_layers=1, num_heads=2, num_kv_heads=1, head_dim=16, mlp_features=64, max_seq_len=16)
    with pytest.raises(ValueError, match="AdamW"):
        dew.Trainer(LMObjective(model, 16, ema_decay=None), dew.OptimConfig(optimizer="lion"), offload="optimizer").engine()
    with pytest.raises(ValueError, match="EMA"):
        dew.Trainer(LMObjective(model, 16, ema_decay=0.99), dew.OptimConfig(), offload="optimizer").engine()
    with pytest.raises(ValueError, match="offload must be"):
        dew.Trainer(LMObjective(model, 16, ema_decay=None), dew.OptimConfig(), offload="everything")


@pytest.mark.gpu
def test_streamed_update_on_the_gpu_matches_resident_update():
    """bf16 compute weights on the device, fp32 masters and moments in pinned host memory crossing on a copy stream."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")

    def make(offload):
        torch.manual_seed(0)
        model = CausalTransformer(vocab_size=512, emb_features=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64, mlp_features=512,
                                  max_seq_len=128, qk_norm=False, tie_embeddings=False).cuda()
        opt = dew.OptimConfig(learning_rate=1e-3, weight_decay=0.1, clip_grads=1.0, optimizer_opts={"b2": 0.95})
        return dew.Trainer(LMObjective(model, 128, ema_decay=None), opt, key=3, microbatches=2, offload=offload, param_dtype=torch.bfloat16)
    a, b = make(None), make("optimizer")
    ea, eb = a.engine(), b.engine()
    eb.bucket_elems = 100_000
    sa, sb = ea.fresh_state(a.key), eb.fresh_state(b.key)
    for i in range(3):
        batch = {"tokens": torch.randint(0, 512, (4, 129), generator=torch.Generator().manual_seed(i)).cuda()}
        sa, ma = ea.step(sa, batch)
        sb, mb = eb.step(sb, batch)
        assert abs(float(ma["loss"].value()) - float(mb["loss"].value())) < 2e-2
    from dew_b200.utils.trees import flatten
    pa, pb = flatten(sa.variables["params"]), flatten(sb.variables["params"])
    assert all(not v.is_cuda for v in pb.values())          # the masters stayed on the host
    worst = max(float((pa[k].cpu().float() - pb[k].float()).abs().max()) for k in pa)
    assert worst < 5e-3, worst
