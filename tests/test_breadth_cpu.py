"""LoRA, quantisation, HF interop, evaluation metrics."""
import pytest
import torch

from dew_b200.eval import metrics as M
from dew_b200.interop.hf import Pretrained, from_hf_state, to_hf_state
from dew_b200.models import CausalTransformer
from dew_b200.nn.lora import LoRALinear, apply_lora, lora_state, merge_all
from dew_b200.nn.quantization import Quantization, dequantize_weight, fake_quant, quantize_variables, quantize_weight
from dew_b200.utils.trees import module_variables


def _lm(**kw):
    torch.manual_seed(0)
    return CausalTransformer(vocab_size=64, emb_features=32, num_layers=2, num_heads=4, num_kv_heads=2, mlp_features=64, max_seq_len=32,
                             tie_embeddings=False, **kw)


def test_lora_trains_only_adapters_and_merges():
    m = _lm()
    x = torch.randint(0, 64, (2, 8))
    before = m(x)
    wrapped = apply_lora(m, ("qkv_proj", "down_proj"), rank=4)
    assert len(wrapped) == 4 and all(("lora_" in n) == p.requires_grad for n, p in m.named_parameters())
    assert torch.allclose(m(x), before, atol=1e-6)                      # B starts at zero
    for mod in m.modules():
        if isinstance(mod, LoRALinear):
            torch.nn.init.normal_(mod.lora_b, std=0.05)
    y = m(x)
    merge_all(m)
    assert torch.allclose(m(x), y, atol=1e-4) and len(lora_state(m)) == 8


def test_quantisation_roundtrips():
    torch.manual_seed(1)
    w = torch.randn(64, 96)
    for kind, tol in (("int8", 0.01), ("float8_e4m3fn", 0.04), ("nvfp4", 0.12)):
        d = dequantize_weight(quantize_weight(w, kind), kind)
        assert d.shape == w.shape and float((d - w).norm() / w.norm()) < tol, kind
    g = fake_quant(w.clone().requires_grad_(), "int8")
    assert g.requires_grad
    m = _lm()
    q = quantize_variables(module_variables(m), Quantization("int8", min_size=1024))
    from dew_b200.utils.trees import flatten
    changed = [k for k, v in flatten(q).items() if not torch.equal(v, flatten(module_variables(m))[k])]
    assert changed and not any("embed" in k or "norm" in k for k in changed)


def test_hf_roundtrip(tmp_path):
    m = _lm(qk_norm=False)
    Pretrained.save(m, tmp_path / "hf")
    m2 = Pretrained.load(tmp_path / "hf")
    x = torch.randint(0, 64, (2, 8))
    assert torch.allclose(m(x), m2(x), atol=1e-6)
    hf = to_hf_state(m)
    assert hf["model.layers.0.self_attn.k_proj.weight"].shape == (2 * 8, 32)
    m3 = _lm(qk_norm=False)
    from_hf_state(m3, hf)
    assert torch.allclose(m(x), m3(x), atol=1e-6)


def test_metrics():
    torch.manual_seed(2)
    a = torch.rand(4, 16, 16, 3) * 2 - 1
    assert float(M.psnr(a, a + 0.01).min()) > 40 and float(M.ssim(a, a).min()) > 0.999
    assert float(M.ssim(a, torch.rand_like(a) * 2 - 1).max()) < 0.5
    f = torch.randn(500, 8)
    assert M.frechet_distance(f, f) < 1e-6 and M.frechet_distance(f, f + 3) > 50
    p = torch.softmax(torch.randn(100, 5) * 3, -1)
    assert 0 <= M.expected_calibration_error(p, p.argmax(-1)) <= 1


def test_nccl_weight_push_orders_chunks_and_aborts_on_failure():
    from dew_b200.inference.nccl import FakeCollectives, NCCLPush, PushFailed, UniqueId
    tensors = {"b.weight": torch.arange(10, dtype=torch.float32), "a.weight": torch.ones(3, 5, dtype=torch.bfloat16)}
    announced = []
    fake = FakeCollectives()
    push = NCCLPush(receivers=2, collectives=fake, announce=lambda *a: announced.append(a), chunk_bytes=16)
    push.push(tensors, version=7)
    assert fake.calls[0] == ("open", 0, 3) and fake.calls[1] == ("all_reduce", 1)
    uid_b64, names, shapes, dtypes, version = announced[0]
    assert names == ["a.weight", "b.weight"] and shapes == [(3, 5), (10,)] and dtypes == ["bfloat16", "float32"] and version == 7
    assert bytes(UniqueId.from_b64(uid_b64).internal) == bytes(fake.unique_id().internal)
    # a.weight: 15 bf16 in 8-element pieces; b.weight: 10 fp32 in 4-element pieces - in name order
    sizes = [c[1] for c in fake.calls if c[0] == "broadcast"]
    assert sizes == [8, 7, 4, 4, 2]
    assert torch.equal(torch.cat(fake.received[2:]), tensors["b.weight"]) and push.pushed == [7]
    push.push(tensors, version=8)                       # the open group is reused: no second rendezvous
    assert sum(c[0] == "open" for c in fake.calls) == 1 and announced[1][0] is None
    bad = FakeCollectives(fail_at=1)
    p2 = NCCLPush(receivers=1, collectives=bad, announce=lambda *a: None, chunk_bytes=16)
    with pytest.raises(PushFailed):
        p2.push(tensors, version=1)
    assert bad.aborted and p2.comm is None and p2.pushed == []


def test_tuning_cache_measures_once_and_persists(tmp_path):
    import time
    from dew_b200.ops.tuning import KernelOp, TuningCache
    calls = []
    def run(name):
        calls.append(name)
        time.sleep(0.002 if name == "slow" else 0.0)
        if name == "refuses":
            raise RuntimeError("no")
    cache = TuningCache(str(tmp_path / "t.json"))
    op = KernelOp("demo", cache)
    assert op.pick((128, 256), ["slow", "fast", "refuses"], run, tune=False) == "slow"          # untuned: first candidate, no timing
    assert calls == []
    assert op.pick((128, 256), ["slow", "fast", "refuses"], run, tune=True) == "fast"
    n = len(calls)
    assert op.pick((128, 256), ["slow", "fast"], run, tune=True) == "fast" and len(calls) == n  # memoised
    again = KernelOp("demo", TuningCache(str(tmp_path / "t.json")))                             # a later process reads the file
    assert again.pick((128, 256), ["slow", "fast"], run, tune=False) == "fast" and len(calls) == n
    assert again.pick((1, 1), ["slow", "fast"], run, tune=False) == "slow"


def test_mixture_is_reproducible_and_restorable_and_scoring_and_clients():
    from dew_b200.data.mixing import Mixture, PhasedStream
    from dew_b200.inference.clients import OpenAIClient
    from dew_b200.inference.scoring import multiple_choice_accuracy, score
    a, b = [("a", i) for i in range(100)], [("b", i) for i in range(100)]
    m1 = iter(Mixture([(a, 3.0), (b, 1.0)], seed=5))
    first = [next(m1) for _ in range(40)]
    assert 20 < sum(r[0] == "a" for r in first) < 38
    m2 = Mixture([(a, 3.0), (b, 1.0)], seed=5)
    it = iter(m2)
    [next(it) for _ in range(25)]
    pos = m2.position()
    m3 = Mixture([(a, 3.0), (b, 1.0)], seed=5); m3.restore(pos)
    assert [next(iter(m3)) for _ in range(1)] + [next(m3) for _ in range(14)] == first[25:40]
    ph = PhasedStream([(2, ["x"] * 10), (4, ["y"] * 10)])
    assert [next(ph) for _ in range(4)] == ["x", "x", "y", "y"]
    torch.manual_seed(0)
    m = CausalTransformer(vocab_size=32, emb_features=32, num_layers=1, num_heads=2, num_kv_heads=2, head_dim=16, mlp_features=64, max_seq_len=32)
    s = score(m, [[1, 2, 3], [4, 5]], [[6, 7], [8, 9, 10]])
    full = torch.log_softmax(m(torch.tensor([[1, 2, 3, 6, 7]])).float(), -1)[0]
    assert abs(s[0][0] - float(full[2, 6] + full[3, 7])) < 1e-4 and s[0][1] == 2 and s[1][1] == 3
    assert 0.0 <= multiple_choice_accuracy(m, [([1, 2], [[3], [4, 5]], 0)]) <= 1.0
    sent = {}
    client = OpenAIClient(model="m", transport=lambda url, body, headers, timeout: sent.update(url=url, body=body) or {"choices": [{"message": {"content": "hi"}}]})
    assert client.chat([{"role": "user", "content": "x"}]) == "hi" and sent["url"].endswith("/chat/completions") and sent["body"]["model"] == "m"


def test_gguf_round_trip_and_block_formats(tmp_path):
    import numpy as np
    import torch
    from dew_b200.interop import gguf
    torch.manual_seed(0)
    tensors = {"tok.weight": torch.randn(8, 64), "blk.0.w": torch.randn(4, 32).half(), "blk.0.b": torch.randn(64).to(torch.bfloat16),
               "blk.0.q": torch.randn(2, 64)}
    path = str(tmp_path / "m.gguf")
    gguf.write(path, {"general.architecture": "llama", "llama.block_count": 1, "tokenizer.ggml.tokens": ["a", "b"], "rope": 10000.0},
               tensors, quantize={"blk.0.q": gguf.Q8_0})
    meta, got = gguf.read(path)
    assert meta["general.architecture"] == "llama" and meta["llama.block_count"] == 1 and meta["tokenizer.ggml.tokens"] == ["a", "b"]
    assert torch.equal(got["tok.weight"], tensors["tok.weight"]) and torch.equal(got["blk.0.w"], tensors["blk.0.w"])
    assert torch.equal(got["blk.0.b"], tensors["blk.0.b"])
    assert (got["blk.0.q"] - tensors["blk.0.q"]).abs().max() < 0.03           # 8-bit blocks
    infos = gguf.read(path, load_tensors=False)[1]
    assert [i.name for i in infos] == list(tensors) and infos[0].shape == (8, 64)
    # Q4_0: value = (nibble - 8) * d, low nibbles first
    d = np.float16(0.5)
    raw = np.zeros(1, dtype=np.dtype([("d", "<f2"), ("q", "u1", (16,))]))
    raw["d"], raw["q"] = d, np.arange(16, dtype=np.uint8) | (np.arange(15, -1, -1, dtype=np.uint8) << 4)
    vals = gguf.dequantize(raw.tobytes(), gguf.Q4_0, (32,))
    assert vals[:16].tolist() == [(i - 8) * 0.5 for i in range(16)] and vals[16:].tolist() == [(15 - i - 8) * 0.5 for i in range(16)]


def test_lpips_is_zero_for_equal_images_and_grows_with_distortion():
    import torch
    from dew_b200.eval.metrics import lpips
    torch.manual_seed(0)
    conv1, conv2 = torch.nn.Conv2d(3, 8, 3, padding=1), torch.nn.Conv2d(8, 12, 3, stride=2, padding=1)

    def feats(x):
        h1 = torch.relu(conv1(x.permute(0, 3, 1, 2)))
        return [h1, torch.relu(conv2(h1))]
    a = torch.rand(3, 16, 16, 3) * 2 - 1
    with torch.no_grad():
        assert float(lpips(a, a, feats).abs().max()) < 1e-8
        small, large = lpips(a, a + 0.05 * torch.randn_like(a), feats), lpips(a, a + 0.5 * torch.randn_like(a), feats)
        assert small.shape == (3,) and bool((large > small).all())
        w = [torch.zeros(8), torch.zeros(12)]
        assert float(lpips(a, -a, feats, w).abs().max()) == 0.0


def test_parity_gate_passes_equal_arms_and_fails_a_wrong_row():
    import pytest
    import torch
    from dew_b200.utils.parity import assert_on_par, assess

    def inputs(seed):
        g = torch.Generator().manual_seed(seed)
        return torch.randn(32, 64, generator=g, dtype=torch.float64), torch.randn(64, 48, generator=g, dtype=torch.float64)

    def truth(seed):
        a, b = inputs(seed)
        return {"y": a @ b, "n": (a @ b).norm(dim=-1)}

    def bf16(seed):
        a, b = inputs(seed)
        y = (a.bfloat16() @ b.bfloat16()).float()
        return {"y": y, "n": y.norm(dim=-1)}

    def fp32(seed):
        a, b = inputs(seed)
        y = a.float() @ b.float()
        return {"y": y, "n": y.norm(dim=-1)}

    found = assert_on_par(fp32, bf16, truth)                  # fp32 is far more exact than the bf16 reference
    assert {f.leaf for f in found} == {"y", "n"} and all(f.ratio < 0.1 for f in found)
    assert all(f.ok for f in assess(bf16, bf16, truth, range(8)))
    over = {f.leaf: f for f in assess(bf16, fp32, truth, range(8))}           # the other way round is over
    assert over["y"].status in ("over", "rows_over")
    assert assess(fp32, bf16, truth, range(3))[0].status == "inconclusive"     # too few seeds decide nothing

    def one_bad_row(seed):
        out = bf16(seed)
        y = out["y"].clone()
        y[5] += 3.0
        return {"y": y, "n": out["n"]}
    with pytest.raises(AssertionError):
        assert_on_par(one_bad_row, bf16, truth)


def test_chat_rendering_roles_and_token_shards(tmp_path):
    import numpy as np
    import pytest
    import torch
    from dew_b200.data import ByteTokenizer
    from dew_b200.data.chat import ChatTemplate, Conversation, Role, chat_batch, render_conversation, render_prompt
    from dew_b200.data.sinks import read_token_shards, write_jsonl, write_token_shards
    tok = ByteTokenizer()
    conv = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "2+2?"}, {"role": "assistant", "content": "4"}]
    r = render_conversation(tok, conv)
    text = bytes(r["tokens"].tolist()).decode()
    assert text == "<|im_start|>system\nbe brief<|im_end|>\n<|im_start|>user\n2+2?<|im_end|>\n<|im_start|>assistant\n4<|im_end|>\n"
    scored = bytes(r["tokens"][r["roles"] == Role.ASSISTANT].tolist()).decode()
    assert scored == "4<|im_end|>\n"                                        # the answer and its closing frame
    assert bytes(r["tokens"][r["roles"] == Role.USER].tolist()).decode() == "2+2?"
    unscored = render_conversation(tok, conv, ChatTemplate(score_close=False))
    assert bytes(unscored["tokens"][unscored["roles"] == Role.ASSISTANT].tolist()).decode() == "4"
    prompt = bytes(render_prompt(tok, conv).tolist()).decode()
    assert prompt.endswith("<|im_start|>assistant\n") and "4<|im_end|>" not in prompt
    batch = chat_batch(tok, [conv, conv[1:]], seq_len=48)
    assert batch["tokens"].shape == (2, 49) and batch["roles"].shape == (2, 49)
    with pytest.raises(ValueError):
        Conversation.of([{"role": "user", "content": "x"}, {"role": "system", "content": "late"}])
    with pytest.raises(ValueError):
        Conversation.of([{"role": "narrator", "content": "x"}])
    # the objective scores the assistant's tokens only
    from dew_b200.models import CausalTransformer
    from dew_b200.objectives import Step
    from dew_b200.objectives.lm import LMObjective
    torch.manual_seed(0)
    m = CausalTransformer(vocab_size=256, emb_features=16, num_layers=1, num_heads=2, num_kv_heads=2, head_dim=8, mlp_features=24, max_seq_len=48)
    obj = LMObjective(m, 48, ema_decay=None, loss_role=int(Role.ASSISTANT))
    stat, _ = obj.loss(None, batch, Step(key=0, train=False))
    assert int(stat.mass) == int((batch["roles"][:, 1:] == Role.ASSISTANT).sum())
    # shards
    docs = [list(range(i, i + 5 + i)) for i in range(7)]
    index = write_token_shards(docs, tmp_path / "shards", shard_tokens=20, vocab_size=256, eos_id=255)
    assert len(index["shards"]) > 1 and index["tokens"] == sum(len(d) + 1 for d in docs)
    back = list(read_token_shards(tmp_path / "shards"))
    assert len(back) == 7 and all(np.array_equal(b, np.array(d + [255])) for b, d in zip(back, docs))
    assert write_jsonl([{"a": 1}, {"a": 2}], tmp_path / "r.jsonl") == 2 and (tmp_path / "r.jsonl").read_text().count("\n") == 2


def test_normuon_and_m3_optimizers_reduce_a_quadratic_and_keep_their_rules():
    import torch
    from dew_b200.optim.config import OptimConfig, newton_schulz
    torch.manual_seed(0)
    target = torch.randn(12, 8)
    for kind, opts, lr in (("normuon", {}, 0.05), ("m3", {"frequency": 3, "alpha": 0.5, "b1": 0.9, "b2": 1.0, "b3": 0.9, "eps": 1e-2}, 1.0)):
        opt = OptimConfig(optimizer=kind, optimizer_opts=opts, learning_rate=lr, weight_decay=0.0).build()
        params = {"layer": {"kernel": torch.zeros(12, 8), "bias": torch.zeros(8)}}
        state = opt.init(params)
        first = None
        for step in range(60):
            w, b = params["layer"]["kernel"], params["layer"]["bias"]
            grads = {"layer": {"kernel": 2 * (w - target), "bias": 2 * (b - 1.0)}}
            loss = float(((w - target) ** 2).sum() + ((b - 1.0) ** 2).sum())
            first = loss if first is None else first
            state, info = opt.update(params, grads, state, step)
        assert loss < (0.5 if kind == "normuon" else 0.8) * first, (kind, first, loss)
        assert int(state["count"]) == 60
    # M3's first step: O2 is zero, so the direction is NS(beta1 g) / sqrt(beta2 g^2 + eps)
    opt = OptimConfig(optimizer="m3", optimizer_opts={"frequency": 2, "b1": 1.0, "b2": 1.0, "eps": 1e-8}, learning_rate=1.0, weight_decay=0.0).build()
    params = {"w": torch.zeros(6, 4)}
    g = torch.randn(6, 4)
    state = opt.init(params)
    state, _ = opt.update(params, {"w": g}, state, 0)
    assert torch.allclose(params["w"], -newton_schulz(g) / torch.sqrt(g * g + 1e-8), atol=1e-5)
    assert float(state["slow"]["w"].abs().sum()) == 0.0 and torch.allclose(state["chunk"]["w"], g)
    state, _ = opt.update(params, {"w": g}, state, 1)            # the chunk closes: slow momentum and its direction appear
    assert torch.allclose(state["slow"]["w"], 0.9 * 2 * g, atol=1e-6) and float(state["chunk"]["w"].abs().sum()) == 0.0
    assert float(state["slow_direction"]["w"].abs().sum()) > 0


def test_qk_clip_bounds_the_logits_of_exceeding_groups_only():
    import torch
    from dew_b200.nn.attention import SelfAttention
    from dew_b200.optim.qk_clip import qk_clip, watch
    torch.manual_seed(0)
    layer = SelfAttention(32, num_heads=4, num_kv_heads=2, head_dim=8, causal=True).train()
    with torch.no_grad():
        w = layer.qkv_proj.weight.view(8, 8, 32)
        w[0:2] *= 12.0                      # the query heads of group 0 run hot
        w[4] *= 12.0                        # and so does their key head
    assert watch(layer) == 1
    x = torch.randn(2, 24, 32)
    layer(x)
    before = layer.qk_max.clone()
    assert before.shape == (4,) and float(before[:2].max()) > 10 > float(before[2:].max())
    # exact: against the dense logits
    q, k, _ = layer.project(x)
    s = torch.einsum("bshd,bthd->bhst", q.float(), k.float().repeat_interleave(2, 2)) / 8 ** 0.5
    s = s.masked_fill(~torch.tril(torch.ones(24, 24, dtype=torch.bool)), float("-inf"))
    assert torch.allclose(before, s.amax((0, 2, 3)), atol=1e-4)
    kept = layer.qkv_proj.weight.detach().clone()
    seen = qk_clip(layer, tau=10.0)
    assert torch.equal(next(iter(seen.values())), before) and layer.qk_max is None
    w2 = layer.qkv_proj.weight.view(8, 8, 32)
    assert torch.equal(w2[2:4], kept.view(8, 8, 32)[2:4]) and torch.equal(w2[5:], kept.view(8, 8, 32)[5:])     # group 1 and V untouched
    layer(x)
    after = layer.qk_max
    assert float(after[:2].max()) <= 10.0 + 1e-3 and torch.allclose(after[2:], before[2:], atol=1e-5)
    qk_clip(layer, tau=10.0)
    watch(layer, False)
    layer(x)
    assert layer.qk_max is None


def test_harness_adapter_scores_and_generates():
    import torch
    from types import SimpleNamespace
    from dew_b200.data import ByteTokenizer
    from dew_b200.eval.harness import HarnessModel
    from dew_b200.inference.scoring import score
    from dew_b200.models import CausalTransformer
    torch.manual_seed(0)
    model = CausalTransformer(vocab_size=259, emb_features=32, num_layers=2, num_heads=2, num_kv_heads=2, head_dim=16, mlp_features=48, max_seq_len=64).eval()
    lm = HarnessModel(model, ByteTokenizer(), max_length=48, batch_size=4, max_gen_tokens=8)
    reqs = [SimpleNamespace(args=("The sky is ", "blue")), SimpleNamespace(args=("The sky is ", "green")), ("", "x")]
    res = lm.loglikelihood(reqs)
    assert len(res) == 3 and all(lp < 0 and isinstance(g, bool) for lp, g in res)
    # the context's trailing space travels with the continuation; the numbers equal a direct scoring call
    direct = score(model, [list(b"The sky is")], [list(b" blue")])[0]
    assert abs(res[0][0] - direct[0]) < 1e-4
    # rolling: a document longer than the window equals the sum of its windows
    doc = "abcdefghij" * 12
    rolled = lm.loglikelihood_rolling([SimpleNamespace(args=(doc,))])[0]
    ids = list(doc.encode())
    want, prev = 0.0, 257
    rest = ids
    for lo in range(0, len(rest), 47):
        win = rest[lo:lo + 47]
        want += score(model, [[prev]], [win], batch=1)[0][0]
        prev = win[-1]
    assert abs(rolled - want) < 1e-3 and rolled < 0
    outs = lm.generate_until([SimpleNamespace(args=("hello", {"until": ["\n"], "max_gen_toks": 6}))])
    assert len(outs) == 1 and isinstance(outs[0], str) and "\n" not in outs[0]


def test_categorical_functions_against_direct_forms():
    import torch
    import torch.nn.functional as F
    from dew_b200.nn import categorical as C
    torch.manual_seed(0)
    logits, ref = torch.randn(5, 7), torch.randn(5, 7)
    labels = torch.randint(0, 7, (5,))
    assert torch.allclose(C.cross_entropy(logits, labels), F.cross_entropy(logits, labels, reduction="none"), atol=1e-6)
    t = torch.softmax(torch.randn(5, 7), -1)
    assert torch.allclose(C.soft_cross_entropy(logits, t), -(t * torch.log_softmax(logits, -1)).sum(-1), atol=1e-6)
    p = torch.softmax(logits, -1)
    assert torch.allclose(C.entropy(logits), -(p * p.log()).sum(-1), atol=1e-6)
    assert torch.allclose(C.kl_divergence(logits, ref), F.kl_div(torch.log_softmax(ref, -1), p, reduction="none").sum(-1), atol=1e-6)
    assert float(C.kl_divergence(logits, logits).abs().max()) < 1e-7
    # masked classes take no probability and add no term; bf16 inputs are widened
    where = torch.tensor([True, True, False, True, True, True, False])
    lp = C.log_probs(logits.bfloat16(), where)
    assert lp.dtype == torch.float32 and torch.isinf(lp[:, 2]).all() and torch.allclose(lp.exp().sum(-1), torch.ones(5), atol=1e-5)
    assert torch.isfinite(C.entropy(logits, where)).all() and torch.isfinite(C.kl_divergence(logits, ref, where)).all()
    sm = C.smoothed(F.one_hot(labels, 7).float(), 0.1, where)
    assert torch.allclose(sm.sum(-1), torch.ones(5)) and float(sm[:, 2].abs().max()) <= 0.9 * 1.0 and torch.all(sm[labels != 2][:, 2] == 0)
    onehot = F.one_hot(labels, 7).float()
    assert torch.allclose(C.brier(logits, onehot), ((p - onehot) ** 2).sum(-1), atol=1e-6)
    assert torch.all(C.spherical(logits, onehot) >= 0) and torch.all(C.ranked_probability(logits, onehot) >= 0)
    assert float(C.ranked_probability(torch.log(onehot + 1e-9) * 50, onehot).max()) < 1e-6
    same = logits[:, None].expand(5, 3, 7)
    assert float(C.group_divergence(same).abs().max()) < 1e-6 and float(C.group_divergence(torch.randn(5, 3, 7)).min()) > 0
    # the block-wise partition equals the whole one
    big = torch.randn(4, 50) * 5
    run = None
    for lo in range(0, 50, 16):
        run = C.rescaled(run, big[:, lo:lo + 16])
    assert torch.allclose(C.log_partition(run), torch.logsumexp(big, -1), atol=1e-5)
    lab = torch.randint(0, 50, (4,))
    assert torch.allclose(C.target_loss(run, big.gather(-1, lab[:, None])[:, 0]), F.cross_entropy(big, lab, reduction="none"), atol=1e-5)
    seg = torch.tensor([0, 0, 2, 2, 2, 3])
    x = torch.randn(6)
    out = C.segment_log_partition(x, seg, 4)
    assert torch.allclose(out[0], torch.logsumexp(x[:2], 0)) and torch.allclose(out[2], torch.logsumexp(x[2:5], 0)) and out[1] == float("-inf")


def test_route_report_cost_model_and_resource_model():
    """The run-time view of the selector, the roofline cost model and the occupancy model (reference: kernel_routes,
    generation.py device facts, launches.py)."""
    from dew_b200.ops import cost, resources
    from dew_b200.ops.selection import Kernel, Op, Requirement, format_route_report, route_report, OPS
    op = Op("toy")
    OPS["toy"] = op
    op.kernels = [Kernel("fast", [Requirement("even", lambda c: c["n"] % 2 == 0, "n must be even")]), Kernel("any", [])]
    assert [op.select({"n": n}) for n in (2, 3, 5)] == ["fast", "any", "any"]
    rep = route_report()["toy"]
    assert rep["fast"]["calls"] == 1 and rep["any"]["calls"] == 2 and rep["any"]["after_refusals"] == {"fast: even": 2}
    assert "after fast: even" in format_route_report({"toy": rep})
    del OPS["toy"]
    dev = cost.Device()
    big = cost.gemm(8192, 4096, 4096, dev=dev)
    assert big.bound == "compute" and 0.15 < big.ms < 0.30
    skinny = cost.gemm(128, 768, 4096, dev=dev)
    assert skinny.bound in ("memory", "launch") and skinny.ms < 0.01
    rows = cost.estimate(0.0, 12288 * 2560 * 2 * 2, "rows", dev=dev)
    assert rows.bound == "memory" and 0.015 < rows.ms < 0.03
    step = cost.decoder_step(8192, 4096, 32, 14336, 32, 8, 128, 128256, 4096, dev=dev)
    assert 250 < step["total_ms"] < 500 and step["gemm_ms"] > 0.6 * step["total_ms"]      # one 8192-token microbatch of the 8 B model
    occ = resources.occupancy(168, resources.LAUNCHES["flash_fwd_kernel"])
    assert occ.ctas_per_sm == 1 and occ.by_shared == 1 and occ.by_tmem == 1 and occ.by_registers == 1
    two = resources.occupancy(96, resources.Launch(128, 100 * 1024, 0))
    assert two.ctas_per_sm == 2 and two.limiter == "shared memory"
    assert resources.occupancy(255, resources.Launch(1024, 0, 0)).limiter == "registers"


def test_lora_variants_quantised_base_and_peft_names():
    from dew_b200.nn.lora import (DoRALinear, LoRAConfig, adapters_disabled, apply_lora_config, from_peft_state, load_lora_state,
                                  lora_state, merge_all, to_peft_state)
    torch.manual_seed(0)
    m = _lm(qk_norm=False)
    x = torch.randint(0, 64, (2, 8))
    base_out = m(x)
    paths = apply_lora_config(m, LoRAConfig(targets=("qkv_proj", "down_proj"), rank=4, rank_pattern={r"layers\.0\.": 2}, rs=True))
    assert any("layers.0" in p for p in paths)
    assert m.layers[0].mixer.qkv_proj.rank == 2 and m.layers[1].mixer.qkv_proj.rank == 4
    assert torch.allclose(m(x), base_out, atol=1e-6)                      # B starts at zero
    for n, p in m.named_parameters():
        if "lora_b" in n:
            torch.nn.init.normal_(p, std=0.05)
    tuned = m(x)
    assert not torch.allclose(tuned, base_out, atol=1e-4)
    with adapters_disabled(m):
        assert torch.allclose(m(x), base_out, atol=1e-6)                   # the base model, no second copy of the weights
    peft = to_peft_state(m)
    assert all(k.startswith("base_model.model.") for k in peft)
    m2 = _lm(qk_norm=False)
    m2.load_state_dict({k: v for k, v in _strip_lora(m.state_dict()).items()}, strict=False)
    apply_lora_config(m2, LoRAConfig(targets=("qkv_proj", "down_proj"), rank=4, rank_pattern={r"layers\.0\.": 2}, rs=True))
    load_lora_state(m2, from_peft_state(peft))
    assert torch.allclose(m2(x), tuned, atol=1e-5)
    merge_all(m)
    assert torch.allclose(m(x), tuned, atol=1e-4)
    # DoRA starts as the base, and merging keeps its output
    d = _lm(qk_norm=False)
    ref = d(x)
    apply_lora_config(d, LoRAConfig(targets=("o_proj",), rank=4, dora=True))
    assert isinstance(d.layers[0].mixer.o_proj, DoRALinear) and torch.allclose(d(x), ref, atol=1e-5)
    for n, p in d.named_parameters():
        if "lora_b" in n:
            torch.nn.init.normal_(p, std=0.05)
    out = d(x)
    merge_all(d)
    assert torch.allclose(d(x), out, atol=1e-4)
    # a quantised frozen base under the adapters
    qm = _lm(qk_norm=False)
    ref = qm(x)
    apply_lora_config(qm, LoRAConfig(targets=("gate_up_proj",), rank=4, quantize_base="int8"))
    assert (qm(x) - ref).abs().max() < 0.05 and not any(n.endswith("gate_up_proj.base.weight") for n, _ in qm.named_parameters())
    with pytest.raises(ValueError, match="no Linear matches"):
        apply_lora_config(_lm(), LoRAConfig(targets=("nothing_like_this",)))


def _strip_lora(sd):
    return {k.replace(".base.", "."): v for k, v in sd.items() if "lora_" not in k and "magnitude" not in k}


def test_quantised_modules_qat_and_calibration():
    from dew_b200.nn.quantization import Calibrator, Quantization, QuantizedLinear, convert_qat, prepare_qat, quantize_model
    torch.manual_seed(1)
    m = _lm(qk_norm=False)
    x = torch.randint(0, 64, (2, 8))
    ref = m(x)
    cal = Calibrator("int8").observe(m)
    m(x)
    cal.close()
    assert cal.scales() and all(v > 0 for v in cal.scales().values())
    report = quantize_model(m, Quantization(kind="int8", min_size=64))
    assert report["bytes_after"] < 0.4 * report["bytes_before"]            # int8 + one fp32 scale per row vs fp32 weights
    assert any(isinstance(mod, QuantizedLinear) for mod in m.modules())
    assert (m(x) - ref).abs().max() < 0.1
    q = _lm(qk_norm=False)
    n = prepare_qat(q, Quantization(kind="int8", min_size=64))
    assert n > 0
    loss = q(x).float().pow(2).mean()
    loss.backward()
    assert all(p.grad is not None for nme, p in q.named_parameters() if nme.endswith("qkv_proj.base.weight"))   # straight-through
    assert convert_qat(q) == n and any(isinstance(mod, QuantizedLinear) for mod in q.modules())
