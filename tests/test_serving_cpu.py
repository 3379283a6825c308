"""Continuous batching on CPU: served tokens equal offline greedy generation, prefix pages are re-used, tickets time
their first token."""
import torch

from dew_b200.inference import PageLedger, Server
from dew_b200.models import CausalTransformer
from dew_b200.nn.kv_cache import KVCache
from dew_b200.sampling.text import Sampling, generate


def _model():
    torch.manual_seed(0)
    return CausalTransformer(vocab_size=101, emb_features=32, num_layers=2, num_heads=4, num_kv_heads=2, mlp_features=64,
                             max_seq_len=128, tie_embeddings=True).eval()


def test_server_matches_offline_generation_with_more_requests_than_slots():
    m = _model()
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(1, 100, (int(n),), generator=g).tolist() for n in (5, 23, 9, 40, 3, 17, 31)]
    server = Server(m, slots=3, capacity=64, kv_cache=KVCache(page_size=8), chunk=16)
    tickets = [server.submit(p, 6) for p in prompts]
    server.run(max_steps=500)
    offline = generate(m, None, prompts, 6, sampling=Sampling(temperature=0.0))
    for r, t in enumerate(tickets):
        assert t.done and t.first_token_time is not None
        assert t.tokens == offline.tokens[r, len(prompts[r]): int(offline.lengths[r])].tolist(), r
    assert server.occupancy == 0 and not server.busy


def test_prefix_pages_are_reused():
    m = _model()
    shared = list(range(1, 33))                       # four full pages of 8
    server = Server(m, slots=2, capacity=64, kv_cache=KVCache(page_size=8), chunk=64)
    a = server.submit(shared + [50, 51], 4)
    server.run(max_steps=100)
    b = server.submit(shared + [60, 61, 62], 4)
    server.run(max_steps=100)
    assert server.ledger.hits >= 4
    ref = generate(m, None, [shared + [60, 61, 62]], 4, sampling=Sampling(temperature=0.0))
    assert b.tokens == ref.tokens[0, 35:39].tolist()


def test_evicted_prefix_pages_return_from_the_host_tier():
    """A small device pool evicts a cached prefix; with a host tier the prefix comes back by copy instead of by recomputation,
    and the served tokens are the same either way."""
    m = _model()
    shared = list(range(1, 33))                       # four full pages of 8
    other = [(7 * i) % 90 + 5 for i in range(40)]

    def serve(host_pages):
        server = Server(m, slots=1, capacity=48, kv_cache=KVCache(page_size=8, pages=6), chunk=64, host_pages=host_pages)
        server.submit(shared + [50, 51], 4)
        server.run(max_steps=100)
        server.submit(other, 4)                       # needs the whole pool: the cached prefix pages are evicted
        server.run(max_steps=100)
        t = server.submit(shared + [60, 61, 62], 4)
        server.run(max_steps=100)
        return server, t

    plain, t0 = serve(0)
    tiered, t1 = serve(8)
    assert plain.ledger.host_hits == 0 and tiered.ledger.host_hits == 4 and tiered.host_tier.spilled >= 4 and tiered.host_tier.fetched == 4
    ref = generate(m, None, [shared + [60, 61, 62]], 4, sampling=Sampling(temperature=0.0))
    assert t0.tokens == t1.tokens == ref.tokens[0, 35:39].tolist()


def test_ledger_accounting():
    led = PageLedger(pages=6, page_size=4)
    s1 = led.seat(list(range(10)), 12)
    assert len(s1.pages) == 3 and led.available() == 3
    led.publish(list(range(10)), s1.pages)
    s2 = led.seat(list(range(10)) + [99], 16)          # shares two full pages
    assert s2.reused_tokens == 8 and s2.pages[:2] == s1.pages[:2]
    led.release(s1.pages)
    led.release(s2.pages)
    assert led.available() == 6


def test_rollout_server_draws_versions_and_rescoring():
    import torch
    from dew_b200.inference.rollouts import NativeRolloutServer, rescore
    from dew_b200.inference.serving import Server
    from dew_b200.models import CausalTransformer
    from dew_b200.utils.trees import module_variables
    torch.manual_seed(0)
    model = CausalTransformer(vocab_size=48, emb_features=32, num_layers=2, num_heads=2, num_kv_heads=2, head_dim=16, mlp_features=48, max_seq_len=64)
    direct = Server(model, slots=4, capacity=32)
    expect = direct([[1, 2, 3], [4, 5, 6, 7]], 6)
    with NativeRolloutServer(Server(model, slots=4, capacity=32), version=3) as rs:
        futs = [rs.submit([1, 2, 3], 6), rs.submit([4, 5, 6, 7], 6)]
        draws = [f.result(timeout=120) for f in futs]
        assert [d.tokens for d in draws] == expect and all(d.version == 3 and not d.stale for d in draws)
        # new weights under a later version: later draws carry it, and differ from the old policy's
        other = {"params": {k: (v + 0.3 * torch.randn_like(v) if v.dtype.is_floating_point else v) for k, v in _flat(module_variables(model)["params"])}}
        rs.load(_unflat(other["params"]), 4)
        later = rs.submit([1, 2, 3], 6).result(timeout=120)
        assert later.version == 4 and later.tokens != draws[0].tokens
        import pytest
        with pytest.raises(ValueError):
            rs.load(None, 2)
        with pytest.raises(ValueError):
            rs.submit(list(range(30)), 10)
    lp = rescore(model, None, draws)
    assert [len(x) for x in lp] == [6, 6] and all(bool((x <= 0).all()) for x in lp)
    # greedy draws are each step's argmax, so every rescored token is its row's most likely one
    tok = torch.tensor([draws[0].prompt + draws[0].tokens])
    with torch.no_grad():
        best = torch.log_softmax(model(tok[:, :-1]).float(), -1).max(-1).values[0, 2:]
    assert torch.allclose(lp[0], best, atol=1e-5)


def _flat(tree, prefix=()):
    out = []
    for k, v in tree.items():
        out += _flat(v, prefix + (k,)) if isinstance(v, dict) else [(prefix + (k,), v)]
    return out


def _unflat(flat):
    root = {}
    for path, v in flat.items():
        node = root
        for k in path[:-1]:
            node = node.setdefault(k, {})
        node[path[-1]] = v
    return {"params": root}


def test_host_banks_stream_layers_and_reproduce_the_resident_model():
    import torch
    from dew_b200.inference.banks import HostBanks
    from dew_b200.models import CausalTransformer
    from dew_b200.sampling.text import Sampling, generate
    torch.manual_seed(0)
    model = CausalTransformer(vocab_size=64, emb_features=32, num_layers=6, num_heads=2, num_kv_heads=2, head_dim=16, mlp_features=48, max_seq_len=32).eval()
    tokens = torch.randint(0, 64, (2, 12))
    with torch.no_grad():
        want = model(tokens)
        text = generate(model, None, [[1, 2, 3]], 6, sampling=Sampling(temperature=0.0)).tokens
    banks = HostBanks(model.layers, "cpu", slots=4)           # 4 does not divide 6 layers: falls back to 3 slots
    assert banks.slots == 3 and banks.host_bytes() == 2 * banks.device_bytes()
    assert all(p.numel() == 0 for p in model.layers[0].parameters())           # nothing of a layer stays on the device between uses
    with torch.no_grad():
        got = model(tokens)
        again = model(tokens)
        text2 = generate(model, None, [[1, 2, 3]], 6, sampling=Sampling(temperature=0.0)).tokens
    assert torch.equal(got, want) and torch.equal(again, want) and torch.equal(text2, text)
    assert banks.copies >= 12                                  # every call streams every layer
    # a reload of one layer's host weights changes the output; releasing restores ordinary parameters
    banks.load(2, {n: torch.zeros_like(t) for n, t in banks.host[2].items()})
    with torch.no_grad():
        assert not torch.equal(model(tokens), want)
    banks.release()
    assert all(p.numel() > 0 for p in model.layers[5].parameters())
    import pytest
    mixed = CausalTransformer(vocab_size=64, emb_features=32, num_layers=2, num_heads=2, num_kv_heads=2, head_dim=16, mlp_features=48, max_seq_len=32,
                              layer_types=("mamba2", "attention"), mixer_options=dict(state_dim=16, head_dim=16))
    with pytest.raises(ValueError):
        HostBanks(mixed.layers, "cpu")


def test_text_generation_task_with_offloaded_layers():
    import torch
    from dew_b200.inference.tasks import TextGeneration
    from dew_b200.models import CausalTransformer
    torch.manual_seed(0)
    model = CausalTransformer(vocab_size=64, emb_features=32, num_layers=4, num_heads=2, num_kv_heads=2, head_dim=16, mlp_features=48, max_seq_len=32).eval()
    task = TextGeneration(model)
    want = task([[1, 2, 3], [4, 5]], max_new_tokens=5).tokens
    off = task.offloaded(slots=2)
    assert torch.equal(off([[1, 2, 3], [4, 5]], max_new_tokens=5).tokens, want)
    assert all(p.numel() == 0 for p in model.layers[1].parameters())
    task.banks.release()


def test_scoring_server_batches_requests_from_threads_and_keeps_refusals_apart():
    import threading
    from dew_b200.decision import BidirectionalBackbone, Choice, Decide, DecisionHead, DecisionModel, Layout, Noul
    from dew_b200.inference.scoring import LikelihoodScoring, ScoringServer, score
    m = _model()
    server = ScoringServer(LikelihoodScoring(m), max_rows=64)
    futures = [server.submit(([1, 2, 3, i + 4], [[5, 6], [7], [8, 9, 10]])) for i in range(5)]
    try:
        server.submit(([1], []))
        raise AssertionError("an empty request must be refused")
    except ValueError:
        pass
    server.run()
    direct = score(m, [[1, 2, 3, 4]] * 3, [[5, 6], [7], [8, 9, 10]])
    got = futures[0].result()
    assert [round(a[0], 4) for a in got] == [round(a[0], 4) for a in direct] and server.metrics()["rows"] == 15 and server.refused == 1
    assert server.metrics()["passes"] == 1                                    # five requests, one pass
    # a decision task served from a thread while four clients submit bodies
    torch.manual_seed(0)
    task = Decide(DecisionModel(BidirectionalBackbone(260, 32, 1, max_len=256), DecisionHead(32, 1)), Layout(shape="state_first", max_len=200, head_max_len=150))
    qs = {"even": Noul("is it even"), "kind": Choice("which", ["a", "b", "c"])}
    body = lambda i: {"state": f"number {i}", "questions": {n: q.wire() for n, q in qs.items()}}
    wire = task.scoring(details=True)
    served = ScoringServer(wire, max_rows=32, max_wait=0.02).start()
    results = {}

    def client(k):
        for i in range(k, 16, 4):
            results[i] = served.submit(body(i)).result(timeout=30)
    threads = [threading.Thread(target=client, args=(k,)) for k in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    served.stop()
    assert sorted(results) == list(range(16)) and served.metrics()["passes"] < 16          # bodies shared passes
    alone = task.systemone(body(5), details=True)
    assert results[5]["answers"] == alone["answers"] and results[5]["usage"]["input_tokens"] == alone["usage"]["input_tokens"]
    try:
        served.submit({"state": "x", "questions": {}})
        raise AssertionError("a body without questions must be refused")
    except ValueError:
        assert wire.metrics()["refused/malformed"] == 1.0


def test_completion_service_speaks_the_openai_shapes_and_streams():
    import json
    import urllib.error
    import urllib.request
    from dew_b200.data import ByteTokenizer
    from dew_b200.inference.http import CompletionService
    torch.manual_seed(0)
    m = CausalTransformer(vocab_size=260, emb_features=32, num_layers=2, num_heads=4, num_kv_heads=2, mlp_features=64, max_seq_len=128, tie_embeddings=True).eval()
    server = Server(m, slots=4, capacity=64, kv_cache=KVCache(page_size=8), chunk=16, tokenizer=ByteTokenizer())
    with CompletionService(server, name="tiny") as svc:
        base = f"http://{svc.address[0]}:{svc.address[1]}"

        def post(path, body):
            req = urllib.request.Request(base + path, data=json.dumps(body).encode(), method="POST")
            with urllib.request.urlopen(req, timeout=60) as r:
                return r.read()
        out = json.loads(post("/v1/completions", {"prompt": "hello", "max_tokens": 5, "temperature": 0}))
        prompt_ids = ByteTokenizer().encode("hello")
        ref = generate(m, None, [list(prompt_ids)], 5, sampling=Sampling(temperature=0.0))
        want = ref.tokens[0, len(prompt_ids): int(ref.lengths[0])].tolist()
        assert out["object"] == "text_completion" and out["model"] == "tiny" and out["choices"][0]["token_ids"] == want
        assert out["usage"] == {"prompt_tokens": len(prompt_ids), "completion_tokens": 5, "total_tokens": len(prompt_ids) + 5} and out["choices"][0]["finish_reason"] == "length"
        by_ids = json.loads(post("/v1/completions", {"prompt": list(prompt_ids), "max_tokens": 5, "temperature": 0}))
        assert by_ids["choices"][0]["token_ids"] == want
        chat = json.loads(post("/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3, "temperature": 0}))
        assert chat["object"] == "chat.completion" and chat["choices"][0]["message"]["role"] == "assistant" and len(chat["choices"][0]["token_ids"]) == 3
        stream = post("/v1/completions", {"prompt": "hello", "max_tokens": 5, "temperature": 0, "stream": True}).decode()
        chunks = [json.loads(l[6:]) for l in stream.splitlines() if l.startswith("data: {")]
        assert [c["choices"][0]["token_ids"][0] for c in chunks[:-1]] == want and chunks[-1]["choices"][0]["finish_reason"] == "length" and "data: [DONE]" in stream
        try:
            post("/v1/completions", {"prompt": "x" * 100, "max_tokens": 50})
            raise AssertionError("a prompt past the row capacity must be refused")
        except urllib.error.HTTPError as e:
            assert e.code == 400 and "capacity" in json.loads(e.read())["error"]["message"]
        with urllib.request.urlopen(base + "/v1/models", timeout=10) as r:
            assert json.loads(r.read())["data"][0]["id"] == "tiny"
        with urllib.request.urlopen(base + "/metrics", timeout=10) as r:
            metrics = r.read().decode()
        assert "dew_serving_requests_total 4" in metrics and "dew_serving_completion_tokens_total 18" in metrics
