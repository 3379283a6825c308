"""One engine drives a text server and scoring servers in alternating passes."""
import pytest
import torch

from dew_b200.inference.engine import Engine
from dew_b200.inference.scoring import Scoring, ScoringRequest, ScoringServer
from dew_b200.inference.serving import Server
from dew_b200.models.causal_transformer import CausalTransformer, TransformerConfig


class Lengths(Scoring):
    """Scores a row by its length; counts its passes."""
    passes = 0

    def admit(self, request):
        if not request:
            raise ValueError("an empty request")
        return ScoringRequest(rows=list(request), payload=len(request))

    def forward(self, rows):
        Lengths.passes += 1
        return [len(r) for r in rows]

    def answer(self, payload, outputs):
        assert len(outputs) == payload
        return list(outputs)


def test_kinds_alternate_and_answer():
    torch.manual_seed(0)
    model = CausalTransformer(TransformerConfig(vocab_size=50, emb_features=32, num_layers=1, num_heads=2, mlp_features=64, max_seq_len=64, qk_norm=False),
                              dtype=torch.float32).eval()
    text = Server(model, slots=2, capacity=64)
    engine = Engine(text=text, scoring={"lengths": ScoringServer(Lengths(), max_rows=3)})
    assert engine.kinds == ["text", "lengths"]
    ticket = engine.submit("text", [1, 2, 3], 6)
    futures = [engine.submit("lengths", ["ab", "cde"]), engine.submit("lengths", ["x"]), engine.submit("lengths", ["four", "fives", "sixsix"])]
    with pytest.raises(KeyError, match="serves no"):
        engine.submit("images", None)
    with pytest.raises(ValueError, match="empty"):
        engine.submit("lengths", [])
    assert engine.busy()
    engine.step()
    # one round: one text step and one scoring pass (the first two requests fill max_rows = 3; the third waits for the next round)
    assert engine.steps == {"text": 1, "lengths": 1} and futures[0].done() and futures[1].done() and not futures[2].done()
    engine.run()
    assert [f.result() for f in futures] == [[2, 3], [1], [4, 5, 6]]
    assert len(ticket.result()) == 6 and not engine.busy()
    assert engine.steps["lengths"] == 2 and engine.steps["text"] >= 6
    m = engine.metrics()
    assert m["lengths/rows"] == 6.0 and m["rounds/lengths"] == 2.0
    # alone, the same generation gives the same tokens: sharing the loop changed nothing it computes
    again = Server(model, slots=2, capacity=64)
    t2 = again.submit([1, 2, 3], 6)
    again.run()
    assert t2.result() == ticket.result()


def test_threaded_engine():
    engine = Engine(scoring={"a": ScoringServer(Lengths()), "b": ScoringServer(Lengths())}).start()
    try:
        fa, fb = engine.submit("a", ["xx"]), engine.submit("b", ["yyy", "z"])
        assert fa.result(timeout=5) == [2] and fb.result(timeout=5) == [3, 1]
    finally:
        engine.stop()
    with pytest.raises(ValueError, match="at least one"):
        Engine()
