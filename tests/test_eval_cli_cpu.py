"""``python -m dew_b200.eval``: the perplexity report of a saved release, and the message when the harness is absent."""
import json

import torch

from dew_b200.eval.__main__ import main
from dew_b200.interop.hf import Pretrained
from dew_b200.models.causal_transformer import CausalTransformer, TransformerConfig


def test_perplexity_of_a_saved_release(tmp_path, capsys):
    torch.manual_seed(0)
    model = CausalTransformer(TransformerConfig(vocab_size=260, emb_features=32, num_layers=1, num_heads=2, mlp_features=64, max_seq_len=64, qk_norm=False,
                                                tie_embeddings=False), dtype=torch.float32)
    Pretrained.save(model, tmp_path / "m", family="llama")
    text = tmp_path / "t.txt"
    text.write_text("the quick brown fox jumps over the lazy dog " * 6)
    assert main(["--model", str(tmp_path / "m"), "--tokenizer", "bytes", "--perplexity", str(text), "--dtype", "float32", "--max-length", "64", "--device", "cpu"]) == 0
    report = json.loads(capsys.readouterr().out)
    assert report["family"] == "llama" and report["perplexity"]["tokens"] >= len(text.read_text())
    # an untrained model over 260 symbols sits near the uniform guess
    assert 100 < report["perplexity"]["per_token_perplexity"] < 700 and 6.0 < report["perplexity"]["bits_per_byte"] < 10.0
    code = main(["--model", str(tmp_path / "m"), "--tokenizer", "bytes", "--tasks", "arc_easy", "--dtype", "float32", "--device", "cpu"])
    try:
        import lm_eval  # noqa: F401
    except ImportError:
        assert code == 2 and "lm_eval" in capsys.readouterr().err
