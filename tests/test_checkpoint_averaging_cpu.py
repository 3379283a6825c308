"""The mean of runs' weights, the tail average of one run, and the greedy soup."""
import pytest
import torch

from dew_b200.checkpoints.averaging import greedy_soup, mean_of


def _tree(v, step=0):
    return {"params": {"layer": {"w": torch.full((2, 3), float(v)), "b": torch.full((3,), float(v), dtype=torch.bfloat16)}}, "count": torch.tensor(step)}


def test_mean_of():
    m = mean_of([_tree(1, 10), _tree(2, 20), _tree(6, 30)])
    assert torch.allclose(m["params"]["layer"]["w"], torch.full((2, 3), 3.0)) and m["params"]["layer"]["b"].dtype == torch.bfloat16
    assert int(m["count"]) == 10                                       # integer leaves are the first tree's
    w = mean_of([_tree(0), _tree(10)], weights=[3, 1])
    assert torch.allclose(w["params"]["layer"]["w"], torch.full((2, 3), 2.5))
    other = _tree(1)
    other["params"]["layer"]["w"] = torch.zeros(3, 3)
    with pytest.raises(ValueError, match="layer/w"):
        mean_of([_tree(1), other])
    missing = _tree(1)
    del missing["params"]["layer"]["b"]
    with pytest.raises(KeyError, match="holds no"):
        mean_of([_tree(1), missing])
    with pytest.raises(KeyError, match="that tree 0 does not"):
        mean_of([missing, _tree(1)])


def test_greedy_soup_keeps_what_helps():
    target = 3.0
    score = lambda t: -abs(float(t["params"]["layer"]["w"].mean()) - target)       # nearer the target is better
    candidates = [_tree(2.5), _tree(3.6), _tree(9.0), _tree(2.0)]
    soup, chosen, best = greedy_soup(candidates, score)
    # 2.5 is the best alone; with 3.6 the mean 3.05 is better; 2.0 then 9.0 would both make it worse
    assert chosen == [0, 1] and best == pytest.approx(-0.05, abs=1e-6)
    assert torch.allclose(soup["params"]["layer"]["w"], torch.full((2, 3), 3.05))
    _, chosen, _ = greedy_soup(candidates, lambda t: abs(float(t["params"]["layer"]["w"].mean()) - target), higher_is_better=False)
    assert chosen == [0, 1]


def test_average_steps_of_a_run(tmp_path):
    import dew_b200 as dew
    from dew_b200.checkpoints.averaging import average_steps
    from dew_b200.models import CausalTransformer
    from dew_b200.objectives.lm import LMObjective
    torch.manual_seed(0)
    model = CausalTransformer(vocab_size=32, emb_features=16, num_layers=1, num_heads=2, mlp_features=32, max_seq_len=16)
    ck = dew.Checkpoints(tmp_path / "run", keep=dew.Keep(3))
    trainer = dew.Trainer(LMObjective(model, 8), dew.OptimConfig(learning_rate=1e-2), checkpoints=ck)
    data = dew.Memory({"tokens": torch.randint(0, 32, (64, 9))}).repeat().batched(8)
    trainer.fit(data, steps=6, checkpoint_every=2, log_every=2)
    ck.wait()
    steps = ck.steps()
    assert len(steps) == 3
    mean = average_steps(ck, last=2)
    from dew_b200.utils.trees import flatten
    a, b = flatten(ck.variables(step=steps[-2])), flatten(ck.variables(step=steps[-1]))
    for path, leaf in flatten(mean).items():
        if torch.is_tensor(leaf) and leaf.is_floating_point():
            assert torch.allclose(leaf.float(), (a[path].float() + b[path].float()) / 2, atol=1e-6), path
