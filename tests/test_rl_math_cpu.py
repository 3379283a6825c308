"""The RL vertical's math and plumbing on fixed tensors: advantages, surrogates, Dreamer's distributions, environments and
rollouts, replay windows, first-episode scoring, DAgger labels, the sandbox, the racing drone and the race's rules."""
import math
import sys

import pytest
import torch

from dew_b200.rl import advantage as A
from dew_b200.rl import distributions as D
from dew_b200.rl import surrogate as S
from dew_b200.rl.aggregation import LABEL, Teacher, imitation_loss, labelled, paired
from dew_b200.rl.env import Driven, Env, TimeLimit, TimeStep, env_rollout, start
from dew_b200.rl.evaluation import episodes, first_episode_rows, first_episodes
from dew_b200.rl.flight import FlightEnv, Racing, commanded, delayed, drawn_course, facings, gate_axes, struck
from dew_b200.rl.quadrotor import GRAVITY, Racer, drawn_body, flown, hovering, quaternion_of, rotation, voltage
from dew_b200.rl.replay import ReplayBuffer
from dew_b200.rl.sandbox import (MathReward, ProcessRunner, Program, ProgramReward, SandboxFleet, SandboxLimits, SubprocessEnvironment, Verdict,
                                 outputs_match)
from dew_b200.rl.simulator import DrivenSimulator, EnvSimulator, simulator_rollout, simulator_start


# ------------------------------------------------------------------------------------------------ advantages
def test_group_rloo_and_gae_advantages():
    r = torch.tensor([1.0, 0.0, 0.0, 1.0, 2.0, 2.0, 2.0, 2.0])
    g = A.group_advantage(r, 4)
    first = r[:4]
    assert torch.allclose(g[:4], (first - first.mean()) / (first.std(correction=1) + 1e-6)) and torch.all(g[4:] == 0)
    assert torch.allclose(A.dr_grpo_advantage(r, 4)[:4], first - first.mean())
    loo = A.rloo_advantage(r, 4)
    assert torch.allclose(loo[:4], (first - first.mean()) * 4 / 3) and abs(float(loo[0]) - (1 - 1 / 3)) < 1e-6
    with pytest.raises(ValueError):
        A.group_advantage(r, 3)
    # GAE against a direct recursion, with padding that must pass values through
    torch.manual_seed(0)
    rewards, values = torch.randn(3, 6), torch.randn(3, 6)
    mask = torch.tensor([[1, 1, 1, 1, 0, 0], [1, 1, 1, 1, 1, 1], [1, 1, 0, 0, 0, 0]], dtype=torch.bool)
    adv, ret = A.gae_advantages(rewards, values, mask, gamma=0.9, lam=0.8)
    for b in range(3):
        T = int(mask[b].sum())
        run, want = 0.0, [0.0] * T
        for t in range(T - 1, -1, -1):
            nxt = float(values[b, t + 1]) if t + 1 < T else 0.0
            run = float(rewards[b, t]) + 0.9 * nxt - float(values[b, t]) + 0.9 * 0.8 * run
            want[t] = run
        assert torch.allclose(adv[b, :T], torch.tensor(want), atol=1e-5)
    assert torch.allclose(ret, adv + values)
    white, _ = A.gae(rewards, values, mask, 0.9, 0.8)
    kept = white[mask]
    assert abs(float(kept.mean())) < 1e-5 and abs(float(kept.var(correction=1)) - 1) < 1e-4 and torch.all(white[~mask] == 0)
    assert torch.isnan(A.masked_mean(torch.tensor([1.0, float("nan")]), torch.tensor([True, False]))) == False
    lam = A.lambda_returns(torch.ones(3, 1), torch.zeros(3, 1), torch.full((3, 1), 0.5), 1.0)
    assert torch.allclose(lam[:, 0], torch.tensor([1.5, 1.0]))


# ------------------------------------------------------------------------------------------------ surrogates
def test_clipped_surrogate_dual_clip_and_reductions():
    logp_old = torch.zeros(2, 3)
    logp = torch.log(torch.tensor([[1.0, 1.5, 0.5], [5.0, 1.0, 0.9]])).requires_grad_()
    adv = torch.tensor([[1.0, 1.0, 1.0], [-1.0, -1.0, 1.0]])
    mask = torch.tensor([[1, 1, 1], [1, 1, 0]], dtype=torch.bool)
    lr = S.token_log_ratio(logp, logp_old)
    terms, m = S.clipped_surrogate_terms(lr, adv, mask, 0.2, 0.3, dual_clip=3.0)
    # positive advantage: ratio 1.5 is clipped at 1.3, ratio 0.5 is not (the pessimistic side keeps the plain term)
    assert torch.allclose(terms[0].detach(), torch.tensor([-1.0, -1.3, -0.5]))
    # negative advantage: ratio 5 would cost 5, the dual clip caps it at 3
    assert torch.allclose(terms[1, :2].detach(), torch.tensor([3.0, 1.0]))
    assert abs(float(m["clip_fraction"]) - 1 / 5) < 1e-6 and abs(float(m["dual_clip_fraction"]) - 1 / 5) < 1e-6
    S.aggregate(terms, mask).backward()
    assert float(logp.grad[0, 1]) == 0.0 and float(logp.grad[1, 0]) == 0.0 and float(logp.grad[0, 2]) != 0.0 and float(logp.grad[1, 2]) == 0.0
    t = torch.tensor([[1.0, 2.0, 3.0], [4.0, 6.0, 100.0]])
    assert float(S.aggregate(t, mask, "token-mean")) == pytest.approx(16 / 5)
    assert float(S.aggregate(t, mask, "seq-mean-token-sum")) == pytest.approx((6 + 10) / 2)
    assert float(S.aggregate(t, mask, "seq-mean-token-mean")) == pytest.approx((2 + 5) / 2)
    assert float(S.aggregate(t, mask, "seq-mean-token-sum-norm")) == pytest.approx((6 / 3 + 10 / 3) / 2)
    with pytest.raises(ValueError):
        S.clipped_surrogate_terms(lr, adv, mask, dual_clip=1.0)


def test_sequence_ratio_cispo_gmpo_and_kl():
    torch.manual_seed(0)
    old = torch.randn(2, 4) * 0.1
    logp = (old + torch.randn(2, 4) * 0.2).requires_grad_()
    mask = torch.tensor([[1, 1, 1, 0], [1, 1, 1, 1]], dtype=torch.bool)
    seq = S.sequence_log_ratio(logp, old, mask)
    want = ((logp - old) * mask).sum(-1) / mask.sum(-1)
    assert torch.allclose(seq.detach(), want.detach()[:, None].expand(2, 4), atol=1e-6)
    seq.sum().backward()
    assert torch.allclose(logp.grad, torch.ones(2, 4))                   # the gradient is each token's own log-probability's
    segs = torch.tensor([[1, 1, 2, 2], [1, 1, 1, 1]])
    sm = S.segment_mean(torch.tensor([[1.0, 3.0, 5.0, 7.0], [1.0, 1.0, 1.0, 5.0]]), torch.ones(2, 4, dtype=torch.bool), segs)
    assert torch.allclose(sm, torch.tensor([[2.0, 2.0, 6.0, 6.0], [2.0, 2.0, 2.0, 2.0]]))
    adv = torch.tensor([[1.0] * 4, [-1.0] * 4])
    lp = logp.detach().clone().requires_grad_()
    terms, m = S.cispo_terms(lp, old, adv, mask, 1.0, 0.28)
    S.aggregate(terms, mask).backward()
    r = (lp.detach() - old).exp().clamp(0.0, 1.28)
    assert torch.allclose(lp.grad, -(r * adv * mask) / mask.sum(), atol=1e-6)           # the clipped ratio weighs a REINFORCE gradient
    g, _ = S.gmpo_terms(lp.detach(), old, adv, mask, 0.4, 0.4)
    d = (lp.detach() - old)
    assert torch.allclose(g[0, 0], -torch.exp((torch.minimum(d[0], d[0].clamp(-0.4, 0.4)) * mask[0]).sum() / 3), atol=1e-5)
    assert torch.allclose(S.reinforce_terms(lp.detach(), adv), -adv * lp.detach())
    ref = lp.detach() + 0.3
    k3 = S.k3_kl(lp.detach(), ref)
    assert torch.all(k3 >= 0) and torch.allclose(k3, torch.full_like(k3, math.exp(0.3) - 0.3 - 1), atol=1e-6)
    small = torch.tensor([1e-4])
    assert abs(float(S.sampled_kl(small)) - 5e-9) < 1e-10                # expm1 keeps the r^2 / 2 term exp(r) - 1 rounds away
    assert float(S.kl_penalty(lp.detach(), ref, "k2")[0, 0]) == pytest.approx(0.045, rel=1e-4)
    v, old_v, ret = torch.tensor([2.0, 0.2]), torch.tensor([0.0, 0.0]), torch.tensor([1.0, 1.0])
    vt, clipped = S.clipped_value_loss_terms(v, old_v, ret, 0.5)
    assert torch.allclose(vt, torch.tensor([0.5 * 1.0, 0.5 * 0.64])) and clipped.tolist() == [0.0, 0.0]


def test_sampler_mismatch_corrections_and_preferences():
    prox = torch.log(torch.tensor([[1.0, 4.0, 0.3], [1.1, 0.9, 1.0]]))
    beh = torch.zeros(2, 3)
    mask = torch.tensor([[1, 1, 1], [1, 1, 0]], dtype=torch.bool)
    w = S.behavior_importance_weights(prox, beh, mask, threshold=2.0)
    assert torch.allclose(w, torch.tensor([[1.0, 2.0, 0.3], [1.1, 0.9, 0.0]]), atol=1e-6) and not w.requires_grad
    band = S.behavior_band_weights(prox, beh, mask, 0.5, 2.0)
    assert torch.allclose(band, torch.tensor([[1.0, 0.0, 0.0], [1.1, 0.9, 0.0]]), atol=1e-6)
    rej = S.sequence_rejection_mask(prox, beh, mask, 0.9, 1.1, geometric=False)
    assert rej.tolist() == [[0, 0, 0], [1, 1, 0]]
    mm = S.mismatch_metrics(prox, beh, mask)
    assert float(mm["ratio_max"]) == pytest.approx(4.0) and float(mm["k3_kl"]) > 0
    one = torch.ones(1, 2, dtype=torch.bool)
    terms, rc, rr = S.preference_logsigmoid_terms(torch.tensor([[-1.0, -1.0]]), torch.tensor([[-2.0, -2.0]]), torch.tensor([[-1.5, -1.5]]),
                                                   torch.tensor([[-1.5, -1.5]]), one, one, beta=0.5)
    assert float(terms) == pytest.approx(-math.log(1 / (1 + math.exp(-1.0)))) and float(rc) == pytest.approx(0.5) and float(rr) == pytest.approx(-0.5)


# ------------------------------------------------------------------------------------------------ distributions
def test_symlog_twohot_unimix_and_tanh_jacobian():
    x = torch.tensor([-1000.0, -1.0, 0.0, 0.5, 3e4])
    assert torch.allclose(D.symexp(D.symlog(x)), x, rtol=1e-4)
    bins = D.twohot_bins()
    assert bins.shape == (255,) and float(bins[127]) == 0.0 and torch.equal(bins, -bins.flip(0))
    assert float(D.twohot_mean(torch.zeros(255), bins)) == 0.0             # uniform probabilities predict zero exactly
    target = torch.tensor([0.0, 2.5, -7.0, 1e12, -1e12])
    enc = D.twohot(target, bins)
    assert torch.allclose(enc.sum(-1), torch.ones(5)) and int((enc[1] > 0).sum()) == 2
    assert torch.allclose((enc[:3] * bins).sum(-1), target[:3], atol=1e-4)
    assert float(enc[3, -1]) == 1.0 and float(enc[4, 0]) == 1.0           # past the ends: all on the last / first bin
    logits = enc[1].clamp_min(1e-30).log()
    assert float(D.twohot_loss(logits, target[1], bins)) == pytest.approx(float(-(enc[1][enc[1] > 0] * enc[1][enc[1] > 0].log()).sum()), abs=1e-5)
    assert float(D.twohot_mean(logits, bins)) == pytest.approx(2.5, abs=1e-4)
    lp = D.unimix_log_probs(torch.tensor([0.0, -1e4, 50.0]), 0.01)
    assert torch.isfinite(lp).all() and float(lp.exp().sum()) == pytest.approx(1.0, abs=1e-6) and float(lp[1].exp()) == pytest.approx(0.01 / 3, rel=1e-4)
    raw = torch.tensor([-20.0, 0.0, 0.3, 20.0], dtype=torch.float64)
    exact = torch.log1p(-torch.tanh(raw[1:3]) ** 2)
    assert torch.allclose(D.tanh_log_jacobian(raw)[1:3], exact) and torch.isfinite(D.tanh_log_jacobian(raw)).all()
    lp = torch.log_softmax(torch.randn(64, 5, generator=torch.Generator().manual_seed(0)), -1).requires_grad_()
    draw = D.onehot_sample(lp, torch.Generator().manual_seed(1))
    assert torch.allclose(draw.sum(-1), torch.ones(64)) and set(draw.detach().round().unique().tolist()) <= {0.0, 1.0}
    (draw * torch.arange(5.0)).sum().backward()
    assert torch.allclose(lp.grad, lp.exp().detach() * torch.arange(5.0), atol=1e-6)       # straight through the probabilities
    assert float(D.normal_entropy(torch.tensor(1.0))) == pytest.approx(0.5 * math.log(2 * math.pi * math.e))


# ------------------------------------------------------------------------------------------------ environments
class Walk(Env):
    """A point on a line: the action moves it, the reward is the move, the episode ends at |x| >= 3."""
    action_size = 1

    def reset(self, key, count):
        x = torch.zeros(count)
        return {"x": x}, TimeStep({"x": x.clone(), "passed": torch.zeros(count)}, torch.zeros(count), torch.zeros(count, dtype=torch.bool),
                                  torch.zeros(count, dtype=torch.bool))

    def step(self, state, action):
        x = state["x"] + action[:, 0]
        return {"x": x}, TimeStep({"x": x.clone(), "passed": x.abs().floor()}, action[:, 0], x.abs() >= 3, torch.zeros_like(x, dtype=torch.bool))


def _right(params, obs, memory, key):
    n = obs["x"].shape[0]
    return torch.ones(n, 1) * params, {"logp": torch.zeros(n)}, memory


def test_rollout_restarts_in_place_time_limit_and_driven():
    env = Walk()
    carry, tr = env_rollout(env, _right, 1.0, start(env, 0, 2), 7)
    assert tr.step.reward.shape == (7, 2) and tr.step.terminated[:, 0].tolist() == [False, False, True, False, False, True, False]
    assert tr.observation["x"][:, 0].tolist() == [0, 1, 2, 0, 1, 2, 0] and carry.episodes == 4 and tr.extras["logp"].shape == (7, 2)
    limited = TimeLimit(Walk(), episode_length=2, action_repeat=2)
    state, ts = limited.reset(0, 1)
    state, ts = limited.step(state, torch.full((1, 1), 0.5))
    assert float(ts.reward) == 1.0 and not bool(ts.done)
    state, ts = limited.step(state, torch.full((1, 1), 0.5))
    assert bool(ts.truncated) and not bool(ts.terminated) and float(state["inner"]["x"]) == 2.0
    state, ts = limited.reset(0, 1)
    state, ts = limited.step(state, torch.full((1, 1), 3.0))              # ends inside the repeats: the second repeat earns nothing
    assert bool(ts.terminated) and float(ts.reward) == 3.0 and float(state["inner"]["x"]) == 3.0
    driven = Driven(Walk())
    state, ts = driven.reset(0, 1)
    assert bool(ts.observation["first"]) and float(ts.observation["reward"]) == 0
    flags = []
    for _ in range(5):
        state, ts = driven.step(state, torch.ones(1, 1))
        flags.append((bool(ts.observation["first"]), bool(ts.observation["last"]), float(ts.observation["x"])))
    assert flags == [(False, False, 1.0), (False, False, 2.0), (False, True, 3.0), (True, False, 0.0), (False, False, 1.0)]
    # the same through a host-stepped simulator
    sim = EnvSimulator(Walk(), 2)
    carry, tr2 = simulator_rollout(sim, _right, 1.0, simulator_start(sim, 0), 7)
    assert torch.equal(tr2.step.terminated, tr.step.terminated) and torch.equal(tr2.observation["x"], tr.observation["x"])
    ds = DrivenSimulator(EnvSimulator(Walk(), 1))
    obs = ds.reset(0)
    seen = []
    for _ in range(5):
        obs, *_ = ds.step(torch.ones(1, 1))
        seen.append((bool(obs["first"]), bool(obs["last"]), float(obs["x"])))
    assert seen == flags


def test_first_episode_scores_replay_windows_and_dagger_labels():
    done = torch.tensor([[0, 0], [1, 0], [0, 0], [0, 1]], dtype=torch.bool)
    assert first_episodes(done).tolist() == [[True, True], [True, True], [False, True], [False, True]]
    score = episodes(_right, Walk(), steps=8, count=3, names=("passed",))(1.0, 0)
    assert score == {"return": 3.0, "steps": 3.0, "terminated": 1.0, "finished": 1.0, "last_reward": 1.0, "passed": 3.0}
    rb = ReplayBuffer(capacity=6, envs=2)
    for t in range(9):
        rb.add({"t": torch.full((2,), float(t)), "env": torch.arange(2.0)})
    assert rb.filled == 6 and rb.windows(4) == 3
    batch = rb.sample(64, 4, torch.Generator().manual_seed(0))
    assert batch["t"].shape == (64, 4) and torch.all(batch["t"][:, 1:] - batch["t"][:, :-1] == 1)      # never across the ring's seam
    assert float(batch["t"].min()) == 3.0 and float(batch["t"].max()) == 8.0 and torch.all(batch["env"] == batch["env"][:, :1])
    with pytest.raises(ValueError):
        rb.sample(1, 7)
    teacher = Teacher(lambda v, obs, m, k: (-obs["x"][:, None] * v, {}, m), 0.5)
    policy = labelled(_right, teacher, beta=0.5)
    action, extras, _ = policy(paired(1.0, teacher), {"x": torch.arange(8.0)}, None, 3)
    assert torch.equal(extras[LABEL][:, 0], -0.5 * torch.arange(8.0)) and 0 < int(extras["teacher_acted"].sum()) < 8
    assert torch.equal(action[extras["teacher_acted"]], extras[LABEL][extras["teacher_acted"]]) and torch.all(action[~extras["teacher_acted"]] == 1)
    assert float(imitation_loss(torch.zeros(8, 1), extras[LABEL], torch.tensor([1, 1, 0, 0, 0, 0, 0, 0]))) == pytest.approx(0.125)


# ------------------------------------------------------------------------------------------------ the sandbox
def test_sandbox_runs_limits_and_scores_programs():
    limits = SandboxLimits(cpu_seconds=2, memory_bytes=512 << 20, wall_seconds=3.0, output_bytes=4096)
    with SandboxFleet(ProcessRunner(), workers=4, limits=limits) as fleet:
        ok, bad, spin, loud, fork = fleet.run([
            fleet.python("print(int(input()) * 2)", "21\n"),
            fleet.python("import sys; sys.exit(3)"),
            fleet.python("while True: pass"),
            fleet.python("print('x' * 100000)"),
            fleet.python("import os, time\nif os.fork() == 0:\n    time.sleep(30)\nprint('parent')"),
        ])
        assert ok.ok and outputs_match(ok, "42") and outputs_match(ok, " 42 \n")
        assert bad.verdict is Verdict.COMPLETED and bad.exit_code == 3 and not outputs_match(bad, "")
        assert spin.verdict is Verdict.TIMED_OUT and spin.seconds < 4.0
        assert loud.verdict is Verdict.OUTPUT_EXCEEDED and len(loud.stdout) <= 4096
        assert fork.ok and fork.seconds < 3.0                             # the forked child is killed with the group
        reward = ProgramReward(fleet)
        scores = reward(["```python\nprint(sum(map(int, input().split())))\n```", "no code", "```python\nprint(0)\n```"],
                        [[("1 2", "3"), ("5 5", "10")]] * 3)
        assert scores == [1.0, 0.0, 0.0]
    with pytest.raises(ValueError):
        Program({"../escape.py": ""}, ("python",))
    with pytest.raises(ValueError):
        Program({}, ())
    math_reward = MathReward()
    assert math_reward("so the answer is \\boxed{\\frac{1}{2}}", "0.5") == 1.0 and math_reward("\\boxed{3}", "4") == 0.0
    assert math_reward("the answer is 1,234", "1234") == 0.0 and MathReward(require_boxed=False)("the answer is 1,234", "1234") == 1.0
    worker = ("import json, sys\nx = 0\nfor line in sys.stdin:\n    m = json.loads(line)\n    x = 0 if m['op'] == 'reset' else x + m['action']\n"
              "    print(json.dumps({'observation': x, 'reward': float(x > 2), 'done': x > 2}), flush=True)\n")
    with SubprocessEnvironment((sys.executable, "-I", "worker.py"), limits, files={"worker.py": worker}) as env:
        assert env.reset()["observation"] == 0
        assert [env.step(1)["observation"] for _ in range(3)] == [1, 2, 3] and env.step(0)["done"] is True


# ------------------------------------------------------------------------------------------------ the drone and the race
def test_racing_drone_hovers_turns_and_sags():
    racer = Racer()
    assert 4 * racer.thrust_coefficient * racer.top_speed ** 2 / (racer.mass * GRAVITY) == pytest.approx(11.95, abs=0.05)
    body = drawn_body(racer, 0, 3, ramp=0.0)
    assert torch.allclose(body["mass"], torch.full((3,), racer.mass)) and float(body["force"].abs().max()) == 0.0
    f = hovering(racer, body, torch.tensor([[0.0, 0.0, 3.0]] * 3), quaternion_of(torch.tensor([0.0, 1.0, -2.0])))
    hover = body["mass"] * GRAVITY
    for i in range(30):
        f, path = flown(racer, body, f, hover, torch.zeros(3, 3), 60.0, i)
    assert path.shape == (3, racer.substeps + 1, 3) and float((f["position"][:, 2] - 3.0).abs().max()) < 0.15
    assert float(f["position"][:, :2].abs().max()) < 1e-3 and torch.allclose(f["orientation"].norm(dim=-1), torch.ones(3), atol=1e-6)
    assert float(voltage(racer, body, f["speed"], f["used"])[0]) < racer.cells * racer.full_voltage      # the load sags the pack
    # a commanded roll rate is reached within 70 ms with little overshoot
    rates = []
    for i in range(12):
        f, _ = flown(racer, body, f, hover, torch.tensor([[3.0, 0.0, 0.0]] * 3), 60.0, i)
        rates.append(float(f["angular_velocity"][0, 0]))
    assert rates[3] > 0.9 * 3.0 and max(rates) < 3.0 * 1.08 and abs(rates[-1] - 3.0) < 0.05
    # full throttle climbs at about (T/W - 1) g less the sag
    f = hovering(racer, body, torch.tensor([[0.0, 0.0, 3.0]] * 3), quaternion_of(torch.zeros(3)))
    for i in range(30):
        f, _ = flown(racer, body, f, torch.full((3,), 4 * racer.thrust_coefficient * racer.top_speed ** 2), torch.zeros(3, 3), 60.0, i)
    assert 20.0 < float(f["velocity"][0, 2]) < 55.0
    wild = drawn_body(racer, 1, 64, ramp=1.0)
    assert 0.9 * racer.mass < float(wild["mass"].min()) and float(wild["mass"].max()) < 1.1 * racer.mass and float(wild["force"].norm(dim=-1).max()) <= 2.0 * 0.8
    R = rotation(quaternion_of(torch.tensor([math.pi / 2])))
    assert torch.allclose(R[0] @ torch.tensor([1.0, 0.0, 0.0]), torch.tensor([0.0, 1.0, 0.0]), atol=1e-6)


def test_race_rules_gates_frames_pillars_and_commands():
    rc = Racing()
    centre, facing = torch.tensor([[5.0, 0.0, 2.0]] * 5), torch.zeros(5)
    none = torch.zeros(5, 1, 4)
    line = lambda a, b: torch.stack([torch.tensor(a), torch.tensor(b)])[None]
    paths = torch.cat([line([4.0, 0.0, 2.0], [6.0, 0.0, 2.0]),            # through the middle
                       line([4.0, 0.4, 2.3], [6.0, 0.4, 2.3]),            # through, off centre
                       line([4.0, 0.8, 2.0], [6.0, 0.8, 2.0]),            # into the frame's bar
                       line([4.0, 2.0, 2.0], [6.0, 2.0, 2.0]),            # past the gate, outside the frame
                       line([6.0, 0.0, 2.0], [4.0, 0.0, 2.0])])           # backwards through the opening: no pass, no crash
    crashed, passed, offset = struck(rc, paths, centre, facing, none)
    assert crashed.tolist() == [False, False, True, False, False] and passed.tolist() == [True, True, False, False, False]
    assert float(offset[0]) == 0.0 and float(offset[1]) == pytest.approx(0.4 / 0.75)
    pillar = torch.tensor([[[5.0, 0.0, 0.3, 3.0]]])
    hit, _, _ = struck(rc, line([4.0, 0.0, 2.0], [4.6, 0.0, 2.0]), torch.tensor([[50.0, 0.0, 2.0]]), torch.zeros(1), pillar)
    over, _, _ = struck(rc, line([4.0, 0.0, 3.5], [4.6, 0.0, 3.5]), torch.tensor([[50.0, 0.0, 2.0]]), torch.zeros(1), pillar)
    assert bool(hit) and not bool(over)
    ground, _, _ = struck(rc, line([0.0, 0.0, 0.5], [0.0, 0.0, 0.1]), torch.tensor([[50.0, 0.0, 2.0]]), torch.zeros(1), none[:1])
    assert bool(ground)
    body = drawn_body(rc.racer, 0, 3, 0.0)
    collective, rates = commanded(rc, body, torch.full((3,), 10.0), torch.tensor([[-1.0, 0, 0, 0], [0.0, 1.0, 0, 0], [1.0, 0, 0, -0.5]]))
    hover = rc.racer.mass * GRAVITY
    assert collective.tolist() == pytest.approx([0.0, hover, 4 * rc.racer.thrust_coefficient * rc.racer.top_speed ** 2], rel=1e-5)
    assert rates[1].tolist() == [10.0, 0.0, 0.0] and rates[2].tolist() == [0.0, 0.0, -5.0]
    pending = torch.zeros(2, 4, 1)
    taken = []
    for t in range(1, 6):
        pending, got = delayed(pending, torch.full((2, 1), float(t)), torch.tensor([0, 2]))
        taken.append(got[:, 0].tolist())
    assert taken == [[1.0, 0.0], [2.0, 0.0], [3.0, 1.0], [4.0, 2.0], [5.0, 3.0]]
    square = torch.tensor([[[0.0, 0, 1], [4.0, 0, 1], [4.0, 4, 1], [0.0, 4, 1]]])
    fc = facings(square, torch.tensor([4]), torch.tensor([True]))
    assert torch.allclose(fc, torch.tensor([[-math.pi / 4, math.pi / 4, 3 * math.pi / 4, -3 * math.pi / 4]]), atol=1e-6)
    fo = facings(square, torch.tensor([4]), torch.tensor([False]))
    assert torch.allclose(fo[0, [0, 3]], torch.tensor([0.0, math.pi]), atol=1e-6)
    n, l = gate_axes(torch.tensor([math.pi / 2]))
    assert torch.allclose(n, torch.tensor([[0.0, 1.0, 0.0]]), atol=1e-6) and torch.allclose(l, torch.tensor([[-1.0, 0.0, 0.0]]), atol=1e-6)
    for fam in ("loop", "chain", "figure8", "layout"):
        course = drawn_course(Racing(families=((fam, 1.0),)), 0, 4, 1.0)
        k = course["count"]
        assert course["centres"].shape == (4, 12, 3) and int(k.min()) >= 4 and float(course["centres"][..., 2].min()) > 1.0
        gaps = (course["centres"][:, 1:] - course["centres"][:, :-1]).norm(dim=-1)
        assert float(gaps[0, : int(k[0]) - 1].min()) > 1.0
    a, b = drawn_course(rc, 5, 3), drawn_course(rc, 5, 3)
    assert torch.equal(a["centres"], b["centres"]) and not torch.equal(a["centres"], drawn_course(rc, 6, 3)["centres"])


def test_flight_env_rewards_progress_and_ends_on_a_crash():
    env = FlightEnv(Racing(), views=("state", "gates", "airframe", "obstacles", "action", "progress"), difficulty=0.0, ramp=0.0)
    state, ts = env.reset(0, 4)
    assert {k: v.shape[-1] for k, v in ts.observation.items()} == {"state": 13, "gates": 24, "airframe": 6, "obstacles": 12, "action": 4, "progress": 3}
    assert torch.allclose(ts.observation["airframe"][:, 1:3], torch.ones(4, 2), atol=1e-5)
    # the next gate's corners, seen from the body, lie ahead (positive x) and centre on the gate
    ahead = ts.observation["gates"].reshape(4, 2, 4, 3)[:, 0]
    assert float(ahead[..., 0].min()) > 1.0 and float(ahead[..., 1].mean(1).abs().max()) < 0.5
    # pitching forward under a little extra throttle approaches the gate: progress is rewarded
    total = torch.zeros(4)
    for t in range(40):
        a = torch.zeros(4, 4)
        a[:, 0] = 0.03
        a[:, 2] = 0.25 if t < 6 else 0.0
        state, ts = env.step(state, a)
        total += ts.reward
        assert not bool(ts.terminated.any())
    assert float(total.min()) > 0.3 and float(state["distance"].max()) < float(6.5)
    # cutting the throttle falls to the ground: a crash ends the episode with the penalty
    for t in range(200):
        state, ts = env.step(state, torch.tensor([[-1.0, 0, 0, 0]] * 4))
        if bool(ts.terminated.all()):
            break
    assert bool(ts.terminated.all()) and float(ts.reward.max()) < -5.0
    with pytest.raises(ValueError):
        FlightEnv(views=("nope",))
