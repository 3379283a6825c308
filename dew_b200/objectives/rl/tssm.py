"""TransDreamer's transformer state-space model (arXiv 2202.09481): a Dreamer world model's dynamics as a causal transformer over the
latents and actions before each step.  At step t the posterior reads the observation alone, ``q(z_t | x_t)``, so a window's latents
are drawn at once; the transformer reads each step's previous latent and action ``(z_{t-1}, a_{t-1})`` and answers the deterministic
state ``h_t``, from which the prior predicts ``z_t``: ``p(z_t | h_t)``.  ``h_t`` therefore holds nothing of ``x_t``, and the prior is a
prediction.  Attention stays within an episode: a step that starts one reads a learned start embedding and attends to nothing before it.

Training runs the window in parallel (``observe``); acting and imagination run the same attention a step at a time over a cache of
keys and values (``step`` with a ``TSSMCache``), so the policy and the imagined rollouts read the function the model was trained as -
the two forms agree to rounding, which the tests hold it to.  Rotary positions count from each episode's start; queries and keys are
RMS-normed; the feed-forward is gated.

Reference: src/dew/objectives/rl/tssm.py.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import ops
from ...rl import distributions as D


@dataclass
class TSSMCache:
    """Per layer, keys and values ``[N, T, heads, head_dim]`` of the steps so far; ``episode [N, T]`` the episode each belongs to (a
    running count of starts), ``position [N]`` the next step's position in its episode."""
    k: List[Optional[torch.Tensor]]
    v: List[Optional[torch.Tensor]]
    episode: Optional[torch.Tensor]
    position: torch.Tensor
    current: torch.Tensor

    def trimmed(self, keep: int) -> "TSSMCache":
        """The last ``keep`` steps only (a bounded context for long rollouts)."""
        cut = lambda t: None if t is None else t[:, -keep:]
        return TSSMCache([cut(t) for t in self.k], [cut(t) for t in self.v], cut(self.episode), self.position, self.current)


class _Block(nn.Module):
    def __init__(self, width: int, heads: int, eps: float = 1e-6):
        super().__init__()
        self.h, self.d = heads, width // heads
        self.norm1, self.norm2 = nn.RMSNorm(width, eps=eps), nn.RMSNorm(width, eps=eps)
        self.qkv, self.out = nn.Linear(width, 3 * width, bias=False), nn.Linear(width, width, bias=False)
        self.q_norm, self.k_norm = nn.RMSNorm(self.d, eps=eps), nn.RMSNorm(self.d, eps=eps)
        inner = (8 * width // 3 + 15) // 16 * 16                       # four widths wide before the gate's 2/3
        self.gate_up, self.down = nn.Linear(width, 2 * inner, bias=False), nn.Linear(inner, width, bias=False)

    def project(self, x, cos, sin, positions):
        B, T, _ = x.shape
        q, k, v = self.qkv(self.norm1(x)).view(B, T, 3, self.h, self.d).unbind(2)
        q, k = self.q_norm(q), self.k_norm(k)
        return ops.rope_reference(q, cos, sin, positions), ops.rope_reference(k, cos, sin, positions), v

    def attend(self, x, q, k, v, visible):
        s = torch.einsum("bshd,bthd->bhst", q.float(), k.float()) * self.d ** -0.5
        p = torch.softmax(s.masked_fill(~visible[:, None], float("-inf")), -1)
        o = torch.einsum("bhst,bthd->bshd", p, v.float()).to(x.dtype)
        x = x + self.out(o.reshape(*x.shape[:2], -1))
        g, u = self.gate_up(self.norm2(x)).chunk(2, -1)
        return x + self.down(F.silu(g) * u)


class TSSM(nn.Module):
    def __init__(self, embed: int, action: int, deter: int = 512, stoch: int = 32, classes: int = 32, layers: int = 4, heads: int = 8, hidden: int = 512,
                 unimix: float = 0.01, max_steps: int = 4096):
        super().__init__()
        self.deter, self.stoch, self.classes, self.unimix, self.action = deter, stoch, classes, unimix, action
        self.inp = nn.Sequential(nn.Linear(stoch * classes + action, deter), nn.RMSNorm(deter), nn.SiLU())
        self.start = nn.Parameter(torch.zeros(deter))
        self.blocks = nn.ModuleList(_Block(deter, heads) for _ in range(layers))
        self.final = nn.RMSNorm(deter)
        self.prior = nn.Sequential(nn.Linear(deter, hidden), nn.RMSNorm(hidden), nn.SiLU(), nn.Linear(hidden, stoch * classes))
        self.post = nn.Sequential(nn.Linear(embed, hidden), nn.RMSNorm(hidden), nn.SiLU(), nn.Linear(hidden, stoch * classes))
        self.max_steps = max_steps
        self._rope = None

    @property
    def features(self) -> int:
        return self.deter + self.stoch * self.classes

    def _tables(self, device):
        if self._rope is None or self._rope[0].device != torch.device(device):
            self._rope = ops.rope_tables(self.max_steps, self.deter // self.blocks[0].h, 10000.0, device)
        return self._rope

    def _logp(self, logits):
        return D.unimix_log_probs(logits.reshape(*logits.shape[:-1], self.stoch, self.classes), self.unimix)

    def draw(self, logp, generator=None, mode: bool = False):
        if mode:
            return F.one_hot(logp.argmax(-1), self.classes).to(logp.dtype).reshape(*logp.shape[:-2], self.stoch * self.classes)
        return D.onehot_sample(logp, generator).reshape(*logp.shape[:-2], self.stoch * self.classes)

    def posterior(self, embed, generator=None, mode: bool = False):
        """``q(z | x)`` from the observation's embedding alone: ``(z, log-probabilities)`` for any leading axes."""
        post = self._logp(self.post(embed))
        return self.draw(post, generator, mode), post

    def _tokens(self, z_prev, a_prev, first):
        x = self.inp(torch.cat([z_prev, a_prev], -1))
        return torch.where(first[..., None], self.start.to(x.dtype).expand_as(x), x)

    # ------------------------------------------------------------------ a window at once
    def observe(self, embed, actions, first, generator=None):
        """``embed [N, T, E]``, ``actions [N, T, A]`` (the action taken *at* each step), ``first [N, T]`` -> ``(h, z, prior, post)`` with
        ``h [N, T, deter]``.  Step t's token is ``(z_{t-1}, a_{t-1})``, or the start embedding where ``first``."""
        N, T, _ = embed.shape
        z, post = self.posterior(embed, generator)
        z_prev = torch.cat([torch.zeros_like(z[:, :1]), z[:, :-1]], 1)
        a_prev = torch.cat([torch.zeros_like(actions[:, :1]), actions[:, :-1]], 1)
        first = first.clone()
        first[:, 0] = True                                               # nothing is known before the window
        x = self._tokens(z_prev, a_prev, first)
        episode = first.long().cumsum(1)
        idx = torch.arange(T, device=embed.device)
        starts = torch.where(first, idx[None].expand(N, T), torch.zeros_like(episode)).cummax(1).values
        positions = idx[None] - starts
        visible = (episode[:, :, None] == episode[:, None, :]) & (idx[None, :, None] >= idx[None, None, :])
        cos, sin = self._tables(embed.device)
        for block in self.blocks:
            q, k, v = block.project(x, cos, sin, positions)
            x = block.attend(x, q, k, v, visible)
        h = self.final(x)
        return h, z, self._logp(self.prior(h)), post

    # ------------------------------------------------------------------ a step at a time
    def initial(self, n: int, device) -> TSSMCache:
        L = len(self.blocks)
        zero = torch.zeros(n, dtype=torch.long, device=device)
        return TSSMCache([None] * L, [None] * L, None, zero, zero.clone())

    def step(self, cache: TSSMCache, z_prev, a_prev, first) -> Tuple[torch.Tensor, torch.Tensor, TSSMCache]:
        """One step from the previous latent and action: ``(h_t, prior log-probabilities, cache)``.  ``first [N]`` starts an episode."""
        N = z_prev.shape[0]
        first = first | (cache.episode is None)
        x = self._tokens(z_prev, a_prev, first)[:, None]
        current = cache.current + first.long()
        position = torch.where(first, torch.zeros_like(cache.position), cache.position)
        episode = current[:, None] if cache.episode is None else torch.cat([cache.episode, current[:, None]], 1)
        visible = (episode == current[:, None])[:, None, :]              # [N, 1, T]
        cos, sin = self._tables(z_prev.device)
        ks, vs = [], []
        for i, block in enumerate(self.blocks):
            q, k, v = block.project(x, cos, sin, position[:, None])
            k = k if cache.k[i] is None else torch.cat([cache.k[i], k], 1)
            v = v if cache.v[i] is None else torch.cat([cache.v[i], v], 1)
            x = block.attend(x, q, k, v, visible)
            ks.append(k), vs.append(v)
        h = self.final(x)[:, 0]
        return h, self._logp(self.prior(h)), TSSMCache(ks, vs, episode, position + 1, current)

    def imagine(self, cache: TSSMCache, z, policy, steps: int, generator=None):
        """Roll the prior forward from latent ``z`` (and the state ``cache`` that produced it): ``policy(feat) -> action``.  Returns the
        features ``[steps, N, deter + stoch * classes]`` and actions ``[steps, N, A]``; ``feat`` of the first imagined step needs the
        ``h`` that came with ``z``, so the caller passes ``policy`` a closure over it for step 0 (``h`` is returned by ``step``)."""
        feats, actions = [], []
        no = torch.zeros(z.shape[0], dtype=torch.bool, device=z.device)
        h = None
        a = policy(None, z)
        for _ in range(steps):
            h, prior, cache = self.step(cache, z, a, no)
            z = self.draw(prior, generator)
            feats.append(torch.cat([h, z], -1))
            a = policy(h, z)
            actions.append(a)
        return torch.stack(feats), torch.stack(actions)
