"""Autoregressive text generation: ``Sampling`` (logits transforms), ``generate``, strategies (sample, beam,
speculative) and stopping.

Parity: src/dew/sampling/text.py (``Sampling`` :137-175, ``generate`` :1076-1083 -> ``Generation(tokens, lengths,
terminated, text)``), src/dew/sampling/decoding.py (logits transforms, stopping), src/dew/sampling/strategies.py
(``Sample``, ``Beam``, ``Speculative``).  Per-row keys: row ``i``'s draws come from ``fold_in(key, i)`` folded with the
step, so a row's continuation does not depend on which rows share its batch.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, List, Optional, Sequence, Tuple

import torch

from ..nn.kv_cache import KVCache, KVStore
from ..utils import keys as K


@dataclass(frozen=True)
class Sampling:
    temperature: float = 1.0
    top_k: Optional[int] = None
    eos_token_ids: Optional[Sequence[int]] = None
    pad_token_id: Optional[int] = None
    top_p: float = 1.0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    no_repeat_ngram_size: int = 0
    min_new_tokens: int = 0
    typical_p: float = 1.0
    stop: Sequence[str] = ()

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0 or self.top_k == 1


@dataclass
class Generation:
    tokens: torch.Tensor            # [rows, prompt + new] padded with pad id
    lengths: torch.Tensor           # [rows] total length of each row
    terminated: torch.Tensor        # [rows] bool: ended on an EOS / stop rather than the token budget
    text: Optional[List[str]] = None
    prompt_lengths: Optional[torch.Tensor] = None

    def new_tokens(self, row: int) -> torch.Tensor:
        return self.tokens[row, int(self.prompt_lengths[row]): int(self.lengths[row])]


def transform_logits(logits: torch.Tensor, history: torch.Tensor, history_len: torch.Tensor, s: Sampling, new_count: int) -> torch.Tensor:
    """Apply the ``Sampling`` transforms to ``logits [R, V]`` given each row's token ``history [R, L]`` (first
    ``history_len[r]`` entries valid)."""
    R, V = logits.shape
    x = logits.float().clone()
    valid = torch.arange(history.shape[1], device=x.device)[None] < history_len[:, None]
    if s.repetition_penalty != 1.0 or s.presence_penalty or s.frequency_penalty:
        counts = torch.zeros(R, V, device=x.device)
        counts.scatter_add_(1, history.clamp(0, V - 1), valid.float())
        seen = counts > 0
        if s.repetition_penalty != 1.0:
            x = torch.where(seen, torch.where(x > 0, x / s.repetition_penalty, x * s.repetition_penalty), x)
        x = x - s.presence_penalty * seen.float() - s.frequency_penalty * counts
    if s.no_repeat_ngram_size > 0:
        n = s.no_repeat_ngram_size
        for r in range(R):
            L = int(history_len[r])
            if L + 1 < n:
                continue
            h = history[r, :L].tolist()
            prefix = tuple(h[L - n + 1:]) if n > 1 else ()
            for i in range(L - n + 1):
                if tuple(h[i:i + n - 1]) == prefix:
                    x[r, h[i + n - 1]] = float("-inf")
    if s.eos_token_ids and new_count < s.min_new_tokens:
        x[:, list(s.eos_token_ids)] = float("-inf")
    if s.greedy:
        return x
    x = x / max(s.temperature, 1e-6)
    if s.top_k is not None and s.top_k < V:
        kth = torch.topk(x, s.top_k, dim=-1).values[:, -1:]
        x = x.masked_fill(x < kth, float("-inf"))
    if s.min_p > 0:
        p = torch.softmax(x, -1)
        x = x.masked_fill(p < s.min_p * p.max(-1, keepdim=True).values, float("-inf"))
    if s.typical_p < 1.0:
        logp = torch.log_softmax(x, -1)
        p = logp.exp()
        ent = -(p * torch.where(p > 0, logp, torch.zeros_like(logp))).sum(-1, keepdim=True)
        dev = (ent + logp).abs()
        order = dev.argsort(-1)
        cp = p.gather(-1, order).cumsum(-1)
        drop_sorted = cp - p.gather(-1, order) >= s.typical_p
        drop = torch.zeros_like(drop_sorted).scatter(-1, order, drop_sorted)
        x = x.masked_fill(drop, float("-inf"))
    if s.top_p < 1.0:
        sp, order = torch.sort(torch.softmax(x, -1), descending=True, dim=-1)
        drop_sorted = sp.cumsum(-1) - sp >= s.top_p
        drop = torch.zeros_like(drop_sorted).scatter(-1, order, drop_sorted)
        x = x.masked_fill(drop, float("-inf"))
    return x


def plain_filters(s: Sampling) -> bool:
    """True when only temperature / top-k / min-p / top-p shape the distribution (what the sampling kernel does itself)."""
    return (s.repetition_penalty == 1.0 and not s.presence_penalty and not s.frequency_penalty and s.no_repeat_ngram_size == 0
            and s.typical_p >= 1.0 and not (s.eos_token_ids and s.min_new_tokens > 0))


def row_uniforms(row_keys: Sequence[int], step: int) -> torch.Tensor:
    """One uniform number per row from the row's keyed generator (the same keys the multinomial draws use)."""
    return torch.stack([torch.rand(1, generator=K.generator(K.fold_in(k, step), "cpu"))[0] for k in row_keys])


def draw(logits: torch.Tensor, s: Sampling, row_keys: Sequence[int], step: int) -> torch.Tensor:
    """Draw from already transformed logits.  On a GPU: the argmax / inverse-CDF kernels (no per-row host round trip)."""
    if logits.is_cuda:
        from ..ops import sample as S
        if S.kernel_ok(logits):
            if s.greedy:
                return S.argmax_rows(logits)
            return S.sample_rows(logits, row_uniforms(row_keys, step))
    if s.greedy:
        return logits.argmax(-1)
    p = torch.softmax(logits, -1)
    out = torch.empty(p.shape[0], dtype=torch.long, device=p.device)
    for r, k in enumerate(row_keys):
        g = K.generator(K.fold_in(k, step), "cpu")
        out[r] = torch.multinomial(p[r].cpu(), 1, generator=g)[0]
    return out


# ---------------------------------------------------------------------------------------------------------------


def _prefill(model, params_call, tokens, lengths, store: KVStore):
    """Run the prompts (right-padded) through the model, filling the cache; returns last-position logits ``[R, V]``."""
    R, S = tokens.shape
    pos = torch.arange(S, device=tokens.device)[None].expand(R, S).clone()
    pos[pos >= lengths[:, None]] = -1
    logits = params_call(tokens, positions=pos, cache=store)
    last = (lengths - 1).clamp_min(0)
    return logits[torch.arange(R, device=tokens.device), last]


def make_cache(model, rows: int, max_len: int, spec: Optional[KVCache] = None, device=None, dtype=None) -> KVStore:
    cfg = model.config
    hd = cfg.head_dim or cfg.emb_features // cfg.num_heads
    p = next(model.parameters())
    kvh = getattr(model, "local_kv_heads", None) or (cfg.num_kv_heads or cfg.num_heads)     # this rank's KV heads under TP
    return KVStore(spec or KVCache(), cfg.num_layers, rows, max_len, kvh, hd,
                   dtype or p.dtype, device or p.device)


def generate(model, params, inputs, max_new_tokens: int, *, key: int = 0, sampling: Sampling = Sampling(), n: int = 1,
             logits: Optional[Callable] = None, stopping: Optional[Callable] = None, strategy: Any = None,
             tokenizer=None, kv_cache: Optional[KVCache] = None, prefix=None, progress=None) -> Generation:
    """Generate continuations of ``inputs`` (a list of token-id lists, a padded tensor with ``lengths``, or strings when
    ``tokenizer`` is given).  ``params`` is a variable tree or ``None`` for the model's own parameters."""
    if strategy is not None and not isinstance(strategy, Sample):
        return strategy.run(model, params, inputs, max_new_tokens, key=key, sampling=sampling, tokenizer=tokenizer)
    dev = next(model.parameters()).device
    if isinstance(inputs, (list, tuple)) and inputs and isinstance(inputs[0], str):
        assert tokenizer is not None, "string prompts need a tokenizer"
        inputs = [tokenizer.encode(t) for t in inputs]
    if isinstance(inputs, torch.Tensor):
        prompts = [row.tolist() for row in inputs]
    else:
        prompts = [list(p) for p in inputs]
    if n > 1:
        prompts = [p for p in prompts for _ in range(n)]
    R = len(prompts)
    plen = torch.tensor([len(p) for p in prompts], device=dev)
    S = int(plen.max())
    pad = sampling.pad_token_id if sampling.pad_token_id is not None else 0
    total = S + max_new_tokens
    tokens = torch.full((R, total), pad, dtype=torch.long, device=dev)
    for r, p in enumerate(prompts):
        tokens[r, :len(p)] = torch.tensor(p, device=dev)

    if params is None:
        call = lambda t, **kw: model(t, **kw)
    else:
        from ..utils.trees import variables_for_call
        named = variables_for_call(model, params)
        call = lambda t, **kw: torch.func.functional_call(model, named, (t,), kw)

    store = make_cache(model, R, total, kv_cache)
    row_keys = [K.fold_in(K.key(key), r) for r in range(R)]
    eos = set(sampling.eos_token_ids or ())
    lengths = plen.clone()
    done = torch.zeros(R, dtype=torch.bool, device=dev)
    terminated = torch.zeros(R, dtype=torch.bool, device=dev)
    with torch.no_grad():
        step_logits = _prefill(model, call, tokens[:, :S], plen, store)
        for step in range(max_new_tokens):
            x = logits(step_logits, tokens, lengths) if logits is not None else step_logits
            x = transform_logits(x, tokens, lengths, sampling, step)
            nxt = draw(x, sampling, row_keys, step)
            nxt = torch.where(done, torch.full_like(nxt, pad), nxt)
            tokens[torch.arange(R, device=dev), lengths.clamp_max(total - 1)] = torch.where(done, tokens[torch.arange(R, device=dev), lengths.clamp_max(total - 1)], nxt)
            hit = torch.tensor([int(t) in eos for t in nxt.tolist()], device=dev) & ~done if eos else torch.zeros_like(done)
            lengths = lengths + (~done).long()
            terminated |= hit
            done |= hit
            if stopping is not None:
                stop_now = stopping(tokens, lengths)
                terminated |= stop_now & ~done
                done |= stop_now
            if sampling.stop and tokenizer is not None:
                for r in range(R):
                    if not bool(done[r]):
                        text = tokenizer.decode(tokens[r, int(plen[r]):int(lengths[r])].tolist())
                        if any(s in text for s in sampling.stop):
                            done[r] = True
                            terminated[r] = True
            if bool(done.all()) or step == max_new_tokens - 1:
                break
            pos = torch.where(done, torch.full_like(lengths, -1), lengths - 1)
            step_logits = call(nxt[:, None], positions=pos[:, None], cache=store)[:, 0]
    text = None
    if tokenizer is not None:
        text = [tokenizer.decode(tokens[r, int(plen[r]):int(lengths[r])].tolist()) for r in range(R)]
    return Generation(tokens, lengths, terminated, text, plen)


# ---------------------------------------------------------------------------------------------------------------
# strategies


@dataclass
class Sample:
    """Plain ancestral sampling (the default strategy)."""


@dataclass
class Beam:
    """Beam search by cumulative log-probability with length penalty."""
    beams: int = 4
    length_penalty: float = 1.0

    def run(self, model, params, inputs, max_new_tokens, *, key=0, sampling=Sampling(), tokenizer=None) -> Generation:
        dev = next(model.parameters()).device
        prompts = [tokenizer.encode(t) for t in inputs] if inputs and isinstance(inputs[0], str) else [list(p) for p in inputs]
        eos = set(sampling.eos_token_ids or ())
        results, lens, term = [], [], []
        call = (lambda t: model(t)) if params is None else (lambda t: torch.func.functional_call(
            model, __import__("dew_b200.utils.trees", fromlist=["variables_for_call"]).variables_for_call(model, params), (t,)))
        with torch.no_grad():
            for p in prompts:
                beams = [(0.0, list(p), False)]
                for _ in range(max_new_tokens):
                    live = [b for b in beams if not b[2]]
                    if not live:
                        break
                    batch = torch.tensor([b[1] for b in live], device=dev)
                    logp = torch.log_softmax(call(batch)[:, -1].float(), -1)
                    cand = [b for b in beams if b[2]]
                    top = torch.topk(logp, self.beams, dim=-1)
                    for i, b in enumerate(live):
                        for lp, tok in zip(top.values[i].tolist(), top.indices[i].tolist()):
                            cand.append((b[0] + lp, b[1] + [tok], tok in eos))
                    score = lambda c: c[0] / (max(1, len(c[1]) - len(p)) ** self.length_penalty)
                    beams = sorted(cand, key=score, reverse=True)[: self.beams]
                best = beams[0]
                results.append(best[1]); lens.append(len(best[1])); term.append(best[2])
        total = max(lens)
        pad = sampling.pad_token_id or 0
        toks = torch.full((len(results), total), pad, dtype=torch.long, device=dev)
        for r, t in enumerate(results):
            toks[r, :len(t)] = torch.tensor(t, device=dev)
        plen = torch.tensor([len(p) for p in prompts], device=dev)
        text = [tokenizer.decode(results[r][len(prompts[r]):]) for r in range(len(results))] if tokenizer else None
        return Generation(toks, torch.tensor(lens, device=dev), torch.tensor(term, device=dev), text, plen)


@dataclass
class Speculative:
    """Greedy speculative decoding: a draft model proposes ``lookahead`` tokens, the target verifies them in one pass
    and keeps the longest agreeing prefix plus its own next token (exact for greedy decoding)."""
    draft: Any = None
    lookahead: int = 4

    def run(self, model, params, inputs, max_new_tokens, *, key=0, sampling=Sampling(), tokenizer=None) -> Generation:
        dev = next(model.parameters()).device
        prompts = [tokenizer.encode(t) for t in inputs] if inputs and isinstance(inputs[0], str) else [list(p) for p in inputs]
        eos = set(sampling.eos_token_ids or ())
        outs, term, accepted, proposed = [], [], 0, 0
        with torch.no_grad():
            for p in prompts:
                seq = list(p)
                ended = False
                while len(seq) - len(p) < max_new_tokens and not ended:
                    d = list(seq)
                    for _ in range(self.lookahead):
                        d.append(int(self.draft(torch.tensor([d], device=dev))[0, -1].argmax()))
                    tgt = model(torch.tensor([d], device=dev))[0].argmax(-1).tolist()
                    keep = 0
                    while keep < self.lookahead and d[len(seq) + keep] == tgt[len(seq) + keep - 1]:
                        keep += 1
                    proposed += self.lookahead
                    accepted += keep
                    new = d[len(seq): len(seq) + keep] + [tgt[len(seq) + keep - 1]]
                    for t in new:
                        if len(seq) - len(p) >= max_new_tokens:
                            break
                        seq.append(t)
                        if t in eos:
                            ended = True
                            break
                outs.append(seq); term.append(ended)
        total = max(len(o) for o in outs)
        pad = sampling.pad_token_id or 0
        toks = torch.full((len(outs), total), pad, dtype=torch.long, device=dev)
        for r, t in enumerate(outs):
            toks[r, :len(t)] = torch.tensor(t, device=dev)
        plen = torch.tensor([len(p) for p in prompts], device=dev)
        gen = Generation(toks, torch.tensor([len(o) for o in outs], device=dev), torch.tensor(term, device=dev),
                         [tokenizer.decode(o[len(p):]) for o, p in zip(outs, prompts)] if tokenizer else None, plen)
        gen.acceptance = accepted / max(1, proposed)
        return gen


@dataclass
class TreeSpeculative:
    """Greedy speculative decoding over a token tree: the draft proposes the ``branching`` most likely continuations at each
    of ``depth`` levels (a tree of candidates), the target scores every node in ONE pass under a tree attention mask (a node
    attends to the prompt and to its own ancestors only), and the longest root path the target agrees with is kept, plus
    the target's own token after it.  Exact for greedy decoding.  Reference: src/dew/sampling/strategies.py ``TreeSpeculative``,
    src/dew/sampling/trees.py."""
    draft: Any = None
    branching: int = 2
    depth: int = 3

    def _tree(self, seq, dev):
        """Nodes as (token, parent index or -1), level by level, from the draft's top-k at every node."""
        nodes = []
        frontier = [(-1, list(seq))]
        for _ in range(self.depth):
            nxt = []
            for parent, ctx in frontier:
                top = torch.topk(self.draft(torch.tensor([ctx], device=dev))[0, -1].float(), self.branching).indices.tolist()
                for tok in top:
                    nodes.append((tok, parent))
                    nxt.append((len(nodes) - 1, ctx + [tok]))
            frontier = nxt
        return nodes

    @staticmethod
    def tree_mask(prefix_len: int, parents) -> torch.Tensor:
        """Boolean attention mask ``[L, L]`` (True = may attend) for prefix tokens followed by the tree's nodes."""
        n = len(parents)
        L = prefix_len + n
        m = torch.zeros(L, L, dtype=torch.bool)
        m[:prefix_len, :prefix_len] = torch.tril(torch.ones(prefix_len, prefix_len, dtype=torch.bool))
        for i, p in enumerate(parents):
            m[prefix_len + i, :prefix_len] = True
            j = i
            while j >= 0:
                m[prefix_len + i, prefix_len + j] = True
                j = parents[j]
        return m

    def _verify(self, model, seq, nodes, dev):
        """The target's greedy token after the prefix and after every node.  Nodes are scored path by path through the
        model's causal interface (each root path is a causal sequence), batched in one call."""
        paths = []
        for i in range(len(nodes)):
            path, j = [], i
            while j >= 0:
                path.append(nodes[j][0])
                j = nodes[j][1]
            paths.append(list(reversed(path)))
        width = max(len(p) for p in paths) if paths else 0
        rows = [list(seq) + p + [0] * (width - len(p)) for p in paths] or [list(seq)]
        logits = model(torch.tensor(rows, device=dev))
        root_next = int(logits[0, len(seq) - 1].argmax())
        after = [int(logits[i, len(seq) + len(p) - 1].argmax()) for i, p in enumerate(paths)]
        return root_next, after

    def run(self, model, params, inputs, max_new_tokens, *, key=0, sampling=Sampling(), tokenizer=None) -> Generation:
        dev = next(model.parameters()).device
        prompts = [tokenizer.encode(t) for t in inputs] if inputs and isinstance(inputs[0], str) else [list(p) for p in inputs]
        eos = set(sampling.eos_token_ids or ())
        outs, term, accepted, rounds = [], [], 0, 0
        with torch.no_grad():
            for p in prompts:
                seq, ended = list(p), False
                while len(seq) - len(p) < max_new_tokens and not ended:
                    nodes = self._tree(seq, dev)
                    root_next, after = self._verify(model, seq, nodes, dev)
                    # walk down from the root while some child carries the target's token
                    new, parent, want = [], -1, root_next
                    while True:
                        child = next((i for i, (tok, par) in enumerate(nodes) if par == parent and tok == want), None)
                        if child is None:
                            break
                        new.append(want)
                        parent, want = child, after[child]
                    accepted += len(new)
                    rounds += 1
                    new.append(want)
                    for t in new:
                        if len(seq) - len(p) >= max_new_tokens:
                            break
                        seq.append(t)
                        if t in eos:
                            ended = True
                            break
                outs.append(seq); term.append(ended)
        total = max(len(o) for o in outs)
        pad = sampling.pad_token_id or 0
        toks = torch.full((len(outs), total), pad, dtype=torch.long, device=dev)
        for r, t in enumerate(outs):
            toks[r, :len(t)] = torch.tensor(t, device=dev)
        plen = torch.tensor([len(p) for p in prompts], device=dev)
        gen = Generation(toks, torch.tensor([len(o) for o in outs], device=dev), torch.tensor(term, device=dev),
                         [tokenizer.decode(o[len(p):]) for o, p in zip(outs, prompts)] if tokenizer else None, plen)
        gen.accepted_per_round = accepted / max(1, rounds)
        return gen
