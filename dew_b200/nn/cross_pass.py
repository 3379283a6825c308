"""Cross-pass messages: a looped decoder's passes coupled through the block summaries the pass before left.  Under ``Loop(messages=n)``
every pass enters the looped block at the prelude's output, the block's layers are cut into blocks of ``n`` (the last shorter where
they do not divide), each pass leaves each block's residual summary in a bank ``[B, S, blocks, D]``, and every sub-layer input of a
later pass merges that bank in before its norm - one ``CrossPassMerge`` per input site.  The first pass reads no bank, so it is the
decoder's own forward; with the gates drawn at zero every later pass is the first again, so a pretrained decoder gains passes without
changing what it computes.  A merge:

    m      = rms_normed(depth_attention(bank))                    the passes' message, at unit RMS
    sigma  = sqrt(mean(u^2) + eps),  u_hat = u / sigma            the sub-layer input u, at unit RMS
    h      = u_hat W_u + m W_m                                    a rank-r controller state
    forget = tanh(h W_f),  gain = tanh(h W_g),  add = tanh(h W_a)
    out    = (1 - forget) u + sigma (gain m + add)

in fp32 whatever the run computes in, cast back to ``u``'s dtype.  ``depth_attention`` is a softmax over the bank's blocks by one learned
pseudo-query per site (a zero query averages them).

Reference: src/dew/nn/cross_pass.py.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .layers import declare


class CrossPassMerge(nn.Module):
    def __init__(self, features: int, rank: int = 16, eps: float = 1e-6, additive: bool = True, dtype=None, device=None):
        super().__init__()
        self.eps, self.additive = eps, additive
        kw = dict(dtype=torch.float32, device=device)
        self.query = declare(nn.Parameter(torch.zeros(features, **kw)), ("embed",), "kernel")
        self.w_u = declare(nn.Parameter(torch.empty(features, rank, **kw)), ("embed", None), "kernel")
        self.w_m = declare(nn.Parameter(torch.empty(features, rank, **kw)), ("embed", None), "kernel")
        # forget | gain | add: drawn at zero, so the merge starts as the identity
        self.w_out = declare(nn.Parameter(torch.zeros(rank, (3 if additive else 2) * features, **kw)), (None, "embed"), "kernel")
        with torch.no_grad():
            self.w_u.normal_(0.0, features ** -0.5)
            self.w_m.normal_(0.0, features ** -0.5)

    def message(self, bank: torch.Tensor) -> torch.Tensor:
        b = bank.float()
        k = b * torch.rsqrt(b.pow(2).mean(-1, keepdim=True) + self.eps)
        m = (torch.softmax(k @ self.query, -1).unsqueeze(-1) * b).sum(-2)
        return m * torch.rsqrt(m.pow(2).mean(-1, keepdim=True) + self.eps)

    def forward(self, u: torch.Tensor, bank: torch.Tensor) -> torch.Tensor:
        uf = u.float()
        sigma = torch.sqrt(uf.pow(2).mean(-1, keepdim=True) + self.eps)
        m = self.message(bank)
        h = (uf / sigma) @ self.w_u + m @ self.w_m
        parts = torch.tanh(h @ self.w_out).chunk(3 if self.additive else 2, -1)
        out = (1 - parts[0]) * uf + sigma * (parts[1] * m + (parts[2] if self.additive else 0.0))
        return out.to(u.dtype)
