"""Multi-stream residual connections: hyper-connections and AltUp.  Both keep several copies of the residual stream and
replace ``h <- h + f(norm(h))`` by a learned read (what the layer sees) and a learned write (how its output and the old
streams form the new streams).

``HyperConnections`` (n streams): read ``x = sum_i alpha_i H_i``; write ``H'_j = sum_i A_ij H_i + beta_j f(x)``.  The static
weights start as the plain residual rotated over the streams (stream ``layer % n`` is read, every stream keeps itself and
receives the output), and the dynamic part adds ``tanh``-bounded, input-dependent corrections computed from the normalised
streams (initialised to zero, so training starts from the static form).
``AltUp`` (K blocks): predict every block from all blocks (``P`` [K x K], identity at start), run the layer on ONE block
(``layer % K``), and correct every block by its gate times the layer's innovation on the active block.

A stack of either with one stream / block reduces to the ordinary pre-norm residual stack.
Reference: ``hyper_connections`` and ``altup`` fields of src/dew/nn/backbones/causal_transformer.py:165-423.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class HyperConnections(nn.Module):
    def __init__(self, features: int, streams: int, layer_index: int, dynamic: bool = True, dtype=None, device=None):
        super().__init__()
        n = streams
        self.n, self.dynamic = n, dynamic
        read = torch.zeros(n)
        read[layer_index % n] = 1.0
        self.alpha = nn.Parameter(read.to(device=device))                       # read weights
        self.mix = nn.Parameter(torch.eye(n, device=device))                    # A: stream i -> stream j
        self.beta = nn.Parameter(torch.ones(n, device=device))                  # write weights
        if dynamic:
            self.norm_weight = nn.Parameter(torch.ones(features, dtype=dtype, device=device))
            self.dyn_alpha = nn.Linear(features, 1, bias=False, dtype=dtype, device=device)
            self.dyn_beta = nn.Linear(features, 1, bias=False, dtype=dtype, device=device)
            self.dyn_mix = nn.Linear(features, n, bias=False, dtype=dtype, device=device)
            self.scale = nn.Parameter(torch.full((3,), 0.01, device=device))
            for lin in (self.dyn_alpha, self.dyn_beta, self.dyn_mix):
                nn.init.zeros_(lin.weight)

    def weights(self, H: torch.Tensor):
        """H ``[B,S,n,d]`` -> alpha ``[B,S,n]``, A ``[B,S,n,n]``, beta ``[B,S,n]`` (static weights plus the dynamic corrections)."""
        B, S, n, d = H.shape
        alpha, mix, beta = self.alpha.float().expand(B, S, n), self.mix.float().expand(B, S, n, n), self.beta.float().expand(B, S, n)
        if self.dynamic:
            hn = F.rms_norm(H.float(), (d,), self.norm_weight.float())
            alpha = alpha + self.scale[0] * torch.tanh(self.dyn_alpha(hn.to(self.dyn_alpha.weight.dtype)).float().squeeze(-1))
            beta = beta + self.scale[1] * torch.tanh(self.dyn_beta(hn.to(self.dyn_beta.weight.dtype)).float().squeeze(-1))
            mix = mix + self.scale[2] * torch.tanh(self.dyn_mix(hn.to(self.dyn_mix.weight.dtype)).float())
        return alpha, mix, beta

    def read(self, H: torch.Tensor):
        alpha, mix, beta = self.weights(H)
        x = torch.einsum("bsn,bsnd->bsd", alpha.to(H.dtype), H)
        return x, (mix, beta)

    def write(self, H: torch.Tensor, out: torch.Tensor, ctx) -> torch.Tensor:
        mix, beta = ctx
        return torch.einsum("bsij,bsid->bsjd", mix.to(H.dtype), H) + beta.to(H.dtype).unsqueeze(-1) * out.unsqueeze(2)


class AltUp(nn.Module):
    def __init__(self, blocks: int, layer_index: int, device=None):
        super().__init__()
        self.k, self.active = blocks, layer_index % blocks
        self.predict = nn.Parameter(torch.eye(blocks, device=device))
        self.gate = nn.Parameter(torch.ones(blocks, device=device))

    def read(self, H: torch.Tensor):
        """H ``[B,S,K,d]``: predicted blocks, and the active one as the layer's input."""
        pred = torch.einsum("ij,bsid->bsjd", self.predict.to(H.dtype), H)
        return pred[:, :, self.active], pred

    def write(self, H: torch.Tensor, out: torch.Tensor, pred: torch.Tensor) -> torch.Tensor:
        """``out`` is the layer's branch output on the active block: its innovation ``(x + out) - x`` corrects every block."""
        return pred + self.gate.to(H.dtype).view(1, 1, -1, 1) * out.unsqueeze(2)


def expand_streams(h: torch.Tensor, n: int) -> torch.Tensor:
    """``[B,S,d] -> [B,S,n,d]``: every stream starts as the embedding."""
    return h.unsqueeze(2).expand(-1, -1, n, -1).contiguous()


def collapse_streams(H: torch.Tensor) -> torch.Tensor:
    """``[B,S,n,d] -> [B,S,d]``: the streams are summed (hyper-connections) / averaged by the caller as needed."""
    return H.sum(2)
