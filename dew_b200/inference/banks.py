"""Parameter banks for generation with a decoder that does not fit the GPU: the layers' weights live in pinned host memory
and stream through a few device-resident slots, one layer at a time, while the previous layer computes.

``HostBanks(model.layers, device, slots=2)`` moves every layer's parameters to pinned host tensors and keeps ``slots`` device
copies of one layer's parameter set.  A forward pre-hook points layer ``i``'s parameters at its slot once the copy stream has
delivered them; a forward hook records that the slot is free and starts the copy of layer ``i + slots`` (wrapping to the
next call's first layers, so a decode loop keeps streaming) on a side stream.  With two slots the host->device copy of the
next layer overlaps the current layer's kernels; PCIe / C2C bandwidth then bounds a decode step at
``layer bytes / link bandwidth`` per layer.  Everything outside the stacked layers (embedding, head, norms) stays resident.

Reference: src/dew/inference/banks.py (``LayerBanks``, ``HeldBanks``, host-resident banks fetched a layer at a time by
``run_stack``), ``Layout.host_parameters`` (src/dew/distributed/placement.py).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch
import torch.nn as nn


def _signature(layer: nn.Module):
    return tuple((n, tuple(p.shape), p.dtype) for n, p in layer.named_parameters())


class HostBanks:
    def __init__(self, layers: Sequence[nn.Module], device, slots: int = 2):
        self.layers = list(layers)
        self.device = torch.device(device)
        L = len(self.layers)
        if L == 0:
            raise ValueError("no layers to bank")
        sigs = {_signature(l) for l in self.layers}
        if len(sigs) != 1:
            raise ValueError("the banked layers must share one parameter signature (same names, shapes and dtypes): bank each "
                             "run of identical layers by itself")
        slots = max(1, min(slots, L))
        while L % slots:                       # layer j always lands in slot j % slots, also across the wrap to the next call
            slots -= 1
        self.slots = slots
        self.cuda = self.device.type == "cuda"
        self.copy_stream = torch.cuda.Stream(self.device) if self.cuda else None
        names = [n for n, _ in self.layers[0].named_parameters()]
        # host copies (pinned where possible), device parameters released
        self.host: List[Dict[str, torch.Tensor]] = []
        for layer in self.layers:
            held = {}
            for n, p in layer.named_parameters():
                t = p.detach().to("cpu").contiguous()
                if self.cuda:
                    t = t.pin_memory()
                held[n] = t
                p.requires_grad_(False)
                p.data = torch.empty(0, dtype=p.dtype, device=self.device)
            self.host.append(held)
        proto = self.host[0]
        self.slot_tensors = [{n: torch.empty_like(proto[n], device=self.device) for n in names} for _ in range(slots)]
        self.resident: List[Optional[int]] = [None] * slots              # which layer each slot holds (or is receiving)
        self.copied = [torch.cuda.Event() if self.cuda else None for _ in range(slots)]
        self.freed = [torch.cuda.Event() if self.cuda else None for _ in range(slots)]
        self.bytes_per_layer = sum(t.numel() * t.element_size() for t in proto.values())
        self.copies = 0
        self._handles = []
        for i, layer in enumerate(self.layers):
            self._handles.append(layer.register_forward_pre_hook(lambda m, a, i=i: self._enter(i)))
            self._handles.append(layer.register_forward_hook(lambda m, a, out, i=i: self._leave(i)))
        for i in range(slots):
            self._fetch(i, first=True)

    # ------------------------------------------------------------------ copies
    def _fetch(self, layer: int, first: bool = False) -> None:
        slot = layer % self.slots
        if self.resident[slot] == layer:
            return
        self.resident[slot] = layer
        self.copies += 1
        if self.cuda:
            with torch.cuda.stream(self.copy_stream):
                if not first:
                    self.copy_stream.wait_event(self.freed[slot])        # the slot's previous layer has finished computing
                for n, t in self.host[layer].items():
                    self.slot_tensors[slot][n].copy_(t, non_blocking=True)
                self.copied[slot].record(self.copy_stream)
        else:
            for n, t in self.host[layer].items():
                self.slot_tensors[slot][n].copy_(t)

    def _enter(self, i: int) -> None:
        slot = i % self.slots
        if self.resident[slot] != i:               # not prefetched (first call after a reset, or a layer called out of order)
            if self.cuda:
                self.freed[slot].record(torch.cuda.current_stream(self.device))
            self._fetch(i)
        if self.cuda:
            torch.cuda.current_stream(self.device).wait_event(self.copied[slot])
        for n, p in self.layers[i].named_parameters():
            p.data = self.slot_tensors[slot][n]

    def _leave(self, i: int) -> None:
        slot = i % self.slots
        if self.cuda:
            self.freed[slot].record(torch.cuda.current_stream(self.device))
        for _, p in self.layers[i].named_parameters():
            p.data = torch.empty(0, dtype=p.dtype, device=self.device)
        self._fetch((i + self.slots) % len(self.layers))

    # ------------------------------------------------------------------ housekeeping
    def device_bytes(self) -> int:
        return self.slots * self.bytes_per_layer

    def host_bytes(self) -> int:
        return len(self.layers) * self.bytes_per_layer

    def load(self, layer: int, tensors: Dict[str, torch.Tensor]) -> None:
        """Replace one layer's host weights (a weight reload); the slot that holds it, if any, is fetched again."""
        for n, t in tensors.items():
            self.host[layer][n].copy_(t)
        slot = layer % self.slots
        if self.resident[slot] == layer:
            self.resident[slot] = None
            self._fetch(layer, first=not self.cuda)

    def release(self) -> None:
        """Undo the banking: every layer gets its own device parameters back and the hooks go away."""
        for h in self._handles:
            h.remove()
        if self.cuda:
            torch.cuda.synchronize(self.device)
        for layer, held in zip(self.layers, self.host):
            for n, p in layer.named_parameters():
                p.data = held[n].to(self.device)
