"""Several mixers side by side on one input."""
from __future__ import annotations

import torch

from ..config.specs import LayerCall, ParallelMixerSpec
from .registry import build_part, register_part


class WeightedSum:
    """The results of mixers that ran side by side, not yet added up: ``terms`` = [(float32 tensor, scale), ...].  A
    block whose stream update can form the sum in its own pass asks for this (``weighted=True``)."""
    __slots__ = ("terms",)

    def __init__(self, terms):
        self.terms = terms


class ParallelMixer:
    """h -> sum_i scales[i] * mixers[i](h).  Mixer i keeps cache entry ``(call.cache, i)``.  The weighted sum is one
    small kernel per mixer over their float32 results, unless the caller takes a :class:`WeightedSum` of two."""

    can_return_weighted = True

    def __init__(self, spec: ParallelMixerSpec, weights, runtime):
        self.spec = spec
        self.rt = runtime
        self.k = runtime.kernels
        self.mixers = [build_part(m, weights, runtime) for m in spec.mixers]

    @property
    def graph_safe(self):
        return all(getattr(m, "graph_safe", False) for m in self.mixers)

    def forward(self, h, ctx, call, weighted=False):
        results = [mixer.forward(h, ctx, LayerCall(call.layer, (call.cache, i), call.store)) for i, mixer in enumerate(self.mixers)]
        if weighted and len(results) == 2 and results[0].data_ptr() != results[1].data_ptr():
            return WeightedSum(list(zip(results, self.spec.scales)))
        total = None
        for d, scale in zip(results, self.spec.scales):
            if total is None:
                total = ctx.buffer("delta_parallel", d.shape, torch.float32)
                self.k.scaled_sum(total, d, scale, accumulate=False)
            else:
                self.k.scaled_sum(total, d, scale, accumulate=True)
        return total


register_part(ParallelMixerSpec, ParallelMixer)
