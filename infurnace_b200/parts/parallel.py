"""Several mixers side by side on one input."""
from __future__ import annotations

import torch

from ..config.specs import LayerCall, ParallelMixerSpec
from .registry import build_part, register_part


class ParallelMixer:
    """h -> sum_i scales[i] * mixers[i](h).  Mixer i keeps cache entry ``(call.cache, i)``.  The weighted sum is one
    small kernel over the mixers' float32 results."""

    def __init__(self, spec: ParallelMixerSpec, weights, runtime):
        self.spec = spec
        self.rt = runtime
        self.k = runtime.kernels
        self.mixers = [build_part(m, weights, runtime) for m in spec.mixers]

    @property
    def graph_safe(self):
        return all(getattr(m, "graph_safe", False) for m in self.mixers)

    def forward(self, h, ctx, call):
        n = h.shape[0]
        total = None
        for i, (mixer, scale) in enumerate(zip(self.mixers, self.spec.scales)):
            d = mixer.forward(h, ctx, LayerCall(call.layer, (call.cache, i), call.store))
            if total is None:
                total = ctx.buffer("delta_parallel", d.shape, torch.float32)
                self.k.scaled_sum(total, d, scale, accumulate=False)
            else:
                self.k.scaled_sum(total, d, scale, accumulate=True)
        return total


register_part(ParallelMixerSpec, ParallelMixer)
