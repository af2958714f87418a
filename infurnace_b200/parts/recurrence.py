"""The HGRN2 mixer: a gated linear recurrence with a matrix state per head in the request's state slot."""
from __future__ import annotations

import torch

from ..config.specs import GatedRecurrenceSpec
from .registry import register_part


class GatedRecurrence:
    """h -> o_proj(norm(S^T q)) with S <- diag(f) S + (1 - f) v^T per head.

    The three projections run as one product against their row-wise concatenation (exact) into float32, because
    everything that enters the recurrence is 32-bit.  One kernel then applies silu to q and the gate formula to f,
    walks this step's tokens of every request in order from the state its slot holds (zero when the slot was
    granted), writes the state back and normalises each head's output.  A whole prompt, a portion and a single
    decoded token are the same call: the state carries what came before."""

    graph_safe = True     # launches depend on the step's sizes only

    def __init__(self, spec: GatedRecurrenceSpec, weights, runtime):
        self.spec = spec
        self.rt = runtime
        self.k = runtime.kernels
        self.w_qfv = torch.cat((weights[spec.q_proj], weights[spec.f_proj], weights[spec.v_proj]), dim=0).contiguous()
        self.w_o = weights[spec.o_proj]
        self.bias, self.lower, self.norm_w = weights[spec.f_bias], weights[spec.lower], weights[spec.out_norm]
        self.hd = spec.num_heads * spec.head_dim
        self.hv = spec.num_heads * spec.value_head_dim
        slabs = getattr(self.k, "gated_scan_slabs", None)
        self.slabs = slabs(spec.head_dim, spec.value_head_dim) if slabs else 1

    def forward(self, h, ctx, call):
        s, k = self.spec, self.k
        n = h.shape[0]
        proj = ctx.buffer("gr_proj", (n, 2 * self.hd + self.hv), torch.float32)
        k.linear(h, self.w_qfv, proj)
        out = ctx.buffer("gr_out", (n, self.hv), self.rt.act_dtype)
        raw = ctx.buffer("gr_raw", (n, self.hv), torch.float32) if self.slabs > 1 else None
        k.gated_scan(proj, 0, self.hd, 2 * self.hd, self.bias, self.lower, self.norm_w, s.eps, ctx.state(call.cache),
                     ctx.state_slots, ctx.cu_q, ctx.seq_lens, out, s.num_heads, s.head_dim, s.value_head_dim, raw=raw,
                     max_q_len=ctx.max_q_len)
        delta = ctx.buffer("delta_mixer", (n, s.hidden_size), torch.float32)
        k.linear(out, self.w_o, delta)
        return delta


register_part(GatedRecurrenceSpec, GatedRecurrence)
