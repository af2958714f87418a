"""Attention over the paged cache whose heads' scores are mixed before the softmax."""
from __future__ import annotations

import torch

from ..config.specs import TalkingAttentionSpec
from .registry import register_part


class TalkingAttention:
    """h -> o_proj(sigmoid(G h) * attention(q, K, V)).

    q | k | (v) | (gate) run as one product against their row-wise concatenation into float32.  One kernel
    normalises the whole q and the whole k of a token (one statistic each over all heads), writes q in the
    cache's dtype and stores the normalised k as the key and the raw k (or v) as the value at the token's
    place in the pages.  The attention kernel reads every key from the pages, this step's included, so a
    prompt cut anywhere sees the same keys; positions enter through the distance bias and the chunk rule,
    both counted from the start of the sequence."""

    graph_safe = True     # launches depend on the step's sizes only

    def __init__(self, spec: TalkingAttentionSpec, weights, runtime):
        self.spec = spec
        self.rt = runtime
        self.k = runtime.kernels
        self.qw = spec.num_heads * spec.head_dim
        self.kw = spec.num_kv_heads * spec.head_dim
        rows = [weights[spec.q_proj], weights[spec.k_proj]]
        self.v_col = self.gate_col = -1
        width = self.qw + self.kw
        if spec.v_proj is not None:
            rows.append(weights[spec.v_proj])
            self.v_col, width = width, width + self.kw
        if spec.gate is not None:
            rows.append(weights[spec.gate])
            self.gate_col, width = width, width + self.qw
        self.width = width
        self.w_all = torch.cat(rows, dim=0).contiguous()
        self.w_o = weights[spec.o_proj]
        self.q_norm_w = weights[spec.q_norm] if spec.q_norm is not None else None
        self.k_norm_w = weights[spec.k_norm] if spec.k_norm is not None else None
        self.talk = weights[spec.talk] if spec.talk is not None else None

    def forward(self, h, ctx, call):
        s, k = self.spec, self.k
        n = h.shape[0]
        proj = ctx.buffer("ta_proj", (n, self.width), torch.float32)
        k.linear(h, self.w_all, proj)
        kv = ctx.kv(call.cache)
        q = ctx.buffer("ta_q", (n, self.qw), self.rt.act_dtype)
        k.wide_norm_store(proj, self.qw, self.kw, self.v_col, s.head_dim, self.q_norm_w, self.k_norm_w, s.eps, q,
                          kv.slot_mapping if call.store else None, kv.pages)
        out = ctx.buffer("ta_out", (n, self.qw), self.rt.act_dtype)
        k.attention_talk(q, s.num_heads, s.num_kv_heads, s.head_dim, kv.pages, kv.block_tables, ctx.cu_q, ctx.seq_lens, out,
                         s.scale, chunk=s.chunk or 0, slope_exponent=s.slope_exponent or 0.0, talk=self.talk,
                         gate=proj if self.gate_col >= 0 else None, gate_col=max(self.gate_col, 0), max_q_len=ctx.max_q_len,
                         max_seq_len=ctx.max_seq_len)
        delta = ctx.buffer("delta_mixer", (n, s.hidden_size), torch.float32)
        k.linear(out, self.w_o, delta)
        return delta


register_part(TalkingAttentionSpec, TalkingAttention)
