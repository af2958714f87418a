"""Embedding, LM head, and the decoder that runs the layers in the schedule's order."""
from __future__ import annotations

import torch

from ..config.specs import EmbeddingSpec, LMHeadSpec, ModelPlan, NormedEmbeddingSpec, SinusoidEmbeddingSpec
from .registry import build_part, register_part


class Embedding:
    """x[t] = table[id_t], widened to float32, no scaling
    (src/infurnace/executor/tinygrad/model.py:95)."""

    def __init__(self, spec: EmbeddingSpec, weights, runtime):
        self.spec = spec
        self.table = weights[spec.weight]
        self.k = runtime.kernels

    def forward(self, ids, out):
        self.k.embed(self.table, ids, out)
        return out


class LMHead:
    """logits = h @ W^T in float32 (model.py:151); W is the embedding table when tied
    (src/infurnace/executor/tinygrad/weights.py:68), read in place."""

    def __init__(self, spec: LMHeadSpec, weights, runtime):
        self.spec = spec
        self.weight = weights[spec.weight]
        self.k = runtime.kernels

    def forward(self, h, out):
        self.k.linear(h, self.weight, out)
        if self.spec.softcap:                  # c * tanh(logits / c), in place
            self.k.softcap(out, float(self.spec.softcap))
        return out


class SinusoidEmbedding:
    """x[t] = table[id_t] + e(p_t) in float32, with e[2i] = sin(p * base^(-2i/width)) and e[2i+1] = the cosine of
    the same angle; p_t is the token's position in its sequence.  It takes the step's context (``uses_context``)
    for the positions, and in bfloat16 mode leaves a bfloat16 copy of the rows for the first layer's products
    (``ctx.shared[STREAM_COPY]``)."""

    uses_context = True

    def __init__(self, spec: SinusoidEmbeddingSpec, weights, runtime):
        self.spec = spec
        self.rt = runtime
        self.table = weights[spec.weight]
        self.k = runtime.kernels
        i = torch.arange((spec.hidden_size + 1) // 2, dtype=torch.float64)
        self.inv_freq = torch.pow(torch.tensor(float(spec.base), dtype=torch.float64),
                                  -2.0 * i / spec.hidden_size).to(runtime.device)

    def forward(self, ids, out, ctx=None):
        half = None
        if self.rt.act_dtype == torch.bfloat16:
            half = ctx.buffer("stream_copy", out.shape, torch.bfloat16)
            ctx.shared[STREAM_COPY] = half
        self.k.embed_sinusoid(self.table, ids, ctx.positions, self.inv_freq, out, half)
        return out


class NormedEmbedding:
    """x[t] = norm(table[id_t]) in float32: the gather writes a scratch buffer and the norm kernel writes the stream.
    With ``keep`` the rows are also copied to a buffer of the step (``ctx.shared[EMBEDDING_ROWS]``) for a later part
    that adds them to the stream again."""

    uses_context = True

    def __init__(self, spec: NormedEmbeddingSpec, weights, runtime):
        self.spec = spec
        self.table = weights[spec.weight]
        self.norm = build_part(spec.norm, weights, runtime)
        self.k = runtime.kernels

    def forward(self, ids, out, ctx=None):
        raw = ctx.buffer("embed_raw", out.shape, torch.float32)
        self.k.embed(self.table, ids, raw)
        self.norm.forward(raw, out)
        if self.spec.keep:
            kept = ctx.buffer("embed_kept", out.shape, torch.float32)
            self.k.add_rows(kept, out, None, accumulate=False)
            ctx.shared[EMBEDDING_ROWS] = kept
        return out


# key of ``ctx.shared`` under which the embedding's rows are kept for the step
EMBEDDING_ROWS = ("embedding_rows",)

# key of ``ctx.shared`` under which a bfloat16 copy of the current residual stream is handed from the part that wrote the
# stream last (an embedding, a block's residual update) to the part that reads it next
STREAM_COPY = ("stream_copy",)

register_part(EmbeddingSpec, Embedding)
register_part(SinusoidEmbeddingSpec, SinusoidEmbedding)
register_part(LMHeadSpec, LMHead)
register_part(NormedEmbeddingSpec, NormedEmbedding)


class DecoderModel:
    """The parts of a :class:`ModelPlan`, built once, and ``forward(ctx)``: the tokens of
    one step through every layer call of the schedule, then the final norm and the head on
    the rows whose logits are wanted (model.py:150-151 does so for the last row)."""

    def __init__(self, plan: ModelPlan, weights, runtime):
        self.plan = plan
        self.rt = runtime
        self.embedding = build_part(plan.embedding, weights, runtime)
        self.layers = [build_part(spec, weights, runtime) for spec in plan.layers]
        self.schedule = plan.resolved_schedule()
        self.final_norm = build_part(plan.final_norm, weights, runtime)
        self.lm_head = build_part(plan.lm_head, weights, runtime)

    @property
    def graph_safe(self) -> bool:
        """True when every layer's launches depend only on the sizes of a step, so that a
        decode step may be recorded once and replayed (a part says so with ``graph_safe``)."""
        return all(getattr(layer, "graph_safe", False) for layer in self.layers)

    def forward(self, ctx):
        n = ctx.num_tokens
        x = ctx.buffer("x", (n, self.plan.hidden_size), torch.float32)
        if getattr(self.embedding, "uses_context", False):
            self.embedding.forward(ctx.token_ids, x, ctx=ctx)
        else:
            self.embedding.forward(ctx.token_ids, x)
        pending = None
        for i, call in enumerate(self.schedule):
            layer = self.layers[call.layer]
            nxt = self.layers[self.schedule[i + 1].layer] if i + 1 < len(self.schedule) else None
            if getattr(layer, "folds_norms", False) and getattr(nxt, "folds_norms", False):
                pending = layer.forward(x, pending, ctx, call, next_layer=nxt)     # may hand over a folded norm
            elif getattr(layer, "hands_over_input", False) and getattr(nxt, "hands_over_input", False):
                pending = layer.forward(x, pending, ctx, call, next_layer=nxt)     # may hand over the next block's input
            else:
                pending = layer.forward(x, pending, ctx, call)
        m = ctx.num_logit_rows
        if m == 0:
            return None
        hn = ctx.buffer("h_final", (m, self.plan.hidden_size), self.rt.act_dtype, rows=m)
        self.final_norm.forward(x, hn, delta=pending, rows=ctx.logit_rows)
        logits = ctx.buffer("logits", (m, self.plan.vocab_size), torch.float32, rows=m)
        self.lm_head.forward(hn, logits)
        return logits
