"""Kafunex: the plan builder (configuration -> layers, order, tensor names).

A post-norm decoder over a float32 residual stream.  The embedding adds a sinusoidal position
vector.  Every layer is x += ls1 * norm1(mixer(x)), then, if it has a feed-forward,
x += ls2 * norm2(ff(x)), where the norms have one number as weight and ls1 / ls2 are per-feature
vectors.  The mixer is either the HGRN2 recurrence (state slots) or chunk-local attention whose
values are its unnormalised keys, with a distance bias, the heads' scores mixed before the softmax,
and a sigmoid gate on the output (paged cache).  The feed-forward is down(relu(up(x))^2).  A final
one-number norm and an untied head follow.  Tensor names: ``embed``, ``l<i>.norm1|norm2|ls1|ls2``,
``l<i>.mix.*``, ``l<i>.mlp.up|down``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.kafunex import ATTENTION, KafunexConfig
from ..config.specs import (
    DenseMLPSpec, GatedRecurrenceSpec, LayerCall, LMHeadSpec, ModelPlan, PostNormBlockSpec, ScalarRMSNormSpec,
    SinusoidEmbeddingSpec, TalkingAttentionSpec,
)
from .registry import register_architecture

POSITION_BASE = 10000.0        # e[2i] = sin(p * base^(-2i/width))
SLOPE_EXPONENT = 8.0           # slope of head j of H: 2^(-8 (j + 1) / H)
MAX_POSITIONS = 1 << 20        # the position vector has no end; block tables need one


def build_kafunex_plan(cfg: KafunexConfig) -> ModelPlan:
    W, eps = cfg.hidden_size, cfg.norm_eps
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = p + "mix."
        if layer.type == ATTENTION:
            mixer = TalkingAttentionSpec(
                hidden_size=W, num_heads=layer.heads, num_kv_heads=layer.kv_heads, head_dim=layer.dim, scale=layer.scale,
                eps=eps, q_proj=m + "q", k_proj=m + "k", o_proj=m + "o", v_proj=None, q_norm=m + "q.norm",
                k_norm=m + "k.norm", talk=m + "talk", gate=m + "g", chunk=layer.chunk, slope_exponent=SLOPE_EXPONENT)
        else:
            mixer = GatedRecurrenceSpec(
                hidden_size=W, num_heads=layer.heads, head_dim=layer.dim, value_head_dim=layer.vdim, eps=eps,
                q_proj=m + "q", f_proj=m + "f", f_bias=m + "f.b", lower=m + "lower", v_proj=m + "v", out_norm=m + "norm",
                o_proj=m + "o")
        ffn = ffn_norm = ffn_scale = None
        if layer.mlp is not None:
            ffn = DenseMLPSpec(W, layer.mlp.ff, "relu2", p + "mlp.up", p + "mlp.down")
            ffn_norm, ffn_scale = ScalarRMSNormSpec(eps, p + "norm2"), p + "ls2"
        layers.append(PostNormBlockSpec(W, mixer, ScalarRMSNormSpec(eps, p + "norm1"), p + "ls1", ffn, ffn_norm, ffn_scale))
    return ModelPlan(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab_size,
        hidden_size=W,
        max_positions=MAX_POSITIONS,
        embedding=SinusoidEmbeddingSpec(cfg.vocab_size, W, "embed", POSITION_BASE),
        layers=tuple(layers),
        schedule=tuple(LayerCall(i) for i in range(len(layers))),
        final_norm=ScalarRMSNormSpec(eps, "final.norm"),
        lm_head=LMHeadSpec(cfg.vocab_size, W, "head", tied=False),
    )


register_architecture("Kafunex", KafunexConfig, build_kafunex_plan)
