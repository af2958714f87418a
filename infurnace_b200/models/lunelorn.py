"""Lunelorn: the plan builder (configuration -> layers, order, tensor names).

A decoder over a float32 residual stream with a norm before and after every sublayer.  The embedding is
normalised.  A layer is x += post1(mixer(pre1(x))), x += post2(ffn(pre2(x))), then a per-layer token input.  Three
mixers, in any order given by config.json's ``layers``: ``retention`` (linear attention with a fixed decay per
head), ``parallel`` (softmax attention with rotary positions on keys and values beside a minGRU recurrence) and
``wkv`` (RWKV-style time mixing).  The feed-forward is a mixture of gated experts.  A range of layers may run
several times in a row with the same weights, each pass with cache entries of its own; before a pass the
embedding's rows (from the second pass on) and a per-pass vector are added to the stream.  A final norm, an untied
head and a soft cap on the logits follow.  Tensor names: ``embed``, ``embed.norm``, ``loop.step``, ``side.embed``,
``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.gate|up|down``,
``l<i>.side.gate|proj|norm``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.lunelorn import PARALLEL, RETENTION, LunelornConfig
from ..config.specs import (
    GatedUnitSpec, LayerCall, LMHeadSpec, ModelPlan, NormedEmbeddingSpec, ParallelMixerSpec, RetentionSpec, RMSNormSpec,
    RotarySpec, RotaryValueAttentionSpec, RoutedExpertsSpec, SandwichBlockSpec, StreamInjectSpec, TimeMixSpec, TokenSideSpec,
)
from .registry import register_architecture

MAX_POSITIONS = 1 << 20        # rotary positions have no end; block tables need one
EXPERT_ACTIVATION = "silu"
SIDE_ACTIVATION = "gelu_tanh"


def _mixer(kind, m, p, W, eps):
    if kind == RETENTION:
        return RetentionSpec(hidden_size=W, num_heads=m["heads"], head_dim=m["dim"], value_head_dim=m["vdim"],
                             decay=tuple(float(x) for x in m["decay"]), key_scale=float(m["dim"]) ** -0.5, eps=eps,
                             q_proj=p + "q", k_proj=p + "k", v_proj=p + "v", g_proj=p + "g", o_proj=p + "o")
    if kind == PARALLEL:
        left, right = m["left"], m["right"]
        lp, rp = p + "left.", p + "right."
        base = float(left["rot"]["base"])
        attention = RotaryValueAttentionSpec(
            hidden_size=W, num_heads=left["heads"], num_kv_heads=left["kv_heads"], head_dim=left["dim"],
            value_head_dim=left["vdim"], scale=float(left["scale"]), eps=eps, q_proj=lp + "q", k_proj=lp + "k", v_proj=lp + "v",
            o_proj=lp + "o", position=RotarySpec(left["dim"], int(left["rot"]["dims"]), base),
            value_norm=True, value_position=RotarySpec(left["vdim"], left["vdim"], base))
        unit = GatedUnitSpec(hidden_size=W, width=right["width"], z_proj=rp + "z", z_bias=rp + "z.b", x_proj=rp + "x",
                             x_bias=rp + "x.b", g_proj=rp + "g", o_proj=rp + "o")
        return ParallelMixerSpec((attention, unit), (float(m["left_scale"]), float(m["right_scale"])))
    return TimeMixSpec(hidden_size=W, num_heads=m["heads"], head_dim=m["dim"], eps=eps,
                       mu=tuple(p + "mu." + s for s in "rkvgw"), r_proj=p + "r", k_proj=p + "k", v_proj=p + "v", g_proj=p + "g",
                       w1=p + "w1", w2=p + "w2", w0=p + "w0", bonus=p + "u", out_norm=p + "norm", o_proj=p + "o",
                       rank=m.get("rank"))


def build_lunelorn_plan(cfg: LunelornConfig) -> ModelPlan:
    W, eps, V = cfg.hidden_size, cfg.norm_eps, cfg.vocab_size
    n = len(cfg.layers)
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        mlp = layer["mlp"]
        ffn = ffn_norm = ffn_post = None
        unused = ()
        if mlp is not None:
            ep = p + "mlp."
            ffn = RoutedExpertsSpec(W, mlp["expert"]["ff"], mlp["router"]["top"], EXPERT_ACTIVATION, ep + "router",
                                    tuple((f"{ep}e{j}.gate", f"{ep}e{j}.up", f"{ep}e{j}.down")
                                          for j in range(mlp["router"]["experts"])))
            ffn_norm, ffn_post = RMSNormSpec(W, eps, p + "norm2"), RMSNormSpec(W, eps, p + "norm2b")
        else:
            unused = (p + "norm2", p + "norm2b")
        side = None
        if cfg.token_side_dim is not None:
            sd = cfg.token_side_dim
            side = TokenSideSpec(W, sd, V, "side.embed", n * sd, i * sd, SIDE_ACTIVATION, p + "side.gate", p + "side.proj",
                                 RMSNormSpec(W, eps, p + "side.norm"))
        layers.append(SandwichBlockSpec(W, RMSNormSpec(W, eps, p + "norm1"), _mixer(layer["type"], layer["mixer"], p + "mix.", W, eps),
                                        RMSNormSpec(W, eps, p + "norm1b"), ffn_norm, ffn, ffn_post, side, unused))
    # the order: layers before the loop, the loop's passes (each opened by an injection step), the rest
    loop = cfg.loop
    schedule = []
    looped = loop is not None and loop.stop > loop.start
    times = loop.times if looped else 0
    for i in range(loop.start if looped else n):
        schedule.append(LayerCall(i))
    for t in range(times):
        layers.append(StreamInjectSpec(W, "loop.step", times, t, add_embedding=t > 0))
        schedule.append(LayerCall(len(layers) - 1))
        schedule.extend(LayerCall(i) for i in range(loop.start, loop.stop))
    if looped:
        schedule.extend(LayerCall(i) for i in range(loop.stop, n))
    return ModelPlan(
        architecture=cfg.architecture,
        vocab_size=V,
        hidden_size=W,
        max_positions=MAX_POSITIONS,
        # a loop over an empty range runs nothing; its per-pass table may still be stored
        embedding=NormedEmbeddingSpec(V, W, "embed", RMSNormSpec(W, eps, "embed.norm"), keep=times > 1,
                                      unused=("loop.step",) if loop is not None and not looped else ()),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=RMSNormSpec(W, eps, "final.norm"),
        lm_head=LMHeadSpec(V, W, "head", tied=False, softcap=cfg.logit_softcap),
    )


register_architecture("Lunelorn", LunelornConfig, build_lunelorn_plan)
