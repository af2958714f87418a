"""Tiny Kafunex configurations and model folders with weights drawn here (not by the package), shaped so that
a fault shows: the query norm weights are scaled up (peaked attention: a wrong, missing or stale key moves the
logits), the forget gates' lower bounds spread over (0, 1) (short and long memories), the head-mixing matrix is
far from the identity, and the layer scales are of size one (every sublayer counts)."""
from __future__ import annotations

import json
import os

import torch


def _attn(heads, kv, dim, scale, chunk, ff):
    m = {"dim": dim, "heads": heads, "kv_heads": kv, "scale": scale, "vdim": dim}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    return {"type": "attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _rec(heads, dim, vdim, ff):
    return {"type": "hgrn2", "mixer": {"dim": dim, "heads": heads, "vdim": vdim},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _config(vocab, width, eps, layers):
    return {"architecture": "Kafunex", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}


TINY = {
    # recurrence first; two chunk sizes (one smaller than a page, neither a multiple of one); a layer without feed-forward
    "K1": dict(config=_config(97, 48, 1e-5, [_rec(2, 8, 12, 40), _attn(4, 2, 16, 0.25, 24, 56), _rec(3, 16, 8, None),
                                              _attn(2, 1, 8, 0.4, 7, 24)]),
               page_size=16, store="float32", seed=5),
    # as many key heads as query heads; no chunk rule on the first layer; one recurrence head; an odd vdim; dims that
    # are no power of two; a chunk of exactly four pages; feed-forwards narrower than the stream
    "K2": dict(config=_config(61, 40, 1e-6, [_attn(6, 6, 8, 0.35, None, 24), _rec(1, 24, 40, 32), _attn(3, 1, 24, 0.2, 32, None),
                                              _rec(2, 40, 33, 16)]),
               page_size=8, store="bfloat16", seed=6),
    # wider: the tensor-core products see k of 256 and 192; a long chunk
    "K3": dict(config=_config(331, 256, 1e-5, [_attn(8, 2, 32, 0.18, 100, 192), _rec(4, 64, 64, 192), _rec(2, 32, 128, None),
                                                _attn(4, 4, 64, 0.125, 48, 320)]),
               page_size=16, store="bfloat16", seed=7),
}


def make_weights(cfg, seed, sharpen=3.0):
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def mat(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * (gain / i ** 0.5)

    def near_one(*shape, spread=0.2):
        return 1.0 + spread * torch.randn(tuple(shape), generator=g)

    w = {"embed": torch.randn(cfg["vocab"], W, generator=g), "head": mat(cfg["vocab"], W), "final.norm": near_one()}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        w[p + "norm1"], w[p + "ls1"] = near_one(), near_one(W)
        if layer["type"] == "attention":
            qw, kw = m["heads"] * m["dim"], m["kv_heads"] * m["dim"]
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.g"] = mat(qw, W), mat(kw, W), mat(qw, W)
            w[p + "mix.q.norm"] = sharpen * near_one(qw)
            w[p + "mix.k.norm"] = near_one(kw)
            w[p + "mix.talk"] = torch.eye(m["heads"]) + 0.5 * torch.randn(m["heads"], m["heads"], generator=g)
            w[p + "mix.o"] = mat(W, qw)
        else:
            hd, hv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            w[p + "mix.q"], w[p + "mix.f"], w[p + "mix.v"] = mat(hd, W), mat(hd, W, 2.0), mat(hv, W)
            w[p + "mix.f.b"] = torch.randn(hd, generator=g)
            w[p + "mix.lower"] = 0.05 + 0.9 * torch.rand(hd, generator=g)
            w[p + "mix.norm"] = near_one(m["vdim"])
            w[p + "mix.o"] = mat(W, hv)
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            w[p + "norm2"], w[p + "ls2"] = near_one(), near_one(W)
            w[p + "mlp.up"], w[p + "mlp.down"] = mat(ff, W), mat(W, ff)
    return w


def make_model_dir(name, root):
    """Write tiny model ``name`` under ``root`` (config.json, model.safetensors) and return the folder.  The values
    are rounded to the storage dtype before they are written, so the oracle and the engine read the same numbers."""
    from safetensors.torch import save_file
    spec = TINY[name]
    d = os.path.join(root, f"tiny{name}")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(spec["config"], f)
    dt = getattr(torch, spec["store"])
    save_file({k: v.to(dt).contiguous() for k, v in make_weights(spec["config"], spec["seed"]).items()},
              os.path.join(d, "model.safetensors"))
    return d


def another_arrangement():
    """(plan, weights, tokens, logits written out in float64) of a one-layer model put together from the same part
    descriptions in another way: a plain embedding, attention with a value projection of its own and nothing else
    (no norms, no mixing of heads, no gate, no distance bias, no chunk rule), a gelu feed-forward, post-norm block."""
    import math
    from infurnace_b200.config.specs import (DenseMLPSpec, EmbeddingSpec, LayerCall, LMHeadSpec, ModelPlan, PostNormBlockSpec,
                                             ScalarRMSNormSpec, TalkingAttentionSpec)
    W, H, G, d, V, F, T = 24, 4, 2, 8, 40, 24, 21
    g = torch.Generator().manual_seed(4)
    bf = lambda t: t.to(torch.bfloat16).float()          # values a bfloat16 engine holds exactly
    w = {"emb": bf(torch.randn(V, W, generator=g)), "q": bf(torch.randn(H * d, W, generator=g) / 3),
         "k": bf(torch.randn(G * d, W, generator=g) / 3), "v": bf(torch.randn(G * d, W, generator=g) / 3),
         "o": bf(torch.randn(W, H * d, generator=g) / 3), "n1": bf(torch.tensor(1.2)), "s1": bf(1 + 0.2 * torch.randn(W, generator=g)),
         "up": bf(torch.randn(F, W, generator=g) / 3), "down": bf(torch.randn(W, F, generator=g) / 3), "n2": bf(torch.tensor(0.8)),
         "s2": bf(1 + 0.2 * torch.randn(W, generator=g)), "nf": bf(torch.tensor(1.1)), "head": bf(torch.randn(V, W, generator=g) / 3)}
    attn = TalkingAttentionSpec(hidden_size=W, num_heads=H, num_kv_heads=G, head_dim=d, scale=0.7, eps=1e-5, q_proj="q", k_proj="k",
                                o_proj="o", v_proj="v", slope_exponent=None)
    block = PostNormBlockSpec(W, attn, ScalarRMSNormSpec(1e-5, "n1"), "s1", DenseMLPSpec(W, F, "gelu_tanh", "up", "down"),
                              ScalarRMSNormSpec(1e-5, "n2"), "s2")
    plan = ModelPlan("other", V, W, 256, EmbeddingSpec(V, W, "emb"), (block,), (LayerCall(0),), ScalarRMSNormSpec(1e-5, "nf"),
                     LMHeadSpec(V, W, "head", tied=False))
    toks = [int(t) for t in torch.randint(0, V, (T,), generator=g)]
    D = torch.float64

    def rms(t):
        return t / torch.sqrt(t.pow(2).mean(-1, keepdim=True) + 1e-5)

    x = w["emb"].to(D)[torch.tensor(toks)]
    q, k, v = (x @ w[n].to(D).t() for n in ("q", "k", "v"))
    q, k, v = q.view(T, H, d), k.view(T, G, d).repeat_interleave(H // G, 1), v.view(T, G, d).repeat_interleave(H // G, 1)
    a = torch.einsum("thd,shd->hts", q, k) * 0.7
    a = a.masked_fill(~torch.tril(torch.ones(T, T, dtype=torch.bool))[None], float("-inf"))
    y = torch.einsum("hts,shd->thd", torch.softmax(a, -1), v).reshape(T, H * d) @ w["o"].to(D).t()
    x = x + rms(y) * w["n1"].to(D) * w["s1"].to(D)
    z = x @ w["up"].to(D).t()
    y = (0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))) @ w["down"].to(D).t()
    x = x + rms(y) * w["n2"].to(D) * w["s2"].to(D)
    return plan, w, toks, (rms(x) * w["nf"].to(D)) @ w["head"].to(D).t()
