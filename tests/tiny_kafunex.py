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
