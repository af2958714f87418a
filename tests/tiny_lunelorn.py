"""Tiny Lunelorn configurations and model folders with weights drawn here (not by the package), shaped so that a
fault shows: query matrices are scaled up (peaked attention: a wrong, missing or stale key moves the logits), decays
spread from short to long memories, blends and bonuses far from 0 and 1, router matrices large enough that the
choice of experts is no close call, and norm weights of size one (every sublayer counts)."""
from __future__ import annotations

import json
import os

import torch


def _moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _ret(heads, dim, vdim, decay, mlp):
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}, "mlp": mlp}


def _par(heads, kv, dim, vdim, rot_dims, base, scale, width, ls, rs, mlp):
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "rot": {"base": base, "dims": rot_dims},
                               "scale": scale}, "left_scale": ls, "right": {"width": width}, "right_scale": rs}, "mlp": mlp}


def _wkv(heads, dim, rank, mlp):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim, "rank": rank}, "mlp": mlp}


def _config(vocab, width, eps, layers, loop=None, side=None, cap=None):
    c = {"architecture": "Lunelorn", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if loop is not None:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    if side is not None:
        c["token_side"] = {"dim": side}
    if cap is not None:
        c["logit_softcap"] = cap
    return c


TINY = {
    # attention first, with keys wider than values and half of a key head rotated; a wkv layer whose heads do not fill the
    # width and that has no feed-forward; the last two layers run three times; every option present
    "L1": dict(config=_config(97, 48, 1e-5, [_par(4, 2, 16, 8, 8, 1000.0, 0.4, 40, 0.8, 1.3, _moe(5, 2, 24)),
                                              _wkv(3, 8, 5, None),
                                              _ret(2, 8, 12, [0.6, 0.97], _moe(4, 1, 16))],
                              loop=(1, 3, 3), side=6, cap=10.0),
               page_size=16, store="float32", seed=11),
    # no loop, no token side input, no soft cap; every expert chosen (top = experts); whole key heads rotated; values
    # wider than keys; one key/value head per query head; pages of 8
    "L2": dict(config=_config(131, 64, 1e-6, [_ret(3, 16, 16, [0.5, 0.9, 0.995], _moe(3, 3, 40)),
                                              _par(6, 6, 8, 16, 8, 50000.0, 0.3, 24, 1.0, 1.0, _moe(6, 2, 8)),
                                              _wkv(2, 32, 4, _moe(2, 1, 32))]),
               page_size=8, store="bfloat16", seed=12),
    # wider: heads of 128 over one key/value head, products with k of 256; the first two layers run twice; one expert of four
    "L3": dict(config=_config(331, 256, 1e-5, [_par(4, 1, 128, 128, 64, 10000.0, 0.09, 96, 1.1, 0.9, _moe(4, 1, 128)),
                                               _ret(4, 64, 64, [0.9, 0.95, 0.98, 0.999], _moe(8, 3, 64)),
                                               _wkv(4, 64, 16, _moe(4, 2, 96))],
                              loop=(0, 2, 2), side=16, cap=30.0),
               page_size=16, store="bfloat16", seed=13),
}


def make_weights(cfg, seed, sharpen=3.0):
    g = torch.Generator().manual_seed(seed)
    W, V, n = cfg["width"], cfg["vocab"], len(cfg["layers"])

    def mat(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * (gain / i ** 0.5)

    def near_one(*shape, spread=0.2):
        return 1.0 + spread * torch.randn(tuple(shape), generator=g)

    w = {"embed": torch.randn(V, W, generator=g), "embed.norm": near_one(W), "head": mat(V, W, 2.0), "final.norm": near_one(W)}
    if cfg.get("loop"):
        w["loop.step"] = 0.5 * torch.randn(cfg["loop"]["times"], W, generator=g)
    side = (cfg.get("token_side") or {}).get("dim")
    if side:
        w["side.embed"] = torch.randn(V, n * side, generator=g)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        w[p + "norm1"], w[p + "norm1b"] = near_one(W), near_one(W)
        if layer["type"] == "retention":
            hd, hv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"] = mat(hd, W), mat(hd, W, 2.0), mat(hv, W)
            w[p + "mix.g"], w[p + "mix.o"] = mat(hv, W, 2.0), mat(W, hv)
        elif layer["type"] == "parallel":
            a, r = m["left"], m["right"]["width"]
            w[p + "mix.left.q"] = mat(a["heads"] * a["dim"], W, sharpen)
            w[p + "mix.left.k"] = mat(a["kv_heads"] * a["dim"], W, sharpen)
            w[p + "mix.left.v"] = mat(a["kv_heads"] * a["vdim"], W)
            w[p + "mix.left.o"] = mat(W, a["heads"] * a["vdim"])
            w[p + "mix.right.z"], w[p + "mix.right.x"], w[p + "mix.right.g"] = mat(r, W, 2.0), mat(r, W, 2.0), mat(r, W, 2.0)
            w[p + "mix.right.z.b"], w[p + "mix.right.x.b"] = torch.randn(r, generator=g), 0.5 * torch.randn(r, generator=g)
            w[p + "mix.right.o"] = mat(W, r)
        else:
            hd, rank = m["heads"] * m["dim"], m["rank"]
            for s in "rkvgw":
                w[p + "mix.mu." + s] = torch.rand(W, generator=g)
            w[p + "mix.r"], w[p + "mix.k"], w[p + "mix.v"], w[p + "mix.g"] = mat(hd, W), mat(hd, W), mat(hd, W), mat(hd, W, 2.0)
            w[p + "mix.w1"], w[p + "mix.w2"] = mat(rank, W, 2.0), mat(hd, rank, 2.0)
            w[p + "mix.w0"] = -1.5 + torch.randn(hd, generator=g)
            w[p + "mix.u"] = 0.5 * torch.randn(m["heads"], m["dim"], generator=g)
            w[p + "mix.norm"] = near_one(hd)
            w[p + "mix.o"] = mat(W, hd)
        if layer["mlp"] is not None:
            e, ff = layer["mlp"]["router"]["experts"], layer["mlp"]["expert"]["ff"]
            w[p + "norm2"], w[p + "norm2b"] = near_one(W), near_one(W)
            w[p + "mlp.router"] = mat(e, W, 3.0)
            for j in range(e):
                w[f"{p}mlp.e{j}.gate"], w[f"{p}mlp.e{j}.up"], w[f"{p}mlp.e{j}.down"] = mat(ff, W, 2.0), mat(ff, W), mat(W, ff)
        if side:
            w[p + "side.gate"], w[p + "side.proj"], w[p + "side.norm"] = mat(side, W, 2.0), mat(W, side), near_one(W)
    return w


def make_model_dir(name, root, config=None, seed=None, store=None):
    """Write tiny model ``name`` under ``root`` (config.json, model.safetensors) and return the folder.  The values
    are rounded to the storage dtype before they are written, so the oracle and the engine read the same numbers."""
    from safetensors.torch import save_file
    spec = TINY.get(name, {})
    config = config or spec["config"]
    d = os.path.join(root, f"tiny{name}")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(config, f)
    dt = getattr(torch, store or spec["store"])
    save_file({k: v.to(dt).contiguous() for k, v in make_weights(config, seed if seed is not None else spec["seed"]).items()},
              os.path.join(d, "model.safetensors"))
    return d


def load_model_dir(d):
    """(config mapping, weights as float64-ready tensors) of a folder written by :func:`make_model_dir`."""
    from safetensors.torch import load_file
    with open(os.path.join(d, "config.json")) as f:
        cfg = json.load(f)
    return cfg, {k: v.float() for k, v in load_file(os.path.join(d, "model.safetensors")).items()}
