"""The Lunelorn decoder stated plainly: one function per mechanism, float64, whole sequences, token-by-token
loops for everything recurrent, no cache and no code of the package.  ``forward(cfg, weights, tokens)`` takes the
config.json mapping, a mapping from tensor name to tensor and one sequence of token ids, and returns the logits
of every position; ``layer_outputs`` is filled with the residual stream after every layer run.

Notation: h is a sublayer's input [T, W]; matrices are stored [out, in] and applied as h @ M.T.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def rotate_pairs(x, positions, base, dims, interleaved=False):
    """Turn the first ``dims`` entries of the last axis of x [T, heads, d]: pair m of dims/2 by the angle
    position * base^(-2m/dims).  Pairs are (m, m + dims/2), or (2m, 2m + 1) when interleaved.  A negative
    position turns the other way."""
    half = dims // 2
    m = torch.arange(half, dtype=F)
    ang = positions.to(F)[:, None] * base ** (-2.0 * m / dims)[None, :]          # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    if interleaved:
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    else:
        a, b = x[..., :half], x[..., half:dims]
        out[..., :half] = a * c - b * s
        out[..., half:dims] = b * c + a * s
    return out


# ------------------------------------------------------------------------------------------------ mixers
def retention(h, w, p, m, eps):
    """Linear attention with one fixed decay per head and no softmax: S <- decay S + k v^T, o = S^T q."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, H, d) * d ** -0.5
    v = (h @ w[p + "v"].T).view(T, H, dv)
    decay = torch.tensor(m["decay"], dtype=F)
    S = torch.zeros(H, d, dv, dtype=F)
    o = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms(o, eps).reshape(T, H * dv) * silu(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def rotary_attention(h, w, p, m, eps):
    """Grouped-query softmax attention, rotary positions on part of q and k, values normalised per head and
    rotated by their position over their whole width, the summed output rotated back by the query's position."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    base, dims = float(m["rot"]["base"]), int(m["rot"]["dims"])
    pos = torch.arange(T)
    q = rotate_pairs((h @ w[p + "q"].T).view(T, H, d), pos, base, dims)
    k = rotate_pairs((h @ w[p + "k"].T).view(T, G, d), pos, base, dims)
    v = rotate_pairs(rms((h @ w[p + "v"].T).view(T, G, dv), eps), pos, base, dv)
    out = torch.zeros(T, H, dv, dtype=F)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(torch.ones(T, T, dtype=torch.bool).triu(1), float("-inf"))
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, g]
    out = rotate_pairs(out, -pos, base, dv)
    return out.reshape(T, H * dv) @ w[p + "o"].T


def min_gru(h, w, p, m):
    """A gated recurrence whose gates read only the current token, element by element."""
    T, n = h.shape[0], m["width"]
    z = torch.sigmoid(h @ w[p + "z"].T + w[p + "z.b"])
    u = h @ w[p + "x"].T + w[p + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    S = torch.zeros(n, dtype=F)
    out = torch.zeros(T, n, dtype=F)
    for t in range(T):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        out[t] = S
    return (out * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def parallel(h, w, p, m, eps):
    return m["left_scale"] * rotary_attention(h, w, p + "left.", m["left"], eps) \
        + m["right_scale"] * min_gru(h, w, p + "right.", m["right"])


def wkv(h, w, p, m, eps):
    """RWKV-style time mixing: every projection reads its own blend of the token and the one before it; the
    decay is per token, head and key channel; the current token enters its own output through a bonus."""
    T, W = h.shape
    H, d = m["heads"], m["dim"]
    prev = torch.cat((torch.zeros(1, W, dtype=F), h[:-1]), dim=0)
    mix = {s: h + (prev - h) * w[p + "mu." + s] for s in "rkvgw"}
    r = (mix["r"] @ w[p + "r"].T).view(T, H, d)
    k = (mix["k"] @ w[p + "k"].T).view(T, H, d)
    v = (mix["v"] @ w[p + "v"].T).view(T, H, d)
    gate = silu(mix["g"] @ w[p + "g"].T)
    dec = torch.exp(-torch.exp(torch.tanh(mix["w"] @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).view(T, H, d)
    u = w[p + "u"].view(H, d)
    S = torch.zeros(H, d, d, dtype=F)
    o = torch.zeros(T, H, d, dtype=F)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S + u[:, :, None] * kv, r[t])
        S = dec[t][:, :, None] * S + kv
    o = rms(o, eps).reshape(T, H * d) * w[p + "norm"] * gate
    return o @ w[p + "o"].T


# ------------------------------------------------------------------------------------------------ feed-forward
def moe(h, w, p, mlp):
    """Each token runs its ``top`` experts with the largest router logits, weighted by the softmax over those."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    logits = h @ w[p + "router"].T
    val, idx = torch.topk(logits, top, dim=-1)
    gate = torch.softmax(val, dim=-1)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for j in range(top):
            e = f"{p}e{int(idx[t, j])}."
            a = silu(h[t] @ w[e + "gate"].T) * (h[t] @ w[e + "up"].T)
            out[t] += gate[t, j] * (a @ w[e + "down"].T)
    return out


# ------------------------------------------------------------------------------------------------ the model
def run_layer(x, i, layer, w, tokens, cfg):
    eps = cfg["norm"]["eps"]
    p = f"l{i}."
    h = rms(x, eps) * w[p + "norm1"]
    kind, m = layer["type"], layer["mixer"]
    if kind == "retention":
        y = retention(h, w, p + "mix.", m, eps)
    elif kind == "parallel":
        y = parallel(h, w, p + "mix.", m, eps)
    elif kind == "wkv":
        y = wkv(h, w, p + "mix.", m, eps)
    else:
        raise ValueError(kind)
    x = x + rms(y, eps) * w[p + "norm1b"]
    if layer.get("mlp") is not None:
        y = moe(rms(x, eps) * w[p + "norm2"], w, p + "mlp.", layer["mlp"])
        x = x + rms(y, eps) * w[p + "norm2b"]
    side = cfg.get("token_side")
    if side:
        sd = side["dim"]
        e = w["side.embed"][tokens][:, i * sd:(i + 1) * sd]
        y = (gelu_tanh(x @ w[p + "side.gate"].T) * e) @ w[p + "side.proj"].T
        x = x + rms(y, eps) * w[p + "side.norm"]
    return x


def forward(cfg, weights, tokens, layer_outputs=None):
    w = {k: v.to(F) if v.is_floating_point() else v for k, v in weights.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = cfg["norm"]["eps"]
    x = rms(w["embed"][tokens], eps) * w["embed.norm"]
    emb = x
    layers = cfg["layers"]
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    order = []                                   # (layer index, pass number or None, first of its pass)
    for i in range(loop["start"]):
        order.append((i, None, False))
    for t in range(loop["times"] if loop["stop"] > loop["start"] else 0):
        for i in range(loop["start"], loop["stop"]):
            order.append((i, t, i == loop["start"]))
    for i in range(max(loop["stop"], loop["start"]), len(layers)):
        order.append((i, None, False))
    for i, t, first in order:
        if first:
            if t > 0:
                x = x + emb
            x = x + w["loop.step"][t]
        x = run_layer(x, i, layers[i], w, tokens, cfg)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    logits = (rms(x, eps) * w["final.norm"]) @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits


def greedy(cfg, weights, prompt, max_tokens):
    """The tokens greedy decoding appends to ``prompt`` (the whole sequence is recomputed for every token)."""
    toks, out = list(prompt), []
    for _ in range(max_tokens):
        nxt = int(torch.argmax(forward(cfg, weights, toks)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
