"""A plain, slow statement of the Kafunex decoder in float64/float32 torch on the CPU, for tests only.

One function per mechanism, whole sequences, no cache, token-by-token loops where the
mechanism is a recurrence.  It shares no code with the package: it takes a configuration as the
nested dict of config.json and the weights as a name -> tensor dict.

Notation.  t, s: positions (from 0).  W: width.  For a layer L its tensors are "l<L>.<...>".
"""
from __future__ import annotations

import math

import torch

DT = torch.float64


def position_vector(positions, width):
    """e[t, 2i] = sin(t * 10000^(-2i/W)), e[t, 2i+1] = cos(same angle)."""
    t = torch.as_tensor(positions, dtype=DT)[:, None]
    i = torch.arange((width + 1) // 2, dtype=DT)[None, :]
    ang = t * torch.pow(torch.tensor(10000.0, dtype=DT), -2.0 * i / width)
    e = torch.zeros(t.shape[0], 2 * ((width + 1) // 2), dtype=DT)
    e[:, 0::2] = ang.sin()
    e[:, 1::2] = ang.cos()
    return e[:, :width]


def rms(v, eps):
    """v / sqrt(mean(v^2) + eps) over the last axis."""
    return v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def hgrn2(h, w, p, m, eps, state=None):
    """The gated linear recurrence.  h: [T, W].  Per head a matrix S [dim, vdim], S_0 = 0:
    f_t = lo + (1 - lo) * sigmoid(F h_t + b);  S_t = f_t[:, None] * S_{t-1} + (1 - f_t)[:, None] * v_t[None, :];
    o_t = S_t^T q_t with q_t = silu(Q h_t).  Each head's o is divided by its root mean square over vdim and
    multiplied by n[vdim]; the heads side by side go through O."""
    H, d, e = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = torch.nn.functional.silu(h @ w[p + "q"].to(DT).t()).view(T, H, d)
    f = torch.sigmoid(h @ w[p + "f"].to(DT).t() + w[p + "f.b"].to(DT))
    lo = w[p + "lower"].to(DT)
    f = (lo + (1 - lo) * f).view(T, H, d)
    v = (h @ w[p + "v"].to(DT).t()).view(T, H, e)
    S = torch.zeros(H, d, e, dtype=DT) if state is None else state
    out = torch.zeros(T, H, e, dtype=DT)
    for t in range(T):
        S = f[t][:, :, None] * S + (1 - f[t])[:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hde,hd->he", S, q[t])
    out = rms(out, eps) * w[p + "norm"].to(DT)
    return out.reshape(T, H * e) @ w[p + "o"].to(DT).t(), S


def head_slopes(H):
    return torch.tensor([2.0 ** (-8.0 * (j + 1) / H) for j in range(H)], dtype=DT)


def attention(h, w, p, m, eps, first_position=0):
    """Chunk-local softmax attention whose values are the unnormalised keys.
    q = Q h, k = K h; qn = rms over ALL of q's entries (one statistic per token) times a weight of that
    length, kn likewise; values are k itself.  a[j, t, s] = scale * qn_j(t) . kn_g(s) - slope_j * (t - s),
    g = j // (H/G); b[j] = sum_i M[j, i] a[i];  visible: s <= t and s // C == t // C;
    o_j(t) = sum_s softmax_s(b[j, t, :]) k_g(s); the heads side by side are multiplied by sigmoid(Gate h) and go through O."""
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    T = h.shape[0]
    q = h @ w[p + "q"].to(DT).t()
    k = h @ w[p + "k"].to(DT).t()
    qn = (rms(q, eps) * w[p + "q.norm"].to(DT)).view(T, H, d)
    kn = (rms(k, eps) * w[p + "k.norm"].to(DT)).view(T, G, d)
    val = k.view(T, G, d)
    rep = H // G
    pos = torch.arange(first_position, first_position + T)
    a = torch.einsum("thd,shd->hts", qn, kn.repeat_interleave(rep, dim=1)) * m["scale"]
    dist = (pos[:, None] - pos[None, :]).to(DT)
    a = a - head_slopes(H)[:, None, None] * dist[None]
    b = torch.einsum("ji,its->jts", w[p + "talk"].to(DT), a)
    vis = pos[None, :] <= pos[:, None]
    size = (m.get("mask") or {}).get("size")
    if size:
        vis &= (pos[None, :] // size) == (pos[:, None] // size)
    b = b.masked_fill(~vis[None], float("-inf"))
    pr = torch.softmax(b, dim=-1)
    o = torch.einsum("hts,shd->thd", pr, val.repeat_interleave(rep, dim=1)).reshape(T, H * d)
    o = o * torch.sigmoid(h @ w[p + "g"].to(DT).t())
    return o @ w[p + "o"].to(DT).t()


def feed_forward(h, w, p):
    """D (relu(U h))^2."""
    return torch.relu(h @ w[p + "up"].to(DT).t()).pow(2) @ w[p + "down"].to(DT).t()


def scalar_norm(v, g, eps):
    """rms(v) times one number."""
    return rms(v, eps) * g.to(DT)


def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of a whole sequence (float64), and the residual stream after every layer."""
    W, eps = cfg["width"], cfg["norm"]["eps"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"].to(DT)[ids] + position_vector(range(len(ids)), W)
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        if layer["type"] == "hgrn2":
            y, _ = hgrn2(x, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "attention":
            y = attention(x, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + scalar_norm(y, w[p + "norm1"], eps) * w[p + "ls1"].to(DT)
        if layer.get("mlp") is not None:
            y = feed_forward(x, w, p + "mlp.")
            x = x + scalar_norm(y, w[p + "norm2"], eps) * w[p + "ls2"].to(DT)
        after.append(x.clone())
    logits = scalar_norm(x, w["final.norm"], eps) @ w["head"].to(DT).t()
    if return_layers:
        return logits, torch.stack(after)
    return logits


def read_model(model_dir):
    """(config.json as a dict, name -> tensor) of a model folder."""
    import json
    import os
    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, load_file(os.path.join(model_dir, "model.safetensors"))


def greedy(cfg, w, prompt, n):
    """n tokens by argmax (lowest index among equals), recomputing the whole sequence each time."""
    toks = list(prompt)
    out = []
    for _ in range(n):
        nxt = int(torch.argmax(forward(cfg, w, toks)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
