"""A plain, slow Zasudra in float64 on the CPU: the oracle of the GPU tests.

One function per mechanism, each written from its equation; whole sequences
only (no cache, no state carried between calls: a position's logits are those of
the whole prefix run at once).  Nothing here is shared with the engine.

Notation: x residual stream [T, W]; n(.) = division by the root mean square with
eps inside the root; positions t = 0 .. T-1; m the residual multiplier.
A layer is  x <- x + m * w1 * n(mixer(x));  x <- x + m * w2 * n(ff(x)):
the sublayers read x itself, the norm sits on their OUTPUT.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_divide(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def bigram_rows(tokens: list, b: dict) -> list:
    """Row of the bigram table for every position: a hash of (previous, current)
    token; the first token of a sequence takes the extra last row."""
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(b["buckets"] if t == 0 else (tokens[t - 1] * b["mul_prev"] + tok * b["mul_cur"]) % b["buckets"])
    return rows


def embed(cfg: dict, w: dict, tokens: list) -> torch.Tensor:
    x = w["embed"][torch.tensor(tokens)]
    b = (cfg.get("embedding") or {}).get("bigram")
    if b:
        x = x + w["bigram"][torch.tensor(bigram_rows(tokens, b))]
    return x


def rotate_interleaved(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, H, D]: coordinate 2i pairs with 2i+1 for i < dims/2; the pair at
    position t turns by the angle t * base^(-2i/dims).  Coordinates >= dims stay."""
    if dims == 0:
        return x
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    ang = positions.to(F64)[:, None, None] * freq[None, None, :]
    even, odd = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = even * torch.cos(ang) - odd * torch.sin(ang)
    out[..., 1:dims:2] = odd * torch.cos(ang) + even * torch.sin(ang)
    return out


def visible_chunked(T: int, size: int) -> torch.Tensor:
    """[T, T] bool: query i sees key j iff j <= i and both lie in the same block of
    ``size`` positions counted from position 0; size 0 = every earlier key."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    vis = j <= i
    if size > 0:
        vis = vis & (i // size == j // size)
    return vis


def softmax_with_sink(s: torch.Tensor, vis: torch.Tensor, sink: float) -> torch.Tensor:
    """Weights exp(s_j) / (exp(sink) + sum_visible exp(s_j)): the sink has no value."""
    s = s.masked_fill(~vis, -math.inf)
    top = torch.clamp(s.max(-1, keepdim=True).values, min=sink)
    e = torch.exp(s - top)
    return e / (e.sum(-1, keepdim=True) + math.exp(sink) * torch.exp(-top))


def projection_norm(y: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm over the WHOLE projection row (all heads at once), then the weight."""
    return rms_divide(y, eps) * weight


def keys_and_values(w: dict, p: str, m: dict, kind: str, h: torch.Tensor, eps: float):
    """The (cached) keys [T, G, D] after norm and rotation and the values [T, G, V] of a layer that owns them."""
    T = h.shape[0]
    G, D = m["kv_heads"], m["dim"]
    k_raw = h @ w[p + "k"].T
    if kind == "attention":
        v = k_raw.view(T, G, D).clone()            # the values are the keys as projected
    else:
        v = (h @ w[p + "v"].T).view(T, G, m.get("vdim") or D)
    k = projection_norm(k_raw, w[p + "k.norm"], eps).view(T, G, D)
    rot = m.get("rot")
    if kind == "attention" and rot:
        k = rotate_interleaved(k, torch.arange(T), rot["dims"], rot["base"])
    return k, v


def attention(w: dict, p: str, m: dict, kind: str, h: torch.Tensor, eps: float, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Grouped-query attention over given keys and values.  kind "attention": rotated
    queries, blocks of positions, a learned sink per head.  kind "attention_2": no
    rotation, every earlier key, a sink of score 0, a sigmoid gate per head."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    V = v.shape[-1]
    q = projection_norm(h @ w[p + "q"].T, w[p + "q.norm"], eps).view(T, H, D)
    if kind == "attention":
        rot = m.get("rot")
        if rot:
            q = rotate_interleaved(q, torch.arange(T), rot["dims"], rot["base"])
        vis = visible_chunked(T, (m.get("mask") or {}).get("size", 0))
        sinks = w[p + "sink"].tolist()
    else:
        vis = visible_chunked(T, 0)
        sinks = [0.0] * H
    out = torch.zeros(T, H, V, dtype=F64)
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a, :] @ k[:, g, :].T) * m["scale"]
        out[:, a, :] = softmax_with_sink(s, vis, sinks[a]) @ v[:, g, :]
    if kind == "attention_2":
        out = out * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return out.reshape(T, H * V) @ w[p + "o"].T


def wkv(w: dict, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    """Time mixing with a decay per head and key channel that depends on the token.
    o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t;  S_t = diag(d_t) S_{t-1} + k_t v_t^T."""
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    prev = torch.cat([torch.zeros(1, h.shape[1], dtype=F64), h[:-1]])
    mix = {s: h + (prev - h) * w[p + "mu." + s] for s in "rkvgw"}
    r = (mix["r"] @ w[p + "r"].T).view(T, H, D)
    k = (mix["k"] @ w[p + "k"].T).view(T, H, D)
    v = (mix["v"] @ w[p + "v"].T).view(T, H, D)
    g = mix["g"] @ w[p + "g"].T
    gate = g * torch.sigmoid(g)
    low = torch.tanh(mix["w"] @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"]
    d = torch.exp(-torch.exp(low)).view(T, H, D)
    u = w[p + "u"].view(H, D)
    o = torch.zeros(T, H, D, dtype=F64)
    for b in range(H):
        S = torch.zeros(D, D, dtype=F64)
        for t in range(T):
            kv = torch.outer(k[t, b], v[t, b])
            o[t, b] = (S + u[b][:, None] * kv).T @ r[t, b]
            S = d[t, b][:, None] * S + kv
    y = rms_divide(o, eps).reshape(T, H * D) * w[p + "norm"] * gate
    return y @ w[p + "o"].T


def route(w: dict, p: str, r: dict, h: torch.Tensor):
    """(chosen experts [T, top], their weights [T, top]): the largest logits, softmax over the chosen only."""
    z = h @ w[p + "router"].T + w[p + "router.b"]
    val, idx = torch.topk(z, r["top"], dim=-1)
    return idx, torch.softmax(val, -1)


def route_margin(w: dict, p: str, r: dict, h: torch.Tensor) -> torch.Tensor:
    """[T]: by how much the last chosen logit beats the best one left out (inf when every
    expert is chosen).  A small margin is a close call that rounding may turn."""
    z = (h @ w[p + "router"].T + w[p + "router.b"]).sort(-1, descending=True).values
    if r["top"] >= z.shape[1]:
        return torch.full((h.shape[0],), math.inf, dtype=F64)
    return z[:, r["top"] - 1] - z[:, r["top"]]


def expert_mixture(w: dict, p: str, mlp: dict, h: torch.Tensor) -> torch.Tensor:
    idx, wt = route(w, p, mlp["router"], h)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e, c in zip(idx[t].tolist(), wt[t]):
            z = torch.relu(w[f"{p}e{e}.up"] @ h[t]) ** 2
            out[t] += c * (w[f"{p}e{e}.down"] @ z)
    return out


def forward(cfg: dict, weights: dict, tokens: list, streams: list | None = None,
            margins: list | None = None) -> torch.Tensor:
    """[T, vocab] logits of one whole sequence; ``streams`` collects x after every layer,
    ``margins`` every router's margin [T]."""
    w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in weights.items()}
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    x = embed(cfg, w, tokens)
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, mx, kind = f"l{i}.", layer["mixer"], layer["type"]
        if kind == "wkv":
            y = wkv(w, p + "mix.", mx, x, eps)
        else:
            src = mx.get("kv_from")
            kept[i] = kept[src] if src is not None else keys_and_values(w, p + "mix.", mx, kind, x, eps)
            y = attention(w, p + "mix.", mx, kind, x, eps, *kept[i])
        x = x + mult * rms_divide(y, eps) * w[p + "norm1"]
        if layer.get("mlp"):
            if margins is not None:
                margins.append(route_margin(w, p + "mlp.", layer["mlp"]["router"], x))
            x = x + mult * rms_divide(expert_mixture(w, p + "mlp.", layer["mlp"], x), eps) * w[p + "norm2"]
        if streams is not None:
            streams.append(x.clone())
    return (rms_divide(x, eps) * w["final.norm"]) @ w["head"].T * cfg.get("logit_scale", 1.0)
