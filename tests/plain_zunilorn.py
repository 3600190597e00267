"""A plain, slow Zunilorn in float64 on the CPU: the oracle of the GPU tests.

One function per mechanism, each written from its equation; whole sequences
only (no cache, no state carried between calls: a position's logits are those of
the whole prefix run at once).  Nothing here is shared with the engine.

Notation: T tokens, W the width, n(.) = division by the root mean square with
eps inside the root, m the residual multiplier, s the number of streams.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_divide(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def softcap(x: torch.Tensor, cap) -> torch.Tensor:
    return x if not cap else cap * torch.tanh(x / cap)


# ------------------------------------------------------------------------------------------------
# rotation
def rotary_frequencies(rot: dict) -> tuple:
    """(frequency of every pair [dims/2], the factor on cos and sin).  Plain: base^(-2i/dims), 1.
    With 'scaling' {factor, original, fast, slow}: pairs that turn fast keep their frequency, slow
    ones are divided by factor, a linear ramp over the pair index lies between; cos and sin are
    multiplied by 0.1 ln(factor) + 1."""
    dims, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(f, dtype=F64), 1.0

    def pair_of(turns):                       # the (real) pair index that makes `turns` turns in `original` positions
        return dims * math.log(sc["original"] / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(pair_of(sc["fast"])), 0)
    hi = min(math.ceil(pair_of(sc["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / sc["factor"] * ramp + fi * (1 - ramp))
    return torch.tensor(out, dtype=F64), 0.1 * math.log(sc["factor"]) + 1.0


def rotate_half(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, H, D]: coordinate i pairs with i + dims/2 for i < dims/2; coordinates >= dims stay."""
    dims = rot["dims"] if rot else 0
    if dims == 0:
        return x
    half = dims // 2
    freq, mag = rotary_frequencies(rot)
    ang = positions.to(F64)[:, None, None] * freq[None, None, :]
    c, s = torch.cos(ang) * mag, torch.sin(ang) * mag
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# ------------------------------------------------------------------------------------------------
# mixers
def attention(m: dict, w: dict, p: str, h: torch.Tensor) -> torch.Tensor:
    """Grouped-query attention: rotation of q and k, a capped score, every earlier key, a learned
    number per head in the softmax's denominator, a sigmoid gate per head from the mixer's input."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    V = m.get("vdim") or D
    pos = torch.arange(T)
    q = rotate_half((h @ w[p + "q"].T).view(T, H, D), pos, m.get("rot"))
    k = rotate_half((h @ w[p + "k"].T).view(T, G, D), pos, m.get("rot"))
    v = (h @ w[p + "v"].T).view(T, G, V)
    gate = torch.sigmoid(h @ w[p + "g"].T)                          # [T, H]
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    out = torch.zeros(T, H, V, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        sc = softcap((q[:, hd] @ k[:, g].T) * m["scale"], m.get("softcap"))
        sc = sc.masked_fill(~causal, -math.inf)
        sink = w[p + "sink"][hd]
        top = torch.maximum(sc.max(-1, keepdim=True).values, sink)
        e = torch.exp(sc - top)
        den = e.sum(-1, keepdim=True) + torch.exp(sink - top)
        out[:, hd] = (e / den) @ v[:, g] * gate[:, hd:hd + 1]
    return out.reshape(T, H * V) @ w[p + "o"].T


def causal_conv(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x [T, C], weight [C, taps]: column taps - 1 - d weighs the input d positions back; nothing lies before position 0."""
    T, taps = x.shape[0], weight.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=x.dtype), x], 0)
    out = bias.expand(T, -1).clone()
    for j in range(taps):
        out = out + padded[j:j + T] * weight[:, j]
    return out


def mamba2(m: dict, w: dict, p: str, h: torch.Tensor, eps: float) -> torch.Tensor:
    """S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T per head, y_t = S_t^T C_t + D x_t; the
    gate silu(z) first, then a root-mean-square division in norm_groups parts."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = torch.nn.functional.softplus(dt + w[p + "dt_bias"], threshold=1e9)        # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * dt)
    y = torch.zeros(T, H, P, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(N, P, dtype=F64)
        for t in range(T):
            S = decay[t, hd] * S + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + w[p + "D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    parts = m.get("norm_groups") or 1
    y = rms_divide(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


# ------------------------------------------------------------------------------------------------
# feed-forwards
def glu(gate: torch.Tensor, up: torch.Tensor, limit) -> torch.Tensor:
    """min(gate, limit) sigmoid(1.702 min(gate, limit)) (clamp(up, -limit, limit) + 1)"""
    if limit is not None:
        gate = torch.clamp(gate, max=limit)
        up = torch.clamp(up, -limit, limit)
    return gate * torch.sigmoid(1.702 * gate) * (up + 1)


def gated_ff(w: dict, p: str, h: torch.Tensor, limit, bias: bool) -> torch.Tensor:
    g, u = h @ w[p + "gate"].T, h @ w[p + "up"].T
    if bias:
        g, u = g + w[p + "gate.b"], u + w[p + "up.b"]
    y = glu(g, u, limit) @ w[p + "down"].T
    return y + w[p + "down.b"] if bias else y


def route(f: dict, w: dict, p: str, h: torch.Tensor) -> tuple:
    """(chosen [T, top], weights [T, top]) over experts + identity outputs: softmax over all, the
    choice by score + correction, the weights from the scores alone, divided by their sum, scaled."""
    r = f["router"]
    s = torch.softmax(h @ w[p + "router"].T, -1)
    choice = s + w[p + "correction"] if (p + "correction") in w else s
    chosen = torch.topk(choice, r["top"], dim=-1).indices
    weights = torch.gather(s, 1, chosen)
    weights = weights / (weights.sum(-1, keepdim=True) + 1e-20) * r.get("scale", 1.0)
    return chosen, weights


def moe_ff(f: dict, w: dict, p: str, h: torch.Tensor) -> torch.Tensor:
    r = f["router"]
    E = r["experts"]
    chosen, weights = route(f, w, p, h)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t].tolist(), weights[t]):
            if e >= E:                                   # an identity expert hands its input on
                out[t] += a * h[t]
            else:
                out[t] += a * gated_ff(w, f"{p}e{e}.", h[t:t + 1], f["expert"].get("limit"), False)[0]
    if f.get("shared"):
        sg = torch.sigmoid(h @ w[p + "shared.sg"].T)                    # [T, 1]
        out = out + sg * gated_ff(w, p + "shared.", h, f["shared"].get("limit"), False)
    return out


def feed_forward(f: dict, w: dict, p: str, h: torch.Tensor) -> torch.Tensor:
    if f["kind"] == "dense":
        return gated_ff(w, p, h, f.get("limit"), True)
    return moe_ff(f, w, p, h)


# ------------------------------------------------------------------------------------------------
# the layer and the model
def run_order(cfg: dict) -> list:
    """Layer indices in the order they run: the span start .. stop-1 `times` times in a row."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b = loop["start"], loop["stop"]
    return list(range(a)) + list(range(a, b)) * loop["times"] + list(range(b, n))


def sublayer(cfg: dict, w: dict, i: int, q: int, h: torch.Tensor) -> torch.Tensor:
    layer = cfg["layers"][i]
    eps = cfg["norm"]["eps"]
    if q == 1:
        fn = mamba2 if layer["type"] == "mamba2" else None
        return mamba2(layer["mixer"], w, f"l{i}.mix.", h, eps) if fn else attention(layer["mixer"], w, f"l{i}.mix.", h)
    return feed_forward(layer["mlp"], w, f"l{i}.mlp.", h)


def layer_forward(cfg: dict, w: dict, i: int, xs: torch.Tensor) -> torch.Tensor:
    """xs [s, T, W] -> the same after layer i.  With hyper-connections a sublayer reads
    u = sum_s in[s] x_s and every stream becomes sum_s mix[s, t] x_s + m out[t] y; without them
    (no 'streams' key) s = 1 and x <- x + m y."""
    m, eps = cfg.get("residual_mult", 1.0), cfg["norm"]["eps"]
    hyper = cfg.get("streams") is not None
    for q in (1, 2):
        if q == 2 and not cfg["layers"][i].get("mlp"):
            break
        if hyper:
            c_in, c_out, c_mix = (w[f"l{i}.hc{q}.{k}"] for k in ("in", "out", "mix"))
            u = torch.einsum("s,stw->tw", c_in, xs)
        else:
            u = xs[0]
        y = sublayer(cfg, w, i, q, rms_divide(u, eps) * w[f"l{i}.norm{q}"])
        if hyper:
            xs = torch.einsum("sr,stw->rtw", c_mix, xs) + m * c_out[:, None, None] * y[None]
        else:
            xs = xs + m * y[None]
    return xs


def forward(cfg: dict, w: dict, tokens: list, layers_out: list = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence; layers_out collects the sum of the streams after every layer run."""
    w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in w.items()}
    x = w["embed"][torch.tensor(tokens)]
    xs = x[None].repeat(cfg.get("streams") or 1, 1, 1)
    for i in run_order(cfg):
        xs = layer_forward(cfg, w, i, xs)
        if layers_out is not None:
            layers_out.append(xs.sum(0))
    x = rms_divide(xs.sum(0), cfg["norm"]["eps"]) * w["final.norm"]
    return softcap(x @ w["embed"].T, cfg.get("logit_softcap"))
