"""A plain, slow implementation of the Fasodra design, one function per mechanism, in torch on the CPU.

It takes a configuration in config.json's form and a dict of tensors by checkpoint name, and shares no code with the
library: every request is computed alone, with full keys and values, one token after the other where the design has a
recurrence. ``dtype`` is the arithmetic's type (float64 by default: the oracle of the tests).
"""
from __future__ import annotations

import math

import torch


# ---------------------------------------------------------------- norms
def layer_norm(x, w, b, eps):
    mean = x.mean(-1, keepdim=True)
    dev = x - mean
    var = (dev * dev).mean(-1, keepdim=True)
    return dev / torch.sqrt(var + eps) * w + b


def rms_divide(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


# ---------------------------------------------------------------- attention pieces
def distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of the distance table for the distance n >= 0: one row per distance below rows / 2, logarithmic steps up to ``far``."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def rotate(x, positions, dims, base):
    """x [t, heads, dim]: the first ``dims`` elements of every head, element i paired with i + dims / 2."""
    half = dims // 2
    f = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    a = positions.to(torch.float64)[:, None] * f[None, :]
    cos, sin = torch.cos(a).to(x.dtype)[:, None, :], torch.sin(a).to(x.dtype)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], -1)


def softmax_attention(q, k, v, scale, visible, bias=None):
    """q [t, H, d], k [t, G, d], v [t, G, e]; visible [t, t] bool; bias [H, t, t] added to the scaled scores."""
    t, H, _ = q.shape
    G = k.shape[1]
    out = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if bias is not None:
            s = s + bias[h]
        s = s.masked_fill(~visible, float("-inf"))
        out.append(torch.softmax(s, -1) @ v[:, g])
    return torch.stack(out, 1)                   # [t, H, e]


def _heads(x, n):
    return x.view(x.shape[0], n, -1)


def _qkv(h, w, p, m):
    lin = lambda name: h @ w[p + name].T + w[p + name + ".b"]
    H, G = m["heads"], m.get("kv_heads") or m["heads"]
    return _heads(lin("q"), H), _heads(lin("k"), G), _heads(lin("v"), G), H, G


def biased_attention(h, w, p, m, eps):
    """The mixer "attention": no rotation, q and k divided by their RMS per head, a learned bias per distance bucket and head,
    and a key is visible only inside the query's chunk of ``mask.size`` positions."""
    t = h.shape[0]
    q, k, v, H, G = _qkv(h, w, p, m)
    q, k = rms_divide(q, eps), rms_divide(k, eps)
    rel = w[p + "rel"]
    rows = rel.shape[0]
    i = torch.arange(t)
    visible = i[None, :] <= i[:, None]
    size = (m.get("mask") or {}).get("size")
    if size:
        visible &= (i[None, :] // size) == (i[:, None] // size)
    by_distance = torch.stack([rel[distance_bucket(n, rows, m["bias_max"])] for n in range(t)])       # [t, H]
    bias = by_distance[(i[:, None] - i[None, :]).clamp(min=0)].permute(2, 0, 1)                       # [H, query, key]
    o = softmax_attention(q, k, v, m["scale"], visible, bias)
    return o.reshape(t, -1) @ w[p + "o"].T


def rotary_attention(h, w, p, m, eps, head_norm=False, gate=False):
    """The left half of the two-sided mixers: causal attention with a rotation of the first rot.dims elements of every head;
    ``head_norm``: q and k RMS-normed per head with a weight of the head's size first; ``gate``: one sigmoid per head on the output."""
    t = h.shape[0]
    q, k, v, H, G = _qkv(h, w, p, m)
    if head_norm:
        q = rms_divide(q, eps) * w[p + "q.norm"]
        k = rms_divide(k, eps) * w[p + "k.norm"]
    rot = m.get("rot")
    pos = torch.arange(t)
    if rot:
        q, k = rotate(q, pos, rot["dims"], rot["base"]), rotate(k, pos, rot["dims"], rot["base"])
    visible = pos[None, :] <= pos[:, None]
    o = softmax_attention(q, k, v, m["scale"], visible)
    if gate:
        o = o * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(t, -1) @ w[p + "o"].T


# ---------------------------------------------------------------- recurrent pieces
def time_mix(h, w, p, m, eps):
    """Time mixing with a decay per head and key channel that depends on the token, and a bonus for the current token."""
    t, W = h.shape
    H, D = m["heads"], m["dim"]
    prev = torch.cat([torch.zeros(1, W, dtype=h.dtype), h[:-1]], 0)
    mix = lambda s: h + (prev - h) * w[p + "mu." + s]
    r = _heads(mix("r") @ w[p + "r"].T, H)
    k = _heads(mix("k") @ w[p + "k"].T, H)
    v = _heads(mix("v") @ w[p + "v"].T, H)
    gate = torch.nn.functional.silu(mix("g") @ w[p + "g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mix("w") @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"]))
    decay = _heads(decay, H)
    u = w[p + "u"]
    S = torch.zeros(H, D, D, dtype=h.dtype)
    out = torch.zeros(t, H, D, dtype=h.dtype)
    for i in range(t):
        kv = k[i][:, :, None] * v[i][:, None, :]                  # [H, D(key), D(value)]
        out[i] = torch.einsum("hkv,hk->hv", S + u[:, :, None] * kv, r[i])
        S = decay[i][:, :, None] * S + kv
    o = rms_divide(out, eps).reshape(t, -1) * w[p + "norm"] * gate
    return o @ w[p + "o"].T


def short_conv(x, taps_w):
    """x [t, channels], taps_w [channels, taps]: the last column multiplies the current token, zeros before the start."""
    t, _ = x.shape
    taps = taps_w.shape[1]
    y = torch.zeros_like(x)
    for j in range(taps):
        shift = taps - 1 - j
        if shift < t:
            y[shift:] += x[:t - shift] * taps_w[:, j]
    return y


def gated_delta(h, w, p, m, eps):
    """The gated delta rule: the state forgets by a decay per head, and a write replaces what the key already reads out."""
    t = h.shape[0]
    H, G, D, V = m["heads"], m.get("kv_heads") or m["heads"], m["dim"], m.get("vdim") or m["dim"]
    silu = torch.nn.functional.silu
    proj = lambda name: silu(short_conv(h @ w[p + name].T, w[p + name + ".conv"])) if (p + name + ".conv") in w else silu(h @ w[p + name].T)
    q, k, v = _heads(proj("q"), G), _heads(proj("k"), G), _heads(proj("v"), H)
    unit = lambda x: x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)
    q, k = unit(q) * D ** -0.5, unit(k)
    beta = torch.sigmoid(h @ w[p + "b"].T)                                                          # [t, H]
    g = torch.exp(-torch.exp(w[p + "A_log"]) * torch.nn.functional.softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    S = torch.zeros(H, D, V, dtype=h.dtype)
    out = torch.zeros(t, H, V, dtype=h.dtype)
    for i in range(t):
        for a in range(H):
            c = a // (H // G)
            S[a] = g[i, a] * S[a]
            u = beta[i, a] * (v[i, a] - S[a].T @ k[i, c])
            S[a] = S[a] + k[i, c][:, None] * u[None, :]
            out[i, a] = S[a].T @ q[i, c]
    o = rms_divide(out, eps) * w[p + "norm"]
    o = o.reshape(t, -1) * silu(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


# ---------------------------------------------------------------- mixers
def mixer(kind, h, w, p, m, eps):
    if kind == "attention":
        return biased_attention(h, w, p, m, eps)
    if kind == "parallel":
        left = rotary_attention(h, w, p + "left.", m["left"], eps, gate=True)
        right = time_mix(h, w, p + "right.", m["right"], eps)
        return m.get("left_scale", 1.0) * left + m.get("right_scale", 1.0) * right
    if kind == "parallel_2":
        left = rotary_attention(h, w, p + "left.", m["left"], eps, head_norm=True)
        right = gated_delta(h, w, p + "right.", m["right"], eps)
        return 0.5 * (rms_divide(left, eps) * w[p + "left.out"] + rms_divide(right, eps) * w[p + "right.out"])
    raise ValueError(kind)


# ---------------------------------------------------------------- feed-forward
def router_scores(h, w, p):
    return torch.softmax(h @ w[p + "router"].T, -1)


def routed_experts(h, w, p, f, margins=None, forced=None):
    """Every token's ``top`` experts by softmax score, their scores divided by their sum; an expert is down(max(up x, 0)^2).
    ``forced`` {position: experts}: choices made elsewhere, taken as they are (the weights are still this function's scores)."""
    experts, top = f["router"]["experts"], f["router"]["top"]
    s = router_scores(h, w, p)
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        order = sorted(range(experts), key=lambda e: (-float(s[i, e]), e))
        chosen = order[:top] if forced is None else list(forced[i])
        if margins is not None:
            # how far, in logits, the last chosen expert is ahead of the best one left out
            margins.append(float(torch.log(s[i, order[top - 1]]) - torch.log(s[i, order[top]])) if top < experts else float("inf"))
        total = sum(s[i, e] for e in chosen) + 1e-20
        for e in chosen:
            a = torch.relu(w[f"{p}e{e}.up"] @ h[i]) ** 2
            out[i] += (s[i, e] / total) * (w[f"{p}e{e}.down"] @ a)
    return out


# ---------------------------------------------------------------- the model
def forward(config, weights, tokens, dtype=torch.float64, layers_out=None, margins=None, forced=None):
    """Logits [len(tokens), vocab] of one request; ``layers_out``: a list that receives the stream after every layer (the sum
    of the streams, where there are several); ``margins``: a list that receives one list of router margins per layer; ``forced``
    {layer: {position: experts}}: router choices to take instead of this implementation's own."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    mult = float(config.get("residual_mult", 1.0))
    streams = int(config.get("streams") or 0)
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    xs = [x.clone() for _ in range(streams)] if streams else None
    norm = lambda name, v: layer_norm(v, w[name], w[name + ".b"], eps)
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        subs = [(1, lambda hh: mixer(layer["type"], hh, w, p + "mix.", layer["mixer"], eps))]
        if layer.get("mlp") is not None:
            mg = [] if margins is not None else None
            if margins is not None:
                margins.append(mg)
            subs.append((2, lambda hh, mg=mg: routed_experts(hh, w, p + "mlp.", layer["mlp"], mg, None if forced is None else forced[i])))
        elif margins is not None:
            margins.append([])
        for qn, fn in subs:
            if streams:
                hc = f"{p}hc{qn}."
                u = sum(w[hc + "in"][s] * xs[s] for s in range(streams))
                y = fn(norm(f"{p}norm{qn}", u))
                xs = [sum(w[hc + "mix"][s, t] * xs[s] for s in range(streams)) + mult * w[hc + "out"][t] * y for t in range(streams)]
            else:
                x = x + mult * fn(norm(f"{p}norm{qn}", x))
        if layers_out is not None:
            layers_out.append(sum(xs) if streams else x.clone())
    if streams:
        x = sum(xs)
    return norm("final.norm", x) @ w["head"].T
