"""A plain, slow implementation of the Sozanex design, written from its equations: one function per mechanism,
whole sequences at a time, full keys and values, nothing cached, nothing absorbed, nothing shared with the library.

``forward(config, weights, tokens)`` takes the config.json dictionary, a dict of tensors by checkpoint name and one
sequence's token ids and returns the logits at every position (and, on request, the stream after every layer run).
``dtype`` is the arithmetic of the matrix products: float64 / float32 give a reference, bfloat16 rounds the products'
operands and results the way a 16-bit implementation does, with everything the design wants in 32-bit kept there.
"""
from __future__ import annotations

import math

import torch


def _mm(x, w, dtype):
    """x Wᵀ with operands rounded to ``dtype``, summed exactly, rounded once to ``dtype``; returned in the work precision."""
    if dtype in (torch.float64, torch.float32):
        return x @ w.to(x.dtype).T
    y = x.to(dtype).double() @ w.to(dtype).double().T
    return y.to(dtype).to(x.dtype)


def _rnd(x, dtype):
    return x if dtype in (torch.float64, torch.float32) else x.to(dtype).to(x.dtype)


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w, var = mean of the squared deviations; no bias."""
    mu = x.mean(-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w.to(x.dtype)


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w.to(x.dtype)


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


# ---------------------------------------------------------------- embedding
def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the bigram table for every position: a hash of (previous, current); the extra last row for the first token."""
    rows = []
    for i, t in enumerate(tokens):
        rows.append(buckets if i == 0 else (tokens[i - 1] * mul_prev + t * mul_cur) % buckets)
    return rows


def embedding(config, weights, tokens, work):
    e = config["embedding"]
    x = weights["embed"].to(work)[tokens] * float(e.get("scale", 1.0))
    b = e.get("bigram")
    if b is not None:
        rows = bigram_rows(tokens, int(b["buckets"]), int(b["mul_prev"]), int(b["mul_cur"]))
        x = x + weights["bigram"].to(work)[rows]
    return x


# ---------------------------------------------------------------- rotations
def llama3_frequencies(rot):
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    s = rot.get("scaling")
    if s is None:
        return f
    factor, low, high, orig = float(s["factor"]), float(s["low"]), float(s["high"]), float(s["original"])
    out = []
    for fi in f:
        wl = 2 * math.pi / fi
        if wl < orig / high:
            out.append(fi)
        elif wl > orig / low:
            out.append(fi / factor)
        else:
            sm = (orig / wl - low) / (high - low)
            out.append((1 - sm) * fi / factor + sm * fi)
    return out


def yarn_frequencies(rot):
    """Returns (frequencies, multiplier of cos and sin)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    s = rot.get("scaling")
    if s is None:
        return f, 1.0
    factor, orig, fast, slow = float(s["factor"]), float(s["original"]), float(s["fast"]), float(s["slow"])
    where = lambda t: dims * math.log(orig / (2 * math.pi * t)) / (2 * math.log(base))
    lo = max(math.floor(where(fast)), 0)
    hi = min(math.ceil(where(slow)), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x, freqs, interleaved, mult=1.0):
    """x [T, heads, dims]: all of the last axis is rotated; position = index along the first axis."""
    T, dims = x.shape[0], x.shape[-1]
    ang = torch.arange(T, dtype=torch.float64)[:, None] * torch.tensor(freqs, dtype=torch.float64)[None, :]
    cos, sin = (ang.cos() * mult).to(x.dtype)[:, None, :], (ang.sin() * mult).to(x.dtype)[:, None, :]
    if interleaved:
        u, v = x[..., 0::2], x[..., 1::2]
        out = torch.empty_like(x)
        out[..., 0::2] = u * cos - v * sin
        out[..., 1::2] = v * cos + u * sin
        return out
    u, v = x[..., : dims // 2], x[..., dims // 2:]
    return torch.cat([u * cos - v * sin, v * cos + u * sin], -1)


# ---------------------------------------------------------------- softmax over visible keys
def masked_attention(q, k, v, scale, window=None, sink=None):
    """q [T, H, d], k [T, H, d], v [T, H, dv] (keys already repeated per query head). Position i sees j <= i, and with a
    window only i - j < window. ``sink`` [H]: one more term exp(sink) in the denominator, with no value."""
    T = q.shape[0]
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & (i - j < window)
    s = s.masked_fill(~seen[None], float("-inf"))
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink.to(s.dtype)[:, None, None])
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink.to(s.dtype)[:, None, None] - m)
    return torch.einsum("hij,jhd->ihd", e / den, v)


# ---------------------------------------------------------------- mixers
def attention_mixer(m, w, p, h, eps, dtype):
    """Grouped-query attention with biases, per-head q/k RMS norm, partial rotate-half rotation and a window."""
    T = h.shape[0]
    H, G, D = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"])
    V = int(m.get("vdim", D))
    lin = lambda name: _mm(h, w[p + name], dtype) + w[p + name + ".b"].to(h.dtype) if (p + name + ".b") in w else _mm(h, w[p + name], dtype)
    q = _rnd(lin("q"), dtype).view(T, H, D)
    k = _rnd(lin("k"), dtype).view(T, G, D)
    v = _rnd(lin("v"), dtype).view(T, G, V)
    if p + "q.norm" in w:
        q = rms_norm(q, w[p + "q.norm"], eps)
        k = rms_norm(k, w[p + "k.norm"], eps)
    rot = m.get("rot")
    if rot is not None:
        r = int(rot["dims"])
        f = llama3_frequencies(rot)
        q = torch.cat([rotate(q[..., :r], f, False), q[..., r:]], -1)
        k = torch.cat([rotate(k[..., :r], f, False), k[..., r:]], -1)
    q, k = _rnd(q, dtype), _rnd(k, dtype)
    rep = H // G
    k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    mask = m.get("mask")
    o = masked_attention(q, k, v, float(m["scale"]), int(mask["size"]) if mask else None)
    o = _rnd(o, dtype).reshape(T, H * V)
    y = _mm(o, w[p + "o"], dtype)
    if p + "o.b" in w:
        y = y + w[p + "o.b"].to(h.dtype)
    return y


def latent_attention_mixer(m, w, p, h, eps, dtype):
    """Attention through latents with one rotated key part shared by the heads, a sink and an output gate."""
    T = h.shape[0]
    H, D, Rd, V, R = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    cq = _rnd(rms_norm(_rnd(_mm(h, w[p + "dq"], dtype), dtype), w[p + "dq.norm"], eps), dtype)
    q = _rnd(_mm(cq, w[p + "uq"], dtype), dtype).view(T, H, D + Rd)
    dkv = _rnd(_mm(h, w[p + "dkv"], dtype), dtype)
    c = _rnd(rms_norm(dkv[:, :R], w[p + "dkv.norm"], eps), dtype)
    k_rot = dkv[:, R:].view(T, 1, Rd)
    f, mult = yarn_frequencies(m["rot"])
    q_rot = _rnd(rotate(q[..., D:], f, True, mult), dtype)
    k_rot = _rnd(rotate(k_rot, f, True, mult), dtype)
    k_plain = _rnd(_mm(c, w[p + "uk"], dtype), dtype).view(T, H, D)
    v = _rnd(_mm(c, w[p + "uv"], dtype), dtype).view(T, H, V)
    qq = torch.cat([q[..., :D], q_rot], -1)
    kk = torch.cat([k_plain, k_rot.expand(T, H, Rd)], -1)
    sink = w[p + "sink"].to(h.dtype) if p + "sink" in w else None
    o = _rnd(masked_attention(qq, kk, v, float(m["scale"]), None, sink), dtype).reshape(T, H * V)
    if p + "g" in w:
        gate = torch.sigmoid(_rnd(_mm(h, w[p + "g"], dtype), dtype))
        o = _rnd(o * gate, dtype)
    return _mm(o, w[p + "o"], dtype)


def feed_forward(f, w, p, h, dtype):
    """W_down relu(W_up h)^2."""
    u = _mm(h, w[p + "up"], dtype)
    a = _rnd(torch.relu(u) ** 2, dtype)
    return _mm(a, w[p + "down"], dtype)


# ---------------------------------------------------------------- the model
def layer_runs(config):
    """The layers in the order they run, with a flag on the first layer of each pass of the loop."""
    n = len(config["layers"])
    loop = config.get("loop")
    if loop is None:
        return [(i, False) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, False) for i in range(a)]
    for _ in range(times):
        runs += [(i, i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(b, n)]


def forward(config, weights, tokens, dtype=torch.float32, work=None, return_layers=False):
    work = work or (torch.float64 if dtype == torch.float64 else torch.float32)
    w = weights
    eps = float(config["norm"]["eps"])
    x = embedding(config, w, list(tokens), work)
    x0 = x
    after = []
    for li, starts_pass in layer_runs(config):
        L = config["layers"][li]
        p = f"l{li}."
        if starts_pass:
            x = _mm(_rnd(torch.cat([x, x0], -1), dtype), w["loop.in"], dtype)
        h = _rnd(layer_norm(x, w[p + "norm1"], eps), dtype)
        mixer = {"attention": attention_mixer, "latent_attention": latent_attention_mixer}[L["type"]]
        y = mixer(L["mixer"], w, p + "mix.", h, eps, dtype)
        x = x + layer_norm(y, w[p + "norm1b"], eps)
        if L.get("mlp") is not None:
            h = _rnd(layer_norm(x, w[p + "norm2"], eps), dtype)
            y = feed_forward(L["mlp"], w, p + "mlp.", h, dtype)
            x = x + layer_norm(y, w[p + "norm2b"], eps)
        after.append(x)
    h = _rnd(layer_norm(x, w["final.norm"], eps), dtype)
    logits = h.to(dtype).double() @ w["head"].to(dtype).double().T if dtype == torch.bfloat16 else h @ w["head"].to(work).T
    logits = logits.float()
    return (logits, torch.stack(after).float()) if return_layers else logits
