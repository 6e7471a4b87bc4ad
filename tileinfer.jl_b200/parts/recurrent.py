"""Two mixers whose memory is a matrix state per head, carried from token to token in 32-bit (the cache's "state" kind), however
long the sequence is.

``time_mix``: time mixing with a decay that depends on the token. With h' the row before h in the sequence (zeros at its start),
each of r, k, v, g, w reads its own blend b_s = h + (h' - h) mu_s:

    r, k, v = W_r b_r, W_k b_k, W_v b_v   [heads, dim]          gate = silu(W_g b_g)
    w = exp(-exp(W_w2 tanh(W_w1 b_w) + w0))                       per head and key channel, 32-bit
    o_t = (S + diag(u) k_t v_t^T)^T r_t ;   S <- diag(w_t) S + k_t v_t^T          (u: a bonus for the current token only)
    out = W_o ( concat_heads(o / rms(o over the head)) * norm * gate )

A sequence keeps S [heads, dim, dim] and its last input row h.

``gated_delta``: the gated delta rule behind short convolutions. q, k [qk_heads, dim] and v [heads, value_dim] are projections of h
(head i reads q/k head i / (heads / qk_heads)); each channel passes a causal convolution over time of ``conv_taps`` taps and SiLU; q
and k become unit vectors per head, x / sqrt(sum x^2 + unit_eps), q also times dim^(-1/2):

    beta = sigmoid(W_b h),   g = exp(-exp(A_log) * softplus(W_a h + dt_bias))       one of each per head, 32-bit
    S <- g S ;   e = beta (v - S^T k) ;   S <- S + k e^T ;   o = S^T q              (the read-out sees the token's own write)
    out = W_o ( o / rms(o over the head) * norm * silu(W_g h) )                       norm [value_dim], shared by the heads

A sequence keeps S [heads, dim, value_dim] and the last taps - 1 rows of the q|k|v projections.

Both ask the cache for ONE state of floats per layer and lay their pieces into it; the recurrences, decays, gates and norms run in
32-bit in every element type (``csrc/recurrent.cu``), the projections in the model's element type.
"""
from __future__ import annotations

import torch

from ..config.spec import MixerSpec, TensorDecl
from ..kernels import ops
from .base import CacheRequest, Mixer, register_mixer
from .linear import Linear


def _f32(rt, t):
    return rt.param(t, keep_dtype=True).float().contiguous()


@register_mixer("time_mix")
class TimeMix(Mixer):
    BLENDS = ("r", "k", "v", "g", "w")

    def __init__(self, spec: MixerSpec, tensors, rt, position):
        self.spec, self.rt = spec, rt
        self.heads, self.dim = spec.num_heads, spec.head_dim
        self.eps = float(spec.options.get("norm_eps", 1e-6))
        n, p = spec.tensor_names, spec.prefix
        get = lambda k: rt.param(tensors[p + n[k]])
        self.mu = torch.stack([rt.param(tensors[p + n["mu"] + s]) for s in self.BLENDS]).contiguous()          # [5, width]
        self.r, self.k, self.v, self.g = (Linear(get(s), rt, "time_mix_" + s) for s in ("r", "k", "v", "g"))
        self.w1, self.w2 = Linear(get("w1"), rt, "time_mix_w1"), Linear(get("w2"), rt, "time_mix_w2")
        if self.w1.out_features != self.w2.in_features:
            raise ValueError(f"time_mix: the decay's two matrices do not fit ({tuple(self.w1.weight.shape)}, {tuple(self.w2.weight.shape)})")
        self.w0, self.u = _f32(rt, tensors[p + n["w0"]]).flatten(), _f32(rt, tensors[p + n["u"]]).flatten()
        self.norm_w = get("norm")
        self.o = Linear(get("o"), rt, "o")
        self.out_name = "mixer.delta"
        self.o.partials_name = "time_mix.partials"

    @classmethod
    def tensors(cls, spec: MixerSpec):
        n, p, o = spec.tensor_names, spec.prefix, spec.options
        W, H, D = spec.hidden_size, spec.num_heads, spec.head_dim
        R = int(o.get("decay_rank", 16))
        std = lambda fan_in: ("normal", fan_in ** -0.5)
        out = [TensorDecl(p + n[s], (H * D, W), std(W)) for s in ("r", "k", "v", "g")]
        out += [TensorDecl(p + n["mu"] + s, (W,), ("const_plus_normal", 0.5, 0.25)) for s in cls.BLENDS]
        out += [TensorDecl(p + n["w1"], (R, W), std(W), free_dims=(0,)), TensorDecl(p + n["w2"], (H * D, R), ("normal", 0.5 * R ** -0.5), free_dims=(1,)),
                TensorDecl(p + n["w0"], (H * D,), ("const_plus_normal", -2.5, 1.0), keep_dtype=True),
                TensorDecl(p + n["u"], (H, D), ("normal", 0.5), keep_dtype=True),
                TensorDecl(p + n["norm"], (H * D,), ("one_plus_normal", 0.1)), TensorDecl(p + n["o"], (W, H * D), std(H * D))]
        return out

    def cache_request(self):
        return CacheRequest("state", shape=(self.heads * self.dim * self.dim + self.spec.hidden_size,), dtype=torch.float32)

    def forward(self, h, step, cache):
        rt = self.rt
        n, W = h.shape
        H, D = self.heads, self.dim
        HD = H * D
        state = cache.state                                   # [slots, H * D * D + W]: the heads' matrices, then the last input row
        blends = rt.buffer("time_mix.blends", (len(self.BLENDS), n, W))
        ops.shift_blend(blends, h, self.mu, state[:, HD * D:], step)
        rows = rt.buffer("time_mix.rows", (n, 3 * HD))
        for i, lin in enumerate((self.r, self.k, self.v)):
            lin.forward(blends[i], rows[:, i * HD:(i + 1) * HD])
        gate = self.g.forward(blends[3], rt.buffer("time_mix.gate", (n, HD)))
        low = self.w1.forward(blends[4], rt.buffer("time_mix.low", (n, self.w1.out_features)))
        ops.tanh(low, low)
        dlog = self.w2.forward(low, rt.buffer("time_mix.dlog", (n, HD), torch.float32), ops.EPI_F32_OUT)
        o = rt.buffer("time_mix.o", (n, HD), torch.float32)
        ops.decay_scan(o, rows, 0, HD, 2 * HD, dlog, self.w0, self.u, state, step, H, D)
        y = rt.buffer("time_mix.normed", (n, HD))
        ops.heads_norm_gate(y, o, gate, self.norm_w, self.eps, H, D)
        return self.o.forward(y, rt.buffer(self.out_name, (n, W)), allow_partials=True)


@register_mixer("gated_delta")
class GatedDelta(Mixer):
    def __init__(self, spec: MixerSpec, tensors, rt, position):
        self.spec, self.rt = spec, rt
        o = spec.options
        self.heads, self.qk_heads, self.dim, self.vdim = spec.num_heads, spec.num_kv_heads or spec.num_heads, spec.head_dim, int(o["value_dim"])
        if self.heads % self.qk_heads:
            raise ValueError(f"gated_delta: {self.heads} heads do not divide into {self.qk_heads} query/key heads")
        self.eps, self.unit_eps = float(o.get("norm_eps", 1e-6)), float(o.get("unit_eps", 1e-6))
        n, p = spec.tensor_names, spec.prefix
        get = lambda k: rt.param(tensors[p + k])
        self.channels = 2 * self.qk_heads * self.dim + self.heads * self.vdim
        self.proj = Linear(torch.cat([get(n[k]) for k in ("q", "k", "v", "g")], 0).contiguous(), rt, "gated_delta_in")
        self.ba = Linear(torch.cat([get(n["beta"]), get(n["a"])], 0).contiguous(), rt, "gated_delta_gates")
        self.conv = None
        if int(o.get("conv_taps") or 0):
            self.conv = torch.cat([get(n[k] + n["conv_suffix"]) for k in ("q", "k", "v")], 0).contiguous()          # [channels, taps]
        self.taps = self.conv.shape[1] if self.conv is not None else 0
        self.a_log, self.dt_bias = _f32(rt, tensors[p + n["A_log"]]).flatten(), _f32(rt, tensors[p + n["dt_bias"]]).flatten()
        self.norm_w = get(n["norm"])
        self.o = Linear(get(n["o"]), rt, "o")
        self.out_name = "mixer.delta"
        self.o.partials_name = "gated_delta.partials"

    @classmethod
    def tensors(cls, spec: MixerSpec):
        n, p, o = spec.tensor_names, spec.prefix, spec.options
        W, H, G, D, V = spec.hidden_size, spec.num_heads, spec.num_kv_heads or spec.num_heads, spec.head_dim, int(o["value_dim"])
        taps = int(o.get("conv_taps") or 0)
        std = lambda fan_in: ("normal", fan_in ** -0.5)
        out = []
        for k, r in (("q", G * D), ("k", G * D), ("v", H * V)):
            out.append(TensorDecl(p + n[k], (r, W), std(W)))
            if taps:
                out.append(TensorDecl(p + n[k] + n["conv_suffix"], (r, taps), ("const_plus_normal", 1.0 / taps, 0.3), free_dims=(1,)))
        out += [TensorDecl(p + n["g"], (H * V, W), std(W)), TensorDecl(p + n["beta"], (H, W), std(W)), TensorDecl(p + n["a"], (H, W), std(W)),
                TensorDecl(p + n["A_log"], (H,), ("normal", 0.5), keep_dtype=True),
                TensorDecl(p + n["dt_bias"], (H,), ("const_plus_normal", -2.0, 1.0), keep_dtype=True),
                TensorDecl(p + n["norm"], (V,), ("one_plus_normal", 0.1)), TensorDecl(p + n["o"], (W, H * V), std(H * V))]
        return out

    def _taps(self):
        return self.taps

    def cache_request(self):
        history = max(0, self.taps - 1) * self.channels
        return CacheRequest("state", shape=(self.heads * self.dim * self.vdim + history,), dtype=torch.float32)

    def forward(self, h, step, cache):
        rt = self.rt
        n, W = h.shape
        H, G, D, V, C = self.heads, self.qk_heads, self.dim, self.vdim, self.channels
        state = cache.state                                   # [slots, H * D * V + (taps - 1) * C]: the matrices, then the rows' history
        rows = rt.buffer("gated_delta.rows", (n, C + H * V))
        self.proj.forward(h, rows)
        ba = self.ba.forward(h, rt.buffer("gated_delta.gates", (n, 2 * H), torch.float32), ops.EPI_F32_OUT)
        qkv = rt.buffer("gated_delta.inputs", (n, C), torch.float32)
        hist = state[:, H * D * V:] if self.taps > 1 else None
        ops.delta_inputs(qkv, rows, self.conv, self.taps, hist, step, G, D, H * V, self.unit_eps)
        if self.taps > 1:
            ops.history_update(hist, rows, self.taps, step, C)
        o = rt.buffer("gated_delta.o", (n, H * V), torch.float32)
        ops.delta_scan(o, qkv, ba, self.a_log, self.dt_bias, state, step, H, G, D, V)
        y = rt.buffer("gated_delta.normed", (n, H * V))
        ops.heads_norm_gate(y, o, rows[:, C:], self.norm_w, self.eps, H, V)
        return self.o.forward(y, rt.buffer(self.out_name, (n, W)), allow_partials=True)
