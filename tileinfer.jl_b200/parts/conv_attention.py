"""Grouped-query attention whose projections pass through a short causal convolution over time, with whole-row q/k norms, a
rotation of part of every head, a sink in the softmax and an output gate.

Per token, from the mixer's input h (every step optional, by the record):

    u = W h + b                      for q [heads, dim], k [kv_heads, dim], v [kv_heads, value_dim]          (``bias``)
    y_t = sum_j c[:, j] * u_(t - taps + 1 + j)       per channel, zeros before the sequence's start             (``conv_taps``)
    q, k <- y / rms(y) * w           over the WHOLE row of q, and of k, before the heads are split              (``row_norm``)
                                     or, with ``head_norm`` too, every head by itself with one weight [dim] per projection
    q, k <- rotation of the first rotary_dim elements of every head (the position encoding's)
    p_ij = exp(scale * q_i . k_j) / (sum_(j' <= i) exp(scale * q_i . k_j') + exp(sink_head))                    (``sink``)
    out = Wo ( concat_heads(sum_j p_ij v_j) * sigmoid(Wg h) ) + bo                                  (``gate``, ``out_bias``)

The output's bias is not added here: the mixer offers it as ``out_bias`` to the block, whose kernel adds it where it reads the
product (a block that does not know of it refuses the mixer).

A sequence keeps its keys (after convolution, norm and rotation) and values (after convolution) in pages, and the last
taps - 1 rows u as a small fixed-size state: the mixer asks the cache for both. With ``kv_source`` the layer has no key and value
tensors and reads the pages of an earlier layer, with queries, convolution state and everything else of its own.

Keys and values of different sizes share the paged attention kernels by filling both up to one row length ``padded`` with zeros
(a zero adds nothing to a score, and the outputs beyond value_dim are dropped by the gate's kernel).

Further options. ``norm_weight`` False: the norms of q and k have no weight (every head is only divided by its root mean square).
``gate`` "head": W_g has one row per head and the whole head is multiplied by that one sigmoid. ``chunk`` c: a key is visible only
inside the query's chunk of c positions, floor(i / c) = floor(j / c), counted from the sequence's start. ``distance_bias`` far: a
learned table ``rel`` [rows, heads] adds rel[bucket(i - j), head] to the scaled score, bucket(n) = n for n < rows / 2 and
min(rows - 1, rows / 2 + floor(ln(n / (rows / 2)) / ln(far / (rows / 2)) * (rows - rows / 2))) beyond: one row per small distance,
logarithmic steps up to ``far``, the last row from there on. In bfloat16 attention with a chunk or a distance bias runs in the
library's paged kernels (tensor-memory and ``mma.sync`` prompt kernels, split-KV decode kernel; the bias comes as a table by distance),
in 32-bit in the plain kernel.

Record: ``num_heads``, ``num_kv_heads``, ``head_dim``, ``scale``, ``window``, ``kv_source``, ``qk_norm_eps`` and the options
``value_dim``, ``conv_taps`` (0: none), ``bias``, ``out_bias``, ``row_norm``, ``head_norm``, ``norm_weight``, ``sink``, ``gate``,
``chunk``, ``distance_bias``.
"""
from __future__ import annotations

import dataclasses
import math

import torch

from ..config.spec import MixerSpec, TensorDecl
from ..kernels import ops
from .base import CacheRequest, Mixer, register_mixer
from .linear import Linear


def distance_buckets(rows: int, far: float, count: int):
    """bucket(n) for n = 0 .. count - 1 (see the module's text); from n = far on it is rows - 1."""
    half = rows // 2
    out = []
    for n in range(count):
        if n < half or half == 0:
            out.append(min(n, rows - 1))
        else:
            out.append(min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half)))))
    return out


def _flags(o):
    return (int(o.get("conv_taps", 0)), bool(o.get("bias", False)), bool(o.get("row_norm", False)), bool(o.get("sink", False)),
            bool(o.get("gate", False)))


@register_mixer("conv_attention")
class ConvAttention(Mixer):
    def __init__(self, spec: MixerSpec, tensors, rt, position):
        self.spec, self.rt = spec, rt
        o = spec.options
        self.nq, self.nkv, self.dim, self.vdim = spec.num_heads, spec.num_kv_heads, spec.head_dim, int(o.get("value_dim", spec.head_dim))
        if self.nkv < 1 or self.nq % self.nkv:
            raise ValueError(f"conv_attention: {self.nq} query heads do not divide into {self.nkv} KV heads")
        self.taps, self.bias_on, self.row_norm, self.sink_on, self.gated = _flags(o)
        self.own_kv = spec.kv_source is None
        # One row length for keys and values in the pages: the larger of the two sizes, in steps of 16 (what the paged kernels take).
        self.padded = max(16, -(-max(self.dim, self.vdim) // 16) * 16)
        if self.padded > ops.MAX_HEAD_DIM:
            raise ValueError(f"conv_attention: heads of {self.dim} / {self.vdim} exceed the attention kernels' {ops.MAX_HEAD_DIM}")
        n, p = spec.tensor_names, spec.prefix
        get = lambda name: rt.param(tensors[p + name])
        kinds = ["q", "k", "v"] if self.own_kv else ["q"]
        mats = [get(n[k]) for k in kinds] + ([get(n["g"])] if self.gated else [])
        self.proj = Linear(torch.cat(mats, 0).contiguous(), rt, "conv_attention_in")
        self.channels = self.nq * self.dim + (self.nkv * (self.dim + self.vdim) if self.own_kv else 0)
        self.bias = torch.cat([get(n[k] + n["bias_suffix"]) for k in kinds]).contiguous() if self.bias_on else None
        self.conv = torch.cat([get(n[k] + n["conv_suffix"]) for k in kinds], 0).contiguous() if self.taps else None
        self.head_norm = bool(o.get("head_norm", False))
        self.gate_per_head = o.get("gate") == "head"
        self.out_bias = get(n["o"] + n["bias_suffix"]) if o.get("out_bias", False) else None
        if self.row_norm and not o.get("norm_weight", True):
            # A norm without a weight: the kernels' weighted norm with ones.
            size = self.dim if self.head_norm else None
            ones = lambda rows: torch.ones(size or rows, dtype=rt.dtype, device=rt.device)
            self.q_norm, self.k_norm = ones(self.nq * self.dim), (ones(self.nkv * self.dim) if self.own_kv else None)
        else:
            self.q_norm = get(n["q"] + n["norm_suffix"]) if self.row_norm else None
            self.k_norm = get(n["k"] + n["norm_suffix"]) if self.row_norm and self.own_kv else None
        self.chunk = int(o.get("chunk") or 0)
        self.distance_bias = self.distance_bias2 = None
        if o.get("distance_bias"):
            rel = rt.param(tensors[p + n["rel"]], keep_dtype=True).float()           # [rows, heads]
            far = float(o["distance_bias"])
            if far <= rel.shape[0] // 2:
                raise ValueError(f"conv_attention: a bias table of {rel.shape[0]} rows has a row per distance below {rel.shape[0] // 2}, "
                                 f"which its farthest distance {far} must exceed")
            count = int(math.ceil(far)) + 1                                            # from `far` on every distance has the last row
            index = torch.tensor(distance_buckets(rel.shape[0], far, count), dtype=torch.long, device=rel.device)
            self.distance_bias = rel[index].t().contiguous()                          # [heads, count]: the bias by distance
            self.distance_bias2 = (self.distance_bias * 1.4426950408889634).contiguous()      # for the kernels that work in base 2
        self.out_name, self.gated_name = "mixer.delta", "conv_attention.gated"
        self.sink = rt.param(tensors[p + n["sink"]], keep_dtype=True).float().contiguous() if self.sink_on else None
        self.o = Linear(get(n["o"]), rt, "o")
        self.o.partials_name = "mixer.partials"
        self.rotation = position.rotation() if position is not None else None
        # What the paged attention kernels see: heads of the padded size.
        self.attn_spec = dataclasses.replace(spec, head_dim=self.padded)

    @classmethod
    def tensors(cls, spec: MixerSpec):
        n, p, o = spec.tensor_names, spec.prefix, spec.options
        W, H, G, D = spec.hidden_size, spec.num_heads, spec.num_kv_heads, spec.head_dim
        V = int(o.get("value_dim", D))
        taps, bias, row_norm, sink, gate = _flags(o)
        std = lambda fan_in: ("normal", fan_in ** -0.5)
        rows = {"q": H * D}
        if spec.kv_source is None:
            rows.update({"k": G * D, "v": G * V})
        out = [TensorDecl(p + n["o"], (W, H * V), std(H * V))]
        if o.get("out_bias", False):
            out.append(TensorDecl(p + n["o"] + n["bias_suffix"], (W,), ("normal", 0.1)))
        for k, r in rows.items():
            out.append(TensorDecl(p + n[k], (r, W), std(W)))
            if bias:
                out.append(TensorDecl(p + n[k] + n["bias_suffix"], (r,), ("normal", 0.1)))
            if taps:
                out.append(TensorDecl(p + n[k] + n["conv_suffix"], (r, taps), ("const_plus_normal", 1.0 / taps, 0.3)))
            if row_norm and k != "v" and o.get("norm_weight", True):
                out.append(TensorDecl(p + n[k] + n["norm_suffix"], (D if o.get("head_norm", False) else r,), ("one_plus_normal", 0.1)))
        if sink:
            out.append(TensorDecl(p + n["sink"], (H,), ("normal", 1.0), keep_dtype=True))
        if gate:
            out.append(TensorDecl(p + n["g"], (H if o.get("gate") == "head" else H * V, W), std(W)))
        if o.get("distance_bias"):
            out.append(TensorDecl(p + n["rel"], (int(o.get("distance_rows", 16)), H), ("normal", 1.0), keep_dtype=True, free_dims=(0,)))
        return out

    def cache_request(self):
        out = []
        if self.own_kv:
            out.append(CacheRequest("paged_kv", kv_heads=self.nkv, head_dim=self.padded, window=self.spec.window))
        if self.taps > 1:
            out.append(CacheRequest("state", shape=(self.taps - 1, self.channels), dtype=torch.float32))
        return tuple(out)

    def decode_plan(self, group):
        if not (self.rt.fast and self.rt.dtype == torch.bfloat16) or not self.own_kv:
            return None
        from ..kernels import fast
        return fast.SplitKvPlan(self.nkv, group.page_size, group.num_pages * group.page_size)

    def forward(self, h, step, cache):
        s, rt = self.spec, self.rt
        n = h.shape[0]
        nq, nkv, D, V, Dp, C = self.nq, self.nkv, self.dim, self.vdim, self.padded, self.channels
        rows = rt.buffer("conv_attention.rows", (n, self.proj.out_features))
        self.proj.forward(h, rows)
        q = rt.buffer("attention.q", (n, nq, Dp))
        meta = step.group(cache.group_index)
        ops.conv_attention_inputs(rows, self.bias, self.conv, self.taps, cache.state, self.q_norm, self.k_norm, s.qk_norm_eps, self.rotation,
                                  q, cache.k, cache.v, step, meta.slot_mapping, nq, nkv, D, V, Dp, cache.page_size, write_kv=self.own_kv,
                                  head_norm=self.head_norm)
        if self.taps > 1:
            ops.conv_state_update(cache.state, rows, self.bias, self.taps, step, C)
        attn = rt.buffer("attention.out", (n, nq * Dp))
        done = False
        if rt.fast:
            from ..kernels import fast
            done = fast.attention(attn, q, cache, meta, step, self.attn_spec, sink=self.sink, chunk=self.chunk, distance_bias2=self.distance_bias2)
        if not done:
            ops.attention_plain(attn, q, cache.k, cache.v, meta.block_table, step.tok_slot, step.positions, s.scale, nq, nkv, Dp,
                                cache.page_size, window=s.window or 0, sink=self.sink, chunk=self.chunk, distance_bias=self.distance_bias)
        if self.gated or Dp != V:
            y = rt.buffer(self.gated_name, (n, nq * V))
            ops.sigmoid_gate(y, attn, rows[:, C:] if self.gated else None, nq, V, Dp, per_head=self.gate_per_head)
        else:
            y = attn                                # no gate and no filling to drop: the heads' outputs as they are
        out = rt.buffer(self.out_name, (n, s.hidden_size))
        return self.o.forward(y, out, allow_partials=True)
