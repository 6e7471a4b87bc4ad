"""Two mixers side by side: both read the same input, and their outputs are added.

    out = left_scale * L' + right_scale * R'
    L' = left(h), or with ``out_norm``: left(h) / rms(left(h) over the model's width) * w_left     (R' likewise)

The record's options ``left`` and ``right`` are the two mixers' own records (any registered kinds); ``left_scale``, ``right_scale``,
``out_norm`` (with ``norm_eps`` and the tensor names ``left_out`` / ``right_out`` of the two weights). The pair asks the cache for what
both ask (pages from one, a state from the other) and hands the layer's view to both. The sum is 32-bit and reaches the stream's
update unrounded. The position encoding of the record is the left mixer's.
"""
from __future__ import annotations

import torch

from ..config.spec import MixerSpec, TensorDecl
from ..kernels import ops
from .base import Mixer, lookup, register_mixer


@register_mixer("pair")
class MixerPair(Mixer):
    def __init__(self, spec: MixerSpec, tensors, rt, position):
        self.spec, self.rt = spec, rt
        o = spec.options
        self.left = lookup("mixer", o["left"].kind)(o["left"], tensors, rt, position)
        self.right = lookup("mixer", o["right"].kind)(o["right"], tensors, rt, None)
        for side, m in (("left", self.left), ("right", self.right)):
            if not hasattr(m, "out_name"):
                raise ValueError(f"pair: a {type(m).__name__} cannot name its output buffer, so it cannot stand beside another mixer")
            if getattr(m, "out_bias", None) is not None:
                raise ValueError("pair: the bias of a mixer's output projection is not added here")
            m.out_name = "pair." + side
            m.o.partials_name = "pair." + side + ".partials"
        self.left_scale, self.right_scale = float(o.get("left_scale", 1.0)), float(o.get("right_scale", 1.0))
        self.out_norm = bool(o.get("out_norm", False))
        self.eps = float(o.get("norm_eps", 1e-6))
        n, p = spec.tensor_names, spec.prefix
        self.w_left = rt.param(tensors[p + n["left_out"]]) if self.out_norm else None
        self.w_right = rt.param(tensors[p + n["right_out"]]) if self.out_norm else None

    @classmethod
    def tensors(cls, spec: MixerSpec):
        o, n, p = spec.options, spec.tensor_names, spec.prefix
        out = list(lookup("mixer", o["left"].kind).tensors(o["left"])) + list(lookup("mixer", o["right"].kind).tensors(o["right"]))
        if o.get("out_norm", False):
            out += [TensorDecl(p + n["left_out"], (spec.hidden_size,), ("one_plus_normal", 0.1)),
                    TensorDecl(p + n["right_out"], (spec.hidden_size,), ("one_plus_normal", 0.1))]
        return out

    def cache_request(self):
        out = []
        for m in (self.left, self.right):
            r = m.cache_request()
            if r is not None:
                out += list(r) if isinstance(r, (tuple, list)) else [r]
        return tuple(out)

    def decode_plan(self, group):
        return self.left.decode_plan(group) or self.right.decode_plan(group)

    def forward(self, h, step, cache):
        a = self.left.forward(h, step, cache)
        b = self.right.forward(h, step, cache)
        out = self.rt.buffer("pair.sum", (1, h.shape[0], self.spec.hidden_size), torch.float32)
        ops.pair_combine(out[0], a, b, self.w_left, self.w_right, self.eps, self.left_scale, self.right_scale, self.rt.dtype)
        return out                                # 32-bit, shaped like one slice of partial sums: the stream's update adds it as it is
