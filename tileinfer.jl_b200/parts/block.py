"""Arrangement of a layer's parts. ``pre_norm``: x += mixer(norm1(x)); x += ffn(norm2(x)). ``parallel``: x += mixer(h) + ffn(h),
h = norm1(x), on a 32-bit stream.
``post_norm``: x += m norm1(mixer(x)); x += m norm2(ffn(x)); x += m token_input(x), on a 32-bit stream.
``sandwich``: x += norm1b(mixer(norm1(x))); x += norm2b(ffn(norm2(x))), on a 32-bit stream.
``hyper``: pre-norm sublayers that read, rewrite and write to several copies of a 32-bit stream through learned tables.

Each residual add is fused with the norm that follows it, so a block receives the already
normed input ``h`` and produces the next block's normed input with ``next_norm`` (the next
block's mixer norm, or the model's final norm), as AntoineBut/TileInfer.jl's step does
(src/model/decoder.jl:173-192).
"""
from __future__ import annotations

import torch

from ..config.spec import TensorDecl
from ..kernels import ops
from .base import register_block
from .norm import StreamCast


def _no_out_bias(mixer, block: str):
    if getattr(mixer, "out_bias", None) is not None:
        raise ValueError(f"a {block} block does not add the bias of a mixer's output projection")


@register_block("pre_norm")
class PreNormBlock:
    def __init__(self, spec, mixer, feed_forward, mixer_norm, feed_forward_norm):
        _no_out_bias(mixer, "pre_norm")
        self.spec = spec
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm

    @property
    def input_norm(self):
        return self.mixer_norm

    def forward(self, x, h, step, cache, next_norm, h_out):
        """x: residual stream (updated in place); h = input_norm(x); writes next_norm(x) to h_out."""
        delta = self.mixer.forward(h, step, cache)
        self.feed_forward_norm.add_forward(x, delta, h)
        delta = self.feed_forward.forward(h, step)
        next_norm.add_forward(x, delta, h_out)
        return h_out


@register_block("post_norm")
class PostNormBlock:
    """The norm sits on each sublayer's output, the sublayers read the stream itself, and every branch is added with
    the multiplier ``residual_mult`` of the layer's options: x += m * norm1(mixer(x)); x += m * norm2(ffn(x)) (a layer
    may have no feed-forward); then, if the layer has a token input, x += m * its normalised output. The stream x is
    32-bit; ``h`` is its rounding to the products' element type, rewritten by the kernel that updates x. The norms
    are of a kind that offers ``branch_add`` (``rmsnorm32``)."""

    def __init__(self, spec, mixer, feed_forward, mixer_norm, feed_forward_norm, token_input=None):
        _no_out_bias(mixer, "post_norm")
        self.spec = spec
        self.mixer, self.feed_forward, self.token_input = mixer, feed_forward, token_input
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self.mult = float(spec.options.get("residual_mult", 1.0))
        self._cast = StreamCast()

    @property
    def input_norm(self):
        return self._cast

    def forward(self, x, h, step, cache, next_norm, h_out):
        branches = [(self.mixer_norm, lambda: self.mixer.forward(h, step, cache))]
        if self.feed_forward is not None:
            branches.append((self.feed_forward_norm, lambda: self.feed_forward.forward(h, step)))
        if self.token_input is not None:
            branches.append((self.token_input.norm, lambda: self.token_input.forward(h, step)))
        for i, (norm, run) in enumerate(branches):
            delta = run()
            last = i + 1 == len(branches)
            norm.branch_add(x, delta, self.mult, h_out if last else h, next_norm if last else self._cast)
        return h_out


@register_block("parallel")
class ParallelBlock:
    """One norm, and both sublayers read its output: h = norm1(x); x += mixer(h) + ffn(h) (a layer may have no feed-forward).
    The stream x is 32-bit; the two outputs are added to it by one kernel that also writes the next reader's normed input. The
    norms are of a kind that offers ``sum_add`` (``rmsnorm32``)."""

    def __init__(self, spec, mixer, feed_forward, mixer_norm, feed_forward_norm=None):
        _no_out_bias(mixer, "parallel")
        self.spec = spec
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, None

    @property
    def input_norm(self):
        return self.mixer_norm

    def forward(self, x, h, step, cache, next_norm, h_out):
        d1 = self.mixer.forward(h, step, cache)
        d2 = self.feed_forward.forward(h, step) if self.feed_forward is not None else None
        next_norm.sum_add(x, d1, d2, h_out)
        return h_out


@register_block("sandwich")
class SandwichBlock:
    """A norm before and after each sublayer: x += post1(mixer(pre1(x))); x += post2(ffn(pre2(x))) (a layer may have no
    feed-forward). The stream x is 32-bit. The kernel that norms a sublayer's output and adds it to x also writes the next
    reader's normed input, so the block receives h = pre1(x) and leaves ``next_norm``(x) in ``h_out``. A mixer whose output
    projection has a bias (``mixer.out_bias``) leaves the bias to that kernel, which adds it before the norm. The norms are of a
    kind that offers ``branch_add`` (``rmsnorm32``, ``layernorm32``)."""

    def __init__(self, spec, mixer, feed_forward, mixer_norm, feed_forward_norm, mixer_post_norm=None, feed_forward_post_norm=None):
        if mixer_post_norm is None or (feed_forward is not None and (feed_forward_norm is None or feed_forward_post_norm is None)):
            raise ValueError("a sandwich block needs a norm before and after each of its sublayers")
        self.spec = spec
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self.mixer_post_norm, self.feed_forward_post_norm = mixer_post_norm, feed_forward_post_norm

    @property
    def input_norm(self):
        return self.mixer_norm

    def forward(self, x, h, step, cache, next_norm, h_out):
        delta = self.mixer.forward(h, step, cache)
        bias = getattr(self.mixer, "out_bias", None)
        if self.feed_forward is None:
            self.mixer_post_norm.branch_add(x, delta, 1.0, h_out, next_norm, bias=bias)
            return h_out
        self.mixer_post_norm.branch_add(x, delta, 1.0, h, self.feed_forward_norm, bias=bias)
        delta = self.feed_forward.forward(h, step)
        self.feed_forward_post_norm.branch_add(x, delta, 1.0, h_out, next_norm)
        return h_out


class StreamsRead:
    """Stands where a block's input norm would when the stream has several copies: h = norm(sum_s a[s] x_s) for x [n, S * size],
    ``a`` the reader's blend (all ones: the sum of the copies, what the model's final norm reads)."""

    def __init__(self, norm, blend, rt):
        self.norm, self.blend = norm, [float(v) for v in blend]
        self.blend_device = torch.tensor(self.blend, dtype=torch.float32, device=rt.device)

    def read_args(self):
        return self.norm.read_args()

    def forward(self, x, out):
        w, b, eps, centred = self.norm.read_args()
        ops.streams_read_norm(out, x, self.blend_device, w, b, eps, centred)
        return out


@register_block("hyper")
class HyperBlock:
    """Pre-norm sublayers on S copies x_1 .. x_S of a 32-bit stream (hyper-connections). For sublayer q (the mixer, then the
    feed-forward, which a layer may lack), with learned a_q [S], c_q [S] and M_q [S, S] (indexed [from, to]):

        u = sum_s a_q[s] x_s;   y = sublayer(norm_q(u));   x_t <- sum_s M_q[s, t] x_s + m c_q[t] y   for all t at once

    m is the option ``residual_mult``. With ``streams`` 0 there is one stream and x += m sublayer(norm(x)): the same kernels with
    S = 1, a = c = [1], M = [[1]]. Option ``tensors``: {1: {"in", "out", "mix"}, 2: {...}} names the learned tables. The kernel that
    writes a sublayer's output back also makes the next reader's normed input, so the block receives h = norm_1(u) and leaves the next
    block's (or the final norm's) input in ``h_out``; the norms are of a kind that offers ``read_args`` (``layernorm32``)."""

    def __init__(self, spec, mixer, feed_forward, mixer_norm, feed_forward_norm, tensors=None, rt=None):
        _no_out_bias(mixer, "hyper")
        self.spec = spec
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        o = spec.options
        self.mult = float(o.get("residual_mult", 1.0))
        self.streams = S = max(1, int(o.get("streams") or 0))
        self.tables = {}
        for q in (1, 2) if feed_forward is not None else (1,):
            if o.get("streams"):
                names = o["tensors"][q]
                get = lambda k: tensors[names[k]].detach().to("cpu", torch.float32)
                a, c, M = get("in").flatten().tolist(), get("out").flatten().tolist(), get("mix").flatten().tolist()
            else:
                a, c, M = [1.0], [1.0], [1.0]
            self.tables[q] = (a, [self.mult * v for v in c], M)
        rt = rt if rt is not None else mixer.rt
        self._read1 = StreamsRead(mixer_norm, self.tables[1][0], rt)
        self._read2 = StreamsRead(feed_forward_norm, self.tables[2][0], rt) if feed_forward is not None else None

    @classmethod
    def tensors(cls, spec):
        o = spec.options
        S = int(o.get("streams") or 0)
        out = []
        if S:
            for q in (1, 2):
                if q == 2 and spec.feed_forward is None:
                    continue
                names = o["tensors"][q]
                out += [TensorDecl(names["in"], (S,), ("const_plus_normal", 1.0 / S, 0.1), keep_dtype=True),
                        TensorDecl(names["out"], (S,), ("const_plus_normal", 1.0, 0.2), keep_dtype=True),
                        TensorDecl(names["mix"], (S, S), ("const_plus_normal", 1.0 / S, 0.15), keep_dtype=True)]
        return out

    @property
    def input_norm(self):
        return self._read1

    def _next(self, nxt):
        """(blend, norm arguments) of whoever reads the stream next: another reader of copies, or a norm that reads their sum."""
        if isinstance(nxt, StreamsRead):
            return nxt.blend, nxt.read_args()
        return [1.0] * self.streams, nxt.read_args()

    def forward(self, x, h, step, cache, next_norm, h_out):
        a1, c1, M1 = self.tables[1]
        delta = self.mixer.forward(h, step, cache)
        if self.feed_forward is None:
            blend, (w, b, eps, centred) = self._next(next_norm)
            ops.streams_update(x, delta, M1, c1, blend, h_out, w, b, eps, centred)
            return h_out
        w, b, eps, centred = self._read2.read_args()
        ops.streams_update(x, delta, M1, c1, self._read2.blend, h, w, b, eps, centred)
        a2, c2, M2 = self.tables[2]
        delta = self.feed_forward.forward(h, step)
        blend, (w, b, eps, centred) = self._next(next_norm)
        ops.streams_update(x, delta, M2, c2, blend, h_out, w, b, eps, centred)
        return h_out
