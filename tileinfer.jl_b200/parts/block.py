"""Arrangement of a layer's parts. ``pre_norm``: x += mixer(norm1(x)); x += ffn(norm2(x)). ``parallel``: x += mixer(h) + ffn(h),
h = norm1(x), on a 32-bit stream.
``post_norm``: x += m norm1(mixer(x)); x += m norm2(ffn(x)); x += m token_input(x), on a 32-bit stream.
``sandwich``: x += norm1b(mixer(norm1(x))); x += norm2b(ffn(norm2(x))), on a 32-bit stream.

Each residual add is fused with the norm that follows it, so a block receives the already
normed input ``h`` and produces the next block's normed input with ``next_norm`` (the next
block's mixer norm, or the model's final norm), as AntoineBut/TileInfer.jl's step does
(src/model/decoder.jl:173-192).
"""
from __future__ import annotations

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
