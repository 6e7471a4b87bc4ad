"""What rewrites the residual stream before a pass over a stretch of layers that runs several times with the same weights.

``concat_linear``: s' = P concat(s, e) for P [hidden, 2 hidden] (the stream's columns first), e being the embedding's output of the same
token. The stream is 32-bit; the product's operands are the two rows rounded to the products' element type, side by side in one
buffer, and its sums go back to the stream in 32-bit.

Interface: ``PassInput(spec, tensors, rt)``; ``begin(x0)`` once per step, after the embedding (keeps what it needs of x0);
``forward(x)`` before each pass, rewriting x in place.
"""
from __future__ import annotations

from ..config.spec import PassInputSpec, TensorDecl
from ..kernels import ops
from .base import Part, _register
from .linear import Linear


def register_pass_input(kind: str, cls=None):
    return _register("pass_input", kind, cls) if cls is not None else (lambda c: _register("pass_input", kind, c))


class PassInput(Part):
    def begin(self, x0):
        raise NotImplementedError

    def forward(self, x):
        raise NotImplementedError


@register_pass_input("concat_linear")
class ConcatLinear(PassInput):
    def __init__(self, spec: PassInputSpec, tensors, rt):
        self.spec, self.rt = spec, rt
        self.linear = Linear(rt.param(tensors[spec.weight_name]), rt, "pass_input")
        if self.linear.in_features != 2 * spec.hidden_size or self.linear.out_features != spec.hidden_size:
            raise ValueError(f"concat_linear: a weight of {tuple(self.linear.weight.shape)} for a width of {spec.hidden_size}")

    @classmethod
    def tensors(cls, spec: PassInputSpec):
        W = spec.hidden_size
        return [TensorDecl(spec.weight_name, (W, 2 * W), ("normal", spec.options.get("init_std", (2 * W) ** -0.5)))]

    def _pair(self, n):
        return self.rt.buffer("pass_input.pair", (n, 2 * self.spec.hidden_size))

    def begin(self, x0):
        W = self.spec.hidden_size
        ops.cast_rows_into(self._pair(x0.shape[0])[:, W:], x0)

    def forward(self, x):
        W = self.spec.hidden_size
        pair = self._pair(x.shape[0])
        ops.cast_rows_into(pair[:, :W], x)
        return self.linear.forward(pair, x, ops.EPI_F32_OUT)
