"""RMSNorm: normalise in 32-bit, round, then scale by the weight in the storage type
(AntoineBut/TileInfer.jl src/ops/reference.jl:17-21); fused with the residual add that
precedes it (src/ops/tile/norm.jl:48-77). No bias, no ``1 + w``."""
from __future__ import annotations

from ..config.spec import NormSpec, TensorDecl
from ..kernels import ops
from .base import Norm, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, spec: NormSpec, tensors, rt):
        self.spec, self.rt = spec, rt
        self.weight = rt.param(tensors[spec.weight_name])
        self.eps = float(spec.eps)

    @classmethod
    def tensors(cls, spec: NormSpec):
        return [TensorDecl(spec.weight_name, (spec.size,), ("one_plus_normal", spec.options.get("init_std", 0.02)))]

    def forward(self, x, out):
        ops.rmsnorm(out, x, self.weight, self.eps)
        return out

    def add_forward(self, x, delta, out):
        """x += delta; out = norm(x). ``delta`` is [n, size] in the model's element type, or 32-bit
        partial sums [s, n, size] of a product that was split over k."""
        if delta.dim() == 3:
            ops.add_rmsnorm(x, None, self.weight, out, self.eps, partials=delta)
        else:
            ops.add_rmsnorm(x, delta, self.weight, out, self.eps)
        return out


@register_norm("rmsnorm32")
class RMSNorm32(Norm):
    """RMS norm computed in 32-bit with one rounding at the end: y = x / sqrt(mean(x^2) + eps) * g(w), g(w) = w, or
    1 + w with the option ``offset`` (the checkpoint keeps the gain minus one). The input may be a 32-bit residual stream.

    Besides ``forward`` it serves blocks that normalise a sublayer's OUTPUT: ``branch_add(x, delta, mult, h, next_norm)``
    does x += mult * norm(delta) on a 32-bit stream and, in the same kernel, prepares the next reader's input
    (``next_norm``: another norm of this kind or a :class:`StreamCast`)."""

    def __init__(self, spec: NormSpec, tensors, rt):
        self.spec, self.rt = spec, rt
        self.weight = rt.param(tensors[spec.weight_name])
        self.eps = float(spec.eps)
        self.offset = bool(spec.options.get("offset", False))

    @classmethod
    def tensors(cls, spec: NormSpec):
        std = spec.options.get("init_std", 0.02)
        init = ("normal", std) if spec.options.get("offset", False) else ("one_plus_normal", std)
        return [TensorDecl(spec.weight_name, (spec.size,), init)]

    def out_args(self):
        return (self.weight, self.eps, self.offset)

    def forward(self, x, out):
        ops.norm32(out, x, self.weight, self.eps, self.offset)
        return out

    def sum_add(self, x, d1, d2, out):
        """x += d1 + d2 on a 32-bit stream (two sublayers that read the same input; ``d2`` may be None), then out = norm(x)."""
        ops.sum_add_norm32(x, d1, d2, out, self.weight, self.eps, self.offset)
        return out

    def branch_add(self, x, delta, mult, h=None, next_norm=None, bias=None):
        """``bias`` [size]: a vector added to ``delta`` before its norm (the bias of the product that made ``delta``)."""
        out_norm = next_norm.out_args() if next_norm is not None else None
        if isinstance(delta, GatheredRows):
            ops.branch_norm_add32(x, delta.rows, self.weight, self.eps, mult, self.offset, h, out_norm, gather=delta.index, bias=bias)
        else:
            ops.branch_norm_add32(x, delta, self.weight, self.eps, mult, self.offset, h, out_norm, bias=bias)
        return h


@register_norm("layernorm32")
class LayerNorm32(RMSNorm32):
    """Layer norm with a weight and no bias, in 32-bit with one rounding at the end: y = (x - mean(x)) / sqrt(var(x) + eps) * w,
    var the mean of the squared deviations. The same kernels as :class:`RMSNorm32` with the "centred" flag, so it serves the
    same blocks (``forward``, ``branch_add``, and as the ``next_norm`` of another norm's ``branch_add``)."""

    def __init__(self, spec: NormSpec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.offset = ops.NORM_CENTRED | (ops.NORM_OFFSET if spec.options.get("offset", False) else 0)
        # Option ``bias``: y + b, with b the tensor of the weight's name plus ``bias_suffix``. Only the kernels that read several copies
        # of the stream (``streams_read_norm``, ``streams_update``) take a bias; the blocks written for them ask for ``read_args``.
        self.bias = rt.param(tensors[spec.weight_name + spec.options.get("bias_suffix", ".b")]) if spec.options.get("bias") else None

    @classmethod
    def tensors(cls, spec: NormSpec):
        out = super().tensors(spec)
        if spec.options.get("bias"):
            out.append(TensorDecl(spec.weight_name + spec.options.get("bias_suffix", ".b"), (spec.size,), ("normal", spec.options.get("init_std", 0.02))))
        return out

    def read_args(self):
        """(weight, bias or None, eps, centred) for the kernels that norm a blend of the stream's copies."""
        if self.offset & ops.NORM_OFFSET:
            raise NotImplementedError("a gain stored minus one is not built for the kernels that read several copies of the stream")
        return (self.weight, self.bias, self.eps, True)

    def _no_bias(self, what):
        if self.bias is not None:
            raise NotImplementedError(f"layernorm32 with a bias does not serve {what}")

    def forward(self, x, out):
        if self.bias is None:
            return super().forward(x, out)
        ones = self.rt.ones1()
        ops.streams_read_norm(out, x, ones, self.weight, self.bias, self.eps, True)
        return out

    def out_args(self):
        self._no_bias("as the next norm of branch_add")
        return super().out_args()

    def branch_add(self, *a, **k):
        self._no_bias("branch_add")
        return super().branch_add(*a, **k)

    def sum_add(self, x, d1, d2, out):
        raise NotImplementedError("layernorm32 does not serve blocks that add two sublayers' outputs at once")


class GatheredRows:
    """A sublayer's output that is still in pieces: row t is the sum of the rows ``index[t, :]`` of ``rows`` (the units a
    token went through). A norm that offers ``branch_add`` adds them up while it reads them."""

    def __init__(self, rows, index):
        self.rows, self.index = rows, index


class StreamCast(Norm):
    """Stands where a block's input norm would: the block's sublayers read the 32-bit stream itself, rounded to the
    element type of the products."""

    def out_args(self):
        return None

    def forward(self, x, out):
        ops.cast_rows(out, x)
        return out
