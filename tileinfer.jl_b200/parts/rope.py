"""Rotary position embedding with optional llama3 frequency scaling.

Tables are computed once on the host the way AntoineBut/TileInfer.jl does
(src/model/rope.jl:15-48): inverse frequencies and angles in 32-bit, cos/sin in 64-bit of
the 32-bit angle, rounded to 32-bit and then to the model's element type. The scaling is
static: it does not depend on the running sequence length. The device table is
``[max_positions, rotary_dim/2, 2]`` float32 holding (cos, sin) already rounded to the
element type; both elements of a pair share the angle.

Two options of the record go beyond what Apertus uses: ``rotary_dim`` (rotate only the first so
many elements of a head; default: all) and ``pairing`` ("half": element i with i + rotary_dim/2,
the default; "interleaved": 2i with 2i + 1). ``table_dtype`` "float32" keeps cos and sin unrounded in a bfloat16 model, and
``angles`` "float64" computes frequencies (their scaling included) and angles in 64-bit and rounds cos and sin once, for
mixers that rotate in 32-bit.

Besides the band-wise scaling of Llama 3 (:class:`Llama3RopeScaling`) the record may carry a :class:`YarnRopeScaling`: with
d(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), dims - 1) and
ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns at f_i / factor * ramp_i + f_i (1 - ramp_i), and the
table's cos and sin are multiplied by 0.1 ln(factor) + 1 (so a rotated vector grows by that factor).
"""
from __future__ import annotations

import math

import torch

from ..config.spec import Llama3RopeScaling, PositionSpec, YarnRopeScaling
from .base import PositionEncoding, Rotation, register_position


def rotary_dim(spec: PositionSpec) -> int:
    D = int(spec.options.get("rotary_dim", spec.head_dim))
    if D < 2 or D % 2 or D > spec.head_dim:
        raise ValueError(f"rotary_dim {D} must be even and between 2 and the head size {spec.head_dim}")
    return D


def inverse_frequencies(spec: PositionSpec) -> torch.Tensor:
    D = rotary_dim(spec)
    theta = torch.tensor(float(spec.theta), dtype=torch.float32)
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float32) / torch.tensor(float(D), dtype=torch.float32)))
    s = spec.scaling
    if s is None:
        return inv
    f32 = lambda v: torch.tensor(float(v), dtype=torch.float32)
    factor, low, high = f32(s.factor), f32(s.low_freq_factor), f32(s.high_freq_factor)
    old = f32(s.original_max_position_embeddings)
    wavelen = 2.0 * f32(math.pi) / inv
    smooth = (old / wavelen - low) / (high - low)
    blended = (1 - smooth) * inv / factor + smooth * inv
    return torch.where(wavelen < old / high, inv, torch.where(wavelen > old / low, inv / factor, blended))


def scaled_frequencies64(spec: PositionSpec):
    """(the pairs' frequencies after the record's scaling, the multiplier of cos and sin), in 64-bit."""
    D = rotary_dim(spec)
    base = float(spec.theta)
    f = [base ** (-2.0 * i / D) for i in range(D // 2)]
    s = spec.scaling
    if s is None:
        return f, 1.0
    if isinstance(s, YarnRopeScaling):
        where = lambda t: D * math.log(s.original / (2.0 * math.pi * t)) / (2.0 * math.log(base))
        lo, hi = max(math.floor(where(s.fast)), 0), min(math.ceil(where(s.slow)), D - 1)
        out = []
        for i, fi in enumerate(f):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(fi / s.factor * ramp + fi * (1.0 - ramp))
        return out, 0.1 * math.log(s.factor) + 1.0
    if isinstance(s, Llama3RopeScaling):
        old, low, high = float(s.original_max_position_embeddings), float(s.low_freq_factor), float(s.high_freq_factor)
        out = []
        for fi in f:
            wavelength = 2.0 * math.pi / fi
            if wavelength < old / high:
                out.append(fi)
            elif wavelength > old / low:
                out.append(fi / s.factor)
            else:
                smooth = (old / wavelength - low) / (high - low)
                out.append((1.0 - smooth) * fi / s.factor + smooth * fi)
        return out, 1.0
    raise ValueError(f"rope: a scaling of type {type(s).__name__} is not known")


@register_position("rope")
class RotaryEmbedding(PositionEncoding):
    def __init__(self, spec: PositionSpec, rt, max_positions: int):
        self.spec = spec
        self.max_positions = int(min(max_positions, spec.max_positions) if spec.max_positions else max_positions)
        exact = spec.options.get("angles") == "float64"
        if isinstance(spec.scaling, YarnRopeScaling) and not exact:
            raise ValueError("rope: YaRN scaling is built for tables with 64-bit angles (options[\"angles\"] = \"float64\")")
        inv = inverse_frequencies(spec) if not exact else None
        self.rotary_dim = rotary_dim(spec)
        pairing = spec.options.get("pairing", "half")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"rope pairing must be \"half\" or \"interleaved\", not {pairing!r}")
        self.interleaved = pairing == "interleaved"
        table = torch.empty(self.max_positions, self.rotary_dim // 2, 2, dtype=torch.float32)
        if exact:                                            # frequencies and angles in 64-bit, one rounding of cos and sin
            f, mult = scaled_frequencies64(spec)
            f = torch.tensor(f, dtype=torch.float64)
        # In blocks, to bound the 64-bit scratch for long contexts.
        for p0 in range(0, self.max_positions, 1 << 15):
            p1 = min(self.max_positions, p0 + (1 << 15))
            if exact:
                ang = torch.arange(p0, p1, dtype=torch.float64)[:, None] * f[None, :]
                table[p0:p1, :, 0], table[p0:p1, :, 1] = (ang.cos() * mult).float(), (ang.sin() * mult).float()
            else:
                ang = torch.arange(p0, p1, dtype=torch.float32)[:, None] * inv[None, :]
                table[p0:p1, :, 0] = ang.double().cos().float()
                table[p0:p1, :, 1] = ang.double().sin().float()
        if rt.dtype != torch.float32 and spec.options.get("table_dtype") != "float32":
            table = table.to(rt.dtype).float()
        self.cos_sin = table.contiguous().to(rt.device)

    def rotation(self) -> Rotation:
        return Rotation(self.cos_sin, self.rotary_dim, self.interleaved)


@register_position("none")
class NoPosition(PositionEncoding):
    def __init__(self, spec, rt, max_positions):
        self.spec = spec
        self.max_positions = max_positions
