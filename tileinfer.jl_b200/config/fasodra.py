"""Typed configuration of the Fasodra design and its lowering to per-layer records.

A Fasodra model is a decoder whose config.json lists its layers one by one (``layers``: ``type``, ``mixer``, ``mlp``), so every
layer may have sizes of its own. What the design fixes lives here and in the parts; what config.json gives is read from it and
nowhere else:

* the stream is 32-bit; a layer is x += m f(norm(x)) per sublayer with a layer norm that has a weight and a bias, m =
  ``residual_mult``; with ``streams`` = s > 0 there are s copies of the stream that every sublayer reads through a learned
  vector, rewrites through a learned s x s matrix and writes to through a second vector (hyper-connections), and whose sum the
  final norm reads;
* mixer ``attention``: grouped-query attention with biases on q, k, v, every query and key head divided by its root mean square
  (no weight), no rotation, a learned bias per (distance bucket, head) added to the scaled score, and with ``mask.size`` a key
  is visible only inside the query's chunk of so many positions, counted from the sequence's start;
* mixer ``parallel``: two mixers read the same input and their outputs are added with ``left_scale`` and ``right_scale``: causal
  attention with a rotation of the first ``rot.dims`` elements of every head and one sigmoid gate per head, beside a time-mixing
  recurrence whose inputs blend the token's row with the one before it and whose decay depends on the token;
* mixer ``parallel_2``: causal attention with a weighted RMS norm of every query and key head before the rotation, beside a gated
  delta rule behind short convolutions; each output is RMS-normed over the model's width and the result is half their sum;
* feed-forward ``moe``: a softmax router, the ``top`` best of ``experts`` units down(max(up h, 0)^2), weights divided by their sum.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .apertus import ConfigError, _require
from .spec import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec

DEFAULT_MAX_POSITIONS = 131072       # config.json gives no limit; tables are sized by the engine's max_context below this


def _need(m: Mapping[str, Any], key: str, where: str):
    if not isinstance(m, Mapping) or key not in m or m[key] is None:
        raise ConfigError(f"config.json: {where} has no \"{key}\"")
    return m[key]


@dataclass(frozen=True)
class AttentionConfig:
    """Softmax attention of any of the three mixers; which options a mixer has is decided by its type."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: Optional[int] = None          # mask.size
    bias_max: Optional[float] = None     # the distance from which on the last bucket of the bias table is used
    rot_dims: int = 0
    rot_base: float = 10000.0

    @classmethod
    def from_dict(cls, m, where, biased: bool):
        rot, mask = m.get("rot"), m.get("mask")
        heads = int(_need(m, "heads", where))
        out = cls(heads, int(m.get("kv_heads") or heads), int(_need(m, "dim", where)), int(m.get("vdim") or _need(m, "dim", where)),
                  float(_need(m, "scale", where)), None if not mask else int(_need(mask, "size", where + ".mask")),
                  float(_need(m, "bias_max", where)) if biased else None,
                  0 if not rot else int(_need(rot, "dims", where + ".rot")), 10000.0 if not rot else float(_need(rot, "base", where + ".rot")))
        if min(out.heads, out.kv_heads, out.dim, out.vdim) < 1 or out.heads % out.kv_heads:
            raise ConfigError(f"{where}: {out.heads} query heads do not divide into {out.kv_heads} key/value heads")
        if out.rot_dims % 2 or out.rot_dims > out.dim:
            raise ConfigError(f"{where}.rot.dims {out.rot_dims} must be even and at most dim {out.dim}")
        if out.chunk is not None and out.chunk < 1:
            raise ConfigError(f"{where}.mask.size must be positive")
        if biased and out.bias_max <= 1:
            raise ConfigError(f"{where}.bias_max must exceed 1")
        return out

    def to_dict(self):
        d = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.bias_max is not None:
            d["bias_max"] = int(self.bias_max) if float(self.bias_max).is_integer() else self.bias_max
        if self.chunk is not None:
            d["mask"] = {"size": self.chunk}
        if self.rot_dims:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        return d


@dataclass(frozen=True)
class TimeMixConfig:
    heads: int
    dim: int

    @classmethod
    def from_dict(cls, m, where):
        out = cls(int(_need(m, "heads", where)), int(_need(m, "dim", where)))
        if min(out.heads, out.dim) < 1:
            raise ConfigError(f"{where}: heads and dim must be positive")
        return out

    def to_dict(self):
        return {"dim": self.dim, "heads": self.heads}


@dataclass(frozen=True)
class DeltaRuleConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int                            # taps of the short convolution; 0 or 1 with one tap means no history

    @classmethod
    def from_dict(cls, m, where):
        heads = int(_need(m, "heads", where))
        out = cls(heads, int(m.get("kv_heads") or heads), int(_need(m, "dim", where)), int(m.get("vdim") or _need(m, "dim", where)),
                  int(m.get("conv") or 0))
        if min(out.heads, out.kv_heads, out.dim, out.vdim) < 1 or out.heads % out.kv_heads or out.conv < 0:
            raise ConfigError(f"{where}: {out.heads} heads do not divide into {out.kv_heads} query/key heads")
        return out

    def to_dict(self):
        d = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "vdim": self.vdim}
        if self.conv:
            d["conv"] = self.conv
        return d


@dataclass(frozen=True)
class PairConfig:
    left: AttentionConfig
    right: Any                           # TimeMixConfig ("parallel") | DeltaRuleConfig ("parallel_2")
    left_scale: float = 1.0
    right_scale: float = 1.0

    def to_dict(self):
        d = {"left": self.left.to_dict(), "right": self.right.to_dict()}
        if isinstance(self.right, TimeMixConfig):
            d.update({"left_scale": self.left_scale, "right_scale": self.right_scale})
        return d


@dataclass(frozen=True)
class MoeConfig:
    ff: int
    experts: int
    top: int

    @classmethod
    def from_dict(cls, m, where):
        kind = _need(m, "kind", where)
        if kind != "moe":
            raise ConfigError(f"{where}.kind \"{kind}\" is not a feed-forward of this design (moe)")
        r = _need(m, "router", where)
        out = cls(int(_need(_need(m, "expert", where), "ff", where + ".expert")), int(_need(r, "experts", where + ".router")),
                  int(_need(r, "top", where + ".router")))
        if out.ff < 1 or not 1 <= out.top <= out.experts:
            raise ConfigError(f"{where}.router: top {out.top} of {out.experts} experts")
        return out

    def to_dict(self):
        return {"expert": {"ff": self.ff}, "kind": "moe", "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class FasodraLayerConfig:
    type: str                          # "attention" | "parallel" | "parallel_2"
    mixer: Any
    mlp: Optional[MoeConfig]


def _mixer_from_dict(kind, m, where):
    if kind == "attention":
        return AttentionConfig.from_dict(m, where, biased=True)
    left = AttentionConfig.from_dict(_need(m, "left", where), where + ".left", biased=False)
    if kind == "parallel":
        return PairConfig(left, TimeMixConfig.from_dict(_need(m, "right", where), where + ".right"),
                          float(m.get("left_scale", 1.0)), float(m.get("right_scale", 1.0)))
    if kind == "parallel_2":
        return PairConfig(left, DeltaRuleConfig.from_dict(_need(m, "right", where), where + ".right"))
    raise ConfigError(f"{where[:-6]}.type \"{kind}\" is not a mixer of this design (attention, parallel, parallel_2)")


@dataclass(frozen=True)
class FasodraConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    streams: int                       # 0: one stream and the plain residual sum
    layers: Tuple[FasodraLayerConfig, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: Tuple[int, ...] = ()

    architecture = "Fasodra"
    model_type = "fasodra"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, c: Mapping[str, Any]) -> "FasodraConfig":
        layers = []
        for i, l in enumerate(_require(c, "layers")):
            where = f"layers[{i}]"
            kind = _need(l, "type", where)
            mlp = l.get("mlp")
            layers.append(FasodraLayerConfig(kind, _mixer_from_dict(kind, _need(l, "mixer", where), where + ".mixer"),
                                             None if mlp is None else MoeConfig.from_dict(mlp, where + ".mlp")))
        eos = c.get("eos_token_id", ())
        eos = (eos,) if isinstance(eos, int) else tuple(eos or ())
        out = cls(vocab=int(_require(c, "vocab")), width=int(_require(c, "width")), norm_eps=float(_need(_require(c, "norm"), "eps", "norm")),
                  residual_mult=float(c.get("residual_mult", 1.0)), streams=int(c.get("streams") or 0), layers=tuple(layers),
                  max_positions=int(c.get("max_positions") or DEFAULT_MAX_POSITIONS), eos_token_ids=eos)
        if out.vocab < 1 or out.width < 1 or not layers:
            raise ConfigError("vocab and width must be positive and layers not empty")
        if not 0 <= out.streams <= 8:
            raise ConfigError(f"streams {out.streams}: at most 8 copies of the stream are built")
        return out

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture,
             "layers": [{"mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict(), "type": l.type} for l in self.layers],
             "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}
        if self.streams:
            d["streams"] = self.streams
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ---- lowering
    def _attention_spec(self, m: AttentionConfig, prefix: str, kind: str) -> MixerSpec:
        """``kind``: "attention" (unweighted head norms, distance bias, chunks), "gated" (rotation, a gate per head) or "normed"
        (weighted head norms, rotation)."""
        position = PositionSpec(kind="none")
        if m.rot_dims:
            position = PositionSpec(kind="rope", head_dim=m.dim, theta=m.rot_base, max_positions=self.max_positions,
                                    options={"rotary_dim": m.rot_dims, "pairing": "half", "table_dtype": "float32", "angles": "float64"})
        options = {"value_dim": m.vdim, "conv_taps": 0, "bias": True, "sink": False, "gate": "head" if kind == "gated" else False,
                   "row_norm": kind != "gated", "head_norm": kind != "gated", "norm_weight": kind == "normed"}
        if kind == "attention":
            options.update({"chunk": m.chunk, "distance_bias": m.bias_max})
        return MixerSpec(kind="conv_attention", prefix=prefix, hidden_size=self.width, num_heads=m.heads, num_kv_heads=m.kv_heads,
                         head_dim=m.dim, qk_norm=kind != "gated", qk_norm_eps=self.norm_eps, scale=m.scale, position=position,
                         tensor_names={"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "rel": "rel", "bias_suffix": ".b", "norm_suffix": ".norm"},
                         options=options)

    def model_spec(self) -> ModelSpec:
        W, eps, s = self.width, self.norm_eps, self.streams
        norm = lambda name: NormSpec("layernorm32", W, eps, name, {"init_std": 0.1, "bias": True, "bias_suffix": ".b"})
        layers = []
        for i, l in enumerate(self.layers):
            p = f"l{i}."
            m = l.mixer
            if l.type == "attention":
                mixer = self._attention_spec(m, p + "mix.", "attention")
            else:
                left = self._attention_spec(m.left, p + "mix.left.", "gated" if l.type == "parallel" else "normed")
                r = m.right
                if l.type == "parallel":
                    right = MixerSpec(kind="time_mix", prefix=p + "mix.right.", hidden_size=W, num_heads=r.heads, head_dim=r.dim,
                                      tensor_names={"r": "r", "k": "k", "v": "v", "g": "g", "o": "o", "mu": "mu.", "w1": "w1", "w2": "w2",
                                                    "w0": "w0", "u": "u", "norm": "norm"},
                                      options={"norm_eps": eps})
                    options = {"left": left, "right": right, "left_scale": m.left_scale, "right_scale": m.right_scale, "out_norm": False}
                else:
                    right = MixerSpec(kind="gated_delta", prefix=p + "mix.right.", hidden_size=W, num_heads=r.heads, num_kv_heads=r.kv_heads,
                                      head_dim=r.dim,
                                      tensor_names={"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "beta": "b", "a": "a", "A_log": "A_log",
                                                    "dt_bias": "dt_bias", "norm": "norm", "conv_suffix": ".conv"},
                                      options={"value_dim": r.vdim, "conv_taps": r.conv, "norm_eps": eps, "unit_eps": 1e-6})
                    options = {"left": left, "right": right, "left_scale": 0.5, "right_scale": 0.5, "out_norm": True, "norm_eps": eps}
                mixer = MixerSpec(kind="pair", prefix=p + "mix.", hidden_size=W, position=left.position,
                                  tensor_names={"left_out": "left.out", "right_out": "right.out"}, options=options)
            ffn = n2 = None
            if l.mlp is not None:
                x = l.mlp
                ffn = FeedForwardSpec("routed_experts", p + "mlp.", W, x.ff, {"router": "router", "expert": "e{}.", "up": "up", "down": "down"},
                                      {"experts": x.experts, "top": x.top, "limit": None, "score": "softmax", "renormalize": True,
                                       "scale_input": False, "gated": False, "activation": "relu2"})
                n2 = norm(p + "norm2")
            hyper = {"residual_mult": self.residual_mult, "streams": s}
            if s:
                hyper["tensors"] = {q: {k: f"{p}hc{q}.{k}" for k in ("in", "out", "mix")} for q in (1, 2)}
            layers.append(LayerSpec("hyper", mixer, norm(p + "norm1"), ffn, n2, options=hyper))
        options = {"residual_dtype": "float32", "embed_init_std": 1.0}
        if s:
            options["streams"] = s
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=W, layers=tuple(layers), order=tuple(range(len(layers))),
            final_norm=norm("final.norm"), embed_name="embed", lm_head_name="head", max_positions=self.max_positions,
            eos_token_ids=self.eos_token_ids, init_std=W ** -0.5, embedding_kind="lookup32", head_kind="linear", options=options)
