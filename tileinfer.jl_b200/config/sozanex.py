"""Typed configuration of the Sozanex design and its lowering to per-layer records.

A Sozanex model is a decoder whose config.json lists its layers one by one (``layers``: ``type``, ``mixer``, ``mlp``), so every
layer may have sizes of its own. What the design fixes lives here and in the parts; what config.json gives is read from it and
nowhere else:

* the stream starts as ``embedding.scale`` times the token's embedding row plus, with ``embedding.bigram``, a row of a second
  table chosen by a hash of the token and the one before it (an extra last row for a sequence's first token); it is kept in 32-bit;
* ``loop``: the layers ``start .. stop - 1`` run ``times`` times in a row with the same weights (every run with a cache of its
  own), and before the first layer of every such pass the stream s becomes P concat(s, e), e being the embedding's output;
* a layer has a layer norm (a weight, no bias) before AND after each sublayer: x += n1b(mixer(n1(x))); x += n2b(ff(n2(x)));
  the model ends with such a norm and the head;
* mixer ``attention``: grouped-query attention (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``) with biases on q, k, v and
  the output, an RMS norm of every query and key head with one weight per projection, a rotation of the first ``rot.dims``
  elements of every head (half-split pairs) whose frequencies may be rescaled band by band (``rot.scaling``: factor, low, high,
  original), and a window of ``mask.size`` keys;
* mixer ``latent_attention``: queries through a normed latent of ``q_rank``; keys and values from a normed latent of ``kv_rank``
  that is all the cache keeps, beside ONE rotated key part of ``rot_dim`` elements shared by the heads (interleaved pairs, YaRN
  scaling ``rot.scaling``: factor, original, fast, slow); every earlier position is visible; a learned sink per head in the
  softmax's denominator; a sigmoid output gate computed from the mixer's input;
* feed-forward ``dense``: down(max(up h, 0)^2); or none.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .apertus import ConfigError, _require
from .spec import (FeedForwardSpec, LayerSpec, Llama3RopeScaling, MixerSpec, ModelSpec, NormSpec, PassInputSpec, PositionSpec,
                   YarnRopeScaling)

DEFAULT_MAX_POSITIONS = 131072       # config.json gives no limit; tables are sized by the engine's max_context below this


def _need(m: Mapping[str, Any], key: str, where: str):
    if not isinstance(m, Mapping) or key not in m or m[key] is None:
        raise ConfigError(f"config.json: {where} has no \"{key}\"")
    return m[key]


@dataclass(frozen=True)
class RotationConfig:
    dims: int
    base: float
    scaling: Optional[Any]             # Llama3RopeScaling (attention) | YarnRopeScaling (latent attention) | None

    @classmethod
    def from_dict(cls, r, where, yarn: bool):
        s = r.get("scaling")
        scaling = None
        if s:
            w = where + ".scaling"
            if yarn:
                scaling = YarnRopeScaling(float(_need(s, "factor", w)), float(_need(s, "original", w)), float(_need(s, "fast", w)),
                                          float(_need(s, "slow", w)))
            else:
                scaling = Llama3RopeScaling(float(_need(s, "factor", w)), float(_need(s, "low", w)), float(_need(s, "high", w)),
                                            int(_need(s, "original", w)))
                if scaling.high_freq_factor == scaling.low_freq_factor:
                    raise ConfigError(f"{w}: low and high must differ")
            if scaling.factor <= 0:
                raise ConfigError(f"{w}.factor must be positive")
        out = cls(int(_need(r, "dims", where)), float(_need(r, "base", where)), scaling)
        if out.dims < 2 or out.dims % 2:
            raise ConfigError(f"{where}.dims {out.dims} must be even and at least 2")
        return out

    def to_dict(self):
        d = {"base": self.base, "dims": self.dims}
        s = self.scaling
        if isinstance(s, YarnRopeScaling):
            d["scaling"] = {"factor": s.factor, "fast": s.fast, "original": s.original, "slow": s.slow}
        elif s is not None:
            d["scaling"] = {"factor": s.factor, "high": s.high_freq_factor, "low": s.low_freq_factor,
                            "original": s.original_max_position_embeddings}
        return d


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]              # mask.size; None: every earlier position is visible
    rot: Optional[RotationConfig]

    @classmethod
    def from_dict(cls, m, where):
        rot, mask = m.get("rot"), m.get("mask")
        out = cls(int(_need(m, "heads", where)), int(m.get("kv_heads") or _need(m, "heads", where)), int(_need(m, "dim", where)),
                  int(m.get("vdim") or _need(m, "dim", where)), float(_need(m, "scale", where)),
                  None if not mask else int(_need(mask, "size", where + ".mask")),
                  None if not rot else RotationConfig.from_dict(rot, where + ".rot", yarn=False))
        if min(out.heads, out.kv_heads, out.dim, out.vdim) < 1 or out.heads % out.kv_heads:
            raise ConfigError(f"{where}: {out.heads} query heads do not divide into {out.kv_heads} key/value heads")
        if out.rot is not None and out.rot.dims > out.dim:
            raise ConfigError(f"{where}.rot.dims {out.rot.dims} exceeds dim {out.dim}")
        if out.window is not None and out.window < 1:
            raise ConfigError(f"{where}.mask.size must be positive")
        return out

    def to_dict(self):
        d = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.window is not None:
            d["mask"] = {"size": self.window}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int                           # unrotated query/key size of a head
    rot_dim: int                       # rotated query/key size (the key's part is shared by the heads); 0: none
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot: Optional[RotationConfig]

    @classmethod
    def from_dict(cls, m, where):
        rot = m.get("rot")
        out = cls(int(_need(m, "heads", where)), int(_need(m, "dim", where)), int(m.get("rot_dim") or 0), int(_need(m, "vdim", where)),
                  int(_need(m, "q_rank", where)), int(_need(m, "kv_rank", where)), float(_need(m, "scale", where)),
                  None if not rot else RotationConfig.from_dict(rot, where + ".rot", yarn=True))
        if min(out.heads, out.dim, out.vdim, out.q_rank, out.kv_rank) < 1 or out.rot_dim < 0:
            raise ConfigError(f"{where}: heads, dim, vdim, q_rank and kv_rank must be positive")
        if (out.rot_dim > 0) != (out.rot is not None) or (out.rot is not None and out.rot.dims != out.rot_dim):
            raise ConfigError(f"{where}: the rotated part of {out.rot_dim} elements needs a rotation of as many (rot.dims)")
        if m.get("mask"):
            raise ConfigError(f"{where}.mask: this mixer sees every earlier position; only the attention mixer has a window")
        return out

    def to_dict(self):
        d = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "q_rank": self.q_rank, "scale": self.scale, "vdim": self.vdim}
        if self.rot_dim:
            d["rot_dim"] = self.rot_dim
            d["rot"] = self.rot.to_dict()
        return d


@dataclass(frozen=True)
class MlpConfig:
    kind: str                          # "dense"
    ff: int

    @classmethod
    def from_dict(cls, m, where):
        kind = _need(m, "kind", where)
        if kind != "dense":
            raise ConfigError(f"{where}.kind \"{kind}\" is not a feed-forward of this design (dense)")
        out = cls("dense", int(_need(m, "ff", where)))
        if out.ff < 1:
            raise ConfigError(f"{where}.ff must be positive")
        return out

    def to_dict(self):
        return {"ff": self.ff, "kind": self.kind}


@dataclass(frozen=True)
class BigramConfig:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class SozanexLayerConfig:
    type: str                          # "attention" | "latent_attention"
    mixer: Any
    mlp: Optional[MlpConfig]


_MIXERS = {"attention": AttentionConfig, "latent_attention": LatentAttentionConfig}


@dataclass(frozen=True)
class SozanexConfig:
    vocab: int
    width: int
    norm_eps: float
    embed_scale: float
    bigram: Optional[BigramConfig]
    loop: Optional[LoopConfig]
    layers: Tuple[SozanexLayerConfig, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: Tuple[int, ...] = ()

    architecture = "Sozanex"
    model_type = "sozanex"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, c: Mapping[str, Any]) -> "SozanexConfig":
        layers = []
        for i, l in enumerate(_require(c, "layers")):
            where = f"layers[{i}]"
            kind = _need(l, "type", where)
            if kind not in _MIXERS:
                raise ConfigError(f"{where}.type \"{kind}\" is not a mixer of this design ({', '.join(_MIXERS)})")
            mlp = l.get("mlp")
            layers.append(SozanexLayerConfig(kind, _MIXERS[kind].from_dict(_need(l, "mixer", where), where + ".mixer"),
                                             None if mlp is None else MlpConfig.from_dict(mlp, where + ".mlp")))
        e = c.get("embedding") or {}
        b = e.get("bigram")
        bigram = None
        if b:
            bigram = BigramConfig(int(_need(b, "buckets", "embedding.bigram")), int(_need(b, "mul_prev", "embedding.bigram")),
                                  int(_need(b, "mul_cur", "embedding.bigram")))
            if bigram.buckets < 1:
                raise ConfigError("embedding.bigram.buckets must be positive")
        lp = c.get("loop")
        loop = None
        if lp:
            loop = LoopConfig(int(_need(lp, "start", "loop")), int(_need(lp, "stop", "loop")), int(_need(lp, "times", "loop")))
            if not 0 <= loop.start < loop.stop <= len(layers) or loop.times < 1:
                raise ConfigError(f"loop: layers {loop.start} .. {loop.stop - 1} run {loop.times} times, of {len(layers)} layers")
        eos = c.get("eos_token_id", ())
        eos = (eos,) if isinstance(eos, int) else tuple(eos or ())
        out = cls(vocab=int(_require(c, "vocab")), width=int(_require(c, "width")), norm_eps=float(_need(_require(c, "norm"), "eps", "norm")),
                  embed_scale=float(e.get("scale", 1.0)), bigram=bigram, loop=loop, layers=tuple(layers),
                  max_positions=int(c.get("max_positions") or DEFAULT_MAX_POSITIONS), eos_token_ids=eos)
        if out.vocab < 1 or out.width < 1 or not layers:
            raise ConfigError("vocab and width must be positive and layers not empty")
        return out

    def to_dict(self) -> dict:
        e = {"scale": self.embed_scale}
        if self.bigram is not None:
            e["bigram"] = {"buckets": self.bigram.buckets, "mul_cur": self.bigram.mul_cur, "mul_prev": self.bigram.mul_prev}
        d = {"architecture": self.architecture, "embedding": e,
             "layers": [{"mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict(), "type": l.type} for l in self.layers],
             "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.loop is not None:
            d["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    def layer_order(self) -> Tuple[Tuple[int, ...], Tuple[int, ...]]:
        """(the layers in the order they run, the places in that order where a pass of the loop starts)."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(range(n)), ()
        a, b, times = self.loop.start, self.loop.stop, self.loop.times
        order = tuple(range(a)) + tuple(range(a, b)) * times + tuple(range(b, n))
        return order, tuple(a + k * (b - a) for k in range(times))

    def model_spec(self) -> ModelSpec:
        W, eps = self.width, self.norm_eps
        norm = lambda name: NormSpec("layernorm32", W, eps, name, {"init_std": 0.1})
        rope_options = lambda dims, pairing: {"rotary_dim": dims, "pairing": pairing, "table_dtype": "float32", "angles": "float64"}
        layers = []
        for i, l in enumerate(self.layers):
            p = f"l{i}."
            m = l.mixer
            position = PositionSpec(kind="none")
            if l.type == "attention":
                if m.rot is not None:
                    position = PositionSpec(kind="rope", head_dim=m.dim, theta=m.rot.base, scaling=m.rot.scaling,
                                            max_positions=self.max_positions, options=rope_options(m.rot.dims, "half"))
                mixer = MixerSpec(kind="conv_attention", prefix=p + "mix.", hidden_size=W, num_heads=m.heads, num_kv_heads=m.kv_heads,
                                  head_dim=m.dim, qk_norm=True, qk_norm_eps=eps, scale=m.scale, window=m.window, position=position,
                                  tensor_names={"q": "q", "k": "k", "v": "v", "o": "o", "bias_suffix": ".b", "norm_suffix": ".norm"},
                                  options={"value_dim": m.vdim, "conv_taps": 0, "bias": True, "out_bias": True, "row_norm": True,
                                           "head_norm": True, "sink": False, "gate": False})
            else:
                if m.rot is not None:
                    position = PositionSpec(kind="rope", head_dim=m.rot_dim, theta=m.rot.base, scaling=m.rot.scaling,
                                            max_positions=self.max_positions, options=rope_options(m.rot.dims, "interleaved"))
                mixer = MixerSpec(kind="latent_attention", prefix=p + "mix.", hidden_size=W, num_heads=m.heads, num_kv_heads=1,
                                  head_dim=m.dim, scale=m.scale, window=None, position=position,
                                  tensor_names={"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm",
                                                "uk": "uk", "uv": "uv", "o": "o", "sink": "sink", "g": "g"},
                                  options={"value_dim": m.vdim, "q_rank": m.q_rank, "kv_rank": m.kv_rank, "latent_norm_eps": eps,
                                           "rot_dim": m.rot_dim, "sink": True, "gate": True})
            ffn = n2 = n2b = None
            if l.mlp is not None:
                ffn = FeedForwardSpec("gelu_mlp", p + "mlp.", W, l.mlp.ff, {"up": "up", "down": "down"},
                                      {"activation": "relu2", "init_std_up": W ** -0.5, "init_std_down": l.mlp.ff ** -0.5})
                n2, n2b = norm(p + "norm2"), norm(p + "norm2b")
            layers.append(LayerSpec("sandwich", mixer, norm(p + "norm1"), ffn, n2, mixer_post_norm=norm(p + "norm1b"),
                                    feed_forward_post_norm=n2b))
        order, starts = self.layer_order()
        options = {"residual_dtype": "float32", "embed_init_std": 1.0, "embed_scale": self.embed_scale}
        if self.bigram is not None:
            options.update({"pair_table": "bigram", "pair_buckets": self.bigram.buckets, "pair_mul_prev": self.bigram.mul_prev,
                            "pair_mul_cur": self.bigram.mul_cur, "pair_init_std": 1.0})
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=W, layers=tuple(layers), order=order,
            final_norm=norm("final.norm"), embed_name="embed", lm_head_name="head", max_positions=self.max_positions,
            eos_token_ids=self.eos_token_ids, init_std=W ** -0.5, embedding_kind="scaled_pair32", head_kind="linear", options=options,
            pass_input=PassInputSpec("concat_linear", W, "loop.in", starts) if starts else None)
