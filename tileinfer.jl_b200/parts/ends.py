"""The two ends of the model: the token embedding and the LM head.

AntoineBut/TileInfer.jl: ``x[t] = E[ids[t]]``, no scaling (src/ops/reference.jl:10); only the first
``vocab_size`` rows of the table are loaded (src/hub/loader.jl:155-156); the head is a product with
32-bit output, the value rounded to the storage type first (src/ops/tile/linear.jl:12-13, 26), and a
tied head is the embedding table itself (src/hub/loader.jl:157-163).
"""
from __future__ import annotations

import torch

from ..config.spec import ModelSpec, TensorDecl
from ..kernels import ops
from .base import CacheRequest, Embedding, Head, register_embedding, register_head
from .linear import Linear


@register_embedding("lookup")
class TokenEmbedding(Embedding):
    def __init__(self, spec: ModelSpec, tensors, rt):
        self.table = rt.param(tensors[spec.embed_name])

    @classmethod
    def tensors(cls, spec: ModelSpec):
        return [TensorDecl(spec.embed_name, (spec.vocab_size, spec.hidden_size), ("normal", spec.init_std), allow_extra_rows=True)]

    def forward(self, token_ids, out, status):
        ops.embed(out, self.table, token_ids, status)
        return out


@register_head("linear")
class LinearHead(Head):
    def __init__(self, spec: ModelSpec, tensors, rt, embedding):
        weight = embedding.table if spec.lm_head_name is None else rt.param(tensors[spec.lm_head_name])
        self.linear = Linear(weight, rt, "lm_head")

    @classmethod
    def tensors(cls, spec: ModelSpec):
        if spec.lm_head_name is None:
            return []
        return [TensorDecl(spec.lm_head_name, (spec.vocab_size, spec.hidden_size), ("normal", spec.init_std))]

    def forward(self, h, logits):
        return self.linear.forward(h, logits, ops.EPI_F32_OUT)


@register_embedding("lookup_learned_positions")
class PositionedEmbedding(Embedding):
    """x = E[token] + P[position]: a learned vector per position (unscaled) added to the token's row, the sum kept in
    32-bit. ``ModelSpec.options["position_table"]`` names P [max_positions, hidden]. The stream it writes is 32-bit
    (``options["residual_dtype"] == "float32"``)."""

    def __init__(self, spec: ModelSpec, tensors, rt):
        self.table = rt.param(tensors[spec.embed_name])
        self.positions = rt.param(tensors[spec.options["position_table"]])

    @classmethod
    def tensors(cls, spec: ModelSpec):
        o = spec.options
        return [TensorDecl(spec.embed_name, (spec.vocab_size, spec.hidden_size), ("normal", o.get("embed_init_std", spec.init_std))),
                TensorDecl(o["position_table"], (spec.max_positions, spec.hidden_size), ("normal", o.get("position_init_std", spec.init_std)))]

    def forward_step(self, step, out, status):
        ops.embed_positions32(out, self.table, self.positions, step.token_ids, step.positions, status)
        return out


@register_embedding("lookup32")
class TokenEmbedding32(Embedding):
    """x = E[token] written to a 32-bit stream (``options["residual_dtype"] == "float32"``), unscaled."""

    def __init__(self, spec: ModelSpec, tensors, rt):
        self.table = rt.param(tensors[spec.embed_name])

    @classmethod
    def tensors(cls, spec: ModelSpec):
        return [TensorDecl(spec.embed_name, (spec.vocab_size, spec.hidden_size), ("normal", spec.options.get("embed_init_std", spec.init_std)))]

    def forward_step(self, step, out, status):
        ops.embed_positions32(out, self.table, None, step.token_ids, step.positions, status)
        return out


@register_embedding("scaled_pair32")
class ScaledPairEmbedding(Embedding):
    """x = scale * E[token] + G[(previous token * a + token * b) mod buckets], written to a 32-bit stream. G has one more row
    than ``buckets``, which a sequence's first token takes. The options of the ModelSpec: ``embed_scale``; ``pair_table`` (the
    name of G; absent: no second table), ``pair_buckets``, ``pair_mul_prev`` (a), ``pair_mul_cur`` (b).

    The previous token of a step's first token is the last token of the step before: the part asks the cache for one 32-bit
    integer per sequence (``cache_request``), reads it where a sequence continues and rewrites it after every step."""

    def __init__(self, spec: ModelSpec, tensors, rt):
        o = spec.options
        self.table = rt.param(tensors[spec.embed_name])
        self.scale = float(o.get("embed_scale", 1.0))
        self.pair = rt.param(tensors[o["pair_table"]]) if o.get("pair_table") else None
        self.buckets, self.mul_prev, self.mul_cur = (int(o.get(k, 0)) for k in ("pair_buckets", "pair_mul_prev", "pair_mul_cur"))

    @classmethod
    def tensors(cls, spec: ModelSpec):
        o = spec.options
        out = [TensorDecl(spec.embed_name, (spec.vocab_size, spec.hidden_size), ("normal", o.get("embed_init_std", spec.init_std)))]
        if o.get("pair_table"):
            out.append(TensorDecl(o["pair_table"], (int(o["pair_buckets"]) + 1, spec.hidden_size), ("normal", o.get("pair_init_std", spec.init_std))))
        return out

    def cache_request(self):
        return CacheRequest("state", shape=(1,), dtype=torch.int32) if self.pair is not None else None

    def forward_step(self, step, out, status, cache=None):
        last = cache.state.view(-1) if cache is not None else None
        ops.embed_bigram32(out, self.table, self.pair, step.token_ids, step.positions, step.tok_slot, last, self.scale, self.buckets,
                           self.mul_prev, self.mul_cur, status)
        if last is not None:
            ops.last_token_update(last, step)
        return out
