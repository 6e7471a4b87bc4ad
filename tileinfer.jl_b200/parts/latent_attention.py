"""Attention through low-rank latents, with only the key/value latent cached.

Per token, from the mixer's input h (no positions are applied anywhere inside):

    cq = rms_w(Wdq h, w_q)          query latent   [q_rank]
    c  = rms_w(Wdkv h, w_kv)        key/value latent [kv_rank], the ONLY thing the cache keeps (one row per position)
    q_h = Wuq_h cq                  per head [dim];   k_h(j) = Wuk_h c(j) [dim];   v_h(j) = Wuv_h c(j) [value_dim]
    out = Wo concat_h( sum_j softmax_j(scale q_h . k_h(j)) v_h(j) )      over the visible j (causal, optional window)

rms_w(y, w) = y / sqrt(mean(y^2) + eps) * w in 32-bit. Keys and values are never built: since q_h . (Wuk_h c) =
(Wuk_h^T q_h) . c, the head's query is carried into the latent's space (one small matrix per head), attention runs
over the cached latents as ONE key/value head of size kv_rank shared by all query heads, with the latent as key and
as value, and the attended latent goes through Wuv_h afterwards. That is multi-query attention, so the library's
paged attention kernels (prefill, split-KV decode, plain) serve it unchanged, window included.

Optional parts, by the record's options:

* ``rot_dim`` > 0: a head's query has ``rot_dim`` more elements after the ``dim`` unrotated ones, Wdkv has ``rot_dim`` more rows
  after the latent's, and those rows (not normed) are ONE key part shared by all heads; both are rotated by the position
  encoding's rotation, and the score is scale (q_h . k_h + q_rot_h . k_rot). The cache's row is then [c, k_rot, zeros] of
  ``pool_row`` elements, and the query carried into that row's space is [Wuk_h^T q_h, q_rot_h, zeros]: one matrix per head
  (Wuk_h^T and an identity block) does both. The attended row's first kv_rank elements are the attended latent; Wuv_h is
  stored with zero columns behind them.
* ``sink``: a learned number per head whose exponential is one more term of the softmax's denominator.
* ``gate``: the heads' outputs are multiplied by sigmoid(Wg h) before Wo; Wg rides along in the down projection.

Sizes and constants come from the record: ``num_heads``, ``head_dim`` (unrotated query/key size), ``scale``, ``window`` and the
options ``value_dim``, ``q_rank``, ``kv_rank``, ``latent_norm_eps``, ``rot_dim``, ``sink``, ``gate``.
"""
from __future__ import annotations

import dataclasses

import torch

from ..config.spec import MixerSpec, TensorDecl
from ..kernels import ops
from .base import CacheRequest, Mixer, register_mixer
from .linear import Linear


# Row lengths for which the paged attention kernels have their fast instances (csrc/attention_decode.cu, attention_prefill.cu).
_FAST_ROWS = (16, 32, 48, 64, 80, 96, 112, 128, 256)


def pool_row(kv_rank: int, rot_dim: int) -> int:
    """Length of a cached row: the latent alone, or the latent and the rotated key part filled up with zeros to the next
    length that the fast attention kernels take (else to a multiple of 16)."""
    if not rot_dim:
        return kv_rank
    need = kv_rank + rot_dim
    return next((r for r in _FAST_ROWS if r >= need), -(-need // 16) * 16)


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    def __init__(self, spec: MixerSpec, tensors, rt, position):
        self.spec, self.rt = spec, rt
        o = spec.options
        self.heads, self.dim, self.vdim = spec.num_heads, spec.head_dim, int(o["value_dim"])
        self.q_rank, self.kv_rank = int(o["q_rank"]), int(o["kv_rank"])
        self.eps = float(o.get("latent_norm_eps", 1e-6))
        self.rot_dim, self.sink_on, self.gated = int(o.get("rot_dim", 0)), bool(o.get("sink", False)), bool(o.get("gate", False))
        self.rotation = position.rotation() if (position is not None and self.rot_dim) else None
        if self.rot_dim and (self.rotation is None or self.rotation.rotary_dim != self.rot_dim):
            raise ValueError(f"latent_attention: a rotated part of {self.rot_dim} elements needs a rotation of as many")
        self.pool_row = pool_row(self.kv_rank, self.rot_dim)
        if self.pool_row > ops.MAX_HEAD_DIM:
            raise ValueError(f"latent_attention: a cached row of {self.kv_rank} + {self.rot_dim} exceeds the attention kernels' {ops.MAX_HEAD_DIM}")
        n, p = spec.tensor_names, spec.prefix
        get = lambda k: rt.param(tensors[p + n[k]])
        # The down projections (and the gate's) read the same input: one product, query latent first.
        self.down = Linear(torch.cat([get("dq"), get("dkv")] + ([get("g")] if self.gated else []), 0).contiguous(), rt, "latent_down")
        self.w_q_norm, self.w_kv_norm = get("dq_norm"), get("dkv_norm")
        self.uq = Linear(get("uq"), rt, "uq")
        H, D, V, R, Rd, P = self.heads, self.dim, self.vdim, self.kv_rank, self.rot_dim, self.pool_row
        # Wuk_h [dim, kv_rank] is used transposed (query -> the cached row's space); stored so, head after head, with an
        # identity block that passes the query's rotated part through and zero rows up to the cached row's length.
        uk_t = get("uk").view(H, D, R).transpose(1, 2)                            # [H, kv_rank, dim]
        uv = get("uv").view(H, V, R)                                              # [H, value_dim, kv_rank]
        if P == R:
            self.uk_t, self.uv = uk_t.contiguous(), uv.contiguous()
        else:
            self.uk_t = torch.zeros((H, P, D + Rd), dtype=uk_t.dtype, device=uk_t.device)
            self.uk_t[:, :R, :D] = uk_t
            if Rd:
                self.uk_t[:, R:R + Rd, D:] = torch.eye(Rd, dtype=uk_t.dtype, device=uk_t.device)
            self.uv = torch.zeros((H, V, P), dtype=uv.dtype, device=uv.device)
            self.uv[:, :, :R] = uv
        self.sink = rt.param(tensors[p + n["sink"]], keep_dtype=True).float().contiguous() if self.sink_on else None
        self.o = Linear(get("o"), rt, "o")
        # What the attention kernels see: one KV head of the cached row's size.
        self.attn_spec = dataclasses.replace(spec, num_kv_heads=1, head_dim=P)

    @classmethod
    def tensors(cls, spec: MixerSpec):
        n, p, o = spec.tensor_names, spec.prefix, spec.options
        W, H, D, V = spec.hidden_size, spec.num_heads, spec.head_dim, int(o["value_dim"])
        Q, R, Rd = int(o["q_rank"]), int(o["kv_rank"]), int(o.get("rot_dim", 0))
        std = lambda fan_in: ("normal", fan_in ** -0.5)
        out = [TensorDecl(p + n["dq"], (Q, W), std(W)), TensorDecl(p + n["dq_norm"], (Q,), ("one_plus_normal", 0.1)),
               TensorDecl(p + n["uq"], (H * (D + Rd), Q), std(Q)), TensorDecl(p + n["dkv"], (R + Rd, W), std(W)),
               TensorDecl(p + n["dkv_norm"], (R,), ("one_plus_normal", 0.1)), TensorDecl(p + n["uk"], (H * D, R), std(R)),
               TensorDecl(p + n["uv"], (H * V, R), std(R)), TensorDecl(p + n["o"], (W, H * V), std(H * V))]
        if o.get("sink", False):
            out.append(TensorDecl(p + n["sink"], (H,), ("normal", 1.0), keep_dtype=True))
        if o.get("gate", False):
            out.append(TensorDecl(p + n["g"], (H * V, W), std(W)))
        return out

    def cache_request(self):
        return CacheRequest("paged_latent", kv_heads=1, head_dim=self.pool_row, window=self.spec.window)

    def decode_plan(self, group):
        if not (self.rt.fast and self.rt.dtype == torch.bfloat16):
            return None
        from ..kernels import fast
        return fast.SplitKvPlan(1, group.page_size, group.num_pages * group.page_size)

    def forward(self, h, step, cache):
        rt, s = self.rt, self.spec
        n = h.shape[0]
        H, D, V, Q, R, Rd, P = self.heads, self.dim, self.vdim, self.q_rank, self.kv_rank, self.rot_dim, self.pool_row
        rows = rt.buffer("latent.down", (n, self.down.out_features))
        # The gate's columns are read as they are by the gate's kernel: only a product without them may come in partial sums.
        rows = self.down.forward(h, rows, allow_partials=n <= 256 and not self.gated)
        cq = rt.buffer("latent.cq", (n, Q))
        meta = step.group(cache.group_index)
        ops.latent_inputs(rows, cq, cache.k, self.w_q_norm, self.w_kv_norm, self.eps, meta.slot_mapping, Q, R, self.rotation,
                          step.positions, P)
        q = rt.buffer("latent.q", (n, H, D + Rd))
        self.uq.forward(cq, q.view(n, H * (D + Rd)))
        if Rd:
            ops.rotate_heads(q, self.rotation, step.positions, first=D)
        fast = None
        if rt.fast:
            from ..kernels import fast
        q_lat = rt.buffer("latent.q_latent", (n, H, P))
        if not (fast is not None and fast.head_linear(q_lat, q, self.uk_t)):
            ops.head_gemm(q_lat, q, self.uk_t)
        attn = rt.buffer("latent.attended", (n, H, P))
        done = False
        if fast is not None:
            done = fast.attention(attn.view(n, H * P), q_lat, cache, meta, step, self.attn_spec, sink=self.sink)
        if not done:
            ops.attention_plain(attn.view(n, H * P), q_lat, cache.k, cache.v, meta.block_table, step.tok_slot, step.positions,
                                s.scale, H, 1, P, cache.page_size, window=s.window or 0, sink=self.sink)
        values = rt.buffer("latent.values", (n, H, V))
        if not (fast is not None and fast.head_linear(values, attn, self.uv)):
            ops.head_gemm(values, attn, self.uv)
        if self.gated:
            gated = rt.buffer("latent.gated", (n, H * V))
            ops.sigmoid_gate(gated, values, rows[:, Q + R + Rd:], H, V, V)
            values = gated
        proj = rt.buffer("mixer.delta", (n, s.hidden_size))
        return self.o.forward(values.view(n, H * V), proj, allow_partials=True)
