"""A routed feed-forward: a router picks ``top`` of ``experts`` small gated units per token; a shared unit may run for
every token and is added.

    z = Wr h (32-bit), score = sigmoid(z); the `top` largest scores choose the experts (ties to the smaller index)
    unit(u; limit) = Wdown( a * sigmoid(slope * a) * (b + shift) ),  a = min(Wgate u, limit),  b = clamp(Wup u, -limit, limit)
    out = sum_chosen unit_e(score_e * h)  [+ unit_shared(h)]         with ``scale_input`` (the score scales the INPUT)
    out = sum_chosen score_e * unit_e(h)  [+ unit_shared(h)]         without it

With ``gated`` False a unit has no gate matrix: unit(u) = Wdown act(Wup u), ``activation`` "relu2" (max(z, 0)^2), no clamp and no
shared unit.

Options of the record: ``experts``, ``top``, ``limit`` (None: no clamp), ``sigmoid_slope``, ``up_shift``, ``scale_input``,
``shared_size`` / ``shared_limit`` (0: no shared unit). ``intermediate_size`` is an expert's size. A router with more rules
(any of the following options) is chosen by ``csrc/routed_experts.cu``'s ``router_select``:

    ``score`` "softmax": s = softmax(z) over all router outputs instead of sigmoid(z)
    ``correction``: a tensor added to s for the CHOICE only (the weights use s)
    ``groups`` (count, keep): the router's outputs form `count` equal groups of neighbours, a group's score is its largest choice
        score, and only members of the `keep` best groups can be chosen
    ``renormalize``: weights = the chosen s divided by (their sum + 1e-20)
    ``pass_through``: the last so many router outputs are not experts: a token that chooses one gets its own input back, times
        the weight (they take part in softmax, groups and the sum like any other)
    ``shared_gate``: a tensor [1, width]; the shared unit's output is multiplied by sigmoid(shared_gate . h), one number per token Tensor names: ``router``, ``expert`` (a prefix pattern with ``{}`` for the expert's number), ``shared``
(a prefix), and inside a unit ``gate``, ``up``, ``down``.

On the device the (token, choice) pairs are grouped by expert and every expert's rows go through its matrices in
tiles (``csrc/routed_experts.cu``, on the tensor cores ``csrc/gemm_tcgen05.cu``); no count is read on the host, so a
one-token step stays capturable. The shared unit rides along as units of an expert's size that every token takes.
"""
from __future__ import annotations

import torch

from ..config.spec import FeedForwardSpec, TensorDecl
from ..kernels import ops
from .base import FeedForward, register_feed_forward
from .linear import Linear
from .norm import GatheredRows


def _has_rules(o) -> bool:
    return bool(o.get("score", "sigmoid") != "sigmoid" or o.get("renormalize") or o.get("groups") or o.get("pass_through")
                or o.get("correction") or o.get("shared_gate"))


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    def __init__(self, spec: FeedForwardSpec, tensors, rt):
        self.spec, self.rt = spec, rt
        o, n, p = spec.options, spec.tensor_names, spec.prefix
        self.experts, self.top = int(o["experts"]), int(o["top"])
        self.limit = float(o["limit"]) if o.get("limit") is not None else float("inf")
        self.slope, self.shift = float(o.get("sigmoid_slope", 1.0)), float(o.get("up_shift", 0.0))
        self.scale_input = bool(o.get("scale_input", False))
        get = lambda name: rt.param(tensors[p + name])
        self.gated = bool(o.get("gated", True))
        if not self.gated and (o.get("activation") != "relu2" or int(o.get("shared_size", 0)) or o.get("limit") is not None):
            raise ValueError("routed_experts: a unit without a gate has the activation relu2, no clamp and no shared unit")
        self.select = _has_rules(o)
        self.softmax, self.renormalize = o.get("score", "sigmoid") == "softmax", bool(o.get("renormalize", False))
        self.pass_through = int(o.get("pass_through", 0))
        self.groups, self.keep = (int(v) for v in (o.get("groups") or (1, 1)))
        if o.get("score", "sigmoid") not in ("sigmoid", "softmax"):
            raise ValueError(f"routed_experts: score {o.get('score')!r} (known: sigmoid, softmax)")
        if self.select and self.scale_input:
            raise ValueError("routed_experts: a router with rules scales the experts' outputs, not their inputs")
        total = self.experts + self.pass_through
        if total % self.groups or not 1 <= self.keep <= self.groups or self.keep * (total // self.groups) < self.top:
            raise ValueError(f"routed_experts: {self.keep} of {self.groups} groups over {total} router outputs for top {self.top}")
        self.correction = rt.param(tensors[p + n["correction"]], keep_dtype=True).float().contiguous() if o.get("correction") else None
        self.gate_on = bool(o.get("shared_gate")) and int(o.get("shared_size", 0)) > 0
        self.router = get(n["router"])
        if self.gate_on:                         # the gate's row rides along as the router product's last output
            self.router = torch.cat([self.router, get(n["shared_gate"]).view(1, -1)], 0).contiguous()
        self.router_linear = Linear(self.router, rt, "router")
        units = [p + n["expert"].format(e) for e in range(self.experts)]
        unit = lambda u, k: rt.param(tensors[u + n[k]])
        F, W = spec.intermediate_size, spec.hidden_size
        gate_up = [torch.cat([unit(u, "gate"), unit(u, "up")], 0) if self.gated else unit(u, "up") for u in units]
        down = [unit(u, "down") for u in units]
        limits = [self.limit] * self.experts
        shared_limit = float(o["shared_limit"]) if o.get("shared_limit") is not None else float("inf")
        # The shared unit runs as further units of an expert's size that every token takes with score one: a gated unit is
        # a sum over its inner rows, so slices of F of them (the last one filled up with zero rows, which add nothing)
        # are units of their own, and the grouped products carry them along with the routed experts.
        self.shared_size = int(o.get("shared_size", 0))
        self.always = -(-self.shared_size // F) if self.shared_size else 0
        if self.shared_size:
            u = p + n["shared"]
            g, up, d = unit(u, "gate"), unit(u, "up"), unit(u, "down")
            pad = self.always * F - self.shared_size
            if pad:
                zeros = torch.zeros(pad, W, dtype=g.dtype, device=g.device)
                g, up = torch.cat([g, zeros], 0), torch.cat([up, zeros], 0)
                d = torch.cat([d, torch.zeros(W, pad, dtype=d.dtype, device=d.device)], 1)
            for c in range(self.always):
                gate_up.append(torch.cat([g[c * F:(c + 1) * F], up[c * F:(c + 1) * F]], 0))
                down.append(d[:, c * F:(c + 1) * F])
                limits.append(shared_limit)
        # Every unit's gate rows then its up rows, unit after unit; the down matrices likewise.
        self.gate_up = torch.stack(gate_up).contiguous()
        self.down = torch.stack(down).contiguous()
        self.limits = torch.tensor(limits, dtype=torch.float32, device=rt.device)
        self.units = self.experts + self.always

    @classmethod
    def tensors(cls, spec: FeedForwardSpec):
        o, n, p = spec.options, spec.tensor_names, spec.prefix
        W, F = spec.hidden_size, spec.intermediate_size
        std = lambda fan_in: ("normal", fan_in ** -0.5)
        total = int(o["experts"]) + int(o.get("pass_through", 0))
        out = [TensorDecl(p + n["router"], (total, W), std(W))]
        if o.get("correction"):
            out.append(TensorDecl(p + n["correction"], (total,), ("normal", 0.02), keep_dtype=True))
        if o.get("shared_gate") and int(o.get("shared_size", 0)):
            out.append(TensorDecl(p + n["shared_gate"], (1, W), std(W)))

        def unit(u, size):
            gate = [TensorDecl(u + n["gate"], (size, W), std(W))] if o.get("gated", True) else []
            return gate + [TensorDecl(u + n["up"], (size, W), std(W)), TensorDecl(u + n["down"], (W, size), std(size))]
        for e in range(int(o["experts"])):
            out += unit(p + n["expert"].format(e), F)
        if int(o.get("shared_size", 0)):
            out += unit(p + n["shared"], int(o["shared_size"]))
        return out

    def forward(self, h, step):
        rt, spec = self.rt, self.spec
        n, W = h.shape
        F, top, E, per_token = spec.intermediate_size, self.top, self.experts, self.top + self.always
        pairs = n * per_token
        fast = None
        if rt.fast:
            from ..kernels import fast
        ids = rt.buffer("experts.ids", (n, per_token), torch.int32)
        scores = rt.buffer("experts.scores", (n, per_token), torch.float32)
        tile = fast.grouped_tile(pairs, self.units) if fast is not None else ops.EXPERT_TILE_ROWS
        max_tiles, rows = ops.expert_plan_sizes(pairs, self.units, tile)
        pair_row = rt.buffer("experts.pair_row", (n, per_token), torch.int32)
        row_pair = rt.buffer("experts.row_pair", (rows,), torch.int32)
        plan = rt.buffer("experts.plan", (1 + max_tiles,), torch.int32)
        xs = rt.buffer("experts.rows", (rows, W))
        logits = None
        if fast is not None:                     # the router's 32-bit sums from a product kernel, where one takes the sizes
            logits = fast.linear_f32(self.router_linear, h, rt.buffer("experts.logits", (n, self.router.shape[0]), torch.float32))
        pass_weight = None
        if self.select:
            pass_weight = rt.buffer("experts.pass_weight", (n,), torch.float32) if self.pass_through else None
            ops.router_select(h, self.router, logits, E, E + self.pass_through, top, ids, scores, pass_weight, softmax=self.softmax,
                              correction=self.correction, groups=self.groups, keep=self.keep, renormalize=self.renormalize,
                              always=self.always, gate=self.gate_on)
        else:
            ops.router_topk(h, self.router, top, ids, scores, logits, always=self.always)
        ops.expert_plan(ids, self.units, tile, pair_row, row_pair, plan)
        ops.expert_gather(xs, h, pair_row, scores, per_token, self.scale_input)
        act = rt.buffer("experts.act", (rows, F))
        gu = rt.buffer("experts.gate_up", (rows, 2 * F if self.gated else F))
        if not self.gated:
            if not (fast is not None and fast.grouped_linear(gu, xs, self.gate_up, plan, tile)):
                ops.grouped_gemm(gu, xs, self.gate_up, plan, tile)
            ops.relu2(act, gu)
        elif fast is not None and fast.grouped_linear(gu, xs, self.gate_up, plan, tile):
            ops.gated_unit_limit(act, gu, 0.0, self.slope, self.shift, plan=plan, tile=tile, limits=self.limits)
        else:
            ops.grouped_gemm(act, xs, self.gate_up, plan, tile, gated=True, limits=self.limits, slope=self.slope, shift=self.shift)
        ys = rt.buffer("experts.out_rows", (rows, W))
        if not (fast is not None and fast.grouped_linear(ys, act, self.down, plan, tile)):
            ops.grouped_gemm(ys, act, self.down, plan, tile)
        if self.scale_input:
            return GatheredRows(ys, pair_row)    # the norm that reads the output adds a token's rows up itself
        out = rt.buffer("feed_forward.delta", (n, W))
        ops.expert_combine(out, ys, pair_row, scores, None, per_token, scale_output=True, h=h if pass_weight is not None else None,
                           pass_weight=pass_weight)
        return out
