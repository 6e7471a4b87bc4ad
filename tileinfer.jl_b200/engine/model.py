"""The decoder: embedding part, the layers in their order, final norm, head part.

Built from a :class:`ModelSpec` alone: every layer's parts are looked up by kind, and the
order in which layers run is the spec's ``order`` list (an entry may repeat a layer; a
mixer may read the storage of an earlier layer). The step itself follows
AntoineBut/TileInfer.jl's ``run_step!`` (src/model/decoder.jl:165-196): embed, first norm,
per layer mixer / add+norm / feed-forward / add+norm, and the LM head on the wanted rows
only, with 32-bit logits.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.spec import ModelSpec, TensorDecl
from ..kernels import ops
from ..parts import Linear, Runtime, lookup


def tensor_declarations(spec: ModelSpec) -> List[TensorDecl]:
    """Every checkpoint tensor a model of this spec reads."""
    decls = list(lookup("embedding", spec.embedding_kind).tensors(spec)) + list(lookup("head", spec.head_kind).tensors(spec))
    decls += lookup("norm", spec.final_norm.kind).tensors(spec.final_norm)
    if spec.pass_input is not None:
        decls += lookup("pass_input", spec.pass_input.kind).tensors(spec.pass_input)
    for layer in spec.layers:
        decls += lookup("norm", layer.mixer_norm.kind).tensors(layer.mixer_norm)
        for post in (layer.mixer_post_norm, layer.feed_forward_post_norm):
            if post is not None:
                decls += lookup("norm", post.kind).tensors(post)
        decls += lookup("mixer", layer.mixer.kind).tensors(layer.mixer)
        if layer.feed_forward is not None:
            if layer.feed_forward_norm is not None:          # an arrangement with one norm for both sublayers has none
                decls += lookup("norm", layer.feed_forward_norm.kind).tensors(layer.feed_forward_norm)
            decls += lookup("feed_forward", layer.feed_forward.kind).tensors(layer.feed_forward)
        if layer.token_input is not None:
            decls += lookup("token_input", layer.token_input.kind).tensors(layer.token_input)
        block_tensors = getattr(lookup("block", layer.block), "tensors", None)
        if block_tensors is not None:                            # an arrangement with learned tables of its own
            decls += block_tensors(layer)
    seen, out = set(), []
    for d in decls:
        if d.name not in seen:
            seen.add(d.name)
            out.append(d)
    return out


def ignorable_tensors(spec: ModelSpec) -> List[str]:
    # A tied checkpoint may still store a copy of the head (src/hub/loader.jl:157-163).
    return ["lm_head.weight"] if spec.lm_head_name is None else []


class DecoderModel:
    def __init__(self, spec: ModelSpec, tensors: Dict[str, torch.Tensor], rt: Runtime, max_positions: int):
        self.spec, self.rt = spec, rt
        self.max_positions = int(min(max_positions, spec.max_positions))
        self.embedding = lookup("embedding", spec.embedding_kind)(spec, tensors, rt)
        self.head = lookup("head", spec.head_kind)(spec, tensors, rt, self.embedding)
        # An embedding that keeps something per sequence (the token before, for one) has the cache entry after the layer runs'.
        ask = getattr(self.embedding, "cache_request", None)
        self._embedding_request = ask() if ask is not None else None
        self._embedding_cache = len(spec.order) if self._embedding_request is not None else None
        self.final_norm = lookup("norm", spec.final_norm.kind)(spec.final_norm, tensors, rt)
        self._positions: Dict[tuple, object] = {}
        self.blocks = []
        for layer in spec.layers:
            position = self._position(layer.mixer.position)
            mixer = lookup("mixer", layer.mixer.kind)(layer.mixer, tensors, rt, position)
            ffn = n2 = None
            if layer.feed_forward is not None:
                ffn = lookup("feed_forward", layer.feed_forward.kind)(layer.feed_forward, tensors, rt)
                if layer.feed_forward_norm is not None:
                    n2 = lookup("norm", layer.feed_forward_norm.kind)(layer.feed_forward_norm, tensors, rt)
            n1 = lookup("norm", layer.mixer_norm.kind)(layer.mixer_norm, tensors, rt)
            extra = {}
            if layer.token_input is not None:
                extra["token_input"] = lookup("token_input", layer.token_input.kind)(layer.token_input, tensors, rt)
            if layer.mixer_post_norm is not None:
                extra["mixer_post_norm"] = lookup("norm", layer.mixer_post_norm.kind)(layer.mixer_post_norm, tensors, rt)
            if layer.feed_forward_post_norm is not None:
                extra["feed_forward_post_norm"] = lookup("norm", layer.feed_forward_post_norm.kind)(layer.feed_forward_post_norm, tensors, rt)
            block_class = lookup("block", layer.block)
            if getattr(block_class, "tensors", None) is not None:
                extra.update({"tensors": tensors, "rt": rt})
            self.blocks.append(block_class(layer, mixer, ffn, n1, n2, **extra))
        self.pass_input = None
        if spec.pass_input is not None:
            self.pass_input = lookup("pass_input", spec.pass_input.kind)(spec.pass_input, tensors, rt)
            if any(not 0 <= occ < len(spec.order) for occ in spec.pass_input.at):
                raise ValueError(f"pass input before layer runs {spec.pass_input.at} of {len(spec.order)}")
        self._pass_starts = frozenset(spec.pass_input.at) if spec.pass_input is not None else frozenset()
        # Called with (index of the layer run, the 32-bit or 16-bit stream after it) when set: for tests and debugging.
        self.observer = None
        self.status = torch.zeros(1, dtype=torch.int32, device=rt.device)
        # The residual stream has the products' element type unless the architecture keeps it in 32-bit.
        self.stream_dtype = torch.float32 if spec.options.get("residual_dtype") == "float32" else rt.dtype
        # Copies of the stream that the layers' arrangement keeps side by side (0: one stream); a row of x holds them all.
        self.streams = int(spec.options.get("streams") or 0)
        if self.streams and self.stream_dtype != torch.float32:
            raise ValueError("several copies of the stream are kept in 32-bit")

    def _position(self, pspec):
        key = (pspec.kind, pspec.head_dim, pspec.theta, pspec.scaling, pspec.max_positions, tuple(sorted(pspec.options.items())))
        if key not in self._positions:
            self._positions[key] = lookup("position", pspec.kind)(pspec, self.rt, self.max_positions)
        return self._positions[key]

    # ---- what the cache has to hold, one entry per position of ``order``
    def cache_requests(self):
        """One entry per layer run; then one for the embedding, if it keeps something per sequence."""
        out = [self.blocks[li].mixer.cache_request() for li in self.spec.order]
        if self._embedding_request is not None:
            out.append(self._embedding_request)
        return out

    def cache_shares(self) -> Dict[int, int]:
        """occurrence -> the earlier occurrence whose storage it reads."""
        shares, last = {}, {}
        for occ, li in enumerate(self.spec.order):
            src = self.spec.layers[li].mixer.kv_source
            if src is not None:
                if src not in last:
                    raise ValueError(f"layer {li} reads the cache of layer {src}, which has not run before it")
                shares[occ] = last[src]
            last[li] = occ
        return shares

    def weight_bytes(self) -> int:
        """Bytes of every weight a step reads once: the parts' matrices and vectors and the head (a tied
        head counts once). The embedding table is not among them: a step reads one row of it per token.
        Parts are walked through their attributes, lists and dicts included (experts kept in a list
        count); position encodings hold tables, not weights, and are left out."""
        from ..parts.base import Part, PositionEncoding
        seen, total = set(), 0

        def visit(obj):
            nonlocal total
            if isinstance(obj, torch.Tensor):
                if obj.is_floating_point() and obj.numel() > 1 and obj.data_ptr() not in seen:
                    seen.add(obj.data_ptr())
                    total += obj.numel() * obj.element_size()
            elif isinstance(obj, (list, tuple)):
                for v in obj:
                    visit(v)
            elif isinstance(obj, dict):
                for v in obj.values():
                    visit(v)
            elif isinstance(obj, (Part, Linear)) and not isinstance(obj, PositionEncoding) and id(obj) not in seen:
                seen.add(id(obj))
                for v in vars(obj).values():
                    visit(v)

        for b in self.blocks:
            visit([b.mixer, b.feed_forward, b.mixer_norm, b.feed_forward_norm, getattr(b, "token_input", None),
                   getattr(b, "mixer_post_norm", None), getattr(b, "feed_forward_post_norm", None)])
        visit([self.final_norm, self.head, self.pass_input])
        return total

    def forward(self, step, cache, logits: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Run the step's tokens; write the logits of ``step.want_idx`` rows to ``logits``."""
        from ..kernels.library import stream_scope
        with stream_scope():
            return self._forward(step, cache, logits)

    def _forward(self, step, cache, logits: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        rt, spec = self.rt, self.spec
        n = step.n_tokens
        stream = rt.buffer("model.x", (n, max(1, self.streams) * spec.hidden_size), self.stream_dtype)
        # With copies of the stream the embedding's output is written once and then laid into every copy.
        x = rt.buffer("model.x0", (n, spec.hidden_size), self.stream_dtype) if self.streams else stream
        h = rt.buffer("model.h", (n, spec.hidden_size))
        embed_step = getattr(self.embedding, "forward_step", None)
        if self._embedding_cache is not None:
            embed_step(step, x, self.status, cache=cache.layer(self._embedding_cache))
        elif embed_step is not None:
            embed_step(step, x, self.status)
        else:
            self.embedding.forward(step.token_ids, x, self.status)
        if self.pass_input is not None:
            self.pass_input.begin(x)
        if self.streams:
            ops.streams_begin(stream, x, self.streams)
            x = stream
        order = spec.order
        self.blocks[order[0]].input_norm.forward(x, h) if order else self.final_norm.forward(x, h)
        for occ, li in enumerate(order):
            if occ in self._pass_starts:
                # The stream is rewritten before this run; the normed input that the run before left is made again.
                self.pass_input.forward(x)
                self.blocks[li].input_norm.forward(x, h)
            nxt = self.blocks[order[occ + 1]].input_norm if occ + 1 < len(order) else self.final_norm
            self.blocks[li].forward(x, h, step, cache.layer(occ), nxt, h)
            if self.observer is not None:
                self.observer(occ, x)
        if logits is None or step.n_want == 0:
            return None
        hw = rt.buffer("model.h_wanted", (step.n_want, spec.hidden_size))
        ops.gather_rows(hw, h, step.want_idx)
        self.head.forward(hw, logits)
        return logits
