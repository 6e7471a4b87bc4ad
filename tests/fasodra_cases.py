"""Small Fasodra configurations for the tests, their random model folders and the comparison against the plain
implementation (``plain_fasodra``).

The configurations differ from one another in every size and constant, and none keeps two sizes equal that a kernel could mix up
(query/key size and value size, heads and key/value heads, chunk and page, the two sides of a pair, the copies of the stream).
"""
from __future__ import annotations

import json
import os

import numpy as np
import torch

import plain_fasodra as plain


def moe(ff, experts, top):
    return {"expert": {"ff": ff}, "kind": "moe", "router": {"experts": experts, "top": top}}


def _attention(heads, kv_heads, dim, vdim, scale, rot=None):
    m = {"dim": dim, "heads": heads, "scale": scale}
    if kv_heads:
        m["kv_heads"] = kv_heads
    if vdim:
        m["vdim"] = vdim
    if rot:
        m["rot"] = {"base": rot[1], "dims": rot[0]}
    return m


def attention(heads, kv_heads, dim, vdim, scale, bias_max, mlp, chunk=None):
    m = _attention(heads, kv_heads, dim, vdim, scale)
    m["bias_max"] = bias_max
    if chunk:
        m["mask"] = {"size": chunk}
    return {"mixer": m, "mlp": mlp, "type": "attention"}


def parallel(left, right_heads, right_dim, mlp, scales=None):
    m = {"left": _attention(*left), "right": {"dim": right_dim, "heads": right_heads}}
    if scales:
        m["left_scale"], m["right_scale"] = scales
    return {"mixer": m, "mlp": mlp, "type": "parallel"}


def parallel_2(left, right, mlp):
    """right: (heads, kv_heads or None, dim, vdim or None, conv or None)."""
    heads, kv_heads, dim, vdim, conv = right
    r = {"dim": dim, "heads": heads}
    if kv_heads:
        r["kv_heads"] = kv_heads
    if vdim:
        r["vdim"] = vdim
    if conv:
        r["conv"] = conv
    return {"mixer": {"left": _attention(*left), "right": r}, "mlp": mlp, "type": "parallel_2"}


def model(vocab, width, eps, layers, mult=None, streams=None):
    d = {"architecture": "Fasodra", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if mult is not None:
        d["residual_mult"] = mult
    if streams:
        d["streams"] = streams
    return d


# Odd sizes that no fast kernel takes: three query heads per key/value head, values longer and shorter than keys, a chunk shorter
# than a page and one that is no multiple of anything, three copies of the stream, a pair without feed-forward, every expert chosen.
CASE_A = model(131, 52, 1e-5, [
    attention(6, 2, 10, 14, 0.4, 20, moe(20, 5, 2), chunk=7),
    parallel((3, 1, 12, 6, 0.3, (6, 500.0)), 3, 10, None, scales=(0.8, 1.3)),
    parallel_2((4, 4, 6, 10, 0.35, (6, 50.0)), (4, 2, 10, 6, 3), moe(12, 3, 3)),
    attention(2, 1, 14, 10, 0.3, 50, moe(28, 4, 1), chunk=33),
], mult=0.7, streams=3)
# Sizes the tensor-core kernels take (widths in steps of 8, heads of 32 and 64): a pair first, a chunk of exactly one page and one
# across pages, two and four query heads per key/value head, four copies of the stream.
CASE_B = model(320, 128, 1e-6, [
    parallel_2((4, 2, 64, 32, 0.11, (16, 20000.0)), (2, 1, 32, 64, 4), moe(64, 8, 2)),
    attention(4, 2, 32, 64, 0.2, 100, moe(32, 16, 4), chunk=64),
    parallel((8, 2, 32, 32, 0.17, (32, 100.0)), 2, 64, moe(64, 8, 3), scales=(1.5, 0.4)),
    attention(2, 1, 64, 32, 0.12, 300, moe(96, 4, 2), chunk=100),
], mult=0.6, streams=4)
# What may be absent is absent: one stream and no multiplier, attention without chunks, key/value heads, value sizes, rotation,
# convolution and the pair's scales left out, a layer without feed-forward, one expert per token.
CASE_C = model(97, 64, 3e-6, [
    parallel((2, None, 16, None, 0.25, None), 1, 16, moe(24, 2, 1)),
    attention(2, None, 16, None, 0.25, 12, None),
    parallel_2((1, None, 32, 16, 0.2, None), (2, None, 16, None, None), moe(40, 6, 2)),
])
CASES = {"A": CASE_A, "B": CASE_B, "C": CASE_C}


def write_folder(case: dict, seed: int, out_dir: str, override=None) -> str:
    """A model folder with random weights for ``case``, made without a device. ``override``: name -> tensor put in place of
    (or beside) the random ones: tensors whose extent no configuration key gives."""
    from tileinfer_b200.config import config_from_dict
    from tileinfer_b200.weights import write_model_folder
    write_model_folder(config_from_dict(case), seed, out_dir, device="cpu")
    from tileinfer_b200.weights.safetensors_io import SafetensorsFile, save_file
    path = os.path.join(out_dir, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n).clone() for n in f.entries}
    del f
    tensors.update({k: v.to(torch.bfloat16) for k, v in (override or {}).items()})
    save_file(tensors, path)
    return out_dir


def load_folder(folder):
    """(config dict, tensors) of a model folder, read with the safetensors package."""
    from safetensors import safe_open
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    W = {}
    with safe_open(os.path.join(folder, "model.safetensors"), "pt") as f:
        for k in f.keys():
            W[k] = f.get_tensor(k)
    return cfg, W


class Model:
    """A case's folder, the plain implementation's view of it and cached reference logits."""

    def __init__(self, name: str, seed: int, tmp: str, case: dict = None, override=None):
        self.name = name
        self.folder = write_folder(case or CASES[name], seed, os.path.join(tmp, f"fasodra_{name}_{seed}"), override)
        self.cfg, self.W = load_folder(self.folder)
        self.vocab = self.cfg["vocab"]
        self._refs = {}

    def reference(self, tokens, forced=None):
        """(logits [n, vocab] in 64-bit arithmetic as numpy, every position's smallest router margin [n]). ``forced``: router
        choices to take instead of the plain implementation's own ({layer: {position: experts}})."""
        if forced is not None:
            return plain.forward(self.cfg, self.W, list(tokens), torch.float64, forced=forced).float().numpy(), np.full(len(tokens), np.inf)
        key = tuple(tokens)
        if key not in self._refs:
            margins = []
            logits = plain.forward(self.cfg, self.W, list(tokens), torch.float64, margins=margins)
            per_layer = [m for m in margins if m]
            smallest = np.min(np.array(per_layer), axis=0) if per_layer else np.full(len(tokens), np.inf)
            self._refs[key] = (logits.float().numpy(), smallest)
        return self._refs[key]

    def layers(self, tokens):
        out = []
        plain.forward(self.cfg, self.W, list(tokens), torch.float64, layers_out=out)
        return [x.float() for x in out]

    def engine(self, dtype: str, **kw):
        from tileinfer_b200.engine import Engine
        args = dict(max_tokens=2048, max_seqs=6, max_context=1024)
        args.update(kw)
        return Engine.load(self.folder, dtype=dtype, **args)


def tolerance(dtype, ref: np.ndarray) -> float:
    scale = max(float(np.abs(ref).max()), 1.0)
    return 1e-4 * scale if dtype == torch.float32 else 8 * scale * 2.0 ** -8


def compare(model: Model, tokens, got: dict, dtype, what: str = "", need: float = 0.5, forced=None):
    """``got``: position -> logits row. With ``forced`` (the router choices that the run under test made) every position must be
    within the tolerance of the plain implementation with the same choices. Without it, every position whose router choices are
    settled must be: a choice that rounding turns changes its own position by an expert's whole share, and the positions behind
    it through the recurrent states and the short chunks, so a position counts as settled when no choice of its own or of the 48
    positions before it rests on a gap of less than 1e-4 in the router's logits (bfloat16: 0.1); at least ``need`` of the
    positions (of 20 or more) must be of that kind."""
    ref, margin = model.reference(tokens, forced)
    close = margin < (0.1 if dtype == torch.bfloat16 else 1e-4)
    unsure = np.array([close[max(0, p - 48):p + 1].any() for p in range(len(close))])
    tol = tolerance(dtype, ref)
    sure = [p for p in got if not unsure[p]]
    if len(got) >= 20:
        assert len(sure) >= need * len(got), f"{what}: only {len(sure)} of {len(got)} positions are free of close router calls"
    for p in sure:
        err = float(np.abs(got[p] - ref[p]).max())
        assert err <= tol, f"{what}: position {p} of {len(tokens)}: |d| = {err:.3g} > {tol:.3g}"
    return len(sure)


class Recorder:
    """Notes the router choices that an engine makes, layer by layer, for the token rows that the test names before every step
    (``rows``: one (request, position) per row of the step). The engine must run without captured graphs."""

    def __init__(self, engine, cfg):
        self.engine = engine
        self.tops = [l["mlp"]["router"]["top"] if l.get("mlp") else 0 for l in cfg["layers"]]
        self.rows, self.choices = [], {}
        engine.model.observer = self

    def __call__(self, layer, x):
        top = self.tops[layer]
        if top:
            ids = self.engine.model.rt.buffer("experts.ids", (x.shape[0], top), torch.int32).cpu().tolist()
            assert len(ids) == len(self.rows)
            for (request, position), row in zip(self.rows, ids):
                self.choices.setdefault(request, {}).setdefault(layer, {})[position] = row

    def of(self, request):
        return self.choices.get(request, {})


def prompts(vocab: int, lengths, seed: int):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
