"""Small Sozanex configurations for the tests, their random model folders and the comparison against the plain
implementation (``plain_sozanex``).

The configurations differ from one another in every size and constant, and none keeps two sizes equal that a kernel could
mix up (query/key size and value size, heads and key/value heads, rotated and unrotated parts, ranks, windows and pages).
"""
from __future__ import annotations

import json
import os

import numpy as np
import torch

import plain_sozanex as plain


def attention(heads, kv_heads, dim, vdim, scale, mlp, window=None, rot=None, scaling=None):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": vdim}
    if window:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = {"base": rot[1], "dims": rot[0]}
        if scaling:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return {"mixer": m, "mlp": mlp, "type": "attention"}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, mlp, base=10000.0, scaling=None):
    m = {"dim": dim, "heads": heads, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale, "vdim": vdim, "rot_dim": rot_dim,
         "rot": {"base": base, "dims": rot_dim}}
    if scaling:
        m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"mixer": m, "mlp": mlp, "type": "latent_attention"}


def dense(ff):
    return {"ff": ff, "kind": "dense"}


def model(vocab, width, eps, scale, layers, bigram=None, loop=None):
    e = {"scale": scale}
    if bigram:
        e["bigram"] = dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))
    d = {"architecture": "Sozanex", "embedding": e, "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if loop:
        d["loop"] = dict(zip(("start", "stop", "times"), loop))
    return d


# Odd sizes that no fast kernel takes: three query heads per key/value head, value size larger than the key's, part of a head
# rotated with band-wise scaled frequencies, a window shorter than a page and one that is no multiple of anything, a latent
# layer without feed-forward whose cached row (26 + 6) is filled up, the loop from the first layer on, three passes.
CASE_A = model(131, 52, 1e-5, 3.0, [
    attention(6, 2, 10, 14, 0.4, dense(60), window=7, rot=(6, 500.0), scaling=(4.0, 1.0, 3.0, 100)),
    latent(3, 12, 6, 10, 20, 26, 0.3, None, base=100.0, scaling=(5.0, 16, 8.0, 1.0)),
    attention(4, 4, 8, 8, 0.35, dense(36), window=33, rot=(8, 50.0)),
], bigram=(97, 31, 5), loop=(0, 2, 3))
# Sizes the tensor-core kernels take (widths in steps of 8, heads of 32 and 64, cached rows of 64 and 128): a latent layer first,
# two and four query heads per key/value head, keys longer and shorter than values, a window of exactly one page and one across
# pages, YaRN ramps that start inside and outside the pairs, the loop in the middle.
CASE_B = model(320, 128, 1e-6, 11.3, [
    latent(4, 32, 16, 48, 64, 48, 0.14, dense(256), base=5000.0, scaling=(6.0, 64, 24.0, 1.0)),
    attention(4, 2, 64, 32, 0.11, dense(256), window=100, rot=(16, 20000.0), scaling=(6.0, 1.0, 3.0, 256)),
    latent(2, 64, 32, 64, 96, 96, 0.1, dense(136), base=1000.0, scaling=(3.0, 40, 16.0, 2.0)),
    attention(4, 1, 32, 64, 0.2, dense(128), window=64, rot=(32, 100.0)),
], bigram=(509, 3, 1), loop=(1, 3, 2))
# What may be absent is absent: no second embedding table, no window, no rotation in the attention layer, no scaling of the
# latent layer's rotation, one latent head, a loop of one pass over one layer (its input projection still runs).
CASE_C = model(97, 64, 3e-6, 1.0, [
    attention(2, 2, 16, 16, 0.25, dense(48)),
    latent(1, 16, 8, 24, 16, 24, 0.2, dense(40), base=30.0),
], loop=(1, 2, 1))
CASES = {"A": CASE_A, "B": CASE_B, "C": CASE_C}


def write_folder(case: dict, seed: int, out_dir: str) -> str:
    """A model folder with random weights for ``case``, made without a device."""
    from tileinfer_b200.config import config_from_dict
    from tileinfer_b200.weights import write_model_folder
    write_model_folder(config_from_dict(case), seed, out_dir, device="cpu")
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

    def __init__(self, name: str, seed: int, tmp: str, case: dict = None):
        self.name = name
        self.folder = write_folder(case or CASES[name], seed, os.path.join(tmp, f"sozanex_{name}_{seed}"))
        self.cfg, self.W = load_folder(self.folder)
        self.vocab = self.cfg["vocab"]
        self._refs = {}

    def reference(self, tokens, dtype) -> np.ndarray:
        key = (tuple(tokens), dtype)
        if key not in self._refs:
            self._refs[key] = plain.forward(self.cfg, self.W, list(tokens), dtype).float().numpy()
        return self._refs[key]

    def engine(self, dtype: str, **kw):
        from tileinfer_b200.engine import Engine
        args = dict(max_tokens=2048, max_seqs=6, max_context=1024)
        args.update(kw)
        return Engine.load(self.folder, dtype=dtype, **args)


def tolerance(dtype, ref: np.ndarray) -> float:
    scale = max(float(np.abs(ref).max()), 1.0)
    return 1e-4 * scale if dtype == torch.float32 else 8 * scale * 2.0 ** -8


def compare(model: Model, tokens, got: dict, dtype, what: str = ""):
    """``got``: position -> logits row; every one within the tolerance of the plain implementation's."""
    ref = model.reference(tokens, dtype)
    tol = tolerance(dtype, ref)
    for p in sorted(got):
        err = float(np.abs(got[p] - ref[p]).max())
        assert err <= tol, f"{what}: position {p} of {len(tokens)}: |d| = {err:.3g} > {tol:.3g}"
    return len(got)


def prompts(vocab: int, lengths, seed: int):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
