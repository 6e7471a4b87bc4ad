"""Tensor-level wrappers of the CUDA kernels.

Each function checks devices, element types and layouts, then launches on the current
stream; outputs are passed in by the caller, so a step made of these calls allocates
nothing and can be captured in a CUDA graph.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import library as _library

from .library import KernelError, check, lib

F32, BF16 = 0, 1
EPI_NONE, EPI_XIELU, EPI_F32_OUT = 0, 1, 2
EPI_GELU_ERF, EPI_GELU_TANH = 4, 5          # GELU of the rounded sum, exact or tanh form (3: raw partial sums, inside the library)
EPI_RELU2 = 6                               # max(rounded sum, 0)^2
MAX_HEAD_DIM = 512      # the largest head the attention kernels take (csrc/attention_inputs.cu, csrc/attention_plain.cu)


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


def _stream() -> int:
    return _library.current_stream()


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtype=None, contiguous=True):
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def random_normal(out, k0: int, k1: int, mean: float, std: float, first: int = 0):
    """out.flat[j] = mean + std * z(first + j) of the counter-based generator with keys (k0, k1)."""
    _need(out, "out")
    check(lib().ti_random_normal(out.data_ptr(), dtype_code(out.dtype), out.numel(), first, k0, k1, mean, std, _stream()),
          "random_normal")


def embed(out, table, ids, status):
    _need(out, "out"); _need(table, "table", out.dtype); _need(ids, "ids", torch.int32); _need(status, "status", torch.int32)
    n, hidden = out.shape
    check(lib().ti_embed(out.data_ptr(), table.data_ptr(), ids.data_ptr(), n, hidden, table.shape[0],
                         dtype_code(out.dtype), status.data_ptr(), _stream()), "embed")


def gather_rows(out, x, idx):
    _need(out, "out"); _need(x, "x", out.dtype); _need(idx, "idx", torch.int32)
    check(lib().ti_gather_rows(out.data_ptr(), x.data_ptr(), idx.data_ptr(), out.shape[0], out.shape[1],
                               dtype_code(out.dtype), _stream()), "gather_rows")


def xielu(out, x, alpha_p, alpha_n, beta, eps):
    _need(out, "out"); _need(x, "x", out.dtype)
    check(lib().ti_xielu(out.data_ptr(), x.data_ptr(), x.numel(), alpha_p, alpha_n, beta, eps,
                         dtype_code(out.dtype), _stream()), "xielu")


def rmsnorm(out, x, w, eps):
    _need(out, "out"); _need(x, "x", out.dtype); _need(w, "w", out.dtype)
    size = x.shape[-1]
    check(lib().ti_rmsnorm(out.data_ptr(), x.data_ptr(), w.data_ptr(), x.numel() // size, size, eps,
                           dtype_code(out.dtype), _stream()), "rmsnorm")


def add_rmsnorm(x, delta, w, h, eps, partials=None):
    """x <- x + delta (or the sum of 32-bit ``partials`` [s, n, size]); h <- RMSNorm(x)·w."""
    _need(x, "x"); _need(w, "w", x.dtype); _need(h, "h", x.dtype)
    n, size = x.shape
    if partials is not None:
        _need(partials, "partials", torch.float32)
        s = partials.shape[0]
        check(lib().ti_add_rmsnorm(x.data_ptr(), None, partials.data_ptr(), s, partials.stride(0), w.data_ptr(),
                                   h.data_ptr(), n, size, eps, dtype_code(x.dtype), _stream()), "add_rmsnorm")
    else:
        _need(delta, "delta", x.dtype)
        check(lib().ti_add_rmsnorm(x.data_ptr(), delta.data_ptr(), None, 0, 0, w.data_ptr(), h.data_ptr(), n, size,
                                   eps, dtype_code(x.dtype), _stream()), "add_rmsnorm")


def add(x, delta):
    _need(x, "x"); _need(delta, "delta", x.dtype)
    check(lib().ti_add(x.data_ptr(), delta.data_ptr(), x.numel(), dtype_code(x.dtype), _stream()), "add")


def attention_inputs(qkv, q_out, k_cache, v_cache, q_norm_w, k_norm_w, eps, rotation, positions, slots,
                     nq, nkv, head_dim, page_size, write_kv=True):
    """qkv [n, (nq + 2 nkv) D] -> q_out [n, nq, D]; k and v rows into the pools at ``slots``. ``qkv`` may
    also be the 32-bit partial sums [s, n, features] of a projection that was split over k. ``rotation``:
    None, or a record with ``cos_sin`` [positions, rotary_dim / 2, 2] float32, ``rotary_dim`` and
    ``interleaved`` (see ``parts.base.Rotation``)."""
    cos_sin = rotation.cos_sin if rotation is not None else None
    rotary, interleaved = (int(rotation.rotary_dim), int(bool(rotation.interleaved))) if rotation is not None else (0, 0)
    if rotation is not None and (rotary < 2 or rotary % 2 or rotary > head_dim or cos_sin.shape[1] * 2 != rotary):
        raise KernelError(f"rotation over {rotary} of {head_dim} elements with a table of {tuple(cos_sin.shape)}")
    _need(qkv, "qkv", contiguous=False); _need(q_out, "q_out")
    _need(positions, "positions", torch.int32)
    if qkv.stride(-1) != 1:
        raise KernelError("qkv rows must be dense")
    if write_kv:
        _need(k_cache, "k_cache", q_out.dtype); _need(v_cache, "v_cache", q_out.dtype); _need(slots, "slots", torch.int32)
    if cos_sin is not None:
        _need(cos_sin, "cos_sin", torch.float32)
    if qkv.dim() == 3:
        _need(qkv, "partial sums", torch.float32)
        args = (None, qkv.stride(1), qkv.data_ptr(), qkv.shape[0], qkv.stride(0))
        n = qkv.shape[1]
    else:
        if qkv.dtype != q_out.dtype:
            raise KernelError(f"qkv must be {q_out.dtype}")
        args = (qkv.data_ptr(), qkv.stride(0), None, 0, 0)
        n = qkv.shape[0]
    check(lib().ti_attention_inputs(*args, q_out.data_ptr(), _ptr(k_cache), _ptr(v_cache),
                                    _ptr(q_norm_w), _ptr(k_norm_w), eps, _ptr(cos_sin), rotary, interleaved, positions.data_ptr(),
                                    _ptr(slots), n, nq, nkv, head_dim, page_size, int(write_kv),
                                    dtype_code(q_out.dtype), _stream()), "attention_inputs")


def attention_plain(out, q, k_cache, v_cache, block_table, tok_slot, positions, scale, nq, nkv, head_dim,
                    page_size, window=0, sink=None, chunk=0, distance_bias=None):
    """``sink`` [nq] float32: one more term exp(sink[head]) in every softmax's denominator (no key, no value). ``chunk`` > 0: a
    key is visible only inside the query's chunk of so many positions (counted from the sequence's start). ``distance_bias``
    [nq, L] float32: entry [head, min(distance, L - 1)] is added to the scaled score."""
    if sink is not None:
        _need(sink, "sink", torch.float32)
    if chunk or distance_bias is not None:
        if distance_bias is not None:
            _need(distance_bias, "distance_bias", torch.float32)
            if distance_bias.dim() != 2 or distance_bias.shape[0] != nq:
                raise KernelError(f"attention: bias table {tuple(distance_bias.shape)} for {nq} heads")
        _need(out, "out"); _need(q, "q", out.dtype); _need(k_cache, "k_cache", out.dtype); _need(v_cache, "v_cache", out.dtype)
        _need(block_table, "block_table", torch.int32); _need(tok_slot, "tok_slot", torch.int32); _need(positions, "positions", torch.int32)
        check(lib().ti_attention_plain_biased(out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), block_table.data_ptr(),
                                              block_table.stride(0), tok_slot.data_ptr(), positions.data_ptr(), scale, q.shape[0], nq, nkv,
                                              head_dim, page_size, window or 0, _ptr(sink), int(chunk or 0), _ptr(distance_bias),
                                              distance_bias.shape[1] if distance_bias is not None else 0, dtype_code(out.dtype), _stream()),
              "attention_plain")
        return
    _need(out, "out"); _need(q, "q", out.dtype); _need(k_cache, "k_cache", out.dtype); _need(v_cache, "v_cache", out.dtype)
    _need(block_table, "block_table", torch.int32); _need(tok_slot, "tok_slot", torch.int32)
    _need(positions, "positions", torch.int32)
    check(lib().ti_attention_plain(out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                   block_table.data_ptr(), block_table.stride(0), tok_slot.data_ptr(),
                                   positions.data_ptr(), scale, q.shape[0], nq, nkv, head_dim, page_size, window or 0,
                                   _ptr(sink), dtype_code(out.dtype), _stream()), "attention_plain")


def gemm_plain(y, x, w, epilogue=EPI_NONE, act=(0.0, 0.0, 0.0, 0.0)):
    """y[n, out] = x[n, in] · w[out, in]ᵀ on the CUDA cores in 32-bit arithmetic."""
    _need(x, "x", contiguous=False); _need(w, "w", x.dtype); _need(y, "y", contiguous=False)
    n, k = x.shape
    out = w.shape[0]
    if w.shape[1] != k or y.shape[0] != n or y.shape[1] != out or x.stride(1) != 1 or y.stride(1) != 1:
        raise KernelError(f"gemm: shapes x {tuple(x.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)} do not fit")
    want = torch.float32 if epilogue == EPI_F32_OUT else x.dtype
    if y.dtype != want:
        raise KernelError(f"gemm: output must be {want}")
    check(lib().ti_gemm_plain(y.data_ptr(), y.stride(0), x.data_ptr(), x.stride(0), w.data_ptr(), n, out, k, epilogue,
                              act[0], act[1], act[2], act[3], dtype_code(x.dtype), _stream()), "gemm_plain")


_argmax_ws = {}


def argmax_workspace(rows: int, vocab: int, device):
    """(values, ids, counters) for ``argmax`` over ``rows`` rows: one per device, grown on demand. The
    counters start at zero and every launch leaves them at zero."""
    chunks = lib().ti_argmax_chunks(vocab)
    key = str(device)
    ws = _argmax_ws.get(key)
    if ws is None or ws[0].numel() < rows * chunks or ws[2].numel() < rows:
        n = max(rows, 64)
        ws = _argmax_ws[key] = (torch.empty(n * 256, dtype=torch.float32, device=device),
                                torch.empty(n * 256, dtype=torch.int32, device=device),
                                torch.zeros(n, dtype=torch.int32, device=device))
    return ws


def argmax(logits, out, workspace=None, also=None):
    """out[row] = the largest logit's id, ties to the smaller id; ``also``: a second int32 vector that gets the same
    tokens (the next step's token ids)."""
    _need(logits, "logits", torch.float32, contiguous=False); _need(out, "out", torch.int32)
    val, idx, cnt = workspace or argmax_workspace(logits.shape[0], logits.shape[1], logits.device)
    check(lib().ti_argmax(logits.data_ptr(), logits.stride(0), logits.shape[0], logits.shape[1], out.data_ptr(), _ptr(also),
                          val.data_ptr(), idx.data_ptr(), cnt.data_ptr(), _stream()), "argmax")


def sample(logits, out, temperature, top_k, top_p, seeds, counters, also=None, cluster_blocks=0):
    """``cluster_blocks``: how many blocks share a row (1, 2, 4 or 8); 0 lets the library choose from the number of
    rows and the vocabulary. The token does not depend on it."""
    _need(logits, "logits", torch.float32, contiguous=False); _need(out, "out", torch.int32)
    _need(seeds, "seeds", torch.int32); _need(counters, "counters", torch.int32)
    check(lib().ti_sample_shared(logits.data_ptr(), logits.stride(0), logits.shape[0], logits.shape[1], temperature, top_k,
                                 top_p, seeds.data_ptr(), counters.data_ptr(), out.data_ptr(), _ptr(also), cluster_blocks,
                                 _stream()), "sample")


# ---------------------------------------------------------------- a residual stream in 32-bit
ACT_GELU_ERF, ACT_GELU_TANH = 0, 1


def embed_positions32(x, table, pos_table, ids, positions, status):
    """x[t] = table[ids[t]] + pos_table[positions[t]], summed and kept in 32-bit; without ``pos_table`` the token's row alone."""
    _need(x, "x", torch.float32); _need(table, "table")
    _need(ids, "ids", torch.int32); _need(positions, "positions", torch.int32); _need(status, "status", torch.int32)
    n, hidden = x.shape
    if pos_table is not None:
        _need(pos_table, "pos_table", table.dtype)
    if table.shape[1] != hidden or (pos_table is not None and pos_table.shape[1] != hidden):
        raise KernelError(f"embed_positions32: table {tuple(table.shape)} for a width of {hidden}")
    check(lib().ti_embed_positions32(x.data_ptr(), table.data_ptr(), _ptr(pos_table), ids.data_ptr(), positions.data_ptr(), n,
                                     hidden, table.shape[0], pos_table.shape[0] if pos_table is not None else 0, dtype_code(table.dtype),
                                     status.data_ptr(), _stream()),
          "embed_positions32")


def embed_bigram32(x, table, pair, ids, positions, tok_slot, last, scale, buckets=0, mul_prev=0, mul_cur=0, status=None):
    """x[t] = table[ids[t]] * scale + pair[(previous id * mul_prev + ids[t] * mul_cur) mod buckets] in 32-bit; the token before comes
    from the step or, at the step's start, from ``last`` [slots] int32; a sequence's first token takes row ``buckets`` of ``pair``
    [buckets + 1, hidden]. ``pair`` None: the scaled row alone."""
    _need(x, "x", torch.float32); _need(table, "table"); _need(ids, "ids", torch.int32); _need(positions, "positions", torch.int32)
    _need(tok_slot, "tok_slot", torch.int32); _need(status, "status", torch.int32)
    n, hidden = x.shape
    if pair is not None:
        _need(pair, "pair", table.dtype); _need(last, "last", torch.int32)
        if tuple(pair.shape) != (buckets + 1, hidden):
            raise KernelError(f"embed_bigram32: second table {tuple(pair.shape)} for {buckets} buckets and a width of {hidden}")
    if table.shape[1] != hidden:
        raise KernelError(f"embed_bigram32: table {tuple(table.shape)} for a width of {hidden}")
    check(lib().ti_embed_bigram32(x.data_ptr(), table.data_ptr(), _ptr(pair), ids.data_ptr(), positions.data_ptr(), tok_slot.data_ptr(), _ptr(last), n,
                                  hidden, table.shape[0], scale, buckets, mul_prev, mul_cur, dtype_code(table.dtype), status.data_ptr(), _stream()),
          "embed_bigram32")


def last_token_update(last, step):
    """last[slot] = the last token that the step brings for the sequence in ``slot``."""
    _need(last, "last", torch.int32)
    check(lib().ti_last_token_update(last.data_ptr(), step.token_ids.data_ptr(), step.cu_seqlens.data_ptr(), step.seq_slots.data_ptr(), step.n_seqs,
                                     _stream()), "last_token_update")


def cast_rows_into(h, x):
    """h[:, :size] = x rounded to h's element type for h a view [n, size] of rows that may be longer (stride(0) >= size); x is 32-bit."""
    _need(h, "h", contiguous=False); _need(x, "x", torch.float32)
    if h.stride(1) != 1 or h.shape != x.shape:
        raise KernelError(f"cast_rows_into: h {tuple(h.shape)} with strides {h.stride()} for x {tuple(x.shape)}")
    check(lib().ti_cast_rows_ld(h.data_ptr(), h.stride(0), x.data_ptr(), x.shape[0], x.shape[1], dtype_code(h.dtype), _stream()), "cast_rows_into")


def rotate_heads(x, rotation, positions, first=0):
    """x [n, heads, row]: the elements [first, first + rotary_dim) of every head are rotated in place by the positions' angles."""
    _need(x, "x"); _need(positions, "positions", torch.int32); _need(rotation.cos_sin, "cos_sin", torch.float32)
    n, heads, row = x.shape
    rot = int(rotation.rotary_dim)
    if rotation.cos_sin.shape[1] * 2 != rot:
        raise KernelError(f"rotate_heads: {rot} elements with a table of {tuple(rotation.cos_sin.shape)}")
    check(lib().ti_rotate_heads(x.data_ptr(), rotation.cos_sin.data_ptr(), positions.data_ptr(), n, heads, row, first, rot,
                                int(bool(rotation.interleaved)), dtype_code(x.dtype), _stream()), "rotate_heads")


def cast_rows(h, x):
    """h = x rounded to h's element type; x is 32-bit."""
    _need(h, "h"); _need(x, "x", torch.float32)
    check(lib().ti_cast_rows(h.data_ptr(), x.data_ptr(), x.numel(), dtype_code(h.dtype), _stream()), "cast_rows")


NORM_OFFSET, NORM_CENTRED = 1, 2          # bits of a norm's flags word: the gain is 1 + w; the row's mean is taken off first


def norm_flags(offset) -> int:
    """``offset`` as the wrappers take it: a bool (the gain is 1 + w) or the flags word itself."""
    return int(offset) if isinstance(offset, int) and not isinstance(offset, bool) else int(bool(offset))


def norm32(y, x, w, eps, offset=False):
    """y = x / rms(x) * (1 + w if offset else w), computed in 32-bit; x is 32-bit or of y's type. ``offset`` may be a flags
    word: with NORM_CENTRED the row's mean is taken off and rms is that of the deviations."""
    _need(y, "y"); _need(x, "x"); _need(w, "w", y.dtype)
    if x.dtype not in (torch.float32, y.dtype):
        raise KernelError(f"norm32: input must be float32 or {y.dtype}")
    size = x.shape[-1]
    check(lib().ti_norm32(y.data_ptr(), x.data_ptr(), int(x.dtype == torch.float32), w.data_ptr(), x.numel() // size, size, eps,
                          norm_flags(offset), dtype_code(y.dtype), _stream()), "norm32")


def branch_norm_add32(x, delta, w, eps, mult, offset=False, h=None, out_norm=None, gather=None, bias=None):
    """x += mult * delta / rms(delta) * g(w) in 32-bit (``delta``: [n, size] of w's type, or 32-bit partial sums
    [s, n, size]); then, with ``h``, h = x rounded, or h = x / rms(x) * g(w_out) for ``out_norm`` = (w_out, eps, offset).
    ``bias`` [size]: added to delta before its norm. ``offset`` (both) may be a flags word (NORM_CENTRED: a layer norm).
    ``gather`` [n, k] int32: row t of the branch is the sum of the rows gather[t, :] of ``delta`` [rows, size]."""
    _need(x, "x", torch.float32); _need(w, "w")
    n, size = x.shape
    g_args = (None, 0)
    if gather is not None:
        _need(gather, "gather", torch.int32); _need(delta, "delta", w.dtype)
        if gather.shape[0] != n or delta.shape[1] != size:
            raise KernelError(f"branch_norm_add32: gather {tuple(gather.shape)}, rows {tuple(delta.shape)} for a stream of {tuple(x.shape)}")
        d_args = (delta.data_ptr(), None, 0, 0)
        g_args = (gather.data_ptr(), gather.shape[1])
    elif delta.dim() == 3:
        _need(delta, "partial sums", torch.float32)
        d_args = (None, delta.data_ptr(), delta.shape[0], delta.stride(0))
    else:
        _need(delta, "delta", w.dtype)
        d_args = (delta.data_ptr(), None, 0, 0)
    if h is not None:
        _need(h, "h", w.dtype)
    w_out, eps_out, offset_out = out_norm if out_norm is not None else (None, 0.0, False)
    if w_out is not None:
        _need(w_out, "w_out", w.dtype)
    if bias is not None:
        _need(bias, "bias", w.dtype)
    check(lib().ti_branch_norm_add32(x.data_ptr(), *d_args, *g_args, _ptr(bias), w.data_ptr(), norm_flags(offset), eps, mult, _ptr(h), _ptr(w_out),
                                     norm_flags(offset_out), eps_out, n, size, dtype_code(w.dtype), _stream()), "branch_norm_add32")


def latent_inputs(rows, cq, pool, wq, wkv, eps, slots, q_rank, kv_rank, rotation=None, positions=None, pool_row=None):
    """rows [n, >= q_rank + kv_rank] (or 32-bit partial sums [s, n, ...]) -> cq [n, q_rank] and the key/value latent of every
    token at its place ``slots[t]`` of ``pool`` [positions, pool_row]; both RMS-normed in 32-bit with plain weights. With
    ``rotation`` the rotary_dim elements after the latents are a key part shared by all heads: rotated by ``positions`` and
    written behind the latent in the pool's row (``pool_row`` >= kv_rank + rotary_dim elements, zeros after)."""
    rot = int(rotation.rotary_dim) if rotation is not None else 0
    pool_row = int(pool_row or kv_rank)
    if rotation is not None:
        _need(rotation.cos_sin, "cos_sin", torch.float32); _need(positions, "positions", torch.int32)
        if rotation.cos_sin.shape[1] * 2 != rot:
            raise KernelError(f"latent_inputs: {rot} rotated elements with a table of {tuple(rotation.cos_sin.shape)}")
    _need(cq, "cq"); _need(pool, "pool", cq.dtype); _need(wq, "wq", cq.dtype); _need(wkv, "wkv", cq.dtype); _need(slots, "slots", torch.int32)
    if rows.dim() == 3:
        _need(rows, "partial sums", torch.float32)
        args = (None, 0, rows.data_ptr(), rows.shape[0], rows.stride(0))
        n, in_row = rows.shape[1], rows.shape[2]
    else:
        _need(rows, "rows", cq.dtype, contiguous=False)
        if rows.stride(1) != 1:
            raise KernelError("latent_inputs: rows must be dense")
        args = (rows.data_ptr(), rows.stride(0), None, 0, 0)
        n, in_row = rows.shape[0], rows.shape[1]
    check(lib().ti_latent_inputs(*args, cq.data_ptr(), pool.data_ptr(), wq.data_ptr(), wkv.data_ptr(), eps, slots.data_ptr(), n,
                                 q_rank, kv_rank, rot, _ptr(rotation.cos_sin) if rotation is not None else None,
                                 int(bool(rotation.interleaved)) if rotation is not None else 0, _ptr(positions), pool_row, in_row,
                                 dtype_code(cq.dtype), _stream()), "latent_inputs")


def head_gemm(y, x, w):
    """y[t, h, :] = w[h] x[t, h, :] for w [heads, out_h, in_h], x [n, heads, in_h], y [n, heads, out_h]."""
    _need(y, "y"); _need(x, "x", y.dtype); _need(w, "w", y.dtype)
    heads, out_h, in_h = w.shape
    n = x.shape[0]
    if tuple(x.shape) != (n, heads, in_h) or tuple(y.shape) != (n, heads, out_h):
        raise KernelError(f"head_gemm: x {tuple(x.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)} do not fit")
    check(lib().ti_head_gemm(y.data_ptr(), heads * out_h, x.data_ptr(), heads * in_h, w.data_ptr(), n, heads, out_h, in_h,
                             dtype_code(y.dtype), _stream()), "head_gemm")


def gelu(out, x, kind=ACT_GELU_ERF):
    _need(out, "out"); _need(x, "x", out.dtype)
    check(lib().ti_gelu(out.data_ptr(), x.data_ptr(), x.numel(), kind, dtype_code(out.dtype), _stream()), "gelu")


def gated_token_embedding(g, table, ids, first):
    """g[t, j] = gelu_tanh(g[t, j]) * table[ids[t], first + j], in place."""
    _need(g, "g"); _need(table, "table", g.dtype); _need(ids, "ids", torch.int32)
    n, dim = g.shape
    check(lib().ti_gated_token_embedding(g.data_ptr(), table.data_ptr(), ids.data_ptr(), n, dim, table.shape[1], first, table.shape[0],
                                         dtype_code(g.dtype), _stream()), "gated_token_embedding")


def gated_unit_limit(y, gu, limit, slope, shift, plan=None, tile=0, limits=None):
    """y[t, j] = a * sigmoid(slope * a) * (b + shift), a = min(gu[t, j], limit), b = clamp(gu[t, ff + j], -limit, limit).
    With ``plan`` (rows in tiles of ``tile`` rows, each tile one unit's) the limit of a row is ``limits[unit]``."""
    _need(y, "y"); _need(gu, "gu", y.dtype)
    n, ff = y.shape
    if tuple(gu.shape) != (n, 2 * ff):
        raise KernelError(f"gated_unit_limit: gu {tuple(gu.shape)} for y {tuple(y.shape)}")
    if plan is not None:
        _need(plan, "plan", torch.int32); _need(limits, "limits", torch.float32)
    check(lib().ti_gated_unit_limit(y.data_ptr(), gu.data_ptr(), n, ff, limit, _ptr(plan), tile, _ptr(limits), slope, shift,
                                    dtype_code(y.dtype), _stream()), "gated_unit_limit")


def router_topk(h, wr, top, ids, scores, logits=None, always=0):
    """ids, scores [n, top + always]: the ``top`` experts of every row with the largest sigmoid(wr h), logits in 32-bit,
    followed by ``always`` units that every row takes (numbered after the experts, score 1). ``logits`` [n, experts]
    float32: the sums wr h if a product kernel has already left them (h is then not read)."""
    if tuple(ids.shape) != (h.shape[0], top + always) or ids.shape != scores.shape:
        raise KernelError(f"router_topk: ids {tuple(ids.shape)}, scores {tuple(scores.shape)} for top {top} + {always}")
    _need(h, "h"); _need(wr, "wr", h.dtype); _need(ids, "ids", torch.int32); _need(scores, "scores", torch.float32)
    n, width = h.shape
    if logits is not None:
        _need(logits, "logits", torch.float32)
        if tuple(logits.shape) != (n, wr.shape[0]):
            raise KernelError(f"router_topk: logits {tuple(logits.shape)} for {n} rows and {wr.shape[0]} experts")
    check(lib().ti_router_topk(h.data_ptr(), wr.data_ptr(), _ptr(logits), n, width, wr.shape[0], top, always, ids.data_ptr(), scores.data_ptr(),
                               dtype_code(h.dtype), _stream()), "router_topk")


EXPERT_TILE_ROWS = 32          # the smallest tile of rows the grouped products take (csrc/tile_gemm.cuh)


def expert_plan_sizes(pairs: int, experts: int, tile: int):
    """(most tiles, rows of the padded layout) for ``pairs`` (token, choice) pairs over ``experts`` experts in tiles of
    ``tile`` rows."""
    tiles = int(lib().ti_expert_plan_max_tiles(pairs, experts, tile))
    return tiles, tiles * tile


def expert_plan(ids, experts, tile, pair_row, row_pair, plan):
    """``row_pair`` [capacity] and ``plan`` [1 + capacity / tile] are filled for the pairs ``ids`` [n, top]."""
    _need(ids, "ids", torch.int32); _need(pair_row, "pair_row", torch.int32); _need(row_pair, "row_pair", torch.int32)
    _need(plan, "plan", torch.int32)
    check(lib().ti_expert_plan(ids.data_ptr(), ids.numel(), experts, tile, row_pair.numel(), pair_row.data_ptr(), row_pair.data_ptr(),
                               plan.data_ptr(), _stream()), "expert_plan")


def expert_gather(xs, h, pair_row, scores, per_token, scale_input=True):
    """xs[pair_row[p]] = score[p] * h[p // per_token] (or h[...] itself) for every pair p; padding rows are not touched."""
    _need(xs, "xs"); _need(h, "h", xs.dtype); _need(pair_row, "pair_row", torch.int32); _need(scores, "scores", torch.float32)
    check(lib().ti_expert_gather(xs.data_ptr(), h.data_ptr(), pair_row.data_ptr(), scores.data_ptr(), pair_row.numel(), per_token,
                                 xs.shape[1], int(bool(scale_input)), dtype_code(xs.dtype), _stream()), "expert_gather")


def grouped_gemm(y, x, w, plan, tile, gated=False, limits=None, slope=0.0, shift=0.0):
    """Rows of x grouped by expert in tiles of ``tile`` rows (``plan``): y[row] = w[expert] x[row], on the CUDA cores;
    ``gated``: w [experts, 2 * out, in] holds gate rows then up rows and y is the clamped gated unit's activation, each
    unit with its own ``limits[unit]``."""
    if gated:
        _need(limits, "limits", torch.float32)
    _need(y, "y"); _need(x, "x", y.dtype); _need(w, "w", y.dtype); _need(plan, "plan", torch.int32)
    experts, rows_w, k = w.shape
    out = rows_w // 2 if gated else rows_w
    if x.shape[1] != k or y.shape[1] != out or x.shape[0] != y.shape[0]:
        raise KernelError(f"grouped_gemm: x {tuple(x.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)} do not fit")
    check(lib().ti_grouped_gemm(y.data_ptr(), x.data_ptr(), w.data_ptr(), plan.data_ptr(), x.shape[0], tile, out, k, int(bool(gated)),
                                _ptr(limits), slope, shift, dtype_code(y.dtype), _stream()), "grouped_gemm")


def expert_combine(out, y, pair_row, scores, shared, top, scale_output=False, h=None, pass_weight=None):
    """out[t] = sum over the token's pairs of (score x) y[row of the pair] (+ shared[t]) (+ pass_weight[t] * h[t]: the share of
    choices that hand their input through; their pairs have no row)."""
    _need(out, "out"); _need(y, "y", out.dtype); _need(pair_row, "pair_row", torch.int32); _need(scores, "scores", torch.float32)
    if shared is not None:
        _need(shared, "shared", out.dtype)
    if pass_weight is not None:
        _need(pass_weight, "pass_weight", torch.float32); _need(h, "h", out.dtype)
    n, width = out.shape
    check(lib().ti_expert_combine(out.data_ptr(), y.data_ptr(), pair_row.data_ptr(), scores.data_ptr(), _ptr(shared), _ptr(h), _ptr(pass_weight),
                                  n, top, width, int(bool(scale_output)), dtype_code(out.dtype), _stream()), "expert_combine")



# ---------------------------------------------------------------- a state carried from token to token; convolved projections
def _rows_or_partials(d, dtype, name):
    """(rows pointer, partials pointer, count, stride) of a sublayer's output: [n, size] of ``dtype`` or 32-bit partial sums [s, n, size]."""
    if d is None:
        return (None, None, 0, 0)
    if d.dim() == 3:
        _need(d, name, torch.float32)
        return (None, d.data_ptr(), d.shape[0], d.stride(0))
    _need(d, name, dtype)
    return (d.data_ptr(), None, 0, 0)


def sum_add_norm32(x, d1, d2, h, w_out, eps_out, offset_out=False):
    """x += d1 + d2 on a 32-bit stream (``d2`` may be None), then h = x / rms(x) * g(w_out) rounded to h's type (``h`` None: the
    stream's update alone)."""
    _need(x, "x", torch.float32)
    n, size = x.shape
    dtype = h.dtype if h is not None else (d1.dtype if d1.dim() == 2 else d2.dtype)
    if h is not None:
        _need(h, "h"); _need(w_out, "w_out", h.dtype)
    check(lib().ti_sum_add_norm32(x.data_ptr(), *_rows_or_partials(d1, dtype, "d1"), *_rows_or_partials(d2, dtype, "d2"), _ptr(h), _ptr(w_out),
                                  int(bool(offset_out)), eps_out, n, size, dtype_code(dtype), _stream()), "sum_add_norm32")


def lightning_scan(o, rows, q_off, k_off, v_off, state, decay, cu_seqlens, seq_slots, batch, heads, dim, vdim, act=True):
    """The recurrence S = a_h S + k v^T, o = S^T q over the step's tokens of every sequence, from and to ``state``
    [slots, heads, dim, vdim] float32. ``rows`` [n, ld]: the projections' output with queries, keys and values from the given
    columns on; ``act``: SiLU on them. o [n, heads * vdim] float32."""
    _need(o, "o", torch.float32); _need(rows, "rows", contiguous=False); _need(state, "state", torch.float32); _need(decay, "decay", torch.float32)
    _need(cu_seqlens, "cu_seqlens", torch.int32); _need(seq_slots, "seq_slots", torch.int32)
    if rows.stride(1) != 1 or tuple(state.shape[1:]) != (heads, dim, vdim) or decay.numel() != heads:
        raise KernelError(f"lightning_scan: rows {tuple(rows.shape)}, state {tuple(state.shape)} for {heads} heads of {dim} x {vdim}")
    check(lib().ti_lightning_scan(o.data_ptr(), rows.data_ptr(), rows.stride(0), q_off, k_off, v_off, state.data_ptr(), decay.data_ptr(),
                                  cu_seqlens.data_ptr(), seq_slots.data_ptr(), rows.shape[0], batch, heads, dim, vdim, int(bool(act)), dtype_code(rows.dtype),
                                  _stream()), "lightning_scan")


def lightning_out(y, o, gate, w, eps):
    """y = o / rms(o) * w * sigmoid(gate), the norm over the whole row in 32-bit; ``gate`` [n, size] (rows may be strided) or None."""
    _need(y, "y"); _need(o, "o", torch.float32); _need(w, "w", y.dtype)
    if gate is not None:
        _need(gate, "gate", y.dtype, contiguous=False)
    n, size = y.shape
    check(lib().ti_lightning_out(y.data_ptr(), o.data_ptr(), _ptr(gate), gate.stride(0) if gate is not None else 0, w.data_ptr(), eps, n, size,
                                 dtype_code(y.dtype), _stream()), "lightning_out")


def conv_attention_inputs(rows, bias, conv, taps, state, q_norm_w, k_norm_w, eps, rotation, q_out, k_cache, v_cache, step, slot_map,
                          nq, nkv, dim, vdim, padded, page_size, write_kv=True, head_norm=False):
    """The step's projected rows (queries, then keys and values with ``write_kv``) -> bias, causal convolution over time (history
    from ``state`` [slots, taps - 1, channels] float32), whole-row RMS norms of q and k (``head_norm``: every head by itself, with
    one weight of the head's size), rotation -> q_out [n, nq, padded] and the keys and values at ``slot_map`` in the pools. ``step``
    gives positions, cu_seqlens, seq_slots, kv_lens."""
    _need(rows, "rows", q_out.dtype, contiguous=False); _need(q_out, "q_out")
    cos_sin = rotation.cos_sin if rotation is not None else None
    rotary = int(rotation.rotary_dim) if rotation is not None else 0
    if rotation is not None and rotation.interleaved:
        raise KernelError("conv_attention_inputs: only the half-split pairing is built")
    if state is not None:
        _need(state, "state", torch.float32)
    check(lib().ti_conv_attention_inputs(rows.data_ptr(), rows.stride(0), _ptr(bias), _ptr(conv), taps, _ptr(state), _ptr(q_norm_w), _ptr(k_norm_w),
                                         eps, _ptr(cos_sin), rotary, q_out.data_ptr(), _ptr(k_cache), _ptr(v_cache), step.positions.data_ptr(),
                                         _ptr(slot_map), step.cu_seqlens.data_ptr(), step.seq_slots.data_ptr(), step.kv_lens.data_ptr(),
                                         rows.shape[0], step.n_seqs, nq, nkv, dim, vdim, padded, page_size, int(bool(write_kv)),
                                         int(bool(head_norm)), dtype_code(q_out.dtype), _stream()), "conv_attention_inputs")


def conv_state_update(state, rows, bias, taps, step, channels):
    """After ``conv_attention_inputs``: every sequence's state becomes its last taps - 1 projected rows."""
    _need(state, "state", torch.float32); _need(rows, "rows", contiguous=False)
    check(lib().ti_conv_state_update(state.data_ptr(), rows.data_ptr(), rows.stride(0), _ptr(bias), taps, step.cu_seqlens.data_ptr(),
                                     step.seq_slots.data_ptr(), step.n_seqs, channels, dtype_code(rows.dtype), _stream()), "conv_state_update")


def sigmoid_gate(y, attn, gate, heads, vdim, padded, per_head=False):
    """y [n, heads * vdim] = attn [n, heads, padded][..., :vdim] * sigmoid(gate [n, heads * vdim]) (``gate`` None: the copy alone);
    ``per_head``: gate is [n, heads], one number for a whole head."""
    _need(y, "y"); _need(attn, "attn", y.dtype)
    if gate is not None:
        _need(gate, "gate", y.dtype, contiguous=False)
    check(lib().ti_sigmoid_gate(y.data_ptr(), attn.data_ptr(), _ptr(gate), gate.stride(0) if gate is not None else 0, y.shape[0], heads, vdim,
                                padded, int(bool(per_head)), dtype_code(y.dtype), _stream()), "sigmoid_gate")


def router_select(h, wr, logits, experts, total, top, ids, scores, pass_weight=None, softmax=True, correction=None, groups=1, keep=1,
                  renormalize=True, always=0, gate=False):
    """The router with groups, a correction for the choice, normalised weights, pass-through choices and a gated always-on unit
    (``csrc/routed_experts.cu``: router_select). ``logits`` [n, >= total (+ 1 with gate)] float32 or None (then from h and wr)."""
    _need(h, "h"); _need(wr, "wr", h.dtype); _need(ids, "ids", torch.int32); _need(scores, "scores", torch.float32)
    n, width = h.shape
    if tuple(ids.shape) != (n, top + always) or ids.shape != scores.shape or wr.shape[0] != total + int(bool(gate)):
        raise KernelError(f"router_select: ids {tuple(ids.shape)}, router {tuple(wr.shape)} for top {top} + {always} of {total}")
    if logits is not None:
        _need(logits, "logits", torch.float32, contiguous=False)
    if correction is not None:
        _need(correction, "correction", torch.float32)
    if pass_weight is not None:
        _need(pass_weight, "pass_weight", torch.float32)
    check(lib().ti_router_select(h.data_ptr(), wr.data_ptr(), _ptr(logits), logits.stride(0) if logits is not None else 0, n, width, experts, total,
                                 int(bool(softmax)), _ptr(correction), groups, keep, top, int(bool(renormalize)), always, int(bool(gate)),
                                 ids.data_ptr(), scores.data_ptr(), _ptr(pass_weight), dtype_code(h.dtype), _stream()), "router_select")


ACT_SILU_GATED, ACT_GELU_TANH_GATED = 0, 1


def gated_act(y, gu, kind):
    """y[t, j] = act(gu[t, j]) * gu[t, ff + j]; kind ACT_SILU_GATED or ACT_GELU_TANH_GATED."""
    _need(y, "y"); _need(gu, "gu", y.dtype)
    n, ff = y.shape
    if tuple(gu.shape) != (n, 2 * ff):
        raise KernelError(f"gated_act: gu {tuple(gu.shape)} for y {tuple(y.shape)}")
    check(lib().ti_gated_act(y.data_ptr(), gu.data_ptr(), n, ff, kind, dtype_code(y.dtype), _stream()), "gated_act")


ACT_RELU2, ACT_TANH = 2, 3


def tanh(out, x):
    """out = tanh(x), rounded once."""
    _need(out, "out"); _need(x, "x", out.dtype)
    check(lib().ti_gelu(out.data_ptr(), x.data_ptr(), x.numel(), ACT_TANH, dtype_code(out.dtype), _stream()), "tanh")


def relu2(out, x):
    """out = max(x, 0)^2, rounded once."""
    _need(out, "out"); _need(x, "x", out.dtype)
    check(lib().ti_gelu(out.data_ptr(), x.data_ptr(), x.numel(), ACT_RELU2, dtype_code(out.dtype), _stream()), "relu2")


# ---------------------------------------------------------------- several copies of the residual stream
def _floats(values):
    import ctypes
    values = [float(v) for v in values]
    return (ctypes.c_float * len(values))(*values)


def streams_begin(x, x0, streams):
    """x [n, streams * size] float32 <- x0 [n, size] in every copy."""
    _need(x, "x", torch.float32); _need(x0, "x0", torch.float32)
    n, size = x0.shape
    check(lib().ti_streams_begin(x.data_ptr(), x0.data_ptr(), n, streams, size, _stream()), "streams_begin")


def streams_read_norm(h, x, a, w, b, eps, centred=True):
    """h = norm(sum_s a[s] x_s) for x [n, S * size] float32, ``a`` [S] float32 on the device; the norm has the weight ``w`` and,
    if not None, the bias ``b``; ``centred``: a layer norm (mean taken off), else an RMS norm."""
    _need(h, "h"); _need(x, "x", torch.float32); _need(a, "a", torch.float32); _need(w, "w", h.dtype)
    n, size = h.shape
    check(lib().ti_streams_read_norm(h.data_ptr(), x.data_ptr(), a.data_ptr(), a.numel(), w.data_ptr(), _ptr(b), eps, int(bool(centred)), n, size,
                                     dtype_code(h.dtype), _stream()), "streams_read_norm")


def streams_update(x, delta, mix, out, in_next, h, w, b, eps, centred=True):
    """x_t <- sum_s mix[s][t] x_s + out[t] * delta for the S copies x [n, S * size] float32 (``mix`` [S * S] and ``out`` [S]: host
    floats, ``out`` already times the branch multiplier); then, with ``h``, h = norm(sum_t in_next[t] x_t) (``in_next`` host floats;
    the norm as in ``streams_read_norm``). ``delta``: rows [n, size] of h's type, or float32 [s, n, size] that are added up."""
    _need(x, "x", torch.float32)
    S = len(out)
    n = x.shape[0]
    size = x.shape[1] // S
    dtype = h.dtype if h is not None else (delta.dtype if delta.dim() == 2 else w.dtype)
    if h is not None:
        _need(h, "h"); _need(w, "w", h.dtype)
    check(lib().ti_streams_update(x.data_ptr(), *_rows_or_partials(delta, dtype, "delta"), _floats(mix), _floats(out),
                                  _floats(in_next) if in_next is not None else None, S, _ptr(h), _ptr(w), _ptr(b), eps, int(bool(centred)), n, size,
                                  dtype_code(dtype), _stream()), "streams_update")


# ---------------------------------------------------------------- recurrences with decays that depend on the token
def shift_blend(out, h, mu, prev, step):
    """out [K, n, W] = h + (row before - h) * mu[k]; ``prev`` [slots, >= W] float32 (rows may be strided) holds every sequence's
    last row and is moved on to the step's last."""
    _need(out, "out"); _need(h, "h", out.dtype); _need(mu, "mu", out.dtype); _need(prev, "prev", torch.float32, contiguous=False)
    n, W = h.shape
    check(lib().ti_shift_blend(out.data_ptr(), h.data_ptr(), mu.data_ptr(), mu.shape[0], prev.data_ptr(), prev.stride(0), step.cu_seqlens.data_ptr(),
                               step.seq_slots.data_ptr(), n, step.n_seqs, W, dtype_code(out.dtype), _stream()), "shift_blend")


def decay_scan(o, rkv, r_off, k_off, v_off, dlog, w0, u, state, step, heads, dim):
    """o_t = (S + diag(u) k v^T)^T r; S <- diag(exp(-exp(dlog_t + w0))) S + k v^T over the step's tokens of every sequence; ``state``
    [slots, >= heads * dim * dim] float32 (rows may be strided); rkv [n, ld] with r, k, v from the given columns on; o, dlog float32."""
    _need(o, "o", torch.float32); _need(rkv, "rkv", contiguous=False); _need(dlog, "dlog", torch.float32); _need(w0, "w0", torch.float32)
    _need(u, "u", torch.float32); _need(state, "state", torch.float32, contiguous=False)
    check(lib().ti_decay_scan(o.data_ptr(), rkv.data_ptr(), rkv.stride(0), r_off, k_off, v_off, dlog.data_ptr(), w0.data_ptr(), u.data_ptr(),
                              state.data_ptr(), state.stride(0), step.cu_seqlens.data_ptr(), step.seq_slots.data_ptr(), rkv.shape[0], step.n_seqs,
                              heads, dim, dtype_code(rkv.dtype), _stream()), "decay_scan")


def delta_inputs(out, proj, conv, taps, hist, step, qk_heads, dim, value_channels, unit_eps):
    """proj [n, 2 * qk_heads * dim + value_channels] -> causal convolution over time (history ``hist`` [slots, >= (taps - 1) * C]
    float32), SiLU, unit q and k heads (q also times dim^-1/2) -> out float32."""
    _need(out, "out", torch.float32); _need(proj, "proj", contiguous=False)
    if hist is not None:
        _need(hist, "hist", torch.float32, contiguous=False)
    check(lib().ti_delta_inputs(out.data_ptr(), proj.data_ptr(), proj.stride(0), _ptr(conv), taps, _ptr(hist), hist.stride(0) if hist is not None else 0,
                                step.cu_seqlens.data_ptr(), step.seq_slots.data_ptr(), proj.shape[0], step.n_seqs, qk_heads, dim, value_channels,
                                unit_eps, dtype_code(proj.dtype), _stream()), "delta_inputs")


def history_update(hist, proj, taps, step, channels):
    """Every sequence's history [slots, >= (taps - 1) * channels] becomes its last taps - 1 rows of ``proj``."""
    _need(hist, "hist", torch.float32, contiguous=False); _need(proj, "proj", contiguous=False)
    check(lib().ti_history_update(hist.data_ptr(), hist.stride(0), proj.data_ptr(), proj.stride(0), taps, step.cu_seqlens.data_ptr(),
                                  step.seq_slots.data_ptr(), step.n_seqs, channels, dtype_code(proj.dtype), _stream()), "history_update")


def delta_scan(o, qkv, ba, a_log, dt_bias, state, step, heads, qk_heads, dim, vdim):
    """The gated delta rule over the step's tokens of every sequence: S <- g S; e = beta (v - S^T k); S <- S + k e^T; o = S^T q with
    beta = sigmoid(ba[:, h]), g = exp(-exp(a_log) softplus(ba[:, heads + h] + dt_bias)). qkv, ba, o float32."""
    _need(o, "o", torch.float32); _need(qkv, "qkv", torch.float32); _need(ba, "ba", torch.float32); _need(a_log, "a_log", torch.float32)
    _need(dt_bias, "dt_bias", torch.float32); _need(state, "state", torch.float32, contiguous=False)
    check(lib().ti_delta_scan(o.data_ptr(), qkv.data_ptr(), qkv.stride(0), ba.data_ptr(), a_log.data_ptr(), dt_bias.data_ptr(), state.data_ptr(),
                              state.stride(0), step.cu_seqlens.data_ptr(), step.seq_slots.data_ptr(), qkv.shape[0], step.n_seqs, heads, qk_heads, dim,
                              vdim, _stream()), "delta_scan")


def heads_norm_gate(y, o, gate, w, eps, heads, vdim):
    """y [n, heads * vdim] = o / rms(o over each head) * w * silu(gate); w [vdim] (shared by the heads) or [heads * vdim]."""
    _need(y, "y"); _need(o, "o", torch.float32); _need(w, "w", y.dtype)
    if gate is not None:
        _need(gate, "gate", y.dtype, contiguous=False)
    if w.numel() not in (vdim, heads * vdim):
        raise KernelError(f"heads_norm_gate: a weight of {w.numel()} for {heads} heads of {vdim}")
    check(lib().ti_heads_norm_gate(y.data_ptr(), o.data_ptr(), _ptr(gate), gate.stride(0) if gate is not None else 0, w.data_ptr(),
                                   int(w.numel() == vdim), eps, y.shape[0], heads, vdim, dtype_code(y.dtype),
                                   _stream()), "heads_norm_gate")


def pair_combine(out, a, b, wa, wb, eps, scale_a, scale_b, dtype):
    """out [n, size] float32 = scale_a * A' + scale_b * B'; with weights A' = A / rms(A) * wa (B likewise), else A' = A. A, B: rows of
    ``dtype`` or float32 partial sums [s, n, size]."""
    _need(out, "out", torch.float32)
    n, size = out.shape
    check(lib().ti_pair_combine(out.data_ptr(), *_rows_or_partials(a, dtype, "a"), *_rows_or_partials(b, dtype, "b"), _ptr(wa), _ptr(wb),
                                int(wa is not None), eps, scale_a, scale_b, n, size, dtype_code(dtype), _stream()), "pair_combine")
