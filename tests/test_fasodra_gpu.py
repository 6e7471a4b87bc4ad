"""The Fasodra design through the engine against the plain implementation (``plain_fasodra``): whole prompts, prompts in portions
down to two tokens, token-by-token decoding, batches of unequal requests against each alone, slots, pages and states that are used
again, long decoding past every chunk, hand-made weights that make one key, a chunk's edge or a distance's bias stand out, every
mechanism and kernel alone, greedy generation through the public entry point and trace replay; in 32-bit and in bfloat16, at three
sets of sizes."""
import math
import tempfile
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import fasodra_cases as fc
import plain_fasodra as plain
from replay_util import Trace, run_trace

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F64 = torch.float64


@pytest.fixture(scope="module")
def models():
    with tempfile.TemporaryDirectory() as tmp:
        yield {name: fc.Model(name, seed, tmp) for name, seed in (("A", 31), ("B", 32), ("C", 33))}


def rows(logits, positions):
    a = logits.detach().float().cpu().numpy()
    return {p: a[i].copy() for i, p in enumerate(positions)}


def engine_of(m, dtype, **kw):
    """(engine, recorder of its router choices or None). In bfloat16 a router choice can rest on a gap that rounding closes, so the
    run's own choices are noted (which needs steps that are not replayed from graphs) and the plain implementation takes the same;
    in 32-bit the engine runs as it is served, graphs and all, and chooses for itself."""
    if dtype == "bfloat16":
        engine = m.engine(dtype, graphs=False, **kw)
        return engine, fc.Recorder(engine, m.cfg)
    return m.engine(dtype, **kw), None


def run_cut(engine, tokens, cuts, recorder=None):
    """One sequence fed in portions of the given sizes (the rest one token at a time); logits at every position."""
    slot = engine.new_sequence()
    got, at = {}, 0
    sizes = list(cuts)
    if recorder is not None:
        recorder.choices.pop(0, None)
    while at < len(tokens):
        n = min(sizes.pop(0) if sizes else 1, len(tokens) - at)
        if recorder is not None:
            recorder.rows = [(0, p) for p in range(at, at + n)]
        got.update(rows(engine.step([(slot, tokens[at:at + n])], [list(range(n))]), range(at, at + n)))
        at += n
    engine.free_sequence(slot)
    engine.check_health()
    return got


def rnd(x, T):
    return x.to(T).to(x.dtype)


# ---------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", sorted(DTYPES))
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompts_and_prompts_in_portions(models, name, dtype):
    m = models[name]
    engine, rec = engine_of(m, dtype)
    forced = lambda: rec.of(0) if rec is not None else None
    for tokens in fc.prompts(m.vocab, [1, 2, 7, 64, 65, 150, 330], 21):
        got = run_cut(engine, tokens, [len(tokens)], rec)
        fc.compare(m, tokens, got, DTYPES[dtype], f"{name} {dtype} whole {len(tokens)}", forced=forced())
    tokens = fc.prompts(m.vocab, [260], 22)[0]
    # Portions that start and end inside and at page borders and inside and at the chunks' edges, two tokens, one token.
    for cuts in ([100, 100, 60], [63, 1, 64, 2, 2, 128], [2, 2, 2, 58, 64, 3, 1, 1, 100, 27], [129, 2, 61, 2, 66], [7, 26, 33, 34, 100, 60]):
        got = run_cut(engine, tokens, cuts, rec)
        fc.compare(m, tokens, got, DTYPES[dtype], f"{name} {dtype} portions {cuts[:4]}", forced=forced())


@pytest.mark.parametrize("dtype", sorted(DTYPES))
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding_from_a_short_prompt(models, name, dtype):
    """A prompt of three tokens, then 250 single tokens: pages fill up while decoding, every chunk's edge is passed by decoded
    tokens alone, and the recurrent states, the rows' history and the row before come from the sequence's state at every step."""
    m = models[name]
    engine, rec = engine_of(m, dtype, max_tokens=512, max_seqs=2)
    tokens = fc.prompts(m.vocab, [253], 23)[0]
    got = run_cut(engine, tokens, [3], rec)
    fc.compare(m, tokens, got, DTYPES[dtype], f"{name} {dtype} long decoding", forced=rec.of(0) if rec is not None else None)


@pytest.mark.parametrize("dtype", sorted(DTYPES))
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_batches_of_unequal_requests_and_reuse_of_slots_pages_and_states(models, name, dtype):
    """Requests of unequal lengths prefilled in one step and decoded together, the shorter ones leaving first; then a second batch
    in the slots, pages and states that the first gave back. Every request is compared with the plain implementation of that
    request alone."""
    m = models[name]
    engine, rec = engine_of(m, dtype, max_tokens=1024, max_seqs=4)
    for seed, lengths, tails in ((31, [1, 40, 129, 300], [0, 12, 40, 3]), (32, [70, 3, 230, 64], [6, 2, 65, 33])):
        reqs = fc.prompts(m.vocab, lengths, seed)
        slots = [engine.new_sequence() for _ in reqs]
        got = [dict() for _ in reqs]
        heads = [len(t) - d for t, d in zip(reqs, tails)]
        if rec is not None:
            rec.choices.clear()
            rec.rows = [(i, p) for i, h in enumerate(heads) for p in range(h)]
        out = engine.step([(s, t[:h]) for s, t, h in zip(slots, reqs, heads)], [list(range(h)) for h in heads])
        a = out.detach().float().cpu().numpy()
        at = 0
        for i, h in enumerate(heads):
            got[i].update({p: a[at + p].copy() for p in range(h)})
            at += h
        fed = list(heads)
        live = [i for i in range(len(reqs)) if fed[i] < len(reqs[i])]
        for i in range(len(reqs)):
            if i not in live:
                engine.free_sequence(slots[i])
        while live:
            if rec is not None:
                rec.rows = [(i, fed[i]) for i in live]
            out = engine.step([(slots[i], [reqs[i][fed[i]]]) for i in live]).detach().float().cpu().numpy()
            for r, i in enumerate(live):
                got[i][fed[i]] = out[r].copy()
                fed[i] += 1
            for i in [i for i in live if fed[i] == len(reqs[i])]:
                engine.free_sequence(slots[i])
            live = [i for i in live if fed[i] < len(reqs[i])]
        engine.check_health()
        for i, t in enumerate(reqs):
            assert sorted(got[i]) == list(range(len(t)))
            fc.compare(m, t, got[i], DTYPES[dtype], f"{name} {dtype} batch seed {seed} request {i}", forced=rec.of(i) if rec is not None else None)
    assert engine.cache.slots.held == 0


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_the_stream_after_every_layer(models, name):
    """In 32-bit: the sum of the stream's copies after each layer equals the plain implementation's, layer by layer."""
    m = models[name]
    engine = m.engine("float32")
    tokens = fc.prompts(m.vocab, [90], 27)[0]
    ref = m.layers(tokens)
    copies = max(1, m.cfg.get("streams") or 0)
    seen = []
    engine.model.observer = lambda occ, x: seen.append((occ, x.detach().float().view(x.shape[0], copies, -1).sum(1).cpu().clone()))
    slot = engine.new_sequence()
    engine.step([(slot, tokens)])
    engine.model.observer = None
    engine.free_sequence(slot)
    assert [occ for occ, _ in seen] == list(range(len(ref)))
    for occ, x in seen:
        assert float((x - ref[occ]).abs().max()) <= 2e-4 * max(1.0, float(ref[occ].abs().max())), f"layer {occ}"


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_other_arrangements_of_layers(dtype):
    """One copy of the stream with learned tables; two copies without a multiplier; each kind of layer alone and first; chunks of
    one and two keys; bias tables of 4 and 30 rows and a decay of rank 3 (extents that only the tensors give); every expert
    chosen; convolutions of one and two taps."""
    T = DTYPES[dtype]
    g = torch.Generator().manual_seed(8)
    att = lambda **kw: fc.attention(3, 1, 12, 6, 0.3, 40, fc.moe(16, 4, 2), **kw)
    par = lambda: fc.parallel((2, 1, 8, 12, 0.3, (4, 77.0)), 2, 6, fc.moe(12, 3, 3), scales=(1.1, 0.7))
    par2 = lambda conv: fc.parallel_2((3, 3, 10, 4, 0.3, (10, 60.0)), (2, 2, 6, 10, conv), None)
    cases = {
        "one copy": (fc.model(71, 40, 1e-5, [att(chunk=5), par()], mult=1.5, streams=1), None),
        "two copies no multiplier": (fc.model(71, 40, 1e-5, [par2(2), att(chunk=2)], streams=2), None),
        "attention only": (fc.model(50, 24, 1e-4, [att(chunk=1), att(chunk=70), att()], mult=0.4, streams=5),
                           {"l0.mix.rel": torch.randn(4, 3, generator=g), "l1.mix.rel": torch.randn(30, 3, generator=g)}),
        "time mixing only": (fc.model(50, 24, 1e-6, [par(), par()], mult=0.9),
                             {"l0.mix.right.w1": torch.randn(3, 24, generator=g) * 0.2, "l0.mix.right.w2": torch.randn(12, 3, generator=g) * 0.3}),
        "delta rule only": (fc.model(33, 32, 1e-5, [par2(1), par2(None), par2(5)], streams=2, mult=0.8), None),
    }
    with tempfile.TemporaryDirectory() as tmp:
        for name, (case, override) in cases.items():
            m = fc.Model(name.replace(" ", "_"), 3, tmp, case, override)
            engine, rec = engine_of(m, dtype, max_tokens=512, max_seqs=2, max_context=256)
            tokens = fc.prompts(m.vocab, [130], 5)[0]
            for cuts in ([130], [2, 64, 3], [70, 1, 1, 58]):
                got = run_cut(engine, tokens, cuts, rec)
                fc.compare(m, tokens, got, T, f"{name} {dtype} {cuts}", forced=rec.of(0) if rec is not None else None)


# ---------------------------------------------------------------- mixers alone
def _random_tensor(d, g, T):
    name, shape = d.name, tuple(d.shape)
    t = torch.randn(shape, generator=g, dtype=F64)
    if len(shape) == 2 and not name.endswith((".conv", ".u", ".rel")):
        t = t * shape[1] ** -0.5
    elif name.endswith(".conv"):
        t = 1.0 / shape[1] + 0.3 * t
    elif name.endswith((".norm", ".out")):
        t = 1 + 0.2 * t
    elif ".mu." in name:
        t = torch.rand(shape, generator=g, dtype=F64)
    elif name.endswith(".w0"):
        t = t - 2.5
    elif name.endswith(".dt_bias"):
        t = t - 2.0
    elif name.endswith((".u", ".A_log", ".b")):
        t = 0.4 * t
    return rnd(t, T)


def _mixer_of(case, layer, T, tensors=None, seed=0, max_positions=1024):
    """The mixer part of one layer of a configuration, built as the model builds it, with random (or given) tensors.
    Returns (mixer, tensors by checkpoint name in 64-bit, the layer's raw record)."""
    from tileinfer_b200.config import config_from_dict
    from tileinfer_b200.parts import Runtime, lookup
    spec = config_from_dict(case).model_spec().layers[layer].mixer
    cls = lookup("mixer", spec.kind)
    g = torch.Generator().manual_seed(seed)
    if tensors is None:
        tensors = {d.name: _random_tensor(d, g, T) for d in cls.tensors(spec)}
    rt = Runtime(T)
    position = lookup("position", spec.position.kind)(spec.position, rt, max_positions) if spec.position.kind != "none" else None
    dev = {k: v.to(T) for k, v in tensors.items()}
    return cls(spec, dev, rt, position), tensors, case["layers"][layer]


def _run_mixer(mixer, T, h, cuts, width, neighbour=None, env=None):
    """One sequence's rows through the mixer in portions (the rest one at a time); with ``neighbour`` another sequence's rows ride
    along in every step, in front."""
    from test_parts_gpu import OneStep
    env = env or OneStep(mixer, T, max_tokens=1024, max_seqs=2)
    slot = env.cache.alloc_slot()
    other = env.cache.alloc_slot() if neighbour is not None else None
    at, out, sizes, k = 0, [], list(cuts), 0
    while at < h.shape[0]:
        n = min(sizes.pop(0) if sizes else 1, h.shape[0] - at)
        entries = [(slot, h[at:at + n].to(T))]
        if other is not None and k < neighbour.shape[0]:
            entries = [(other, neighbour[k:k + 1].to(T))] + entries
        r = env.run(mixer, entries, width)
        out.append(r[len(entries) - 1:] if len(entries) > 1 else r)
        at += n
        k += 1
    env.cache.free_slot(slot)
    if other is not None:
        env.cache.free_slot(other)
    return torch.cat(out)


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_every_mixer_alone(dtype):
    """Each layer's mixer of the three configurations against the plain mixer: whole, token by token, in portions whose edges
    fall inside, at and outside the chunks' edges and the pages' borders, beside another sequence in the batch, and once more in
    the slot, pages and state that the run before gave back."""
    from test_parts_gpu import OneStep
    T = DTYPES[dtype]
    g = torch.Generator().manual_seed(3)
    for case in (fc.CASE_A, fc.CASE_B, fc.CASE_C):
        width, eps = case["width"], case["norm"]["eps"]
        for layer in range(len(case["layers"])):
            mixer, W, raw = _mixer_of(case, layer, T, seed=layer)
            total = 200
            h = rnd(torch.randn(total, width, generator=g, dtype=F64), T)
            other = rnd(torch.randn(40, width, generator=g, dtype=F64), T)
            ref = plain.mixer(raw["type"], h, W, f"l{layer}.mix.", raw["mixer"], eps).float()
            chunk = (raw["mixer"].get("mask") or {}).get("size", 50)
            env = OneStep(mixer, T, max_tokens=1024, max_seqs=2)
            for cuts in ([total], [1], [chunk - 1, 2, chunk, chunk + 1, 3], [64, 64, 2, 2, 60], [2, 2, 2, 2]):
                got = _run_mixer(mixer, T, h, cuts, width, neighbour=other if cuts[0] in (1, 64) else None, env=env)
                err = (got - ref).abs().max(-1).values
                tol = (1e-4 if T == torch.float32 else 8 * 2.0 ** -8) * max(1.0, float(ref.abs().max()))
                assert float(err.max()) <= tol, (f"{raw['type']} layer {layer} width {width} cuts {cuts[:3]}: worst {float(err.max()):.3g} at "
                                                 f"{int(err.argmax())}, first bad {int((err > tol).float().argmax())}")


# ---------------------------------------------------------------- weights made by hand
def _marked_rows(total, mark_at, W=16):
    """Ordinary tokens are the unit vector e1; the marked one is e0 with a little e2."""
    h = torch.zeros(total, W, dtype=F64)
    h[:, 1] = 1.0
    h[mark_at] = 0.0
    h[mark_at, 0], h[mark_at, 2] = 1.0, 0.25
    return h


NORMED = 1.0 / math.sqrt(1.0625 / 16)            # what dividing by the root mean square makes of the marked row's e0


def _identity_attention(W, heads, scale, bias_max, rel, chunk=None, q_to_e0=True):
    eye = torch.eye(W, dtype=F64)
    case = fc.model(8, W, 1e-6, [fc.attention(heads, heads, W, W, scale, bias_max, None, chunk=chunk)])
    tensors = {"l0.mix.o": torch.cat([eye if i == 0 else torch.roll(eye, 8, 0) for i in range(heads)], 1), "l0.mix.rel": rel}
    for k in "qkv":
        tensors[f"l0.mix.{k}"] = eye.repeat(heads, 1)
        tensors[f"l0.mix.{k}.b"] = torch.zeros(heads * W, dtype=F64)
    if q_to_e0:
        for i in range(heads):
            tensors["l0.mix.q"][i * W, 1], tensors["l0.mix.q"][i * W + 1, 1] = 1.0, 0.0        # e1 -> e0: ordinary tokens ask along e0
    return case, tensors


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_a_marked_key_is_seen_inside_its_chunk_and_not_beyond(dtype):
    """One head of identity weights whose query projection sends e1 to e0 and a bias table of zeros: every ordinary query scores the
    marked key scale * 4 * 3.88 = 23 above the others, so the output's e2 is the marked value's 0.25 for every query of the marked
    key's chunk behind it, and exactly zero from the next chunk's first position on. Chunks of 1, 2, a page, a page and one, and no
    multiple of anything; the edge inside a prompt, at a portion's first token and among single tokens; the marker at a chunk's
    first and last place, on both sides of a page border, and far into the sequence."""
    T = DTYPES[dtype]
    W, scale = 16, 1.5
    for chunk, mark_at, cuts, total in ((1, 5, [20], 20), (2, 4, [20], 20), (2, 63, [64], 70), (7, 0, [1], 20), (7, 62, [66, 1, 4], 80),
                                        (64, 3, [140], 140), (64, 64, [100, 27], 200), (65, 64, [65], 140), (65, 0, [40, 25, 1, 30], 100),
                                        (100, 129, [128, 1, 1, 64], 260), (100, 100, [199, 2], 260), (100, 227, [230], 335), (33, 300, [1], 340)):
        case, tensors = _identity_attention(W, 1, scale, 50, torch.zeros(8, 1, dtype=F64), chunk=chunk)
        mixer, _, _ = _mixer_of(case, 0, T, tensors)
        out = _run_mixer(mixer, T, _marked_rows(total, mark_at), cuts, W)[:, 2]
        last = min((mark_at // chunk + 1) * chunk, total)          # the first position that no longer sees the marker
        assert float(out[:mark_at].abs().max()) == 0.0 if mark_at else True
        if last > mark_at + 1:
            seen = out[mark_at + 1:last]
            assert float((seen - 0.25).abs().max()) <= (1e-4 if T == torch.float32 else 0.01) * 0.25, \
                f"chunk {chunk}, marker at {mark_at}, cuts {cuts}: {seen[:2].tolist()} .. {seen[-2:].tolist()}"
        assert last == total or float(out[last:].abs().max()) == 0.0, \
            f"chunk {chunk}, marker at {mark_at}, cuts {cuts}: seen at {mark_at + int(out[mark_at:].abs().nonzero().max())}, edge {last}"


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_the_bias_of_a_distance_reaches_the_softmax(dtype):
    """With a scale of zero every score is its distance's bias alone, so a marked key's share seen from distance n is
    exp(rel[bucket(n), head]) over the sum of that over all visible keys: compared with the closed form for two heads with
    different tables, distances up to 300 (far beyond where the last bucket begins), from a prompt and from single tokens."""
    T = DTYPES[dtype]
    W, far, rows_ = 16, 40.0, 10
    g = torch.Generator().manual_seed(5)
    rel = rnd(torch.randn(rows_, 2, generator=g, dtype=F64) * 1.5, T)
    rel[rows_ - 1, 0] = 2.0                                         # the last bucket of head 0 outweighs many near keys
    case, tensors = _identity_attention(W, 2, 0.0, far, rel, q_to_e0=False)
    mixer, _, _ = _mixer_of(case, 0, T, tensors)
    for mark_at, cuts, total in ((0, [1], 120), (3, [310], 310), (64, [70, 2, 100], 260)):
        out = _run_mixer(mixer, T, _marked_rows(total, mark_at), cuts, W)
        for head in range(2):
            seen = out[:, (2 + 8 * head) % W]
            for i in list(range(mark_at, min(total, mark_at + 45))) + [total - 1]:
                weights = [math.exp(float(rel[plain.distance_bucket(i - j, rows_, far), head])) for j in range(i + 1)]
                want = 0.25 * weights[mark_at] / sum(weights)
                assert abs(float(seen[i]) - want) <= (1e-4 if T == torch.float32 else 0.03) * want + 1e-7, \
                    f"head {head}, marker at {mark_at}, query {i}: {float(seen[i])} for {want}"


# ---------------------------------------------------------------- kernels alone
def _step(lengths, slots):
    cu = [0]
    for n in lengths:
        cu.append(cu[-1] + n)
    return SimpleNamespace(cu_seqlens=torch.tensor(cu, dtype=torch.int32, device="cuda"), seq_slots=torch.tensor(slots, dtype=torch.int32, device="cuda"),
                           n_seqs=len(lengths))


def test_decay_scan_alone():
    """The time-mixing recurrence against a loop in 64-bit, at key sizes that are no multiple of a thread's rows or a block's
    columns: sequences of unequal lengths in one launch, continued from the state in later launches (portions of 1, 2 and 37
    tokens), a neighbour that must not see the other's state, and a slot whose state was zeroed and is used again. One marked
    token's trace in the state fades by the product of the decays exactly."""
    from tileinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(11)
    for T in (torch.float32, torch.bfloat16):
        for H, D in ((3, 24), (2, 64), (1, 130), (20, 64), (5, 64)):          # the last two: blocks of 32 and of 16 columns
            HD, extra = H * D, 5
            lengths = [70, 1, 23]
            total = sum(lengths)
            rkv = rnd(torch.randn(total, 3 * HD, generator=g, dtype=F64) * 0.5, T)
            dlog = torch.randn(total, HD, generator=g, dtype=F64).float().double()
            w0 = (torch.randn(HD, generator=g, dtype=F64) - 2.0).float().double()
            u = torch.randn(HD, generator=g, dtype=F64).float().double()
            state = torch.zeros(4, H * D * D + extra, dtype=torch.float32, device="cuda")
            ref, at = torch.zeros(total, HD, dtype=F64), 0
            decay = torch.exp(-torch.exp(dlog + w0))
            final = {}
            for b, n in enumerate(lengths):
                S = torch.zeros(H, D, D, dtype=F64)
                for t in range(at, at + n):
                    r, k, v = (rkv[t, i * HD:(i + 1) * HD].view(H, D) for i in range(3))
                    kv = k[:, :, None] * v[:, None, :]
                    ref[t] = torch.einsum("hkv,hk->hv", S + u.view(H, D)[:, :, None] * kv, r).reshape(-1)
                    S = decay[t].view(H, D)[:, :, None] * S + kv
                final[b] = S
                at += n
            o = torch.zeros(total, HD, dtype=torch.float32, device="cuda")
            slots = [2, 0, 3]
            args = lambda: (dlog.float().cuda(), w0.float().cuda(), u.float().cuda(), state)
            # every sequence in portions: 37 tokens (or all it has), then 2, then one at a time
            fed = [0, 0, 0]
            starts = [0, lengths[0], lengths[0] + lengths[1]]
            for portion in (37, 2) + (1,) * 40:
                live = [b for b in range(3) if fed[b] < lengths[b]]
                if not live:
                    break
                take = [min(portion, lengths[b] - fed[b]) for b in live]
                idx = torch.cat([torch.arange(starts[b] + fed[b], starts[b] + fed[b] + n) for b, n in zip(live, take)])
                part = torch.zeros(len(idx), HD, dtype=torch.float32, device="cuda")
                d_part = dlog[idx].float().cuda().contiguous()
                ops.decay_scan(part, rkv[idx].to(T).cuda().contiguous(), 0, HD, 2 * HD, d_part, args()[1], args()[2], state, _step(take, [slots[b] for b in live]), H, D)
                o[idx.cuda()] = part
                for b, n in zip(live, take):
                    fed[b] += n
            tol = (2e-5 if T == torch.float32 else 2e-5) * max(1.0, float(ref.abs().max()))
            assert float((o.cpu().double() - ref).abs().max()) <= tol, f"{T} {H} heads of {D}"
            for b in range(3):
                got = state[slots[b], :H * D * D].view(H, D, D).cpu().double()
                assert float((got - final[b]).abs().max()) <= 1e-4 * max(1.0, float(final[b].abs().max()))
            assert float(state[1].abs().max()) == 0.0 and float(state[:, H * D * D:].abs().max()) == 0.0          # untouched slot and tail


def test_delta_scan_alone():
    """The gated delta rule against a loop in 64-bit at key and value sizes that differ and are no multiple of anything, grouped
    query/key heads, unequal sequences, portions continued from the state."""
    from tileinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(12)
    for H, G, D, V in ((4, 2, 24, 40), (2, 2, 64, 32), (1, 1, 130, 70), (6, 1, 16, 16), (20, 4, 32, 64), (5, 5, 48, 64)):      # the last two: blocks of 32 and of 16 columns
        C = 2 * G * D + H * V
        lengths = [50, 1, 19]
        total = sum(lengths)
        qkv = torch.randn(total, C, generator=g, dtype=F64).float().double()
        unit = lambda x: x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)
        qkv[:, :G * D] = (unit(qkv[:, :G * D].view(total, G, D)) * D ** -0.5).reshape(total, -1)
        qkv[:, G * D:2 * G * D] = unit(qkv[:, G * D:2 * G * D].view(total, G, D)).reshape(total, -1)
        qkv = qkv.float().double()
        ba = torch.randn(total, 2 * H, generator=g, dtype=F64).float().double()
        a_log, dt_bias = (torch.randn(H, generator=g, dtype=F64) * 0.5).float().double(), (torch.randn(H, generator=g, dtype=F64) - 1.0).float().double()
        beta = torch.sigmoid(ba[:, :H])
        decay = torch.exp(-torch.exp(a_log) * torch.nn.functional.softplus(ba[:, H:] + dt_bias))
        ref, at, final = torch.zeros(total, H * V, dtype=F64), 0, {}
        for b, n in enumerate(lengths):
            S = torch.zeros(H, D, V, dtype=F64)
            for t in range(at, at + n):
                for h in range(H):
                    c = h // (H // G)
                    q, k, v = qkv[t, c * D:(c + 1) * D], qkv[t, G * D + c * D:G * D + (c + 1) * D], qkv[t, 2 * G * D + h * V:2 * G * D + (h + 1) * V]
                    S[h] = decay[t, h] * S[h]
                    e = beta[t, h] * (v - S[h].T @ k)
                    S[h] = S[h] + k[:, None] * e[None, :]
                    ref[t, h * V:(h + 1) * V] = S[h].T @ q
            final[b] = S
            at += n
        state = torch.zeros(4, H * D * V + 7, dtype=torch.float32, device="cuda")
        o = torch.zeros(total, H * V, dtype=torch.float32, device="cuda")
        slots, fed, starts = [1, 3, 0], [0, 0, 0], [0, lengths[0], lengths[0] + lengths[1]]
        for portion in (17, 2) + (1,) * 40:
            live = [b for b in range(3) if fed[b] < lengths[b]]
            if not live:
                break
            take = [min(portion, lengths[b] - fed[b]) for b in live]
            idx = torch.cat([torch.arange(starts[b] + fed[b], starts[b] + fed[b] + n) for b, n in zip(live, take)])
            part = torch.zeros(len(idx), H * V, dtype=torch.float32, device="cuda")
            ops.delta_scan(part, qkv[idx].float().cuda().contiguous(), ba[idx].float().cuda().contiguous(), a_log.float().cuda(), dt_bias.float().cuda(), state,
                           _step(take, [slots[b] for b in live]), H, G, D, V)
            o[idx.cuda()] = part
            for b, n in zip(live, take):
                fed[b] += n
        assert float((o.cpu().double() - ref).abs().max()) <= 3e-5 * max(1.0, float(ref.abs().max())), f"{H}/{G} heads of {D} x {V}"
        for b in range(3):
            got = state[slots[b], :H * D * V].view(H, D, V).cpu().double()
            assert float((got - final[b]).abs().max()) <= 1e-4 * max(1.0, float(final[b].abs().max()))
        assert float(state[2].abs().max()) == 0.0


def test_blends_history_and_convolution_alone():
    """The blend with the row before (from the step, from the state, from nothing at a sequence's start) and the convolution over
    time with taps 1, 10, 100, 1000 whose digits show which row every tap read, with the history coming from the step, from the
    state and from before the start; portions shorter than the taps."""
    from tileinfer_b200.kernels import ops
    T = torch.float32
    W, K = 12, 3
    g = torch.Generator().manual_seed(13)
    h = torch.randn(30, W, generator=g)
    mu = torch.rand(K, W, generator=g)
    prev = torch.cat([torch.zeros(1, W), h[:-1]])
    want = h[None] + (prev - h)[None] * mu[:, None, :]
    state = torch.zeros(3, 5 + W, device="cuda")
    got, at = [], 0
    for n in (1, 2, 20, 1, 6):
        out = torch.zeros(K, n, W, device="cuda")
        ops.shift_blend(out, h[at:at + n].cuda().contiguous(), mu.cuda(), state[:, 5:], _step([n], [1]))
        got.append(out.cpu())
        at += n
    assert float((torch.cat(got, 1) - want).abs().max()) <= 1e-6
    assert float((state[1, 5:].cpu() - h[-1]).abs().max()) == 0.0 and float(state[0].abs().max()) == 0.0 and float(state[:, :5].abs().max()) == 0.0
    # the convolution: one q/k head of 2 and one value head of 3; rows count 1, 2, 3, ...
    G, D, HV, taps = 1, 2, 3, 4
    C = 2 * G * D + HV
    proj = torch.arange(1, 13, dtype=torch.float32)[:, None].repeat(1, C)
    conv = torch.tensor([[1000.0, 100.0, 10.0, 1.0]]).repeat(C, 1)
    digits = plain.short_conv(proj.double(), conv.double())                                     # 1, 12, 123, 1234, 2345, ...
    assert digits[:5, 0].tolist() == [1.0, 12.0, 123.0, 1234.0, 2345.0]
    silu = torch.nn.functional.silu(digits)
    hist = torch.zeros(2, 9 + (taps - 1) * C, device="cuda")
    got, at = [], 0
    for n in (1, 1, 2, 5, 3):
        out = torch.zeros(n, C, device="cuda")
        rows = proj[at:at + n].cuda().contiguous()
        ops.delta_inputs(out, rows, conv.cuda(), taps, hist[:, 9:], _step([n], [1]), G, D, HV, 1e-6)
        ops.history_update(hist[:, 9:], rows, taps, _step([n], [1]), C)
        got.append(out.cpu())
        at += n
    got = torch.cat(got).double()
    assert float((got[:, 2 * G * D:] - silu[:, 2 * G * D:]).abs().max()) <= 1e-3                # values: the activated convolution itself
    unit_q = silu[:, :D] / torch.sqrt((silu[:, :D] ** 2).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    unit_k = silu[:, D:2 * D] / torch.sqrt((silu[:, D:2 * D] ** 2).sum(-1, keepdim=True) + 1e-6)
    assert float((got[:, :D] - unit_q).abs().max()) <= 1e-6 and float((got[:, D:2 * D] - unit_k).abs().max()) <= 1e-6
    assert hist[1, 9:].view(taps - 1, C)[:, 0].tolist() == [10.0, 11.0, 12.0] and float(hist[0].abs().max()) == 0.0


def test_stream_copies_and_small_kernels_alone():
    """The copies of the stream (begin, read through a norm with a bias, update with the next reader's input) against the
    equations in 64-bit for 1, 2 and 5 copies, from rows and from 32-bit partial sums; the per-head norm with its gate; the sum of
    two mixers with and without their norms; the gate per head; the squared rectifier."""
    from tileinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(14)
    for T in (torch.float32, torch.bfloat16):
        n, size = 9, 40
        for S in (1, 2, 5):
            x0 = torch.randn(n, size, generator=g)
            x = torch.zeros(n, S * size, device="cuda")
            ops.streams_begin(x, x0.cuda(), S)
            assert float((x.view(n, S, size).cpu() - x0[:, None]).abs().max()) == 0.0
            old = (torch.randn(n, S, size, generator=g) * 3 + 5).double()
            a, c, M, a2 = (torch.randn(S, generator=g).double(), torch.randn(S, generator=g).double(), torch.randn(S, S, generator=g).double(),
                           torch.randn(S, generator=g).double())
            w, b = rnd(1 + 0.2 * torch.randn(size, generator=g).double(), T), rnd(torch.randn(size, generator=g).double(), T)
            ln = lambda v: plain.layer_norm(v, w, b, 1e-5)
            x = old.float().cuda().view(n, S * size).contiguous()
            h = torch.zeros(n, size, dtype=T, device="cuda")
            ops.streams_read_norm(h, x, a.float().cuda(), w.to(T).cuda(), b.to(T).cuda(), 1e-5, True)
            want = ln(torch.einsum("s,nsd->nd", a, old))
            tol = 2e-5 if T == torch.float32 else 2.0 ** -7
            assert float((h.float().cpu() - want).abs().max()) <= tol * max(1.0, float(want.abs().max()))
            y = rnd(torch.randn(n, size, generator=g).double(), T)
            for form in ("rows", "partials"):
                x = old.float().cuda().view(n, S * size).contiguous()
                delta = y.to(T).cuda() if form == "rows" else torch.stack([0.25 * y, 0.75 * y]).float().cuda()
                ops.streams_update(x, delta, M.flatten().tolist(), (0.7 * c).tolist(), a2.tolist(), h, w.to(T).cuda(), b.to(T).cuda(), 1e-5, True)
                new = torch.einsum("st,nsd->ntd", M, old) + 0.7 * c[None, :, None] * y[:, None, :]
                assert float((x.view(n, S, size).cpu().double() - new).abs().max()) <= 1e-5 * float(new.abs().max())
                want = ln(torch.einsum("t,ntd->nd", a2, new))
                assert float((h.float().cpu() - want).abs().max()) <= tol * max(1.0, float(want.abs().max()))
        # the norm of every head with a weight shared by the heads or of the whole row, and the gate
        H, V = 3, 20
        o = torch.randn(n, H * V, generator=g).double() * 4
        gate = rnd(torch.randn(n, H * V + 8, generator=g).double(), T)
        for w in (rnd(1 + 0.2 * torch.randn(V, generator=g).double(), T), rnd(1 + 0.2 * torch.randn(H * V, generator=g).double(), T)):
            yk = torch.zeros(n, H * V, dtype=T, device="cuda")
            ops.heads_norm_gate(yk, o.float().cuda(), gate.to(T).cuda()[:, 8:], w.to(T).cuda(), 1e-5, H, V)
            want = plain.rms_divide(o.view(n, H, V), 1e-5) * (w.view(H, V) if w.numel() == H * V else w)
            want = want.reshape(n, -1) * torch.nn.functional.silu(gate[:, 8:])
            assert float((yk.float().cpu() - want).abs().max()) <= (2e-5 if T == torch.float32 else 2.0 ** -7) * max(1.0, float(want.abs().max()))
        # two mixers side by side
        A, B = rnd(torch.randn(n, size, generator=g).double(), T), rnd(torch.randn(n, size, generator=g).double() * 3, T)
        wa, wb = rnd(1 + 0.2 * torch.randn(size, generator=g).double(), T), rnd(1 + 0.2 * torch.randn(size, generator=g).double(), T)
        out = torch.zeros(n, size, device="cuda")
        ops.pair_combine(out, A.to(T).cuda(), torch.stack([0.5 * B, 0.5 * B]).float().cuda(), wa.to(T).cuda(), wb.to(T).cuda(), 1e-5, 0.5, 0.5, T)
        want = 0.5 * (plain.rms_divide(A, 1e-5) * wa + plain.rms_divide(B, 1e-5) * wb)
        assert float((out.cpu() - want).abs().max()) <= 1e-5 * max(1.0, float(want.abs().max()))
        ops.pair_combine(out, A.to(T).cuda(), B.to(T).cuda(), None, None, 1e-5, 1.2, -0.3, T)
        assert float((out.cpu() - (1.2 * A - 0.3 * B)).abs().max()) <= 1e-5 * 4
        # one gate per head; the squared rectifier
        attn = rnd(torch.randn(n, H, 32, generator=g).double(), T)
        gh = rnd(torch.randn(n, H, generator=g).double(), T)
        yk = torch.zeros(n, H * V, dtype=T, device="cuda")
        ops.sigmoid_gate(yk, attn.to(T).cuda(), gh.to(T).cuda(), H, V, 32, per_head=True)
        want = (attn[:, :, :V] * torch.sigmoid(gh)[:, :, None]).reshape(n, -1)
        assert float((yk.float().cpu() - want).abs().max()) <= (1e-6 if T == torch.float32 else 2.0 ** -8) * 4
        z = rnd(torch.randn(n, size, generator=g).double(), T)
        out_t = torch.zeros(n, size, dtype=T, device="cuda")
        ops.relu2(out_t, z.to(T).cuda())
        assert float((out_t.float().cpu() - torch.relu(z) ** 2).abs().max()) <= (1e-6 if T == torch.float32 else 2.0 ** -8) * 10


def _dense_attention(q, k, v, scale, start, chunk, bias):
    """q [n, H, D] at positions start .. start + n - 1 over keys k, v [L, G, D]: exact attention in 64-bit with the chunk rule and
    the bias table [H, count] by distance."""
    n, H, D = q.shape
    L, G, _ = k.shape
    qp, kp = torch.arange(start, start + n)[:, None], torch.arange(L)[None, :]
    vis = kp <= qp
    if chunk:
        vis &= (kp // chunk) == (qp // chunk)
    out = torch.zeros(n, H, D, dtype=F64)
    for h in range(H):
        s = (q[:, h].double() @ k[:, h // (H // G)].double().T) * scale
        if bias is not None:
            s = s + bias[h].double()[(qp - kp).clamp(0, bias.shape[1] - 1)]
        out[:, h] = torch.softmax(s.masked_fill(~vis, float("-inf")), -1) @ v[:, h // (H // G)].double()
    return out


@pytest.mark.parametrize("nq,nkv,D,chunk,count", [(8, 2, 64, 100, 241), (6, 3, 32, 64, 0), (16, 1, 128, 7, 30), (40, 2, 64, 0, 500), (4, 4, 96, 333, 64),
                                                  (16, 4, 128, 256, 0), (4, 4, 64, 0, 0)])
def test_chunked_and_biased_attention_kernels_alone(nq, nkv, D, chunk, count):
    """The paged kernels that take the chunk rule and the bias by distance (plain, the prompt kernels on ``mma.sync`` and, for heads of
    64 and 128, on tensor memory, the split-KV decode kernel with 1 to 32 parts) against exact attention: sequences of unequal lengths, some continuing from cached
    positions, shuffled pages, chunks that are no multiple of a page, more than sixteen query heads per key/value head, distances
    beyond the table's end. One key that lies just outside the last query's chunk is made huge and must not show."""
    from test_kernels_gpu import close, dev, paged
    from tileinfer_b200.kernels import ops
    from tileinfer_b200.kernels.library import check, lib
    torch.manual_seed(17)
    dtype = torch.bfloat16
    r = lambda x: x.to(dtype).float()
    total = [300, 1, 130, 513, 64]                  # cached length after the step
    fresh = [300, 1, 30, 200, 64]                   # tokens of the step (the rest was cached before)
    B = len(total)
    ks = [r(torch.randn(L, nkv, D)) for L in total]
    vs = [r(torch.randn(L, nkv, D)) for L in total]
    qs = [r(torch.randn(n, nq, D)) for n in fresh]
    if chunk:
        edge = (512 // chunk) * chunk                # the first key of the last query's chunk in sequence 3
        if edge > 0:
            ks[3][edge - 1] = r(qs[3][-1, 1] * 9.0)[None].expand(nkv, D)
    bias = torch.randn(nq, count) * 1.5 if count else None
    scale = 1 / math.sqrt(D)
    n_pages = sum(-(-L // 64) for L in total) + 3
    kp, vp, table = paged(ks, vs, 64, n_pages, 13, dtype)
    want = torch.cat([_dense_attention(qs[b], ks[b], vs[b], scale, total[b] - fresh[b], chunk, bias) for b in range(B)]).float()
    q = dev(torch.cat(qs), dtype)
    cu = [0]
    for n in fresh:
        cu.append(cu[-1] + n)
    bias_d = dev(bias) if bias is not None else None
    bias2 = dev(bias * 1.4426950408889634) if bias is not None else None
    slots, cu_d, lens_d = (dev(torch.arange(1, B + 1, dtype=torch.int32)), dev(torch.tensor(cu, dtype=torch.int32)),
                           dev(torch.tensor(total, dtype=torch.int32)))
    tok_slot = dev(torch.cat([torch.full((n,), b + 1, dtype=torch.int32) for b, n in enumerate(fresh)]))
    positions = dev(torch.cat([torch.arange(total[b] - fresh[b], total[b], dtype=torch.int32) for b in range(B)]))
    out = torch.full((cu[-1], nq, D), float("nan"), dtype=dtype, device="cuda")
    ops.attention_plain(out, q, kp, vp, table, tok_slot, positions, scale, nq, nkv, D, 64, chunk=chunk, distance_bias=bias_d)
    close(out, want, dtype, ulps=5.0)
    st = torch.cuda.current_stream().cuda_stream
    tpt = 128 // (nq // nkv)
    tiles = sum(-(-n // tpt) for n in fresh)
    out = torch.full((cu[-1], nq, D), float("nan"), dtype=dtype, device="cuda")
    check(lib().ti_attention_prefill_biased(out.data_ptr(), q.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(), table.stride(0),
                                            slots.data_ptr(), cu_d.data_ptr(), lens_d.data_ptr(), B, tiles, scale, nq, nkv, D, 64, 0, None, chunk,
                                            bias2.data_ptr() if bias2 is not None else None, count, st), "attention_prefill")
    close(out, want, dtype, ulps=5.0)
    if D in (64, 128):
        from tileinfer_b200.kernels import fast
        tpb = 2 * (128 // (nq // nkv))
        blocks = sum(-(-n // tpb) for n in fresh)
        status = fast.status_word()
        out = torch.full((cu[-1], nq, D), float("nan"), dtype=dtype, device="cuda")
        check(lib().ti_attention_prefill_tc_biased(out.data_ptr(), q.data_ptr(), kp.data_ptr(), vp.data_ptr(), kp.shape[0], table.data_ptr(), table.stride(0),
                                                   slots.data_ptr(), cu_d.data_ptr(), lens_d.data_ptr(), B, cu[-1], blocks, scale, nq, nkv, D, 64, 0,
                                                   status.data_ptr(), None, chunk, bias2.data_ptr() if bias2 is not None else None, count, st),
              "attention_prefill_tc")
        fast.check_status()
        close(out, want, dtype, ulps=5.0)
    # one token per sequence: the last query of each
    last = [c - 1 for c in cu[1:]]
    qd = dev(torch.cat(qs)[last], dtype)
    for splits in (1, 3, 32):
        out = torch.full((B, nq, D), float("nan"), dtype=dtype, device="cuda")
        ws_o = torch.full((B * splits, nq, D), float("nan"), device="cuda")
        ws_ml = torch.full((B * splits, nq, 2), float("nan"), device="cuda")
        check(lib().ti_attention_decode_biased(out.data_ptr(), qd.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(), table.stride(0),
                                               slots.data_ptr(), lens_d.data_ptr(), None, None, ws_o.data_ptr(), ws_ml.data_ptr(), scale, B, nq, nkv,
                                               D, 64, splits, 0, None, chunk, bias2.data_ptr() if bias2 is not None else None, count, st), "attention_decode")
        close(out, want[last], dtype, ulps=5.0)


def test_bfloat16_steps_take_the_fast_kernels(models):
    """Case B's sizes are ones the fast kernels take: a prompt and a one-token step in bfloat16 go through the tensor-core products,
    the grouped products of the experts and the paged attention kernels (those with the chunk rule and the bias in the biased
    layers), not through their plain stand-ins."""
    from tileinfer_b200.kernels import library
    m = models["B"]
    engine = m.engine("bfloat16", graphs=False)
    slot = engine.new_sequence()
    library.call_counts.clear()
    engine.step([(slot, fc.prompts(m.vocab, [600], 61)[0])])
    engine.step([(slot, [5])])
    engine.free_sequence(slot)
    engine.check_health()
    used = dict(library.call_counts)
    assert used.get("ti_attention_prefill_tc_biased", 0) == 2 and used.get("ti_attention_decode_biased", 0) == 2, used
    assert used.get("ti_attention_prefill_tc", 0) + used.get("ti_attention_prefill", 0) == 2 and used.get("ti_attention_decode_shared", 0) == 2, used
    assert used.get("ti_decay_scan", 0) == 2 and used.get("ti_delta_scan", 0) == 2 and used.get("ti_streams_update", 0) == 16, used
    assert used.get("ti_gemm_tcgen05", 0) > 0 and used.get("ti_gemm_tcgen05_grouped", 0) > 0, used
    assert "ti_attention_plain" not in used and "ti_attention_plain_biased" not in used and "ti_attention_prefill_biased" not in used, used


# ---------------------------------------------------------------- through the public entry points
def test_greedy_generation_through_the_public_entry_point(models):
    """``generate`` (batches, scheduler, sampler, decode loop) on several prompts at once, more than there are slots, in 32-bit:
    every generated token is the plain implementation's most likely next token for the same prefix."""
    import tileinfer_b200 as ti
    for name in ("A", "B"):
        m = models[name]
        engine = ti.load_model(m.folder, dtype="float32", max_context=256, max_seqs=3)
        reqs = fc.prompts(m.vocab, [3, 41, 90, 17, 1], 41)
        outs = ti.generate(engine, reqs, max_new_tokens=40, stop_ids=[])
        assert [len(o) for o in outs] == [40] * 5
        for p, o in zip(reqs, outs):
            ref, _ = m.reference(p + o)
            for k, tok in enumerate(o):
                row = ref[len(p) + k - 1]
                assert row[tok] >= row.max() - 1e-4 * max(1.0, float(np.abs(row).max())), f"{name} token {k}: generated {tok}, plain argmax {int(row.argmax())}"


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_trace_replay(models, dtype):
    """The same requests through ``bin/trace_run``: whole, with the tail one by one, and in two batches one after the other (the
    second in the first one's slots, pages and states)."""
    m = models["B"]
    reqs = {f"r{i}": t for i, t in enumerate(fc.prompts(m.vocab, [1, 9, 70, 130, 200], 51))}
    t = Trace()
    t.whole(reqs)
    t.tail_one_by_one(reqs, tail=20)
    names = list(reqs)
    t.batch({r: reqs[r] for r in names[:3]}, {r: min(len(reqs[r]) - 1, 4 + 3 * i) for i, r in enumerate(names[:3])}, tag="x")
    t.batch({r: reqs[r] for r in names[2:]}, {r: min(len(reqs[r]) - 1, 30) for r in names[2:]}, tag="y")
    with tempfile.TemporaryDirectory() as out:
        got = run_trace(m.folder, dtype, t, out, sum(-(-len(x) // 64) * 64 for x in reqs.values()), m.vocab)
    by_request = {}
    for (rid, pos), row in got.items():
        by_request.setdefault(rid, {})[pos] = row
    assert len(by_request) == 5 + 5 + 3 + 3
    for rid, g in by_request.items():
        fc.compare(m, reqs[rid[1:]], g, DTYPES[dtype], f"replay {dtype} {rid}", need=0.0)
