"""The Sozanex design through the engine against the plain implementation (``plain_sozanex``): whole prompts, prompts in
portions down to two tokens, token-by-token decoding, batches of unequal requests against each alone, slots and pages that
are used again, long decoding past every window, hand-made weights that make one key, one sink or a window's edge stand out,
every mechanism and kernel alone, greedy generation through the public entry point and trace replay; in 32-bit and in
bfloat16, at three sets of sizes."""
import math
import tempfile

import numpy as np
import pytest
import torch

import plain_sozanex as plain
import sozanex_cases as sc
from replay_util import Trace, run_trace

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F64 = torch.float64


@pytest.fixture(scope="module")
def models():
    with tempfile.TemporaryDirectory() as tmp:
        yield {name: sc.Model(name, seed, tmp) for name, seed in (("A", 21), ("B", 22), ("C", 23))}


def rows(logits, positions):
    a = logits.detach().float().cpu().numpy()
    return {p: a[i].copy() for i, p in enumerate(positions)}


def run_cut(engine, tokens, cuts):
    """One sequence fed in portions of the given sizes (the rest one token at a time); logits at every position."""
    slot = engine.new_sequence()
    got, at = {}, 0
    sizes = list(cuts)
    while at < len(tokens):
        n = min(sizes.pop(0) if sizes else 1, len(tokens) - at)
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
    engine = m.engine(dtype)
    for tokens in sc.prompts(m.vocab, [1, 2, 7, 64, 65, 150, 420], 21):
        got = run_cut(engine, tokens, [len(tokens)])
        sc.compare(m, tokens, got, DTYPES[dtype], f"{name} {dtype} whole {len(tokens)}")
    tokens = sc.prompts(m.vocab, [300], 22)[0]
    # Portions that start and end inside and at page borders and inside and at the windows' edges, two tokens, one token.
    for cuts in ([100, 100, 100], [63, 1, 64, 2, 2, 128, 40], [2, 2, 2, 58, 64, 3, 1, 1, 120, 47], [129, 2, 61, 2, 70, 36], [7, 26, 31, 36, 100, 100]):
        got = run_cut(engine, tokens, cuts)
        sc.compare(m, tokens, got, DTYPES[dtype], f"{name} {dtype} portions {cuts[:4]}")


@pytest.mark.parametrize("dtype", sorted(DTYPES))
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding_from_a_short_prompt(models, name, dtype):
    """A prompt of three tokens, then almost 300 single tokens: pages fill up while decoding, every window passes over decoded
    tokens alone, and the token before each step's token comes from the sequence's state."""
    m = models[name]
    engine = m.engine(dtype, max_tokens=512, max_seqs=2)
    tokens = sc.prompts(m.vocab, [300], 23)[0]
    got = run_cut(engine, tokens, [3])
    sc.compare(m, tokens, got, DTYPES[dtype], f"{name} {dtype} long decoding")


@pytest.mark.parametrize("dtype", sorted(DTYPES))
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_batches_of_unequal_requests_and_reuse_of_slots_and_pages(models, name, dtype):
    """Requests of unequal lengths prefilled in one step and decoded together, the shorter ones leaving first; then a second
    batch in the slots, pages and last-token states that the first gave back. Every request is compared with the plain
    implementation of that request alone."""
    m = models[name]
    engine = m.engine(dtype, max_tokens=1024, max_seqs=4)
    for seed, lengths, tails in ((31, [1, 40, 129, 330], [0, 12, 40, 3]), (32, [70, 3, 260, 64], [6, 2, 65, 33])):
        reqs = sc.prompts(m.vocab, lengths, seed)
        slots = [engine.new_sequence() for _ in reqs]
        got = [dict() for _ in reqs]
        heads = [len(t) - d for t, d in zip(reqs, tails)]
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
            sc.compare(m, t, got[i], DTYPES[dtype], f"{name} {dtype} batch seed {seed} request {i}")
    assert engine.cache.slots.held == 0


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_other_arrangements_of_layers(dtype):
    """No loop at all; a loop over every layer; one kind of mixer alone; a single layer that runs four times; windows of one and
    of two keys; one bucket in the second table; multipliers whose products leave 32 bits."""
    T = DTYPES[dtype]
    a = lambda **kw: sc.attention(3, 1, 12, 6, 0.3, sc.dense(28), rot=(4, 77.0), scaling=(2.0, 1.0, 8.0, 30), **kw)
    l = lambda **kw: sc.latent(2, 10, 4, 14, 12, 22, 0.25, sc.dense(20), base=60.0, scaling=(4.0, 20, 6.0, 1.5), **kw)
    cases = {
        "no loop": sc.model(71, 40, 1e-5, 2.5, [l(), a(window=5)], bigram=(53, 7, 3)),
        "all looped": sc.model(71, 40, 1e-5, 0.5, [a(window=2), l()], bigram=(1, 5, 9), loop=(0, 2, 2)),
        "attention only": sc.model(50, 24, 1e-4, 4.0, [a(window=1), a(window=70)], bigram=(11, 2000003, 1000033), loop=(1, 2, 3)),
        "latent only": sc.model(50, 24, 1e-6, 1.5, [l(), l()], loop=(0, 1, 2)),
        "one layer four times": sc.model(33, 32, 1e-5, 6.0, [sc.latent(1, 8, 2, 8, 8, 14, 0.3, None, base=9.0)], bigram=(29, 1, 1), loop=(0, 1, 4)),
    }
    with tempfile.TemporaryDirectory() as tmp:
        for name, case in cases.items():
            m = sc.Model(name.replace(" ", "_"), 3, tmp, case)
            engine = m.engine(dtype, max_tokens=512, max_seqs=2, max_context=256)
            tokens = sc.prompts(m.vocab, [130], 5)[0]
            for cuts in ([130], [2, 64, 3], [70, 1, 1, 58]):
                sc.compare(m, tokens, run_cut(engine, tokens, cuts), T, f"{name} {dtype} {cuts}")


@pytest.mark.parametrize("name", ["A", "B"])
def test_the_stream_after_every_layer_run(models, name):
    """In 32-bit: the residual stream after each layer run (a looped layer once per pass, the pass input before its first layer)
    equals the plain implementation's, run by run."""
    m = models[name]
    engine = m.engine("float32")
    tokens = sc.prompts(m.vocab, [90], 27)[0]
    _, ref = plain.forward(m.cfg, m.W, tokens, torch.float32, return_layers=True)
    seen = []
    engine.model.observer = lambda occ, x: seen.append((occ, x.detach().float().cpu().clone()))
    slot = engine.new_sequence()
    engine.step([(slot, tokens)])
    engine.model.observer = None
    engine.free_sequence(slot)
    assert [occ for occ, _ in seen] == list(range(ref.shape[0]))
    for occ, x in seen:
        assert float((x - ref[occ]).abs().max()) <= 2e-4 * max(1.0, float(ref[occ].abs().max())), f"layer run {occ}"


# ---------------------------------------------------------------- mixers alone
def _mixer_of(case, layer, T, tensors=None, seed=0, max_positions=1024):
    """The mixer part of one layer of a configuration, built as the model builds it, with random (or given) tensors.
    Returns (mixer, tensors by checkpoint name in 64-bit, the layer's raw mixer record)."""
    from tileinfer_b200.config import config_from_dict
    from tileinfer_b200.parts import Runtime, lookup
    spec = config_from_dict(case).model_spec().layers[layer].mixer
    cls = lookup("mixer", spec.kind)
    g = torch.Generator().manual_seed(seed)
    if tensors is None:
        tensors = {}
        for d in cls.tensors(spec):
            t = torch.randn(tuple(d.shape), generator=g, dtype=F64)
            if len(d.shape) == 2:
                t = t * d.shape[1] ** -0.5
            elif d.name.endswith("norm"):
                t = 1 + 0.2 * t
            elif d.name.endswith(".b"):
                t = 0.3 * t
            tensors[d.name] = t if d.name.endswith("sink") else rnd(t, T)
    rt = Runtime(T)
    position = lookup("position", spec.position.kind)(spec.position, rt, max_positions) if spec.position.kind != "none" else None
    dev = {k: (v.float() if k.endswith("sink") else v.to(T)) for k, v in tensors.items()}
    return cls(spec, dev, rt, position), tensors, case["layers"][layer]["mixer"]


def _run_mixer(mixer, T, h, cuts, width, neighbour=None):
    """One sequence's rows through the mixer in portions (the rest one at a time); with ``neighbour`` another sequence's rows ride
    along in every step, in front."""
    from test_parts_gpu import OneStep
    env = OneStep(mixer, T, max_tokens=1024, max_seqs=2)
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
    got = torch.cat(out)
    bias = getattr(mixer, "out_bias", None)
    return got + bias.float().cpu() if bias is not None else got


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_attention_mixer_alone(dtype):
    """Biases, head-wise q/k norm with one weight per projection, partial half-split rotation with scaled bands, grouped heads,
    keys and values of different sizes and a window, against the plain mixer: whole, token by token and in portions whose edges
    fall inside, at and outside the window, beside another sequence in the batch."""
    T = DTYPES[dtype]
    g = torch.Generator().manual_seed(3)
    for case, layer, total in ((sc.CASE_A, 0, 150), (sc.CASE_A, 2, 150), (sc.CASE_B, 1, 260), (sc.CASE_B, 3, 200), (sc.CASE_C, 0, 140)):
        mixer, W, m = _mixer_of(case, layer, T, seed=layer)
        width = case["width"]
        h = rnd(torch.randn(total, width, generator=g, dtype=F64), T)
        other = rnd(torch.randn(40, width, generator=g, dtype=F64), T)
        ref = plain.attention_mixer(m, W, f"l{layer}.mix.", h, case["norm"]["eps"], T if T == torch.bfloat16 else F64).float()
        window = (m.get("mask") or {}).get("size", 50)
        for cuts in ([total], [1], [window - 1, 2, window, window + 1, 3], [64, 64, 2, 2, 60], [2, 2, 2, 2]):
            got = _run_mixer(mixer, T, h, cuts, width, neighbour=other if cuts[0] in (1, 64) else None)
            err = (got - ref).abs().max(-1).values
            tol = (1e-4 if T == torch.float32 else 6 * 2.0 ** -8) * max(1.0, float(ref.abs().max()))
            assert float(err.max()) <= tol, f"layer {layer} cuts {cuts[:3]}: worst {float(err.max()):.3g} at {int(err.argmax())}, first bad {int((err > tol).float().argmax())}"


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_latent_attention_mixer_alone(dtype):
    """Normed latents, the rotated key part shared by the heads (interleaved pairs, YaRN), the sink and the output gate, against
    the plain mixer, which builds every head's keys and values in full."""
    T = DTYPES[dtype]
    g = torch.Generator().manual_seed(4)
    for case, layer, total in ((sc.CASE_A, 1, 150), (sc.CASE_B, 0, 260), (sc.CASE_B, 2, 200), (sc.CASE_C, 1, 140)):
        mixer, W, m = _mixer_of(case, layer, T, seed=10 + layer)
        width = case["width"]
        h = rnd(torch.randn(total, width, generator=g, dtype=F64), T)
        other = rnd(torch.randn(40, width, generator=g, dtype=F64), T)
        ref = plain.latent_attention_mixer(m, W, f"l{layer}.mix.", h, case["norm"]["eps"], T if T == torch.bfloat16 else F64).float()
        for cuts in ([total], [1], [63, 2, 64, 3], [2, 2, 2, 2], [130, 1, 1, 5]):
            got = _run_mixer(mixer, T, h, cuts, width, neighbour=other if cuts[0] in (1, 63) else None)
            err = (got - ref).abs().max(-1).values
            tol = (1e-4 if T == torch.float32 else 8 * 2.0 ** -8) * max(1.0, float(ref.abs().max()))
            assert float(err.max()) <= tol, f"layer {layer} cuts {cuts[:3]}: worst {float(err.max()):.3g} at {int(err.argmax())}, first bad {int((err > tol).float().argmax())}"


# ---------------------------------------------------------------- weights made by hand
def _marked_rows(total, mark_at, W=16):
    """Ordinary tokens are the unit vector e1; the marked one is e0 with a little e2."""
    h = torch.zeros(total, W, dtype=F64)
    h[:, 1] = 1.0
    h[mark_at] = 0.0
    h[mark_at, 0], h[mark_at, 2] = 1.0, 0.25
    return h


NORMED = 1.0 / math.sqrt(1.0625 / 16)            # what the RMS norm makes of the marked row's e0 (its e2: a quarter of that)


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_a_marked_key_is_seen_up_to_the_windows_edge_and_not_beyond(dtype):
    """One head of identity weights whose query projection sends e1 to e0: every ordinary query scores the marked key
    scale * 4 * 3.88 = 23 above the others, so the output's e2 is the marked value's 0.25 while the marked key is among the
    last ``window`` positions and exactly zero from the next position on. Windows of 1, 2, a page, a page and one, and no
    multiple of anything; the edge inside a prompt, at a portion's first token, and among single tokens; marker on both sides
    of a page border."""
    T = DTYPES[dtype]
    W, scale = 16, 1.5
    eye = torch.eye(W, dtype=F64)
    for window, mark_at, cuts, total in ((1, 5, [20], 20), (2, 5, [20], 20), (2, 63, [64], 70), (7, 0, [1], 20), (7, 60, [66, 1, 4], 80),
                                         (64, 3, [140], 140), (64, 63, [100, 27], 200), (65, 64, [65], 140), (65, 0, [40, 25, 1, 30], 100),
                                         (100, 29, [128, 1, 1, 64], 260), (100, 130, [229, 2], 260), (100, 27, [30], 135)):
        case = sc.model(8, W, 1e-6, 1.0, [sc.attention(1, 1, W, W, scale, None, window=window)])
        tensors = {"l0.mix.o": eye.clone(), "l0.mix.o.b": torch.zeros(W, dtype=F64), "l0.mix.q.norm": torch.ones(W, dtype=F64), "l0.mix.k.norm": torch.ones(W, dtype=F64)}
        for k in "qkv":
            tensors[f"l0.mix.{k}"] = eye.clone()
            tensors[f"l0.mix.{k}.b"] = torch.zeros(W, dtype=F64)
        tensors["l0.mix.q"][0, 1], tensors["l0.mix.q"][1, 1] = 1.0, 0.0
        mixer, _, _ = _mixer_of(case, 0, T, tensors)
        out = _run_mixer(mixer, T, _marked_rows(total, mark_at), cuts, W)[:, 2]
        last = min(mark_at + window, total)                        # the first position that no longer sees the marker
        assert float(out[:mark_at].abs().max()) == 0.0 if mark_at else True
        if last > mark_at + 1:
            seen = out[mark_at + 1:last]
            assert float((seen - 0.25).abs().max()) <= (1e-4 if T == torch.float32 else 0.01) * 0.25, \
                f"window {window}, marker at {mark_at}, cuts {cuts}: {seen[:2].tolist()} .. {seen[-2:].tolist()}"
        assert last == total or float(out[last:].abs().max()) == 0.0, \
            f"window {window}, marker at {mark_at}, cuts {cuts}: seen at {mark_at + int(out[mark_at:].abs().nonzero().max())}, edge {last}"


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_one_far_latent_stands_out_among_hundreds_and_the_sink_takes_its_share(dtype):
    """The latent mixer with identity-like weights (ranks as wide as the input, one head, no rotated contribution): an ordinary
    query (4 e0 after the latent's norm) scores the marked latent 4 * 3.88 * scale = 23 and the others 0, so the output's e2 is
    the marked latent's e2 (0.97) times the marker's share times the half-open gate, seen from every later position however
    far, across page borders, from prompts and from single tokens. A sink as large as the marked score halves the share; one
    far below changes nothing; with two heads each sink acts on its own head."""
    T = DTYPES[dtype]
    W, Rd, scale = 16, 4, 1.5
    eye = torch.eye(W, dtype=F64)
    marked_score = scale * 4.0 * NORMED
    for sinks, shares in (([-30.0], [1.0]), ([marked_score], [0.5]), ([marked_score, -30.0], [0.5, 1.0])):
        H = len(sinks)
        case = sc.model(8, W, 1e-6, 1.0, [sc.latent(H, W, Rd, W, W, W, scale, None, base=100.0)])
        uq = torch.zeros(H, W + Rd, W, dtype=F64)
        uq[:, :W] = eye
        uq[:, 0, 1], uq[:, 1, 1] = 1.0, 0.0                             # e1 -> e0: ordinary tokens ask along e0
        dkv = torch.zeros(W + Rd, W, dtype=F64)
        dkv[:W] = eye
        tensors = {"l0.mix.dq": eye.clone(), "l0.mix.dq.norm": torch.ones(W, dtype=F64), "l0.mix.uq": uq.reshape(H * (W + Rd), W),
                   "l0.mix.dkv": dkv, "l0.mix.dkv.norm": torch.ones(W, dtype=F64), "l0.mix.uk": eye.repeat(H, 1), "l0.mix.uv": eye.repeat(H, 1),
                   "l0.mix.sink": torch.tensor(sinks, dtype=F64), "l0.mix.g": torch.zeros(H * W, W, dtype=F64),
                   "l0.mix.o": torch.cat([torch.eye(W, dtype=F64) * (1.0 if i == 0 else 0.0) for i in range(H)], 1)}
        # The output projection reads head 0 as it is; a second head lands eight elements further on.
        if H == 2:
            tensors["l0.mix.o"][:, W:] = torch.roll(eye, 8, 0)
        mixer, _, _ = _mixer_of(case, 0, T, tensors)
        for mark_at, cuts, total in ((0, [1], 150), (63, [64], 200), (64, [140], 330), (5, [300], 310), (128, [129], 260), (2, [2, 2, 60, 2], 100)):
            out = _run_mixer(mixer, T, _marked_rows(total, mark_at), cuts, W)
            for head, share in enumerate(shares):
                want = 0.25 * NORMED * share * 0.5
                seen = out[mark_at + 1:, (2 + 8 * head) % W]
                assert float((seen - want).abs().max()) <= (0.005 if T == torch.float32 else 0.04) * want, \
                    f"sinks {sinks}, head {head}, marker at {mark_at}: {seen[:3].tolist()} .. {seen[-3:].tolist()}, want {want}"
            assert float(out[:mark_at, 2].abs().max()) == 0.0 if mark_at else True


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_the_rotated_key_part_follows_the_distance(dtype):
    """The latent mixer with scores from the rotated part alone: every token's rotated query and key part is the same vector
    (1, 0) per pair up to the query's length a_t, so the score of a query at distance d from a key is scale * c^2 * a_t *
    sum_i cos(d f_i), c the multiplier of cos and sin, whatever the positions themselves; values carry each position's index in binary digits. Compared with that
    closed form in 64-bit: whole, in portions and token by token."""
    T = DTYPES[dtype]
    W, Rd, scale, total = 16, 6, 0.9, 90
    rot = {"base": 40.0, "dims": Rd, "scaling": {"factor": 3.0, "original": 12, "fast": 4.0, "slow": 0.5}}
    case = sc.model(8, W, 1e-6, 1.0, [sc.latent(1, W, Rd, W, W, W, scale, None, base=40.0, scaling=(3.0, 12, 4.0, 0.5))])
    eye = torch.eye(W, dtype=F64)
    uq = torch.zeros(W + Rd, W, dtype=F64)
    uq[W + 0, 15] = uq[W + 2, 15] = uq[W + 4, 15] = 0.25                # a quarter of the normed query latent's e15 per pair
    dkv = torch.zeros(W + Rd, W, dtype=F64)
    dkv[:W] = eye
    dkv[W + 0, 15] = dkv[W + 2, 15] = dkv[W + 4, 15] = 1.0              # the rotated key part is not normed
    tensors = {"l0.mix.dq": eye.clone(), "l0.mix.dq.norm": torch.ones(W, dtype=F64), "l0.mix.uq": uq, "l0.mix.dkv": dkv,
               "l0.mix.dkv.norm": torch.ones(W, dtype=F64), "l0.mix.uk": torch.zeros(W, W, dtype=F64), "l0.mix.uv": eye.clone(),
               "l0.mix.sink": torch.tensor([-30.0], dtype=F64), "l0.mix.g": torch.zeros(W, W, dtype=F64), "l0.mix.o": eye.clone()}
    mixer, _, _ = _mixer_of(case, 0, T, tensors)
    h = torch.zeros(total, W, dtype=F64)
    h[:, 15] = 1.0
    for t in range(total):
        for b in range(7):
            h[t, b] = 0.5 * ((t >> b) & 1)
    h = rnd(h, T)
    f, c = plain.yarn_frequencies(rot)
    d = (torch.arange(total)[:, None] - torch.arange(total)[None, :]).to(F64)
    values = h / torch.sqrt((h * h).mean(-1, keepdim=True) + 1e-6)
    # The query latent is normed with the digits in it: its e15, and so every pair's query, is 0.25 values[t, 15], not 1.
    s = scale * c * c * (0.25 * values[:, 15:16]) * sum(torch.cos(d * fi) for fi in f)
    s = s.masked_fill(d < 0, float("-inf"))
    ref = (torch.softmax(s, -1) @ values * 0.5).float()
    for cuts in ([total], [1], [2, 2, 30, 2, 40], [64, 2]):
        got = _run_mixer(mixer, T, h, cuts, W)
        assert float((got - ref).abs().max()) <= (2e-4 if T == torch.float32 else 0.03) * float(ref.abs().max()), f"cuts {cuts}"


# ---------------------------------------------------------------- kernels alone
def _tol(T, ref):
    return (1e-5 if T == torch.float32 else 2.0 ** -7) * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_small_kernels_alone(dtype):
    """The pair embedding with the token before coming from the step, from the state and from nowhere (products beyond 32 bits);
    the state's update; the layer norm; the stream's update by a normed sublayer output with a bias, from rows and from partial
    sums, with the next layer norm; the rotation of a part of every head in both pairings; the squared rectifier."""
    from types import SimpleNamespace
    from tileinfer_b200.kernels import ops
    from tileinfer_b200.parts.base import Rotation
    T = DTYPES[dtype]
    g = torch.Generator().manual_seed(9)
    R = lambda *shape, s=1.0: rnd(torch.randn(*shape, generator=g).to(F64) * s, T)
    dev = lambda t: t.to(T).cuda()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    # Three sequences in one step: slot 2 goes on from position 7 (its last token, 11, is in the state), slot 0 starts, slot 1
    # goes on by one token.
    vocab, size = 23, 40
    for buckets, a, b in ((13, 5, 3), (1, 9, 4), (1009, 2000003, 1000033)):
        table, pair = R(vocab, size), R(buckets + 1, size)
        ids = [4, 9, 9, 22, 0, 17, 1, 6]
        positions = [7, 8, 9, 0, 1, 2, 3, 30]
        tok_slot = [2, 2, 2, 0, 0, 0, 0, 1]
        last = i32([-1, 21, 11, 5])
        x = torch.empty(len(ids), size, dtype=torch.float32, device="cuda")
        status = torch.zeros(4, dtype=torch.int32, device="cuda")
        ops.embed_bigram32(x, dev(table), dev(pair), i32(ids), i32(positions), i32(tok_slot), last, 2.5, buckets, a, b, status)
        before = [11, 4, 9, None, 22, 0, 17, 21]
        rows = [buckets if p is None else (p * a + t * b) % buckets for p, t in zip(before, ids)]
        ref = table[ids] * 2.5 + pair[rows]
        assert float((x.cpu() - ref.float()).abs().max()) <= 1e-5 * float(ref.abs().max())
        step = SimpleNamespace(token_ids=i32(ids), cu_seqlens=i32([0, 3, 7, 8]), seq_slots=i32([2, 0, 1]), n_seqs=3)
        ops.last_token_update(last, step)
        assert last.tolist() == [1, 6, 9, 5]
        x2 = torch.empty(len(ids), size, dtype=torch.float32, device="cuda")
        ops.embed_bigram32(x2, dev(table), None, i32(ids), i32(positions), i32(tok_slot), None, 0.5, 0, 0, 0, status)
        assert float((x2.cpu() - (table[ids] * 0.5).float()).abs().max()) <= 1e-6 * float(table.abs().max())
        assert int(status.abs().sum()) == 0
    # Layer norm and the stream's update. Rows with a large mean, so that a norm that forgets to take it off shows.
    n, size, eps = 37, 72, 1e-5
    centred = ops.NORM_CENTRED
    x = torch.randn(n, size, generator=g) * 2 + 5
    w, w2, bias = R(size), R(size), R(size, s=0.5)
    h = torch.empty(n, size, dtype=T, device="cuda")
    ops.norm32(h, x.cuda(), dev(w), eps, centred)
    ref = plain.layer_norm(x.to(F64), w, eps)
    assert float((h.float().cpu() - ref.float()).abs().max()) <= _tol(T, ref)
    d = rnd(R(n, size, s=3.0) + 4, T)
    parts = torch.randn(3, n, size, generator=g) + 1
    for delta, ref_d, use_bias in ((d, d, True), (d, d, False), (parts, parts.sum(0).to(F64), True)):
        xs = x.clone().cuda()
        arg = delta.float().cuda() if delta.dim() == 3 else dev(delta)
        ops.branch_norm_add32(xs, arg, dev(w), eps, 1.0, centred, h=h, out_norm=(dev(w2), eps, centred), bias=dev(bias) if use_bias else None)
        ref_x = x.to(F64) + plain.layer_norm(ref_d + (bias if use_bias else 0), w, eps)
        assert float((xs.cpu() - ref_x.float()).abs().max()) <= 2e-5 * float(ref_x.abs().max())
        ref_h = plain.layer_norm(ref_x, w2, eps)
        assert float((h.float().cpu() - ref_h.float()).abs().max()) <= _tol(T, ref_h)
    # Rotation of the elements [first, first + dims) of every head.
    for interleaved, first, dims, row, mult in ((True, 10, 6, 16, 1.3), (False, 0, 4, 12, 1.0), (True, 0, 8, 8, 1.0), (False, 6, 10, 16, 0.7)):
        f = [0.9 ** i for i in range(dims // 2)]
        P = 50
        ang = torch.arange(P, dtype=F64)[:, None] * torch.tensor(f, dtype=F64)[None, :]
        table = torch.stack([ang.cos() * mult, ang.sin() * mult], -1).float().contiguous().cuda()
        q = R(P, 3, row)
        order = torch.randperm(P, generator=g)
        got = dev(q[order]).contiguous()
        ops.rotate_heads(got, Rotation(table, dims, interleaved), order.to(torch.int32).cuda(), first=first)
        ref = q.clone()
        ref[..., first:first + dims] = plain.rotate(q[..., first:first + dims], f, interleaved, mult)
        assert float((got.float().cpu()[torch.argsort(order)] - ref.float()).abs().max()) <= _tol(T, ref)
    # max(z, 0)^2 behind a product.
    xin, wgt = R(n, 48), R(56, 48, s=0.3)
    y = torch.empty(n, 56, dtype=T, device="cuda")
    ops.gemm_plain(y, dev(xin), dev(wgt), ops.EPI_RELU2)
    z = xin @ wgt.T
    ref = torch.relu(rnd(z, T)) ** 2
    assert float((y.float().cpu() - ref.float()).abs().max()) <= 2 * _tol(T, ref)
    assert float(y.float().cpu()[z < -1e-3].abs().max()) == 0.0


def test_the_pass_input_reads_the_stream_and_the_embedding():
    """s' = P concat(s, e): with P = [2 I, 3 I] the stream after the pass input of a model without layers' contributions would be
    2 s + 3 e; checked on the part alone, for rows that differ in x and x0."""
    from tileinfer_b200.config.spec import PassInputSpec
    from tileinfer_b200.parts import Runtime, lookup
    for T in (torch.float32, torch.bfloat16):
        size, n = 24, 9
        rt = Runtime(T)
        cls = lookup("pass_input", "concat_linear")
        spec = PassInputSpec(kind="concat_linear", hidden_size=size, weight_name="loop.in", at=(0,))
        eye = torch.eye(size)
        g = torch.Generator().manual_seed(2)
        mix = torch.randn(size, 2 * size, generator=g) * 0.2
        for W in (torch.cat([2 * eye, 3 * eye], 1), mix):
            part = cls(spec, {"loop.in": W.to(T).cuda()}, rt)
            x0 = rnd(torch.randn(n, size, generator=g), T)
            x = rnd(torch.randn(n, size, generator=g), T)
            xs = x.clone().cuda()
            part.begin(x0.cuda())
            out = part.forward(xs)
            out = out.sum(0) if out.dim() == 3 else out
            ref = torch.cat([x, x0], 1).double() @ rnd(W, T).double().T
            assert out.dtype == torch.float32
            assert float((out.cpu() - ref.float()).abs().max()) <= (1e-5 if T == torch.float32 else 2.0 ** -7) * float(ref.abs().max())


# ---------------------------------------------------------------- through the public entry points
def test_greedy_generation_through_the_public_entry_point(models):
    """``generate`` (batches, scheduler, sampler, decode loop) on several prompts at once, more than there are slots, in 32-bit:
    every generated token is the plain implementation's most likely next token for the same prefix. The token before each
    generated token reaches the pair embedding through the sequence's state."""
    import tileinfer_b200 as ti
    for name in ("A", "B"):
        m = models[name]
        engine = ti.load_model(m.folder, dtype="float32", max_context=256, max_seqs=3)
        reqs = sc.prompts(m.vocab, [3, 41, 90, 17, 1], 41)
        outs = ti.generate(engine, reqs, max_new_tokens=40, stop_ids=[])
        assert [len(o) for o in outs] == [40] * 5
        for p, o in zip(reqs, outs):
            ref = plain.forward(m.cfg, m.W, p + o, torch.float32).numpy()
            for k, tok in enumerate(o):
                row = ref[len(p) + k - 1]
                assert row[tok] >= row.max() - 1e-4, f"{name} token {k}: generated {tok}, plain argmax {int(row.argmax())}"


@pytest.mark.parametrize("dtype", sorted(DTYPES))
def test_trace_replay(models, dtype):
    """The same requests through ``bin/trace_run``: whole, with the tail one by one, and in two batches one after the other (the
    second in the first one's slots, pages and last-token states)."""
    m = models["B"]
    reqs = {f"r{i}": t for i, t in enumerate(sc.prompts(m.vocab, [1, 9, 70, 130, 200], 51))}
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
        sc.compare(m, reqs[rid[1:]], g, DTYPES[dtype], f"replay {dtype} {rid}")


def test_bfloat16_steps_take_the_fast_kernels(models):
    """Case B's sizes are ones the fast kernels take: a prompt and a decode step in bfloat16 go through the tensor-core products
    and the paged attention kernels (with a sink in the latent layers), not through their plain stand-ins."""
    from tileinfer_b200.kernels import library
    m = models["B"]
    engine = m.engine("bfloat16", graphs=False)
    slot = engine.new_sequence()
    library.call_counts.clear()
    engine.step([(slot, sc.prompts(m.vocab, [600], 61)[0])])
    engine.step([(slot, [5])])
    engine.free_sequence(slot)
    engine.check_health()
    used = dict(library.call_counts)
    runs = len(engine.model.spec.order)
    latent_runs = sum(1 for i in engine.model.spec.order if m.cfg["layers"][i]["type"] == "latent_attention")
    assert runs == 6 and latent_runs == 3
    assert used.get("ti_attention_prefill_tc_sink", 0) == latent_runs and used.get("ti_attention_decode_sink", 0) == latent_runs, used
    assert used.get("ti_attention_prefill_tc", 0) == runs - latent_runs and used.get("ti_attention_decode_shared", 0) == runs - latent_runs, used
    assert used.get("ti_latent_inputs", 0) == 2 * latent_runs and used.get("ti_conv_attention_inputs", 0) == 2 * (runs - latent_runs), used
    assert used.get("ti_embed_bigram32", 0) == 2 and used.get("ti_last_token_update", 0) == 2, used
    assert used.get("ti_gemm_tcgen05", 0) > 0 and "ti_attention_plain" not in used and "ti_gemm_plain" not in used, used
