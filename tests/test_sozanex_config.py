"""The Sozanex configuration on the CPU: what config.json keys are read, what may be absent, what is refused, which tensors a
model declares, the order of the layer runs, the rotation tables, the round trip through a model folder, what the cache is
asked for, and the plain implementation's own pieces."""
import copy
import json
import math

import pytest
import torch

import plain_sozanex as plain
import sozanex_cases as sc
from tileinfer_b200.config import ConfigError, SozanexConfig, config_from_dict, resolve_architecture
from tileinfer_b200.engine.model import tensor_declarations


def test_registry_resolves_the_design_by_its_name():
    assert resolve_architecture({"architecture": "Sozanex"}).config_class is SozanexConfig
    assert resolve_architecture({"architectures": ["Sozanex"]}).config_class is SozanexConfig
    assert resolve_architecture({"architecture": "Zudepel"}).name == "Zudepel"


@pytest.mark.parametrize("name", sorted(sc.CASES))
def test_round_trip_and_lowering(name):
    case = sc.CASES[name]
    cfg = config_from_dict(case)
    assert SozanexConfig.from_dict(cfg.to_dict()) == cfg
    assert cfg.to_dict() == case
    spec = cfg.model_spec()
    assert spec.options["residual_dtype"] == "float32" and spec.embedding_kind == "scaled_pair32" and spec.final_norm.kind == "layernorm32"
    assert spec.options["embed_scale"] == case["embedding"]["scale"] and ("pair_table" in spec.options) == ("bigram" in case["embedding"])
    runs = [i for i, _ in plain.layer_runs(case)]
    assert list(spec.order) == runs
    starts = [k for k, (_, first) in enumerate(plain.layer_runs(case)) if first]
    assert (list(spec.pass_input.at) if spec.pass_input else []) == starts
    for l, raw in zip(spec.layers, case["layers"]):
        m = raw["mixer"]
        assert l.block == "sandwich" and l.mixer_post_norm is not None and (l.feed_forward is None) == (raw["mlp"] is None)
        assert (l.feed_forward_norm is None) == (raw["mlp"] is None) == (l.feed_forward_post_norm is None)
        assert (l.mixer.num_heads, l.mixer.head_dim, l.mixer.options["value_dim"], l.mixer.scale) == (m["heads"], m["dim"], m["vdim"], m["scale"])
        assert l.mixer.window == (m.get("mask") or {}).get("size")
        if raw["type"] == "attention":
            assert l.mixer.kind == "conv_attention" and l.mixer.num_kv_heads == m["kv_heads"] and l.mixer.options["head_norm"]
            assert l.mixer.options["out_bias"] and not l.mixer.options["sink"] and not l.mixer.options["gate"]
            if "rot" in m:
                assert l.mixer.position.options["pairing"] == "half" and l.mixer.position.options["rotary_dim"] == m["rot"]["dims"]
            else:
                assert l.mixer.position.kind == "none"
        else:
            o = l.mixer.options
            assert l.mixer.kind == "latent_attention" and (o["q_rank"], o["kv_rank"], o["rot_dim"]) == (m["q_rank"], m["kv_rank"], m["rot_dim"])
            assert o["sink"] and o["gate"] and l.mixer.position.options["pairing"] == "interleaved"
        if raw["mlp"]:
            assert l.feed_forward.options["activation"] == "relu2" and l.feed_forward.intermediate_size == raw["mlp"]["ff"]


def test_declared_tensors():
    decls = {d.name: tuple(d.shape) for d in tensor_declarations(config_from_dict(sc.CASE_A).model_spec())}
    assert decls["embed"] == (131, 52) and decls["bigram"] == (98, 52) and decls["loop.in"] == (52, 104) and decls["head"] == (131, 52)
    assert all(decls[f"l{i}.{n}"] == (52,) for i in (0, 2) for n in ("norm1", "norm1b", "norm2", "norm2b")) and decls["final.norm"] == (52,)
    assert decls["l1.norm1b"] == (52,) and "l1.norm2" not in decls and not any(n.startswith("l1.mlp") for n in decls)
    assert decls["l0.mix.q"] == (60, 52) and decls["l0.mix.k"] == (20, 52) and decls["l0.mix.v"] == (28, 52) and decls["l0.mix.o"] == (52, 84)
    assert decls["l0.mix.q.b"] == (60,) and decls["l0.mix.v.b"] == (28,) and decls["l0.mix.o.b"] == (52,)
    assert decls["l0.mix.q.norm"] == (10,) and decls["l0.mix.k.norm"] == (10,) and "l0.mix.sink" not in decls
    assert decls["l1.mix.dq"] == (20, 52) and decls["l1.mix.uq"] == (3 * 18, 20) and decls["l1.mix.dkv"] == (32, 52) and decls["l1.mix.dkv.norm"] == (26,)
    assert decls["l1.mix.uk"] == (36, 26) and decls["l1.mix.uv"] == (30, 26) and decls["l1.mix.sink"] == (3,) and decls["l1.mix.g"] == (30, 52)
    assert decls["l1.mix.o"] == (52, 30) and decls["l0.mlp.up"] == (60, 52) and decls["l2.mlp.down"] == (52, 36)
    decls = {d.name for d in tensor_declarations(config_from_dict(sc.CASE_C).model_spec())}
    assert "bigram" not in decls and "loop.in" in decls


def test_what_is_refused():
    def broken(change):
        c = copy.deepcopy(sc.CASE_B)
        change(c)
        with pytest.raises(ConfigError):
            config_from_dict(c)
    broken(lambda c: c["layers"][0].update(type="lightning"))
    broken(lambda c: c["layers"][1]["mixer"].update(kv_heads=3))
    broken(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=66))
    broken(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7))
    broken(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=8))          # the rotated part and its rotation differ
    broken(lambda c: c["layers"][0]["mixer"].pop("q_rank"))
    broken(lambda c: c["layers"][0]["mixer"].update(mask={"size": 8}))       # only the attention mixer has a window
    broken(lambda c: c["layers"][2]["mlp"].update(kind="moe"))
    broken(lambda c: c["loop"].update(stop=5))
    broken(lambda c: c["loop"].update(start=3))
    broken(lambda c: c["loop"].update(times=0))
    broken(lambda c: c["embedding"]["bigram"].update(buckets=0))
    broken(lambda c: c["layers"][1]["mixer"]["mask"].update(size=0))
    broken(lambda c: c.pop("norm"))


def test_rotation_tables_follow_the_scalings():
    """The position part's table against the plain implementation's frequencies: band-wise scaled (all three bands occur), YaRN
    (with its multiplier), and unscaled; cos and sin of 64-bit angles."""
    from tileinfer_b200.config.spec import PositionSpec
    from tileinfer_b200.parts import Runtime, lookup
    rt = Runtime(torch.float32, "cpu", "plain")
    for case in sc.CASES.values():
        cfg = config_from_dict(case)
        for l, raw in zip(cfg.model_spec().layers, case["layers"]):
            rot = raw["mixer"].get("rot")
            if rot is None:
                continue
            part = lookup("position", "rope")(l.mixer.position, rt, 700)
            f, mult = plain.yarn_frequencies(rot) if raw["type"] == "latent_attention" else (plain.llama3_frequencies(rot), 1.0)
            ang = torch.arange(700, dtype=torch.float64)[:, None] * torch.tensor(f, dtype=torch.float64)[None, :]
            r = part.rotation()
            assert r.rotary_dim == rot["dims"] and r.interleaved == (raw["type"] == "latent_attention")
            assert float((r.cos_sin[:, :, 0].double() - ang.cos() * mult).abs().max()) < 1e-6
            assert float((r.cos_sin[:, :, 1].double() - ang.sin() * mult).abs().max()) < 1e-6
    s = sc.CASE_A["layers"][0]["mixer"]["rot"]
    f, f0 = plain.llama3_frequencies(s), plain.llama3_frequencies({"dims": s["dims"], "base": s["base"]})
    ratios = [a / b for a, b in zip(f, f0)]
    assert ratios[0] == 1.0 and abs(ratios[-1] - 0.25) < 1e-12 and 0.25 < ratios[1] < 1.0
    y = sc.CASE_B["layers"][0]["mixer"]["rot"]
    f, mult = plain.yarn_frequencies(y)
    assert abs(mult - (0.1 * math.log(6.0) + 1)) < 1e-12 and f[0] == 1.0 and abs(f[-1] * 6.0 / 5000.0 ** (-14 / 16) - 1) < 1e-12


def test_what_the_cache_is_asked_for():
    """Every layer run has storage of its own (a looped layer as many as it has runs); windows reach the cache's groups; the
    latent layers' rows hold the latent and the rotated key part; the embedding keeps one integer per sequence."""
    from tileinfer_b200.parts.latent_attention import pool_row
    assert pool_row(48, 16) == 64 and pool_row(96, 32) == 128 and pool_row(26, 6) == 32 and pool_row(100, 40) == 256
    assert pool_row(300, 4) == 304 and pool_row(70, 0) == 70


def test_plain_pieces():
    assert plain.bigram_rows([3, 4, 4, 0], 7, 5, 2) == [7, (15 + 8) % 7, (20 + 8) % 7, 20 % 7]
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=torch.float64)
    y = plain.layer_norm(x, torch.ones(4), 0.0)
    assert abs(float(y.mean())) < 1e-12 and abs(float((y * y).mean()) - 1.0) < 1e-12
    q = torch.zeros(3, 1, 2, dtype=torch.float64); k = torch.zeros(3, 1, 2, dtype=torch.float64)
    v = torch.tensor([[[1.0]], [[2.0]], [[4.0]]], dtype=torch.float64)
    out = plain.masked_attention(q, k, v, 1.0, window=2, sink=torch.tensor([0.0]))
    assert torch.allclose(out[:, 0, 0], torch.tensor([1 / 2, 3 / 3, 6 / 3], dtype=torch.float64))
    r = plain.rotate(torch.tensor([[[1.0, 0.0, 0.0, 1.0]], [[1.0, 0.0, 0.0, 1.0]]], dtype=torch.float64), [math.pi / 2, math.pi], True)
    assert torch.allclose(r[1, 0], torch.tensor([0.0, 1.0, -0.0, -1.0], dtype=torch.float64), atol=1e-12)
    assert [i for i, _ in plain.layer_runs(sc.CASE_A)] == [0, 1, 0, 1, 0, 1, 2]


def test_the_command_line_writes_a_model_folder_of_this_design(tmp_path, capsys):
    """``tileinfer random config.json out`` goes through the registry: a Sozanex config.json gives a folder that loads back, with
    the loop's input projection, the second table's extra row and the latent layer's tensors in it."""
    from tileinfer_b200.cli import cli
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(sc.CASE_A))
    out = tmp_path / "model"
    assert cli(["random", str(cfg_path), str(out), "--seed", "3"]) == 0
    cfg, W = sc.load_folder(str(out))
    assert cfg["architecture"] == "Sozanex" and cfg["loop"] == {"start": 0, "stop": 2, "times": 3}
    assert W["loop.in"].shape == (52, 104) and W["bigram"].shape == (98, 52)
    assert W["l1.mix.dkv"].shape == (26 + 6, 52) and W["l1.mix.sink"].shape == (3,) and W["l0.mix.q.norm"].shape == (10,)
    assert W["l0.mix.o.b"].shape == (52,) and "l1.mlp.up" not in W
