"""The Fasodra configuration on the CPU: keys read and refused, the round trip, the records and tensors it lowers to, what the
cache is asked for, and pieces of the plain implementation against closed forms."""
import copy
import math

import pytest
import torch

import fasodra_cases as fc
import plain_fasodra as plain
from tileinfer_b200.config import ConfigError, config_from_dict
from tileinfer_b200.engine.model import tensor_declarations


@pytest.mark.parametrize("name", sorted(fc.CASES))
def test_round_trip_and_registry(name):
    case = fc.CASES[name]
    cfg = config_from_dict(case)
    assert type(cfg).__name__ == "FasodraConfig"
    again = config_from_dict(cfg.to_dict())
    assert again == cfg
    spec = cfg.model_spec()
    assert spec.architecture == "Fasodra" and len(spec.layers) == len(case["layers"]) and spec.order == tuple(range(len(case["layers"])))
    assert spec.options["residual_dtype"] == "float32" and spec.options.get("streams", 0) == (case.get("streams") or 0)
    for layer, raw in zip(spec.layers, case["layers"]):
        assert layer.block == "hyper" and layer.mixer_norm.kind == "layernorm32" and layer.mixer_norm.options["bias"]
        assert (layer.feed_forward is None) == (raw["mlp"] is None)
        assert layer.mixer.kind == ("conv_attention" if raw["type"] == "attention" else "pair")


def test_what_is_refused():
    bad = copy.deepcopy(fc.CASE_A)
    bad["layers"][0]["type"] = "convolution"
    with pytest.raises(ConfigError):
        config_from_dict(bad)
    for path, value in ((("layers", 0, "mixer", "heads"), 5), (("layers", 0, "mlp", "router", "top"), 9), (("layers", 1, "mixer", "left", "rot", "dims"), 7),
                        (("layers", 2, "mixer", "right", "kv_heads"), 3), (("streams",), 9), (("layers", 0, "mlp", "kind"), "dense")):
        bad = copy.deepcopy(fc.CASE_A)
        at = bad
        for k in path[:-1]:
            at = at[k]
        at[path[-1]] = value
        with pytest.raises(ConfigError):
            config_from_dict(bad)
    bad = copy.deepcopy(fc.CASE_A)
    del bad["layers"][0]["mixer"]["bias_max"]
    with pytest.raises(ConfigError):
        config_from_dict(bad)


def test_declared_tensors():
    names = {d.name: d for d in tensor_declarations(config_from_dict(fc.CASE_A).model_spec())}
    assert names["l0.mix.rel"].free_dims == (0,) and names["l0.mix.rel"].shape[1] == 6
    assert "l0.mix.q.norm" not in names and names["l2.mix.left.q.norm"].shape == (6,)
    assert names["l1.mix.left.g"].shape == (3, 52) and names["l1.mix.right.mu.w"].shape == (52,)
    assert names["l1.mix.right.w1"].free_dims == (0,) and names["l1.mix.right.w2"].free_dims == (1,) and names["l1.mix.right.u"].shape == (3, 10)
    assert names["l2.mix.right.q.conv"].shape == (20, 3) and names["l2.mix.right.v.conv"].shape == (24, 3) and names["l2.mix.right.b"].shape == (4, 52)
    assert names["l2.mix.left.out"].shape == (52,) and names["l2.mix.right.norm"].shape == (6,)
    assert names["l0.hc1.mix"].shape == (3, 3) and names["l0.hc2.in"].shape == (3,) and "l1.hc2.in" not in names and "l1.norm2" not in names
    assert names["l0.mlp.e4.up"].shape == (20, 52) and "l0.mlp.e0.gate" not in names and names["final.norm.b"].shape == (52,)
    plain_names = {d.name for d in tensor_declarations(config_from_dict(fc.CASE_C).model_spec())}
    assert not any(".hc" in n for n in plain_names) and "l2.mix.right.q.conv" not in plain_names and "l0.mix.left.g" in plain_names


def test_what_the_cache_is_asked_for():
    from tileinfer_b200.config.spec import MixerSpec
    spec = config_from_dict(fc.CASE_A).model_spec()
    pair = spec.layers[2].mixer
    assert isinstance(pair.options["left"], MixerSpec) and pair.options["right"].kind == "gated_delta" and pair.options["out_norm"]
    assert spec.layers[1].mixer.options["right"].kind == "time_mix" and spec.layers[1].mixer.options["left_scale"] == 0.8
    assert spec.layers[0].mixer.options["chunk"] == 7 and spec.layers[0].mixer.options["distance_bias"] == 20.0


def test_distance_buckets():
    from tileinfer_b200.parts.conv_attention import distance_buckets
    for rows, far in ((16, 200), (6, 20), (10, 50), (12, 100), (32, 128), (8, 9)):
        lib = distance_buckets(rows, far, int(far) + 40)
        mine = [plain.distance_bucket(n, rows, far) for n in range(int(far) + 40)]
        assert lib == mine
        half = rows // 2
        assert mine[:half] == list(range(half)) and mine[int(far)] == rows - 1 and max(mine) == rows - 1
        assert all(b >= a for a, b in zip(mine, mine[1:]))


def test_plain_pieces():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 12, generator=g, dtype=torch.float64) + 3.0
    w, b = torch.randn(12, generator=g, dtype=torch.float64), torch.randn(12, generator=g, dtype=torch.float64)
    ref = torch.nn.functional.layer_norm(x, (12,), w, b, 1e-5)
    assert float((plain.layer_norm(x, w, b, 1e-5) - ref).abs().max()) < 1e-12
    # A convolution whose taps are 1, 10, 100 shows which row every tap read.
    rows = torch.arange(1, 6, dtype=torch.float64)[:, None]
    y = plain.short_conv(rows, torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64))
    assert y[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0, 345.0]
    # A rotation by position p turns the pair (1, 0) to (cos, sin) of p * base^(-2 i / dims).
    q = torch.zeros(4, 1, 6, dtype=torch.float64)
    q[:, 0, 0], q[:, 0, 1], q[:, 0, 5] = 1.0, 1.0, 7.0
    r = plain.rotate(q, torch.arange(4), 4, 100.0)
    for p in range(4):
        assert abs(float(r[p, 0, 0]) - math.cos(p)) < 1e-12 and abs(float(r[p, 0, 2]) - math.sin(p)) < 1e-12
        assert abs(float(r[p, 0, 1]) - math.cos(p * 0.1)) < 1e-12 and float(r[p, 0, 5]) == 7.0
