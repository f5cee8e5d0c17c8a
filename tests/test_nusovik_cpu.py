"""CPU side of the Nusovik integration: configuration, registry, cache geometry, the distance-bias lookup,
and sanity of the float64 oracle itself (causality, chunk edges, the sink, the convolution's reach, the
recurrences against their closed forms)."""
import json
import math

import pytest
import torch

from oracle import nusovik_oracle as O
from tests.test_nusovik_gpu import CONFIGS
from vila_b200.model.nusovik import NusovikConfig, NusovikForCausalLM, distance_rows
from vila_b200.model.registry import LANGUAGE_MODELS, language_model_architecture

F64 = torch.float64


def random_weights(cfg_dict, rows, seed=0):
    g = torch.Generator().manual_seed(seed)
    shapes = NusovikConfig.from_dict(cfg_dict).tensor_shapes()
    out = {}
    for n, s in shapes.items():
        s = tuple(rows if k < 0 else k for k in s)
        out[n] = (torch.randn(s, generator=g) * (0.1 if len(s) == 1 else 1.5 / s[-1] ** 0.5)).to(torch.bfloat16)
    return out


@pytest.mark.parametrize("name", list(CONFIGS))
def test_config_round_trip_shapes_and_cache_geometry(name):
    d, rows = CONFIGS[name]
    cfg = NusovikConfig.from_dict(d)
    assert cfg.to_dict() == json.loads(json.dumps(d))
    shapes = cfg.tensor_shapes()
    model = NusovikForCausalLM(cfg, "cpu")
    pools, states = model.latent_widths(), model.state_shapes()
    for i, spec in enumerate(d["layers"]):
        assert (f"l{i}.norm2" in shapes) == (spec["mlp"] is not None)
        m = spec["mixer"]
        if spec["type"] == "parallel":
            a, r = m["left"], m["right"]
            assert pools[i] == 2 * a["kv_heads"] * a["dim"] and shapes[f"l{i}.mix.left.rel"] == (-1, a["heads"])
            assert states[(i, "ssm")] == (r["heads"], r["vdim"], r["state"])
            chans, taps = r["heads"] * r["vdim"] + 2 * r["groups"] * r["state"], r["conv"]
            assert shapes[f"l{i}.mix.right.in"][0] == r["heads"] * r["vdim"] + chans + r["heads"]
        else:
            assert i not in pools and states[(i, "ssm")] == (m["inner"], m["state"])
            chans, taps = m["inner"], m["conv"]
        assert states.get((i, "conv")) == ((taps - 1, chans) if taps > 1 else None)


def test_bad_configs_are_refused():
    for change in (lambda d: d["layers"][0].update(type="something_else"),
                   lambda d: d["layers"][0]["mixer"]["left"].update(kv_heads=3),       # 4 heads over 3 key heads
                   lambda d: d["layers"][0]["mixer"]["left"].update(vdim=16),          # the values are the keys
                   lambda d: d["layers"][0]["mixer"]["right"].update(groups=4),        # 6 heads in 4 groups
                   lambda d: d["layers"][0]["mixer"]["right"].update(norm_groups=7),
                   lambda d: d["layers"][1]["mixer"].update(conv=0),
                   lambda d: d["layers"][0]["mlp"].update(kind="moe")):
        d = json.loads(json.dumps(CONFIGS["odd"][0]))
        change(d)
        with pytest.raises(ValueError):
            NusovikConfig.from_dict(d)


def test_registry_names_the_architecture(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(CONFIGS["ones"][0]))
    assert language_model_architecture(tmp_path) == "Nusovik" and LANGUAGE_MODELS["Nusovik"] is NusovikForCausalLM


def test_weights_are_checked_against_the_config():
    d, rows = CONFIGS["ones"]
    w = random_weights(d, rows)
    model = NusovikForCausalLM(NusovikConfig.from_dict(d), "cpu", torch.float32).load_weights(w)
    assert model.layers[0].dist_bias.shape == (d["layers"][0]["mixer"]["left"]["bias_max"] + 1, 1)
    bad = dict(w)
    bad["l1.mix.x"] = bad["l1.mix.x"][:-1]
    with pytest.raises(ValueError):
        NusovikForCausalLM(NusovikConfig.from_dict(d), "cpu", torch.float32).load_weights(bad)
    del bad["l0.mix.left.sink"]
    with pytest.raises(KeyError):
        NusovikForCausalLM(NusovikConfig.from_dict(d), "cpu", torch.float32).load_weights(bad)


def test_distance_rows_of_the_bias_table():
    for rows, far in ((10, 40), (16, 100), (6, 300), (7, 33), (32, 256), (2, 5)):
        got = distance_rows(rows, far)
        assert got == [O.distance_bucket(n, rows, far) for n in range(far + 1)]
        assert got[:rows // 2] == list(range(rows // 2)) and got[-1] == rows - 1 and got == sorted(got)
    # log-spaced part: with 16 rows up to distance 256 the rows 8 .. 15 start at 8 * 32^(k / 8)
    got = distance_rows(16, 256)
    for k in range(8):
        first = got.index(8 + k)
        assert first == math.ceil(8 * 32 ** (k / 8) - 1e-9)


def test_oracle_is_causal_and_chunked():
    d, rows = CONFIGS["odd"]
    w = random_weights(d, rows, seed=1)
    toks = torch.randint(0, d["vocab"], (60,), generator=torch.Generator().manual_seed(2)).tolist()
    a = O.forward(d, w, toks)
    other = list(toks)
    other[40] = (other[40] + 1) % d["vocab"]
    b = O.forward(d, w, other)
    assert torch.equal(a[:40], b[:40]) and not torch.allclose(a[40:], b[40:])
    # the attention alone: a key in the previous chunk does not reach a query, one in its own chunk does
    m = d["layers"][0]["mixer"]["left"]          # chunk 24
    W = {k: v.to(F64) for k, v in w.items()}
    h = torch.randn(60, d["width"], dtype=F64, generator=torch.Generator().manual_seed(3))
    base = O.chunked_sink_attention(h, W, "l0.mix.left.", m, 1e-5)
    h2 = h.clone()
    h2[23] += 1.0                                 # last position of chunk 0
    moved = O.chunked_sink_attention(h2, W, "l0.mix.left.", m, 1e-5)
    assert torch.equal(base[24:], moved[24:]) and not torch.allclose(base[23], moved[23])
    h2 = h.clone()
    h2[24] += 1.0                                 # first position of chunk 1
    moved = O.chunked_sink_attention(h2, W, "l0.mix.left.", m, 1e-5)
    assert not torch.allclose(base[47], moved[47]) and torch.equal(base[48:], moved[48:])


def test_oracle_sink_takes_weight():
    d, rows = CONFIGS["ones"]
    w = random_weights(d, rows, seed=4)
    m = d["layers"][0]["mixer"]["left"]
    h = torch.randn(9, d["width"], dtype=F64, generator=torch.Generator().manual_seed(5))
    W = {k: v.to(F64) for k, v in w.items()}
    W["l0.mix.left.sink"] = torch.full((1,), 40.0, dtype=F64)
    assert float(O.chunked_sink_attention(h, W, "l0.mix.left.", m, 1e-5).abs().max()) < 1e-9


def test_oracle_convolution_reach_and_recurrence_closed_forms():
    u = torch.zeros(10, 2, dtype=F64)
    u[3] = 1.0
    wconv = torch.tensor([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]], dtype=F64)      # tap 2 meets the newest input
    out = O.causal_conv(u, wconv, torch.zeros(2, dtype=F64))
    assert out[3].tolist() == [3.0, 6.0] and out[4].tolist() == [2.0, 5.0] and out[5].tolist() == [1.0, 4.0]
    assert float(out[:3].abs().max()) == 0.0 and float(out[6:].abs().max()) == 0.0
    # softplus for large and small arguments
    z = torch.tensor([-50.0, 0.0, 50.0], dtype=F64)
    assert torch.allclose(O.softplus(z), torch.tensor([math.exp(-50.0), math.log(2.0), 50.0], dtype=F64))
