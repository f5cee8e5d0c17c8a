"""CPU side of the Ludazen integration: configuration, registry, cache geometry, the frequency table, and
sanity of the float64 oracle itself (the window's reach, kept first tokens, shared latent rows, where the
routing weight enters an expert)."""
import json
import math

import pytest
import torch

from oracle import ludazen_oracle as O
from tests.test_ludazen_gpu import CONFIGS
from vila_b200.model.ludazen import LudazenConfig, LudazenForCausalLM, RotaryConfig
from vila_b200.model.registry import LANGUAGE_MODELS, language_model_architecture

F64 = torch.float64


def random_weights(cfg_dict, seed=0):
    g = torch.Generator().manual_seed(seed)
    shapes = LudazenConfig.from_dict(cfg_dict).tensor_shapes()
    return {n: (torch.randn(s, generator=g) * (0.1 if len(s) == 1 else 1.5 / s[-1] ** 0.5)).to(torch.bfloat16)
            for n, s in shapes.items()}


@pytest.mark.parametrize("name", list(CONFIGS))
def test_config_round_trip_shapes_and_cache_geometry(name):
    d = CONFIGS[name]
    cfg = LudazenConfig.from_dict(d)
    assert cfg.to_dict() == json.loads(json.dumps(d))
    shapes = cfg.tensor_shapes()
    model = LudazenForCausalLM(cfg, "cpu")
    rows = model.latent_widths()
    for i, spec in enumerate(d["layers"]):
        m, mlp = spec["mixer"], spec["mlp"]
        assert (f"l{i}.norm2" in shapes) == (mlp is not None)
        if spec["type"] == "attention":
            assert shapes[f"l{i}.mix.talk"] == (m["heads"], m["heads"]) and shapes[f"l{i}.mix.temp"] == (m["heads"],)
            assert rows[i] == m["kv_heads"] * (m["dim"] + m["vdim"])
        else:
            own = "kv_from" not in m
            assert (f"l{i}.mix.dkv" in shapes) == own and (i in rows) == own
            assert shapes[f"l{i}.mix.q"] == (m["heads"] * (m["dim"] + m["rot_dim"]), d["width"])
            if own:
                assert rows[i] == m["kv_rank"] + m["rot_dim"]
        if mlp and mlp["kind"] == "moe":
            assert (f"l{i}.mlp.shared.gate" in shapes) == ("shared" in mlp)
            assert f"l{i}.mlp.e{mlp['router']['experts'] - 1}.down" in shapes
            assert f"l{i}.mlp.e{mlp['router']['experts']}.down" not in shapes
        if mlp and mlp["kind"] == "dense":
            assert shapes[f"l{i}.mlp.act"] == (2,) and shapes[f"l{i}.mlp.up.b"] == (mlp["ff"],)
    assert model.state_shapes() == {}


def test_bad_configs_are_refused():
    for change in (lambda d: d["layers"][0].update(type="something_else"),
                   lambda d: d["layers"][1]["mixer"].update(kv_heads=2),             # 3 heads over 2 key heads
                   lambda d: d["layers"][1]["mixer"]["rot"].update(dims=14),         # more than the head has
                   lambda d: d["layers"][0]["mixer"]["rot"].update(dims=4),          # not the rotated part's size
                   lambda d: d["layers"][2]["mixer"].update(kv_from=1),              # not a latent layer
                   lambda d: d["layers"][2]["mixer"].update(kv_from=2),              # itself
                   lambda d: d["layers"][2]["mixer"].update(kv_rank=24),             # another width than its source
                   lambda d: d["layers"][3]["mlp"]["router"].update(top=6),          # more than there are
                   lambda d: d["layers"][1]["mlp"].update(kind="other"),
                   lambda d: d["layers"][1]["mixer"]["mask"].update(size=0)):
        d = json.loads(json.dumps(CONFIGS["odd"]))
        change(d)
        with pytest.raises(ValueError):
            LudazenConfig.from_dict(d)


def test_registry_names_the_architecture(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(CONFIGS["plain"]))
    assert language_model_architecture(tmp_path) == "Ludazen"
    assert LANGUAGE_MODELS["Ludazen"] is LudazenForCausalLM


def test_missing_and_misshapen_tensors_are_refused():
    cfg = LudazenConfig.from_dict(CONFIGS["plain"])
    w = random_weights(CONFIGS["plain"])
    bad = dict(w)
    del bad["l0.mix.temp"]
    with pytest.raises(KeyError):
        LudazenForCausalLM(cfg, "cpu").load_weights(bad)
    bad = dict(w)
    bad["l1.mix.uk"] = bad["l1.mix.uk"][:, :-1]
    with pytest.raises(ValueError):
        LudazenForCausalLM(cfg, "cpu").load_weights(bad)


def test_frequency_table():
    """plain: powers of the base; rescaled: fast pairs kept, slow pairs divided, a ramp between; the product
    and the oracle agree to the last bits"""
    plain = RotaryConfig.from_dict({"base": 100.0, "dims": 8})
    assert plain.frequencies() == [100.0 ** (-2.0 * i / 8) for i in range(4)] and plain.magnitude == 1.0
    rd = {"base": 10000.0, "dims": 32, "scaling": {"factor": 4.0, "original": 128, "fast": 16.0, "slow": 1.0}}
    rc = RotaryConfig.from_dict(rd)
    f, f0 = rc.frequencies(), [10000.0 ** (-2.0 * i / 32) for i in range(16)]
    assert f[0] == f0[0] and f[15] == f0[15] / 4.0
    ratio = [a / b for a, b in zip(f, f0)]
    assert all(x >= y for x, y in zip(ratio, ratio[1:])) and 0.25 < ratio[4] < 1.0   # monotone ramp, strictly inside somewhere
    assert torch.allclose(torch.tensor(f, dtype=F64), O.rotary_frequencies(rd), rtol=1e-15)
    assert rc.magnitude == pytest.approx(0.1 * math.log(4.0) + 1.0) and rc.magnitude == O.rotary_magnitude(rd)
    assert rc.to_dict() == rd


def test_rotation_layouts_of_the_oracle():
    """both layouts keep the length of every pair, leave the columns past rot.dims alone, and make scores depend
    on the distance only; position 0 is the identity"""
    rd = {"base": 50.0, "dims": 6}
    v = torch.randn(9, 2, 10, dtype=F64, generator=torch.Generator().manual_seed(1))
    for layout, pairs in (("halves", [(0, 3), (1, 4), (2, 5)]), ("pairs", [(0, 1), (2, 3), (4, 5)])):
        r = O.rotate(v, rd, layout)
        assert torch.equal(r[0], v[0]) and torch.equal(r[..., 6:], v[..., 6:])
        for a, b in pairs:
            assert torch.allclose(r[..., a] ** 2 + r[..., b] ** 2, v[..., a] ** 2 + v[..., b] ** 2)
        same = v[:1].expand(9, 2, 10).contiguous()      # the same vector at every position
        r = O.rotate(same, rd, layout)
        d1, d2 = (r[2, 0, :6] * r[5, 0, :6]).sum(), (r[4, 0, :6] * r[7, 0, :6]).sum()
        assert torch.allclose(d1, d2)
    assert not torch.allclose(O.rotate(v, rd, "halves"), O.rotate(v, rd, "pairs"))


def test_window_mask_reach():
    m = O.window_mask(12, 4, 2)
    assert m[9].nonzero().flatten().tolist() == [0, 1, 6, 7, 8, 9]
    assert m[3].nonzero().flatten().tolist() == [0, 1, 2, 3] and m[0].nonzero().flatten().tolist() == [0]
    assert O.window_mask(5, 1)[4].nonzero().flatten().tolist() == [4]


def test_oracle_window_kept_tokens_and_future():
    """changing a token changes the logits of exactly the positions whose masks (through all layers) can reach it"""
    d = {"architecture": "Ludazen", "norm": {"eps": 1e-6}, "vocab": 31, "width": 24, "layers": [
        {"type": "attention", "mlp": None, "mixer": dict(heads=2, kv_heads=1, dim=6, vdim=6, scale=0.4, rot={"base": 100.0, "dims": 4},
                                                        mask={"size": 3, "keep_first": 2})}]}
    W = random_weights(d, 3)
    toks = list(range(3, 23))
    base = O.forward(d, W, toks)
    for j, reach in ((1, set(range(1, 20))), (5, {5, 6, 7}), (19, {19})):
        t2 = list(toks)
        t2[j] = 30
        diff = (O.forward(d, W, t2) - base).abs().amax(-1)
        assert {i for i in range(20) if diff[i] > 1e-12} == reach, j


def test_oracle_shared_latent_rows_and_expert_input_weight():
    d = CONFIGS["odd"]
    W = {k: v.to(F64) for k, v in random_weights(d, 4).items()}
    h = torch.randn(7, d["width"], dtype=F64, generator=torch.Generator().manual_seed(2))
    m0, m2 = d["layers"][0]["mixer"], d["layers"][2]["mixer"]
    c, kr = O.latent_rows(W, "l0.mix.", h, m0, 1e-6)
    assert c.shape == (7, m0["kv_rank"]) and kr.shape == (7, m0["rot_dim"])
    assert torch.allclose(kr[0], (h @ W["l0.mix.dkv"].T)[0, m0["kv_rank"]:])       # position 0 is not turned
    # the borrowing layer works from those rows with its own expansions
    assert O.latent_attention(W, "l2.mix.", h, m2, c, kr).shape == (7, d["width"])
    # one expert, weight w on the input: expert(w h), which is not w expert(h)
    mlp = {"router": {"top": 1}}
    W1 = {"router": torch.zeros(1, 5, dtype=F64), "e0.gate": torch.randn(4, 5, dtype=F64), "e0.up": torch.randn(4, 5, dtype=F64),
          "e0.down": torch.randn(5, 4, dtype=F64)}
    x = torch.randn(3, 5, dtype=F64)
    out = O.expert_ff(W1, "", x, mlp)                   # sigmoid(0) = 1/2 for every token
    assert torch.allclose(out, O.gated_unit(W1, "e0.", 0.5 * x))
    assert not torch.allclose(out, 0.5 * O.gated_unit(W1, "e0.", x))
    # the two-sided activation is continuous with slope 1/2 at 0 and quadratic above
    z = torch.tensor([-1e-9, 0.0, 1e-9, 2.0], dtype=F64)
    a = O.xielu(z, 0.3, -0.2)
    assert abs(float(a[0])) < 1e-8 and float(a[1]) == 0.0 and abs(float(a[2])) < 1e-8
    assert float(a[3]) == pytest.approx(math.log1p(math.exp(0.3)) * 4.0 + 1.0)
