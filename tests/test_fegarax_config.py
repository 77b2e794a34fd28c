"""Fegarax without a GPU: config.json is read into typed fields, optional keys switch mechanisms off, refusals name the
key, the model's tensor list is what a checkpoint of this design holds, and the parts the model is built from carry the
configuration's constants."""
import json
import math

import pytest
import torch

import plain_fegarax as plain
from fegarax_models import CONFIGS, make_model_dir, random_weights


def test_config_is_chosen_by_the_architecture_key_and_round_trips(tmp_path):
    from marin_b200.config import FegaraxConfig, load_config

    cfg = load_config(make_model_dir(str(tmp_path / "a"), "A"))
    assert isinstance(cfg, FegaraxConfig)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.streams, cfg.embedding_scale, cfg.norm_eps) == (97, 64, 2, 3.0, 1e-5)
    assert [layer.mixer["mask"] for layer in cfg.layers] == [{"size": 13}, {"size": 5}, None, {"size": 64}]
    assert [layer.mixer["v_mix"] for layer in cfg.layers] == [False, True, True, True]
    assert cfg.layers[1].mlp is None and cfg.layers[2].mixer["rot"] is None and cfg.layers[1].mixer["rot"]["scaling"] is None
    again = FegaraxConfig.from_dict(json.loads(json.dumps(cfg.to_json_dict())))
    assert again.to_json_dict() == cfg.to_json_dict()
    plain_cfg = load_config(make_model_dir(str(tmp_path / "b"), "B"))
    assert plain_cfg.streams is None and plain_cfg.embedding_scale == 1.0


@pytest.mark.parametrize("damage, word", [
    (lambda c: c["layers"][0].__setitem__("type", "mamba"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_heads"), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("heads", 3), "kv heads"),
    (lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "size"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "dense"), "mlp.kind"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 6), "top"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.__setitem__("streams", 0), "streams"),
    (lambda c: c.__setitem__("width", "wide"), "width"),
])
def test_config_refusals_name_the_key(damage, word):
    from marin_b200.config import ConfigError, FegaraxConfig

    raw = json.loads(json.dumps(CONFIGS["A"]))
    damage(raw)
    with pytest.raises(ConfigError, match=word):
        FegaraxConfig.from_dict(raw)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_the_models_tensor_list_is_the_checkpoints(tmp_path, name):
    from marin_b200.config import load_config
    from marin_b200.engine import build_model
    from marin_b200.weights import WeightError, load_tensors

    d = make_model_dir(str(tmp_path / "m"), name)
    weights = random_weights(CONFIGS[name], 3)
    model = build_model(load_config(d))
    specs = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    assert specs == {k: tuple(v.shape) for k, v in weights.items()}
    assert model.spec.streams == (CONFIGS[name].get("streams") or 0)
    assert model.capturable()
    load_tensors(d, model.tensor_specs(), model.spec.ignorable)
    from fegarax_models import write_model

    damaged = dict(weights)
    damaged.pop("l0.mix.q.b")
    damaged["l0.mix.extra"] = torch.zeros(3, dtype=torch.bfloat16)
    write_model(str(tmp_path / "bad"), CONFIGS[name], damaged)
    with pytest.raises(WeightError) as err:
        load_tensors(str(tmp_path / "bad"), model.tensor_specs(), model.spec.ignorable)
    assert "l0.mix.q.b" in str(err.value) and "l0.mix.extra" in str(err.value)


def test_the_parts_carry_the_configurations_constants():
    from marin_b200.config import FegaraxConfig
    from marin_b200.engine import build_model

    model = build_model(FegaraxConfig.from_dict(CONFIGS["A"]))
    mixers = [b.mixer for b in model.blocks]
    assert [m.chunk for m in mixers] == [13, 5, None, 64]
    assert [(m.value_mix, m.first_of_mix) for m in mixers] == [(None, False), ("v", True), ("v", False), ("v", False)]
    assert all(m.sink and m.gate and m.bias and m.qk_norm == "whole" for m in mixers)
    assert [type(m.position).__name__ for m in mixers] == ["RescaledRotary", "Rotary", "NoPosition", "Rotary"]
    assert [m.position.rotary_dim for m in mixers] == [8, 24, 0, 2]
    assert [type(b).__name__ for b in model.blocks] == ["HyperConnectionBlock"] * 4 and model.blocks[1].feedforward is None
    ffs = [b.feedforward for b in model.blocks if b.feedforward is not None]
    assert [(f.experts, f.top, f.intermediate, f.score, f.weight_on, f.renormalize) for f in ffs] == [
        (5, 2, 40, "sigmoid", "input", False), (3, 3, 24, "sigmoid", "input", False), (7, 3, 16, "sigmoid", "input", False)]
    assert model.embedding.scale == 3.0 and model.head.tied
    # value heads of their own width: each layout is a cache group of its own
    needs = model.cache_needs()
    assert [(n.kv_heads, n.head_dim, n.v_head_dim) for n in needs] == [(2, 16, 24), (1, 24, 40), (1, 16, 40), (1, 32, 40)]
    plain_model = build_model(FegaraxConfig.from_dict(CONFIGS["B"]))
    assert [type(b).__name__ for b in plain_model.blocks] == ["PreNormBlock"] * 2 and plain_model.spec.streams == 0


@pytest.mark.parametrize("rot", [
    {"base": 100.0, "dims": 8, "scaling": {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}},
    {"base": 10000.0, "dims": 32, "scaling": {"factor": 2.0, "original": 4096, "fast": 1.0, "slow": 1.0}},
    {"base": 10000.0, "dims": 16, "scaling": {"factor": 16.0, "original": 64, "fast": 4.0, "slow": 2.0}},
    {"base": 5000.0, "dims": 64, "scaling": {"factor": 8.0, "original": 128, "fast": 16.0, "slow": 2.0}},
    {"base": 7.0, "dims": 6, "scaling": {"factor": 1.5, "original": 1000, "fast": 0.01, "slow": 0.001}},
])
def test_rescaled_frequencies_follow_the_ramp(rot):
    from marin_b200.parts import lookup

    part = lookup("position", "rope_yarn")(head_dim=rot["dims"] + 8, theta=rot["base"], rotary_dim=rot["dims"], **rot["scaling"])
    want, mag = plain.rotary_frequencies(rot)
    got = torch.tensor(part.frequencies(), dtype=torch.float64)
    assert torch.allclose(got, want, rtol=1e-12, atol=0) and abs(part.magnitude - mag) < 1e-15
    assert abs(mag - (0.1 * math.log(rot["scaling"]["factor"]) + 1.0)) < 1e-15
    base = torch.tensor([rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)], dtype=torch.float64)
    ratio = got / base
    assert ((ratio <= 1.0 + 1e-12) & (ratio >= 1.0 / rot["scaling"]["factor"] - 1e-12)).all()


def test_the_plain_routing_and_the_margins():
    g = torch.Generator().manual_seed(1)
    W = {"r.router": torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]])}
    for e in range(3):
        W[f"r.e{e}.gate"], W[f"r.e{e}.up"], W[f"r.e{e}.down"] = torch.randn(4, 2, generator=g), torch.randn(4, 2, generator=g), torch.randn(2, 4, generator=g)
    mlp = {"router": {"experts": 3, "top": 1}}
    h = torch.tensor([[2.0, -1.0], [-1.0, 3.0], [1.0, 1.5]], dtype=torch.float64)
    assert torch.allclose(plain.router_margins(h, W, "r.", mlp), torch.tensor([1.0, 1.0, 1.0], dtype=torch.float64))
    out = plain.routed_experts(h, W, "r.", mlp)
    for t, e in enumerate((0, 1, 2)):
        z = float(h[t] @ W["r.router"][e].double())
        x = h[t] / (1.0 + math.exp(-z))
        gate, up = W[f"r.e{e}.gate"].double() @ x, W[f"r.e{e}.up"].double() @ x
        assert torch.allclose(out[t], W[f"r.e{e}.down"].double() @ (gate * torch.sigmoid(gate) * up))
