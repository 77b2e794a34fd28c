"""Lakulix without a GPU: config.json is read into typed fields, refusals name the key, the model's tensor list is what a
checkpoint of this design holds, sizes that only tensor shapes give are taken from the checkpoint, the loop becomes a
schedule whose every run owns a cache or state, and the distance buckets are what the plain implementation computes."""
import json
import math
import os

import pytest
import torch

import plain_lakulix as plain
from lakulix_models import CONFIGS, make_model_dir, random_weights


def test_config_is_chosen_by_the_architecture_key_and_round_trips(tmp_path):
    from marin_b200.config import ConfigError, LakulixConfig, load_config

    d = make_model_dir(str(tmp_path / "m"), "A")
    cfg = load_config(d)
    assert isinstance(cfg, LakulixConfig)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.max_position_embeddings, cfg.norm_eps, cfg.logit_softcap) == (97, 64, 160, 1e-5, 8.0)
    assert cfg.layer_runs == [0, 1, 2, 1, 2, 1, 2] == plain.layer_runs(CONFIGS["A"][0])
    # sizes that only the checkpoint's shapes give
    assert cfg.layers[0].mixer["bias_rows"] == 10 and cfg.layers[2].mixer["decay_rank"] == 8
    again = LakulixConfig.from_dict(json.loads(json.dumps(cfg.to_json_dict())))
    assert again.to_json_dict() == cfg.to_json_dict()
    no_loop = load_config(make_model_dir(str(tmp_path / "b"), "B"))
    assert no_loop.layer_runs == [0, 1, 2] and no_loop.logit_softcap is None


@pytest.mark.parametrize("damage, word", [
    (lambda c: c["layers"][0].__setitem__("type", "mamba"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_heads"), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("decay", [0.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["q_temp"].__setitem__("every", 0), "every"),
    (lambda c: c["loop"].__setitem__("stop", 9), "loop"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "experts"), "mlp.kind"),
    (lambda c: c.__setitem__("logit_softcap", -1.0), "logit_softcap"),
])
def test_config_refusals_name_the_key(damage, word):
    from marin_b200.config import ConfigError, LakulixConfig

    raw = json.loads(json.dumps(CONFIGS["A"][0]))
    damage(raw)
    with pytest.raises(ConfigError, match=word):
        LakulixConfig.from_dict(raw)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_the_models_tensor_list_is_the_checkpoints(tmp_path, name):
    from marin_b200.config import load_config
    from marin_b200.engine import build_model
    from marin_b200.weights import WeightError, load_tensors

    d = make_model_dir(str(tmp_path / "m"), name)
    raw, shapes = CONFIGS[name]
    weights = random_weights(raw, shapes, 3)
    model = build_model(load_config(d))
    specs = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    assert specs == {k: tuple(v.shape) for k, v in weights.items()}
    tensors = load_tensors(d, model.tensor_specs(), model.spec.ignorable)
    assert tensors["l0.norm1.alpha"].shape == ()
    # every run of a looped layer owns a cache or a state of its own; attention keeps values of their own width
    needs = model.cache_needs()
    assert len(needs) == len(plain.layer_runs(raw)) and all(n is not None for n in needs)
    from marin_b200.parts import PagedKV, StateNeed
    for run, i in enumerate(plain.layer_runs(raw)):
        m = raw["layers"][i]["mixer"]
        if raw["layers"][i]["type"] == "attention":
            assert needs[run] == PagedKV(m["kv_heads"], m["dim"], None, m["vdim"])
        elif raw["layers"][i]["type"] == "lightning":
            assert needs[run] == StateNeed((m["heads"], m["dim"], m["vdim"]), torch.float32)
        else:
            assert needs[run] == StateNeed((m["heads"] * m["dim"] * m["dim"] + raw["width"],), torch.float32)
    # a checkpoint that lacks a tensor is refused with its name
    os.remove(os.path.join(d, "model.safetensors"))
    from safetensors.torch import save_file
    weights.pop("l1.norm1.alpha")
    save_file(weights, os.path.join(d, "model.safetensors"))
    with pytest.raises(WeightError, match="l1.norm1.alpha"):
        load_tensors(d, model.tensor_specs(), model.spec.ignorable)


def test_cache_with_value_heads_of_their_own_width():
    from marin_b200.cache import CacheManager
    from marin_b200.parts import PagedKV

    cache = CacheManager([PagedKV(2, 16, None, 24), PagedKV(2, 16, None)], [None, None], 4, 8, 2)
    assert len(cache.groups) == 2                                 # another value width is another group
    assert cache.bytes_per_page(torch.float32) == 4 * 4 * 2 * (16 + 24) + 4 * 4 * 2 * 32
    cache.allocate("cpu", torch.float32)
    assert cache.groups[0].k.shape == (1, 8, 2, 4, 16) and cache.groups[0].v.shape == (1, 8, 2, 4, 24)


@pytest.mark.parametrize("rows, farthest", [(10, 40), (7, 25.5), (16, 100), (32, 128), (2, 3), (1, 5)])
def test_distance_buckets_agree_with_the_plain_ones_and_saturate(rows, farthest):
    from marin_b200.parts.mixer import distance_bucket

    half = rows // 2
    for n in range(0, int(farthest) + 40):
        got = distance_bucket(n, rows, farthest)
        if half >= 1 and farthest > half:
            assert got == plain.distance_bucket(n, rows, farthest), n
        assert 0 <= got < rows
        if n < half:
            assert got == n
        if n >= farthest:
            assert got == rows - 1
    if half >= 1 and farthest > half:
        seq = [distance_bucket(n, rows, farthest) for n in range(int(farthest) + 3)]
        assert seq == sorted(seq)


def test_random_weights_mode_writes_a_model_the_loader_takes(tmp_path):
    from marin_b200.config import LakulixConfig, load_config
    from marin_b200.engine import build_model
    from marin_b200.weights import load_tensors, write_random_model

    raw = json.loads(json.dumps(CONFIGS["B"][0]))
    raw["layers"][1]["mixer"]["bias_rows"] = 6
    raw["layers"][0]["mixer"]["decay_rank"] = 5
    d = write_random_model(str(tmp_path / "r"), LakulixConfig.from_dict(raw), seed=4)
    cfg = load_config(d)
    model = build_model(cfg)
    tensors = load_tensors(d, model.tensor_specs(), model.spec.ignorable)
    assert tensors["l1.mix.rel"].shape == (6, 2) and tensors["l0.mix.w1"].shape == (5, 96)
    assert tensors["l1.mix.pb"].dtype == torch.float32 and tensors["l0.mix.r"].dtype == torch.bfloat16
