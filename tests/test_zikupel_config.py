"""The Zikupel configuration reader and model builder on the CPU: what config.json keys mean, what is refused and in
which words, which tensors a model wants, how its cache is laid out, and the random-weights folder."""
import copy
import json

import pytest
import torch

from pico_vllm_b200.errors import ConfigError, WeightError
from pico_vllm_b200.registry import build_model, config_from_dict
from test_zikupel_gpu import SHAPES


def test_round_trip_and_fields():
    for raw in SHAPES.values():
        cfg = config_from_dict(raw)
        assert cfg.architecture == "Zikupel" and config_from_dict(cfg.to_dict()) == cfg
    cfg = config_from_dict(SHAPES["a"])
    assert cfg.vocab_size == 211 and cfg.layers[0].type == "lightning" and cfg.layers[0].mixer.decay == (0.5, 0.9, 0.995)
    assert cfg.layers[0].mlp.shared_ff == 24 and cfg.layers[3].mlp.shared_ff is None and cfg.layers[2].mlp is None
    att = cfg.layers[1].mixer
    assert (att.rot.dims, att.rot.scaling.factor, att.softcap) == (16, 8.0, 6.0) and cfg.layers[2].mixer.rot.scaling is None
    assert cfg.layers[2].mixer.softcap is None
    one = copy.deepcopy(SHAPES["a"])
    one["layers"][0]["mixer"]["decay"] = 0.75                  # a single number stands for all heads
    assert config_from_dict(one).layers[0].mixer.decay == (0.75, 0.75, 0.75)


@pytest.mark.parametrize("edit,word", [
    (lambda r: r["layers"][1].__setitem__("type", "window"), "'type'"),
    (lambda r: r["layers"][1]["mixer"].__setitem__("kv_heads", 3), "multiple"),
    (lambda r: r["layers"][1]["mixer"].__setitem__("vdim", 16), "'vdim'"),
    (lambda r: r["layers"][1]["mixer"]["rot"].__setitem__("dims", 34), "'dims'"),
    (lambda r: r["layers"][1]["mixer"]["rot"].__setitem__("dims", 7), "'dims'"),
    (lambda r: r["layers"][0]["mixer"].__setitem__("decay", [0.5, 0.9]), "'decay'"),
    (lambda r: r["layers"][0]["mlp"]["router"].__setitem__("top", 6), "'top'"),
    (lambda r: r["layers"][0]["mlp"].__setitem__("kind", "sparse"), "'kind'"),
    (lambda r: r["layers"][1]["mixer"].pop("scale"), "'scale'"),
    (lambda r: r.pop("norm"), "norm"),
    (lambda r: r.__setitem__("layers", []), "'layers'"),
])
def test_what_the_reader_refuses(edit, word):
    raw = copy.deepcopy(SHAPES["a"])
    edit(raw)
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw, where="cfg")
    assert word in str(e.value) and str(e.value).startswith("cfg")


def test_tensor_names_and_cache_layout():
    from pico_vllm_b200.cache.manager import CacheManager
    from pico_vllm_b200.weights.loader import wanted_tensors
    model = build_model(config_from_dict(SHAPES["a"]))
    want = wanted_tensors(model)
    assert want["embed"] == (211, 96) and want["head"] == (211, 96) and want["final.norm"] == (96,)
    assert want["l0.mix.q"] == (48, 96) and want["l0.mix.v"] == (72, 96) and want["l0.mix.norm"] == (72,)
    assert want["l0.mlp.router"] == (5, 96) and want["l0.mlp.e4.up"] == (40, 96) and want["l0.mlp.shared.down"] == (96, 24)
    assert "l0.mlp.e0.gate" not in want and "l0.mix.q.b" not in want
    assert want["l1.mix.q"] == (128, 96) and want["l1.mix.k.b"] == (64,) and want["l1.mix.q.norm"] == (32,)
    assert want["l1.mix.g"] == (128, 96) and want["l1.mix.o"] == (96, 128) and "l1.mix.v" not in want
    assert want["l1.mlp.gate"] == (72, 96) and "l2.norm2" not in want and "l3.mlp.shared.up" not in want
    # two attention layers with different heads: two page groups; two linear layers: two state tensors, S transposed
    cm = CacheManager(model.cache_entries, 16, 8, 3, 128, torch.float32, "cpu")
    assert len(cm.groups) == 2 and sorted(cm.states) == [0, 3]
    assert cm.states[0].shape == (3, 3, 24, 16) and cm.states[3].shape == (3, 2, 16, 48) and cm.states[0].dtype == torch.float32
    assert cm.groups[0].tensors["k"].shape == (1, 8, 2, 16, 32) and cm.groups[1].tensors["v"].shape == (1, 8, 2, 16, 64)
    # a head of 24 is kept in rows of 32
    c = build_model(config_from_dict(SHAPES["c"]))
    assert c.cache_entries[0].head_dim == 32 and c.cache_entries[2].head_dim == 48


def test_the_norm_weights_are_stored_around_zero_and_heads_are_padded():
    from pico_vllm_b200.engine.core import _prepare_precision
    from pico_vllm_b200.weights import random_tensors
    from pico_vllm_b200.weights.loader import load_state_dict
    cfg = config_from_dict(SHAPES["c"])
    tensors = random_tensors(cfg, 3, std=0.1, dtype=torch.bfloat16)
    assert abs(float(tensors["l0.norm1"].float().mean())) < 0.1 and abs(float(tensors["l0.mix.q.norm"].float().mean()) - 1) < 0.1
    model = build_model(cfg)
    load_state_dict(model, tensors, torch.float32, "cpu")
    blk = model.blocks[0]
    assert torch.equal(blk.norm1b.weight, tensors["l0.norm1"].float() + 1.0)
    mixer = blk.mixer                                            # 5 heads of 24 in rows of 32
    assert mixer.proj_weight.shape == ((5 + 5 + 5) * 32, 100) and mixer.o_weight.shape == (100, 5 * 32)
    w = mixer.proj_weight.view(15, 32, 100)
    assert float(w[:, 24:].abs().max()) == 0.0 and torch.equal(w[0, :24], tensors["l0.mix.q"].float()[:24])
    assert torch.equal(w[5, :24], tensors["l0.mix.k"].float()[:24]) and torch.equal(w[10, :24], tensors["l0.mix.g"].float()[:24])
    assert float(mixer.o_weight.view(100, 5, 32)[:, :, 24:].abs().max()) == 0.0
    bad = dict(tensors)
    bad.pop("l1.mix.norm")
    bad["l0.mlp.e0.gate"] = torch.zeros(28, 100)
    with pytest.raises(WeightError) as e:
        load_state_dict(build_model(cfg), bad, torch.float32, "cpu")
    assert e.value.missing == ["l1.mix.norm"] and e.value.unexpected == ["l0.mlp.e0.gate"]


def test_stretched_frequencies():
    """The rotary part against the formula written out here: which dimensions keep their frequency, which are divided by
    the factor, and the factor on cos and sin."""
    import math
    from pico_vllm_b200.parts import YarnRotary
    rot = YarnRotary(64, 10000.0, 32, factor=8.0, original=128, fast=16.0, slow=2.0)
    f = rot.frequencies().double()
    plain_f = 10000.0 ** (-2.0 * torch.arange(16, dtype=torch.float64) / 32)
    dim_of = lambda turns: 32 * math.log(128 / (2 * math.pi * turns)) / (2 * math.log(10000.0))
    lo, hi = max(math.floor(dim_of(16.0)), 0), min(math.ceil(dim_of(2.0)), 31)
    assert 0 <= lo < hi < 16
    assert torch.allclose(f[:lo + 1], plain_f[:lo + 1], rtol=1e-6) and torch.allclose(f[hi:], plain_f[hi:] / 8.0, rtol=1e-6)
    mid = (lo + hi) // 2
    ramp = (mid - lo) / (hi - lo)
    assert abs(float(f[mid]) - float(plain_f[mid]) * (ramp / 8.0 + 1 - ramp)) < 1e-6 * float(plain_f[mid])
    assert abs(rot.mult - (0.1 * math.log(8.0) + 1.0)) < 1e-12
    assert YarnRotary(64, 10000.0, 32).mult == 1.0 and torch.allclose(YarnRotary(64, 10000.0, 32).frequencies().double(), plain_f, rtol=1e-6)


def test_random_model_folder(tmp_path):
    from pico_vllm_b200.weights import write_random_model
    folder = write_random_model(config_from_dict(SHAPES["b"]), 4, str(tmp_path / "m"))
    raw = json.load(open(tmp_path / "m" / "config.json"))
    assert raw["architecture"] == "Zikupel" and config_from_dict(raw) == config_from_dict(SHAPES["b"])
