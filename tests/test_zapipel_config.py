"""Host side of the Zapipel design: its config.json reader, the registry, tensor names, cache entries shared
between layers, and the random-weights folder."""
import copy
import json

import pytest
import torch

from pico_vllm_b200.errors import ConfigError, WeightError
from pico_vllm_b200.registry import build_model, config_from_dict
from pico_vllm_b200.weights.loader import check_tensors, wanted_tensors


def _mixer(**over):
    m = dict(heads=3, dim=16, vdim=8, q_rank=24, kv_rank=40, scale=0.3)
    m.update(over)
    return m


RAW = dict(architecture="Zapipel", vocab=100, width=48, norm=dict(eps=1e-5), logit_scale=0.7, logit_softcap=11.0,
           layers=[dict(type="latent_attention", mixer=_mixer(), mlp=dict(kind="dense", ff=64)),
                   dict(type="latent_attention", mixer=_mixer(heads=2, kv_from=0), mlp=None),
                   dict(type="latent_attention", mixer=_mixer(kv_rank=16),
                        mlp=dict(kind="moe", expert=dict(ff=24), router=dict(experts=4, top=2))),
                   dict(type="latent_attention", mixer=_mixer(kv_rank=16, kv_from=2), mlp=dict(kind="dense", ff=32))])


def test_config_round_trip_and_registry():
    cfg = config_from_dict(RAW)
    assert cfg.architecture == "Zapipel" and cfg.vocab_size == 100
    assert config_from_dict(cfg.to_dict()) == cfg
    assert cfg.layers[1].mlp is None and cfg.layers[1].mixer.kv_from == 0
    assert cfg.layers[2].mlp.experts == 4 and cfg.layers[2].mlp.top == 2
    no_cap = {k: v for k, v in RAW.items() if k not in ("logit_softcap", "logit_scale")}
    cfg2 = config_from_dict(no_cap)
    assert cfg2.logit_softcap is None and cfg2.logit_scale == 1.0


@pytest.mark.parametrize("edit,word", [
    (lambda r: r["layers"][1]["mixer"].update(kv_from=1), "earlier"),
    (lambda r: r["layers"][3]["mixer"].update(kv_from=1), "no latents of its own"),
    (lambda r: r["layers"][3]["mixer"].update(kv_rank=24), "differs"),
    (lambda r: r["layers"][0].update(type="window_attention"), "not a mixer"),
    (lambda r: r["layers"][2]["mlp"]["router"].update(top=5), "exceeds"),
    (lambda r: r["layers"][0]["mlp"].update(kind="gelu"), "not a feed-forward"),
    (lambda r: r["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda r: r.pop("norm"), "norm"),
    (lambda r: r.update(layers=[]), "layers"),
])
def test_config_errors_name_the_key(edit, word):
    raw = copy.deepcopy(RAW)
    edit(raw)
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    assert word in str(e.value)


def test_tensor_names_and_shared_cache_entries():
    model = build_model(config_from_dict(RAW))
    want = wanted_tensors(model)
    assert want["embed"] == (100, 48) and want["head"] == (100, 48) and want["final.norm"] == (48,)
    assert want["l0.mix.dkv"] == (40, 48) and want["l0.mix.uk"] == (48, 40) and want["l0.mix.uv"] == (24, 40)
    assert want["l0.mix.g"] == (3, 48) and want["l0.mix.o"] == (48, 24) and want["l0.mix.dq.norm"] == (24,)
    assert "l1.mix.dkv" not in want and "l1.mix.dkv.norm" not in want and "l3.mix.dkv" not in want
    assert "l1.norm2" not in want and "l1.norm2b" not in want and "l1.norm1b" in want
    assert want["l2.mlp.router"] == (4, 48) and want["l2.mlp.router.b"] == (4,) and want["l2.mlp.e3.down"] == (48, 24)
    # two entries: layers 0 and 2 keep latents (rows of 48 and 16 elements), layers 1 and 3 read them
    assert [(c.block, c.cache, c.store) for c in model.order] == [(0, 0, True), (1, 0, False), (2, 1, True), (3, 1, False)]
    assert [s.rank for s in model.cache_entries] == [48, 16]
    have = dict(want)
    have.pop("l2.mlp.router.b")
    have["l1.mix.dkv"] = (40, 48)
    have["head"] = (48, 100)
    with pytest.raises(WeightError) as e:
        check_tensors(model, have, "folder")
    assert e.value.missing == ["l2.mlp.router.b"] and e.value.unexpected == ["l1.mix.dkv"] and e.value.wrong_shape == ["head"]


def test_cache_groups_follow_the_latent_size():
    from pico_vllm_b200.cache.manager import CacheManager
    model = build_model(config_from_dict(RAW))
    cache = CacheManager(model.cache_entries, 8, 6, 2, 48, torch.float32, "cpu")
    assert len(cache.groups) == 2
    views = cache.views()
    assert views[0].tensors["latent"].shape == (6, 1, 8, 48) and views[1].tensors["latent"].shape == (6, 1, 8, 16)
    assert views[0].k is views[0].v is views[0].tensors["latent"]          # one tensor read as keys and as values
    slot = cache.acquire("a")
    cache.append(slot, 20)
    cache.commit(slot)
    assert [g.pool.in_use for g in cache.groups] == [3, 3]
    cache.release(slot)
    cache.check()
    assert [g.pool.in_use for g in cache.groups] == [0, 0]


def test_random_model_folder(tmp_path):
    from pico_vllm_b200.config.base import read_config_json
    from pico_vllm_b200.weights import write_random_model
    from pico_vllm_b200.weights.loader import load_weights
    cfg = config_from_dict(RAW)
    folder = write_random_model(cfg, 3, str(tmp_path / "m"))
    assert config_from_dict(read_config_json(folder)) == cfg
    model = build_model(cfg)
    load_weights(model, folder, torch.bfloat16, "cpu")
    mixer = model.blocks[0].mixer
    assert mixer.down_weight.shape == (80, 48)            # 24 + 40 + 3 rows, padded to a multiple of 16
    assert mixer.uk_weight.shape == (3, 16, 48) and float(mixer.uk_weight[:, :, 40:].abs().max()) == 0.0
    assert mixer.uv_weight.shape == (3, 48, 8) and float(mixer.uv_weight[:, 40:].abs().max()) == 0.0
    assert model.blocks[1].mixer.down_weight.shape == (32, 48)     # no key/value part: 24 + 2 rows
    ff = model.blocks[2].feed_forward
    assert ff.gate_up_weight.shape == (4, 48, 48) and ff.down_weight.shape == (4, 48, 24)
    assert ff.router_weight.dtype == torch.float32 and ff.router_bias.dtype == torch.float32
    assert model.blocks[0].norm1.weight.dtype == torch.float32


def test_a_model_without_positions_is_as_long_as_its_cache():
    """Nothing in this design limits a request's length; the pool the engine is given does."""
    from pico_vllm_b200.config import EngineConfig
    from pico_vllm_b200.engine.core import make_cache, max_model_len
    model = build_model(config_from_dict(RAW))
    cfg = EngineConfig(dtype="float32", page_size=16, max_cache_tokens=8192, device="cpu")
    assert max_model_len(model, cfg) is None
    assert make_cache(model, cfg).max_seq_len == 8192
    assert make_cache(model, EngineConfig(dtype="float32", max_cache_tokens=8192, max_model_len=100, device="cpu")).max_seq_len == 100
