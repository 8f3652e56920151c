"""The Movudra configuration, its plan and what the cache makes of it (no GPU)."""
import copy

import numpy as np
import pytest
import torch

import movudra_helpers as mh
import plain_movudra as pmv
import questwend_b200  # noqa: F401
from questwend_b200.cache import CacheManager
from questwend_b200.config import ConfigError, config_from_dict, get_architecture, load_config
from questwend_b200.config.movudra import DEFAULT_LOW_RANK, MovudraConfig
from questwend_b200.parts.base import KVSpec, StateSpec


def plan_of(cfgd):
    cfg = config_from_dict(cfgd)
    return cfg, get_architecture(cfg.architecture).plan(cfg)


def test_the_architecture_key_names_the_design_and_every_size_is_read():
    cfg, plan = plan_of(mh.MIXED)
    assert isinstance(cfg, MovudraConfig) and (cfg.vocab, cfg.width, cfg.norm_eps) == (96, 64, 1e-5)
    assert [l["type"] for l in cfg.layers] == ["channel_delta", "latent_attention", "mamba2", "latent_attention",
                                               "channel_delta", "mamba2"]
    assert [l.mixer.kind for l in plan.layers] == ["gated_delta_channelwise", "latent_attention", "mamba2",
                                                   "latent_attention", "gated_delta_channelwise", "mamba2"]
    assert [None if l.feed_forward is None else l.feed_forward.kind for l in plan.layers] == [
        "biased_mlp", "routed_experts", None, "routed_experts", "routed_experts", "biased_mlp"]
    lat = plan.layers[3]
    assert (lat.mixer.params["window"], lat.mixer.params["heads"], lat.position.params["rotary_dim"]) == (70, 5, 8)
    assert "factor" not in lat.position.params and plan.layers[1].position.params["factor"] == 8.0
    assert config_from_dict(cfg.to_dict()) == cfg


def test_tensor_names_and_shapes():
    _, plan = plan_of(mh.MIXED)
    shapes = {t.name: tuple(t.shape) for t in plan.manifest()}
    assert shapes["embed"] == (96, 64) and shapes["head"] == (96, 64) and shapes["final.norm"] == (64,)
    assert shapes["l0.mix.q"] == (48, 64) and shapes["l0.mix.v"] == (144, 64) and shapes["l0.mix.v.conv"] == (144, 4)
    assert shapes["l0.mix.a2"] == (96, DEFAULT_LOW_RANK) and shapes["l0.mix.dt_bias"] == (96,) and shapes["l0.mix.norm"] == (24,)
    assert shapes["l0.mlp.up.b"] == (96,) and shapes["l0.mlp.down.b"] == (64,)
    assert shapes["l1.mix.uq"] == (3 * 32, 48) and shapes["l1.mix.dkv"] == (48, 64) and shapes["l1.mix.sink"] == (3,)
    assert shapes["l1.mix.uk"] == (72, 40) and shapes["l1.mix.uv"] == (60, 40)
    assert shapes["l1.mlp.e5.gate"] == (40, 64) and shapes["l1.mlp.router"] == (6, 64) and "l1.mlp.e6.gate" not in shapes
    assert shapes["l2.mix.in"] == (2 * 96 + 2 * 3 * 24 + 6, 64) and shapes["l2.mix.conv"] == (96 + 144, 3)
    assert shapes["l2.mix.norm"] == (96,) and "l2.norm2" not in shapes and "l2.norm1" in shapes


def test_low_ranks_come_from_the_tensors_shapes():
    cfg = config_from_dict(mh.MIXED)
    done = cfg.with_tensor_shapes({"l0.mix.a1": (20, 64), "l0.mix.g1": (12, 64), "l4.mix.a1": (4, 64)})
    assert (done.layers[0]["mixer"]["decay_rank"], done.layers[0]["mixer"]["gate_rank"]) == (20, 12)
    assert done.layers[4]["mixer"]["decay_rank"] == 4 and "gate_rank" not in done.layers[4]["mixer"]
    assert "decay_rank" not in cfg.layers[0]["mixer"]                     # the first object is as it was
    plan = get_architecture(done.architecture).plan(done)
    assert {t.name: tuple(t.shape) for t in plan.manifest()}["l0.mix.a2"] == (96, 20)
    assert config_from_dict(done.to_dict()) == done


def test_load_config_reads_the_shapes_of_a_folder(tmp_path):
    sized = copy.deepcopy(mh.ONES)
    sized["layers"][0]["mixer"]["decay_rank"] = 8
    folder = mh.write_folder(str(tmp_path / "m"), mh.ONES, mh.draw_weights(sized, 0))
    cfg = load_config(folder)
    assert cfg.layers[0]["mixer"]["decay_rank"] == 8 and cfg.layers[0]["mixer"]["gate_rank"] == DEFAULT_LOW_RANK


@pytest.mark.parametrize("path,value,word", [
    (("vocab",), None, "vocab"), (("width",), 0, "width"), (("norm", "eps"), -1.0, "eps"), (("layers",), [], "layers"),
    (("layers", 0, "type"), "lstm", "type"), (("layers", 0, "mixer", "heads"), 4, "kv_heads"),
    (("layers", 0, "mixer", "conv"), 17, "conv"), (("layers", 1, "mixer", "rot", "dims"), 7, "dims"),
    (("layers", 1, "mixer", "rot", "dims"), 10, "dims"), (("layers", 1, "mixer", "kv_rank"), 600, "kv_rank"),
    (("layers", 1, "mixer", "scale"), None, "scale"), (("layers", 1, "mlp", "router", "top"), 7, "top"),
    (("layers", 1, "mlp", "kind"), "sparse", "kind"), (("layers", 2, "mixer", "groups"), 4, "groups"),
    (("layers", 2, "mixer", "norm_groups"), 5, "norm_groups"), (("layers", 2, "mixer", "state"), 513, "state"),
    (("layers", 1, "mixer", "rot", "scaling", "factor"), None, "factor")])
def test_a_bad_value_is_refused_with_its_key(path, value, word):
    d = copy.deepcopy(mh.MIXED)
    at = d
    for k in path[:-1]:
        at = at[k]
    if value is None:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        config_from_dict(d)


def test_the_cache_holds_one_row_per_token_and_both_states():
    cfg, plan = plan_of(mh.MIXED)
    from questwend_b200.engine.model import Model
    from questwend_b200.parts.base import Runtime
    model = Model(plan, Runtime(torch.device("cpu"), torch.float32))
    units = model.cache_units()
    assert units[1][0] == KVSpec(1, 48, 5, values=False) and units[3][0] == KVSpec(1, 36, 70, values=False)
    assert units[0][1] == (StateSpec((3, 240), torch.float32), StateSpec((6, 24, 16), torch.float32))
    assert units[5][1] == (StateSpec((0, 112), torch.float32), StateSpec((2, 40, 16), torch.float32))
    cache = CacheManager(units, 256, 3, 256, torch.float32, "cpu")
    assert cache.n_groups() == 2
    u1, u0 = cache.unit_cache(1), cache.unit_cache(0)
    assert u1.v_pool is None and tuple(u1.k_pool.shape) == (4, 1, 64, 48)
    assert isinstance(u0.state, tuple) and tuple(u0.state[1].shape) == (3, 6, 24, 16)
    a, b = cache.open(2)
    u0.state[0][b].fill_(3.0)
    u0.state[1][b].fill_(5.0)
    cache.close([b])
    (again,) = cache.open(1)
    assert again == b and float(u0.state[0][b].abs().sum()) == 0.0 and float(u0.state[1][b].abs().sum()) == 0.0


def test_the_plain_implementation_cut_anywhere_is_itself():
    """The plain functions are causal: a prefix's rows do not depend on what follows (what a cache must reproduce)."""
    w = mh.draw_weights(mh.ONES, 3)
    tokens = np.random.default_rng(0).integers(0, 32, 20).tolist()
    whole = pmv.forward(mh.ONES, w, tokens)
    assert np.allclose(pmv.forward(mh.ONES, w, tokens[:7]), whole[:7], rtol=0, atol=1e-9)


def test_the_benchmark_s_sizes_are_configurations():
    """``bench.py --model movudra`` builds these two: both must parse, and the Movudra one within the kernels' limits."""
    import bench
    cfg, plan = plan_of(bench.movudra_sizes())
    assert len(plan.layers) == 6 and [l["type"] for l in cfg.layers[:3]] == ["channel_delta", "latent_attention", "mamba2"]
    assert sum(int(np.prod(t.shape)) for t in plan.manifest()) > 2e9
    small = bench.movudra_sizes(width=1024, repeats=1, window=128, vocab=1000)
    assert config_from_dict(small).layers[1]["mixer"]["mask"]["size"] == 128
    beside = config_from_dict(bench.qwen3_beside())
    assert (beside.hidden_size, beside.num_hidden_layers, beside.vocab_size) == (2048, 6, 32768)
