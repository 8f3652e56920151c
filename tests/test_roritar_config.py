"""Roritar without a GPU: configuration, plan and schedule, what the cache is asked for, and the plain implementation's
own mechanisms against closed forms."""
import copy

import numpy as np
import pytest

import plain_roritar as pr
import roritar_helpers as rh
import questwend_b200  # noqa: F401
from questwend_b200.cache.manager import CacheManager, group_pages_for
from questwend_b200.config import ConfigError
from questwend_b200.config.registry import config_from_dict, get_architecture
from questwend_b200.parts.base import KVSpec


def test_config_reads_every_size_and_round_trips():
    cfg = config_from_dict(rh.MIXED)
    assert cfg.architecture == "Roritar" and cfg.width == 64 and cfg.vocab == 96 and cfg.loop == (1, 4, 3)
    assert cfg.layers[0]["mixer"]["mask"] == {"size": 20, "pool": 5} and cfg.layers[2]["mlp"] is None
    assert cfg.logit_scale == 1.5 and cfg.logit_softcap == 9.0
    assert config_from_dict(cfg.to_dict()) == cfg
    ones = config_from_dict(rh.ONES)
    assert ones.logit_scale == 1.0 and ones.logit_softcap == 0.0 and ones.layers[2]["mixer"]["mask"] is None


def test_schedule_repeats_the_looped_run():
    assert config_from_dict(rh.MIXED).schedule() == [0, 1, 2, 3, 1, 2, 3, 1, 2, 3, 4]
    assert config_from_dict(rh.ONES).schedule() == [0, 1, 2, 3]
    assert pr.schedule(rh.MIXED) == config_from_dict(rh.MIXED).schedule()
    no_loop = copy.deepcopy(rh.MIXED)
    del no_loop["loop"]
    assert config_from_dict(no_loop).schedule() == [0, 1, 2, 3, 4]
    plan = get_architecture("Roritar").plan(config_from_dict(rh.MIXED))
    assert [r.layer for r in plan.schedule] == [0, 1, 2, 3, 1, 2, 3, 1, 2, 3, 4]


@pytest.mark.parametrize("path, value, word", [
    (("layers", 0, "type"), "conv", "'type'"), (("layers", 1, "mixer", "blocks"), 5, "'width'"),
    (("layers", 0, "mixer", "kv_heads"), 3, "'heads'"), (("layers", 0, "mixer", "rot", "dims"), 7, "'dims'"),
    (("layers", 0, "mixer", "rot", "dims"), 32, "'dims'"), (("layers", 0, "mixer", "dim"), 20, "key sizes"),
    (("layers", 0, "mixer", "vdim"), 264, "value sizes"), (("layers", 1, "mixer", "conv"), 17, "taps"),
    (("loop", "stop"), 6, "loop"), (("layers", 0, "mlp", "kind"), "moe", "'kind'"), (("logit_softcap",), -1.0, "logit_softcap"),
    (("layers", 0, "mixer", "rot", "layout"), "spiral", "'layout'")])
def test_config_refuses_with_the_keys_name(path, value, word):
    bad = copy.deepcopy(rh.MIXED)
    at = bad
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        config_from_dict(bad)
    assert word in str(e.value)


def test_manifest_names_and_shapes():
    plan = get_architecture("Roritar").plan(config_from_dict(rh.MIXED))
    shapes = {t.name: tuple(t.shape) for t in plan.manifest() if not t.ignored}
    w = rh.draw_weights(rh.MIXED)
    assert shapes == {k: v.shape for k, v in w.items()}
    assert shapes["l1.mix.ra"] == (3, 16, 16) and shapes["l0.mix.v"] == (2 * 16, 64) and shapes["l0.mix.o"] == (64, 4 * 16)
    assert "l2.norm2" not in shapes and shapes["l0.mlp.act"] == (2,)


def test_cache_rows_per_block_and_values_of_another_size():
    import torch
    tokens, blocks = KVSpec(2, 24, 20, value_dim=16), KVSpec(2, 24, 20, value_dim=16, stride=5)
    assert group_pages_for(blocks, 319) == 1 and group_pages_for(blocks, 320) == 1 and group_pages_for(blocks, 325) == 2
    cache = CacheManager([((tokens, blocks), None, None), (tokens, None, None)], 640, 4, 640, torch.float32, "cpu")
    assert cache.n_groups() == 2
    unit = cache.unit_cache(0)
    assert unit.k_pool.shape[1:] == (2, 64, 24) and unit.v_pool.shape[1:] == (2, 64, 16)
    assert len(unit.more) == 1 and unit.more[0].group_id != unit.group_id and unit.more[0].v_pool.shape[1:] == (2, 64, 16)
    assert cache.unit_cache(1).group_id == unit.group_id and cache.unit_cache(1).more == ()
    (s,) = cache.open(1)
    cache.reserve({s: 100})
    assert [len(g.pages[s]) for g in cache._groups] == [2, 1]          # 100 tokens, 20 complete blocks
    cache.advance(s, 100)
    assert cache.room(s) == 28                                         # the tokens' second page ends at 128
    cache.reserve({s: 330})
    assert [len(g.pages[s]) for g in cache._groups] == [6, 2]          # 66 blocks need a second page
    cache.close([s])
    assert cache.free_pages() == [g.pool.n for g in cache._groups]


def test_plain_scan_against_closed_form():
    rng = np.random.default_rng(0)
    T, C = 9, 5
    u, r, i = rng.standard_normal((T, C)), rng.uniform(size=(T, C)), rng.uniform(size=(T, C))
    lam = rng.standard_normal(C)
    S = pr.rglru_scan(u, r, i, lam)
    a = np.exp(-8.0 * r * np.log1p(np.exp(lam))[None])
    for t in range(T):
        want = sum(np.prod(a[s + 1:t + 1], axis=0) * np.sqrt(1 - a[s] ** 2) * i[s] * u[s] for s in range(t + 1))
        assert np.allclose(S[t], want, rtol=1e-12)


def test_plain_visibility():
    assert pr.visible(0, 4, 2) == (0, 0) and pr.visible(3, 4, 2) == (0, 0) and pr.visible(4, 4, 2) == (1, 0)
    assert pr.visible(5, 4, 2) == (2, 1) and pr.visible(6, 4, 2) == (3, 1) and pr.visible(7, 4, 2) == (4, 2)
    assert pr.visible(9, 3, 0) == (7, 0) and pr.visible(9, 1, 1) == (9, 9)


def test_plain_turn_is_undone_and_relative():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((6, 2, 8))
    pos = np.arange(3, 9)
    for layout in ("halves", "interleaved"):
        y = pr.turn(x, pos, 100.0, 8, layout)
        assert np.allclose(pr.turn(y, pos, 100.0, 8, layout, sign=-1.0), x)
        assert np.allclose(pr.turn(x, pos, 100.0, 4, layout)[..., 4:], x[..., 4:])
    a, b = rng.standard_normal((1, 1, 8)), rng.standard_normal((1, 1, 8))
    d1 = (pr.turn(a, [7], 50.0, 8) * pr.turn(b, [4], 50.0, 8)).sum()
    d2 = (pr.turn(a, [13], 50.0, 8) * pr.turn(b, [10], 50.0, 8)).sum()
    assert abs(d1 - d2) < 1e-12


def test_plain_activation_branches():
    z = np.array([-2.0, 0.0, 3.0])
    out = pr.xielu(z, 0.3, -0.2)
    sp = lambda v: np.log1p(np.exp(v))
    assert np.allclose(out, [(0.5 + sp(-0.2)) * (np.exp(-2.0) - 1 + 2.0) - 1.0, 0.0, sp(0.3) * 9 + 1.5])


def test_info_counts_rows_per_run_and_per_block(tmp_path, capsys):
    import json
    from questwend_b200 import cli
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(rh.MIXED))
    assert cli.main(["--random", str(cfg), "--info"]) == 0
    info = json.loads(capsys.readouterr().out)
    assert info["config"]["architecture"] == "Roritar" and info["layers"] == 5
    # per token: keys and values of every attention RUN (the looped layer counts three times), plus a block row's share
    want = 2 * (24 + 16) * 2 * (1 + 1 / 5) + 3 * 3 * (16 + 40) * 2 * (1 + 1 / 12) + 1 * (8 + 8) * 2 * (1 + 1 / 7)
    assert abs(info["memory"]["cache_bytes_per_token"] - want) < 0.1
    # per sequence: convolution tails and states of every recurrent run
    assert info["memory"]["state_bytes_per_sequence"] == 4 * 3 * ((4 - 1) * 48 + 48) + 4 * 3 * ((2 - 1) * 80 + 80)
    assert info["parameters"] == sum(v.size for v in rh.draw_weights(rh.MIXED).values())
