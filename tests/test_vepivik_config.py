"""Vepivik without a GPU: registry, schedule and cache plan, tensor names, rotary frequencies, refused configurations."""

import copy
import math

import pytest
import torch

import plain_vepivik as plain
from yalis_b200.config.presets import preset
from yalis_b200.config.registry import ConfigError, parse_config
from yalis_b200.engine.model import Model
from yalis_b200.parts.base import PagedKV
from yalis_b200.parts.rotary import yarn_frequencies


def spec_of(name):
    arch, cfg = parse_config(preset(name))
    return arch, cfg, arch.model_spec(cfg)


def test_the_registry_knows_the_design_and_round_trips_its_configuration():
    for which in "ABCD":
        raw = preset(f"vepivik-tiny-{which}")
        arch, cfg = parse_config(raw)
        assert arch.name == "Vepivik" and arch.config_to_dict(cfg) == raw


def test_a_layer_that_reads_anothers_rows_is_a_schedule_entry_that_reads_its_cache():
    _, _, spec = spec_of("vepivik-tiny-A")
    assert [e.cache_of for e in spec.schedule] == [None, None, 0, None, None]
    model = Model(spec)
    reqs = model.cache_requests()
    # the rows of layer 0 are kept for the widest window among itself (20) and its reader (33)
    assert reqs[0] == reqs[2] == PagedKV(1, 24 + 8, 33, v_head_dim=0)
    assert reqs[1] == PagedKV(2, 12, 9, v_head_dim=20)
    assert reqs[4] == PagedKV(1, 16 + 6, 11, v_head_dim=0)
    names = set(model.expected_tensors())
    assert "l0.mix.dkv" in names and "l0.mix.dkv.norm" in names and "l2.mix.dkv" not in names and "l2.mix.uk" in names
    assert "l2.norm2" not in names and "l2.mlp.router" not in names            # a layer without feed-forward
    assert "l1.mlp.e5.down" in names and "l3.mlp.shared.up" not in names and "l0.mlp.shared.down" in names
    assert "head" not in names and spec.head_name is None and spec.embedding_scale == 2.5


def test_page_groups_by_how_long_rows_are_kept():
    from yalis_b200.cache.storage import plan_groups
    _, _, spec = spec_of("vepivik-tiny-A")
    groups = {g.name: g for g in plan_groups(Model(spec).cache_requests(), 16, 64, 1024, 4, 64)}
    assert set(groups) == {"kv_window_33", "kv_window_9", "kv_window_16", "kv_window_11"}


@pytest.mark.parametrize("dims, base, factor, original, fast, slow", [(24, 5000.0, 3.0, 1024, 24.0, 1.5), (8, 100.0, 4.0, 32, 8.0, 2.0),
                                                                      (4, 20.0, 3.0, 16, 4.0, 0.5), (32, 500000.0, 40.0, 8192, 32.0, 1.0)])
def test_yarn_frequencies_against_the_plain_ones(dims, base, factor, original, fast, slow):
    rot = {"dims": dims, "base": base, "scaling": {"factor": factor, "original": original, "fast": fast, "slow": slow}}
    want, mag = plain.rotary_frequencies(rot)
    got, got_mag = yarn_frequencies(dims, base, factor, original, fast, slow)
    assert got.dtype == torch.float32 and got_mag == pytest.approx(mag) and mag == pytest.approx(0.1 * math.log(factor) + 1)
    torch.testing.assert_close(got.double(), torch.tensor(want, dtype=torch.float64), rtol=1e-7, atol=0)
    plain_f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    assert want[0] == pytest.approx(plain_f[0]) or factor == 1.0            # the fastest pair keeps its frequency ...
    assert want[-1] <= plain_f[-1]                                             # ... slow pairs are slowed, never sped up


def test_refused_configurations():
    base = preset("vepivik-tiny-A")

    def broken(change):
        raw = copy.deepcopy(base)
        change(raw)
        with pytest.raises(ConfigError):
            parse_config(raw)

    broken(lambda r: r["layers"][2]["mixer"].update(kv_from=4))                       # a later layer
    broken(lambda r: r["layers"][2]["mixer"].update(kv_from=1))                       # not a latent layer
    broken(lambda r: r["layers"][2]["mixer"].update(kv_rank=20))                      # rows of another size
    broken(lambda r: r["layers"][1]["mixer"].update(kv_heads=3))
    broken(lambda r: r["layers"][0]["mlp"]["router"].update(top=9))
    broken(lambda r: r["layers"][0]["mlp"].update(kind="dense"))
    broken(lambda r: r["layers"][0].update(type="retention"))
    broken(lambda r: r["layers"][4]["mixer"]["rot"].update(dims=8))                   # more sizes than the rotated part
    broken(lambda r: r.pop("norm"))
    raw = copy.deepcopy(base)
    raw["layers"][0]["mixer"]["kv_from"] = None                                         # spelled out, still its own
    parse_config(raw)


def test_flops_count_the_experts_a_token_uses():
    _, _, spec = spec_of("vepivik-tiny-C")
    ff = Model(spec).blocks[0].feed_forward
    assert ff.matrix_flops_per_token() == 2.0 * 128 * (16 + 2 * 4 * 32 + 2 * 64)
