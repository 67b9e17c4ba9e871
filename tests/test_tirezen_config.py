"""Tirezen's configuration, schedule and tensor names, the parts' bookkeeping that needs no GPU."""

import copy

import pytest
import torch

from yalis_b200.cache.storage import CacheStorage, group_page_bytes, plan_groups
from yalis_b200.config.presets import preset
from yalis_b200.config.registry import ConfigError, architecture_names, load_config, parse_config
from yalis_b200.engine.model import Model
from yalis_b200.ops.recurrent import StateLayout
from yalis_b200.parts.base import PagedKV, PagedKVCache, SlotState, SlotStateCache, cache_leaves, stack_rows

import plain_tirezen as plain
from tirezen_models import tirezen_dir


def test_architecture_is_registered_and_chosen_by_the_config():
    assert "Tirezen" in architecture_names()
    arch, cfg = parse_config(preset("tirezen-tiny-A"))
    assert arch.name == "Tirezen" and cfg.width == 64 and cfg.loop.times == 3


def test_schedule_repeats_the_looped_layers_with_their_additions():
    arch, cfg = parse_config(preset("tirezen-tiny-A"))           # loop over layers 0..1, three times, then layer 2
    spec = arch.model_spec(cfg)
    assert [e.layer for e in spec.schedule] == [0, 1, 0, 1, 0, 1, 2]
    firsts = [(i, e.before.embedding, e.before.row) for i, e in enumerate(spec.schedule) if e.before is not None]
    assert firsts == [(0, False, 0), (2, True, 1), (4, True, 2)]
    assert all(e.cache_of is None for e in spec.schedule)        # every pass keeps its own
    assert [(i, p, f) for i, p, f in plain.layer_order(preset("tirezen-tiny-A"))] == \
        [(0, 0, True), (1, 0, False), (0, 1, True), (1, 1, False), (0, 2, True), (1, 2, False), (2, None, False)]
    arch, cfg = parse_config(preset("tirezen-tiny-B"))
    spec = arch.model_spec(cfg)
    assert [e.layer for e in spec.schedule] == [0, 1, 2] and not spec.extra_tensors


def test_a_layer_without_feed_forward_has_no_such_part_or_tensor():
    arch, cfg = parse_config(preset("tirezen-tiny-A"))
    model = Model(arch.model_spec(cfg))
    assert "feed_forward" not in model.blocks[2].parts
    names = set(model.expected_tensors())
    assert "l2.mlp.up" not in names and "l1.mlp.up" in names and "loop.step" in names
    assert {"l1.mix.left.q.b", "l1.mix.left.k.norm", "l1.mix.right.a2", "l1.mix.right.q.conv", "l2.mix.A_log",
            "l0.mix.g", "final.norm", "head", "embed"} <= names


def test_low_rank_sizes_come_from_the_tensors_of_a_folder():
    d = tirezen_dir("B")
    import json, os
    raw = json.load(open(os.path.join(d, "config.json")))
    assert "decay_rank" not in raw["layers"][1]["mixer"]["right"]
    arch, cfg = load_config(d)
    assert cfg.layers[1]["mixer"]["right"]["decay_rank"] == 5 and cfg.layers[1]["mixer"]["right"]["gate_rank"] == 12
    with pytest.raises(ConfigError, match="decay_rank"):
        parse_config(raw)


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="window"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=18), "rot"),
    (lambda c: c["layers"][0].update(mlp={"kind": "experts", "ff": 8}), "mlp"),
    (lambda c: c.update(loop={"start": 2, "stop": 1, "times": 2}), "loop"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_bad_configurations_are_refused_with_the_key(change, message):
    raw = copy.deepcopy(preset("tirezen-tiny-A"))
    change(raw)
    with pytest.raises(ConfigError, match=message):
        parse_config(raw)


def test_config_round_trip():
    arch, cfg = parse_config(preset("tirezen-tiny-C"))
    again = arch.parse_config(arch.config_to_dict(cfg))
    assert again == cfg


def test_state_layout_and_stacked_rows():
    lay = StateLayout(heads=3, dim=6, vdim=10, conv_channels=66, taps=5)
    assert lay.dim_padded == 8 and lay.state_floats == 3 * 10 * 8 and lay.tail_floats == 66 * 4
    assert lay.total % 4 == 0 and lay.total >= lay.state_floats + lay.tail_floats
    w, spans = stack_rows([torch.ones(5, 3), 2 * torch.ones(9, 3), 3 * torch.ones(2, 3)])
    assert spans == [(0, 5), (8, 17), (24, 26)] and w.shape == (32, 3)
    assert float(w[5:8].abs().sum()) == 0 and float(w[8:17].mean()) == 2


def test_a_mixer_that_keeps_pages_and_a_state_gets_both():
    arch, cfg = parse_config(preset("tirezen-tiny-A"))
    model = Model(arch.model_spec(cfg))
    requests = model.cache_requests()
    assert isinstance(requests[0], SlotState) and isinstance(requests[1], dict)
    leaves = list(cache_leaves(requests[1]))
    assert isinstance(leaves[0], PagedKV) and leaves[0].head_dim == 16 and leaves[0].value_dim == 8
    cache_of = [None] * len(requests)
    assert group_page_bytes(requests, cache_of, 16, 2) == {"kv_all": 3 * 2 * 16 * (16 + 8) * 2}   # three passes keep keys
    groups = plan_groups(requests, 16, 8, 128, 4, 64)
    storage = CacheStorage(requests, cache_of, groups, 4, "cpu", torch.float32)
    entry = storage.entries[1]
    assert isinstance(entry["left"], PagedKVCache) and entry["left"].k.shape == (8, 2, 16, 16) and entry["left"].v.shape == (8, 2, 16, 8)
    assert isinstance(entry["right"], SlotStateCache) and entry["right"].state.shape[0] == 5
    assert storage.entries[3]["left"].k.data_ptr() != entry["left"].k.data_ptr()      # the second pass has its own
    entry["right"].state[2] += 1.0
    storage.reset_slot(2)
    assert float(entry["right"].state[2].abs().sum()) == 0
