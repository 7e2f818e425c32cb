"""Topidra without a device: configuration, the order of layer runs, the spec's tensors, and what
the cache manager makes of it."""

import json

import pytest
import torch

import layover_b200 as lb
from layover_b200.cache import CacheManager
from layover_b200.config.base import load_config, resolve_architecture
from layover_b200.models import assemble, spec_for_config
from layover_b200.parts.base import PagedKVNeed, StateNeed
from plain_topidra import layer_runs
from topidra_configs import CONFIGS, attention, config, lightning


@pytest.mark.parametrize("name", list(CONFIGS))
def test_config_round_trip_and_registry(name, tmp_path):
    raw = CONFIGS[name]
    cfg = lb.TopidraConfig.from_hf_dict(raw)
    assert lb.TopidraConfig.from_hf_dict(cfg.to_hf_dict()) == cfg
    assert resolve_architecture(raw).config_class is lb.TopidraConfig
    (tmp_path / "config.json").write_text(json.dumps(raw))
    arch, again = load_config(tmp_path)
    assert arch.name == "Topidra" and again == cfg


@pytest.mark.parametrize("name", list(CONFIGS))
def test_layer_runs_follow_the_loop(name):
    raw = CONFIGS[name]
    cfg = lb.TopidraConfig.from_hf_dict(raw)
    assert cfg.layer_runs() == layer_runs(raw)
    spec = spec_for_config(cfg)
    assert [(e.layer, e.adds_embedding) for e in spec.schedule] == layer_runs(raw)
    loop = raw["loop"]
    span = loop["stop"] - loop["start"]
    assert len(spec.schedule) == len(raw["layers"]) + span * (loop["times"] - 1)
    assert sum(e.adds_embedding for e in spec.schedule) == (loop["times"] - 1 if span else 0)


def test_refusals():
    good = CONFIGS["mid_loop"]
    for change, match in [
        (lambda c: c["layers"][0].update(type="conv"), "unknown type"),
        (lambda c: c["layers"][2]["mixer"].pop("scale"), "lacks"),
        (lambda c: c["layers"][2]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
        (lambda c: c["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
        (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "mlp kind"),
        (lambda c: c["loop"].update(stop=9), "does not fit"),
        (lambda c: c.pop("width"), "lacks"),
    ]:
        raw = json.loads(json.dumps(good))
        change(raw)
        with pytest.raises(ValueError, match=match):
            lb.TopidraConfig.from_hf_dict(raw)


def test_the_specs_tensors_have_the_checkpoints_names_and_shapes():
    raw = config(50, 24, [lightning(2, 4, 6, 0.9), attention(4, 2, 8, 12, 5, 0.1, ff=10)])
    specs = {s.name: tuple(s.shape) for s in spec_for_config(lb.TopidraConfig.from_hf_dict(raw)).tensor_specs()}
    assert specs == {
        "embed": (50, 24), "head": (50, 24), "final.norm": (24,),
        "l0.norm1": (24,), "l0.norm1b": (24,),
        "l0.mix.q": (8, 24), "l0.mix.k": (8, 24), "l0.mix.v": (12, 24), "l0.mix.g": (12, 24), "l0.mix.o": (24, 12),
        "l0.mix.norm": (12,),
        "l1.norm1": (24,), "l1.norm1b": (24,), "l1.norm2": (24,), "l1.norm2b": (24,),
        "l1.mix.q": (32, 24), "l1.mix.k": (16, 24), "l1.mix.v": (24, 24), "l1.mix.q.norm": (32,), "l1.mix.k.norm": (16,),
        "l1.mix.sink": (4,), "l1.mix.g": (4, 24), "l1.mix.o": (24, 48),
        "l1.mlp.gate": (10, 24), "l1.mlp.up": (10, 24), "l1.mlp.down": (24, 10),
    }


def test_every_pass_has_a_cache_or_state_of_its_own():
    raw = CONFIGS["mid_loop"]
    model = assemble(spec_for_config(lb.TopidraConfig.from_hf_dict(raw)))
    needs = model.cache_needs()
    assert len(needs) == 10 and all(reads is None for _, _, reads in needs)
    cache = CacheManager(needs, 12, 4, torch.float32, "cpu", max_requests=3)
    # layers 1 and 2 run four times: four state layers and four page layers of their kinds
    by_need = {g.need: g.entries for g in cache.paged + cache.states}
    assert by_need[StateNeed((1, 24, 40), torch.float32)] == [1, 3, 5, 7]
    assert by_need[PagedKVNeed(2, 16, 12, 8)] == [2, 4, 6, 8]
    assert by_need[PagedKVNeed(1, 8, 7, 16)] == [9]
    assert by_need[StateNeed((2, 16, 8), torch.float32)] == [0]
    group = next(g for g in cache.paged if g.need.v_head_dim == 8)
    assert group.pool is None and group.k_store.shape == (4, 13, 2, 4, 16) and group.v_store.shape == (4, 13, 2, 4, 8)
    views = {cache.view(i).state.data_ptr() for i in (1, 3, 5, 7)}
    assert len(views) == 4


def test_windows_give_pages_back_and_slots_are_zeroed_on_reuse():
    raw = CONFIGS["mid_loop"]
    model = assemble(spec_for_config(lb.TopidraConfig.from_hf_dict(raw)))
    cache = CacheManager(model.cache_needs(), 6, 4, torch.float32, "cpu", max_requests=2)
    seq = cache.open("a")
    for total in range(1, 60):
        cache.grow(seq, total)
        cache.commit(seq, total)
        cache.check()
        # windows of 12 and 7 tokens on pages of 4 never hold more than 4 and 3 pages
        assert all(g.allocator.num_used <= (4 if g.need.window == 12 else 3) for g in cache.paged)
    for group in cache.states:
        group.pool[:, seq.slot] = 7.0
    slot = seq.slot
    cache.close(seq)
    again = cache.open("b")
    assert again.slot == slot and all(float(g.pool[:, slot].abs().max()) == 0.0 for g in cache.states)
    cache.check()


def test_presets_and_random_folders(tmp_path):
    cfg = lb.preset("topidra-tiny")
    assert isinstance(cfg, lb.TopidraConfig)
    folder = lb.write_model_folder(cfg, tmp_path / "m", seed=3)
    arch, again = load_config(folder)
    assert again == cfg
    from safetensors.torch import load_file

    stored = load_file(str(folder / "model.safetensors"))
    assert set(stored) == {s.name for s in spec_for_config(cfg).tensor_specs()}
