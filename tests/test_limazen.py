"""Limazen without a device: configuration, the spec's tensors and parts, and what the cache manager
makes of a chunked mask."""

import json

import pytest
import torch

import layover_b200 as lb
from layover_b200.cache import CacheManager
from layover_b200.config.base import load_config, resolve_architecture
from layover_b200.models import assemble, spec_for_config
from layover_b200.parts.base import PagedKVNeed
from limazen_configs import CONFIGS, config, dense, layer, moe


@pytest.mark.parametrize("name", list(CONFIGS))
def test_config_round_trip_and_registry(name, tmp_path):
    raw = CONFIGS[name]
    cfg = lb.LimazenConfig.from_hf_dict(raw)
    assert lb.LimazenConfig.from_hf_dict(cfg.to_hf_dict()) == cfg
    assert resolve_architecture(raw).config_class is lb.LimazenConfig
    (tmp_path / "config.json").write_text(json.dumps(raw))
    arch, again = load_config(tmp_path)
    assert arch.name == "Limazen" and again == cfg


def test_refusals():
    good = CONFIGS["mixed_kinds"]
    for change, match in [
        (lambda c: c["layers"][0].update(type="conv"), "unknown type"),
        (lambda c: c["layers"][2]["mixer"].pop("scale"), "lacks"),
        (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
        (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=14), "rot"),
        (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot"),
        (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "mask.size"),
        (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "mlp kind"),
        (lambda c: c["layers"][1]["mlp"]["router"].update(top=6), "top"),
        (lambda c: c["layers"][3]["mixer"].update(vdim=24), "same kv_heads and vdim"),
        (lambda c: c.update(logit_softcap=-1.0), "logit_softcap"),
        (lambda c: c.pop("width"), "lacks"),
    ]:
        raw = json.loads(json.dumps(good))
        change(raw)
        with pytest.raises(ValueError, match=match):
            lb.LimazenConfig.from_hf_dict(raw)


def test_the_specs_tensors_have_the_checkpoints_names_and_shapes():
    raw = config(50, 24, [layer(4, 2, 8, 6, 5, 4, 100.0, 2.0, 0.1, True, dense(10)),
                          layer(4, 2, 8, 6, 5, 8, 100.0, None, 0.1, True, moe(2, 1, 12, shared=14)),
                          layer(2, 1, 4, 10, 9, 2, 100.0, None, 0.1, False, None)], cap=9.0)
    spec = spec_for_config(lb.LimazenConfig.from_hf_dict(raw))
    specs = {s.name: tuple(s.shape) for s in spec.tensor_specs()}
    want = {"embed": (50, 24), "head": (50, 24), "final.norm": (24,), "final.norm.b": (24,)}
    for i, (heads, kv, d, e) in enumerate([(4, 2, 8, 6), (4, 2, 8, 6), (2, 1, 4, 10)]):
        want.update({f"l{i}.norm1": (24,), f"l{i}.norm1.b": (24,),
                     f"l{i}.mix.q": (heads * d, 24), f"l{i}.mix.q.b": (heads * d,), f"l{i}.mix.k": (kv * d, 24),
                     f"l{i}.mix.k.b": (kv * d,), f"l{i}.mix.v": (kv * e, 24), f"l{i}.mix.v.b": (kv * e,),
                     f"l{i}.mix.g": (heads * e, 24), f"l{i}.mix.o": (24, heads * e)})
    want.update({"l0.mlp.up": (10, 24), "l0.mlp.down": (24, 10), "l1.mix.vmix": (),
                 "l1.mlp.router": (2, 24), "l1.mlp.shared.gate": (14, 24), "l1.mlp.shared.up": (14, 24),
                 "l1.mlp.shared.down": (24, 14), "l1.mlp.shared.sg": (1, 24)})
    for e in range(2):
        want.update({f"l1.mlp.e{e}.gate": (12, 24), f"l1.mlp.e{e}.up": (12, 24), f"l1.mlp.e{e}.down": (24, 12)})
    assert specs == want
    # the blend weight of the layer whose values are kept (and of layers that do not blend) may be stored, and is not read
    assert spec.ignorable_tensors == {"l0.mix.vmix", "l2.mix.vmix"}
    assert spec.logit_softcap == 9.0 and spec.residual_dtype == "float32"
    model = assemble(spec)
    blends = [block.mixer.value_blend for block in model.blocks]
    assert blends == ["keep", "blend", None]
    assert [type(block.feed_forward).__name__ for block in model.blocks] == ["MLP", "RoutedExperts", "NoneType"]
    assert model.blocks[0].mixer.position.rotated == 4 and model.blocks[0].mixer.position.linear_factor == 2.0


def test_a_chunked_mask_gives_back_the_pages_of_finished_chunks():
    raw = CONFIGS["mixed_kinds"]
    model = assemble(spec_for_config(lb.LimazenConfig.from_hf_dict(raw)))
    needs = model.cache_needs()
    assert [need for _, need, _ in needs] == [PagedKVNeed(2, 12, None, 20, 24), PagedKVNeed(1, 24, None, 8, 10),
                                             PagedKVNeed(2, 12, None, 20, 24), PagedKVNeed(2, 8, None, 20, 24)]
    cache = CacheManager(needs, 24, 4, torch.float32, "cpu", max_requests=2)
    assert [g.entries for g in cache.paged] == [[0, 2], [1], [3]]
    seq = cache.open("a")
    for total in range(1, 120):
        cache.grow(seq, total)
        cache.commit(seq, total)
        cache.check()
        for group, table in zip(cache.paged, seq.tables):
            chunk = group.need.chunk
            start = total // chunk * chunk           # the next token's chunk begins here
            assert table.first_live == start // 4
            assert group.allocator.num_used == -(-total // 4) - start // 4 <= chunk // 4 + 2
    # in portions that cross chunk borders: the pages of the portion's first chunk stay until the step is done
    other = cache.open("b")
    cache.grow(other, 23); cache.commit(other, 23)
    cache.grow(other, 23 + 30)
    assert [t.first_live for t in other.tables] == [0, 5, 0]
    cache.commit(other, 53)
    assert [t.first_live for t in other.tables] == [12, 12, 12]
    assert cache.peak_blocks(1, 500, 16) == (10 - 1 + 16) // 4 + 2
    cache.close(seq); cache.close(other); cache.check()


def test_presets_and_random_folders(tmp_path):
    cfg = lb.preset("limazen-tiny")
    assert isinstance(cfg, lb.LimazenConfig)
    folder = lb.write_model_folder(cfg, tmp_path / "m", seed=3)
    arch, again = load_config(folder)
    assert again == cfg
    from safetensors.torch import load_file

    stored = load_file(str(folder / "model.safetensors"))
    assert set(stored) == {s.name for s in spec_for_config(cfg).tensor_specs()}
    assert stored["l1.mix.vmix"].shape == () and float(stored["l1.mix.q.b"].abs().max()) > 0
