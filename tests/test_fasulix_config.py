"""Fasulix on the host: configuration reader, model spec, tensor list and cache layout (no GPU)."""
import copy

import pytest

from fasulix_util import FX_A, FX_B, FX_C, FX_D


def _describe(cfg):
    from rllm_b200.config import resolve_architecture
    from rllm_b200.models.decoder import DecoderModel
    arch = resolve_architecture(cfg)
    spec = arch.build_spec(arch.parse_config(cfg))
    spec.validate()
    return spec, DecoderModel(spec)


def test_the_architecture_is_found_by_its_name_and_every_size_comes_from_the_configuration():
    spec, model = _describe(FX_A)
    assert (spec.hidden_size, spec.vocab_size, len(spec.layers)) == (88, 211, 6)
    shapes = {t.name: t.shape for t in model.tensor_specs()}
    assert shapes["embed"] == (211, 88) and shapes["final.norm"] == (88,)
    assert shapes["l0.mix.dq"] == (40, 88) and shapes["l0.mix.uq"] == (3 * 24, 40)
    assert shapes["l0.mix.dkv"] == (48 + 8, 88) and shapes["l0.mix.uk"] == (3 * 16, 48)
    assert shapes["l0.mix.uv"] == (3 * 24, 48) and shapes["l0.mix.sink"] == (3,) and shapes["l0.mix.o"] == (88, 72)
    assert "l2.mix.sink" not in shapes and "l3.mix.dkv" not in shapes and "l3.mix.dkv.norm" not in shapes
    assert shapes["l1.mix.z"] == (72, 88) and shapes["l1.mix.x.b"] == (72,) and shapes["l1.mix.o"] == (88, 72)
    assert shapes["l1.mlp.router"] == (3, 88) and shapes["l1.mlp.e2.down"] == (88, 40)
    assert "l2.mlp.router" not in shapes and "l2.rg2" not in shapes and "l2.norm2" not in shapes   # no feed-forward
    ignored = [n for part in model.parts() for n in part.ignored_tensors()]
    assert {"l2.rg2", "l2.rg2.b", "l2.norm2", "l2.norm2b", "l3.mix.dkv", "l3.mix.dkv.norm", "l2.mix.sink"} <= set(ignored)
    assert [shapes[f"l{i}.dwa"] for i in range(6)] == [(i + 2,) for i in range(6)]
    assert shapes["l4.rg1"] == (88, 88) and shapes["l4.rg2.b"] == (88,)


def test_cache_layout_rows_are_shared_and_a_shared_slot_keeps_the_widest_window():
    from rllm_b200.parts.spec import KVPagesNeed, StateNeed
    spec, model = _describe(FX_A)
    lay = model.layout
    assert [r.cache for r in spec.order] == [0, 1, 2, 2, 4, 0]
    # layer 5 (window 20) reads the causal layer 0: every key stays.  Layer 3 (window 37) reads layer 2
    # (window 9): the slot keeps 37.
    assert lay.groups[lay.run_group[0]] == KVPagesNeed(1, 56, None, values=False)
    assert lay.run_group[5] == lay.run_group[0] and lay.run_owner[5] == 0
    assert lay.groups[lay.run_group[2]] == KVPagesNeed(1, 56, 37, values=False)
    assert lay.run_group[3] == lay.run_group[2] and lay.run_owner[3] == 2
    assert lay.groups[lay.run_group[1]] == StateNeed((72,)) and lay.groups[lay.run_group[4]] == StateNeed((100,))
    assert model.depth_levels == 7


@pytest.mark.parametrize("breakage,words", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "mixer type"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_from", 3), "earlier layer"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_from", 1), "keeps no rows"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_rank", 32), "must be equal"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 4), "top 4 of 3"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "lacks 'scale'"),
    (lambda c: c.pop("width"), "lacks 'width'"),
])
def test_a_configuration_that_cannot_be_a_model_is_refused_with_the_reason(breakage, words):
    from rllm_b200.config import ConfigError, resolve_architecture
    cfg = copy.deepcopy(FX_A)
    breakage(cfg)
    with pytest.raises(ConfigError, match=words):
        resolve_architecture(cfg).parse_config(cfg)


def test_llama_and_fasulix_are_both_registered():
    from rllm_b200.config import ARCHITECTURES, resolve_architecture
    resolve_architecture(FX_B)
    assert {"Fasulix", "LlamaForCausalLM"} <= set(ARCHITECTURES)


def test_a_model_of_recurrences_only_keeps_no_pages():
    from rllm_b200.parts.spec import StateNeed
    spec, model = _describe(FX_D)
    assert model.layout.groups == [StateNeed((48,)), StateNeed((16,))]
    spec, model = _describe(FX_C)
    assert [type(g).__name__ for g in model.layout.groups] == ["StateNeed", "StateNeed", "KVPagesNeed"]
    assert model.layout.groups[2].head_dim == 26 and model.layout.groups[2].values is False
