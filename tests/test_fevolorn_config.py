"""Fevolorn on the host: configuration reader, model spec, tensor list and cache layout (no GPU)."""
import copy

import pytest

from fevolorn_util import FV_A, FV_B, FV_C
from rllm_b200.config.fevolorn_config import FevolornConfig
from rllm_b200.config.model_config import ConfigError
from rllm_b200.config.registry import resolve_architecture
from rllm_b200.models.decoder import DecoderModel
from rllm_b200.parts.spec import KVPagesNeed, StateNeed


def build(cfg):
    arch = resolve_architecture(cfg)
    return DecoderModel(arch.build_spec(arch.parse_config(cfg)))


def test_the_order_repeats_a_range_of_layers_and_every_run_owns_its_slot():
    cfg = FevolornConfig.from_json(FV_A)
    assert cfg.order() == (0, 1, 2, 1, 2, 1, 2, 3)
    model = build(FV_A)
    assert [r.layer for r in model.spec.order] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [r.cache for r in model.spec.order] == list(range(8))
    assert model.spec.streams == 3
    assert FevolornConfig.from_json(FV_B).order() == (0, 1, 2) and build(FV_B).spec.streams == 1
    assert FevolornConfig.from_json(FV_C).order() == (0, 1, 0, 1)


def test_a_parallel_mixer_keeps_pages_and_two_states():
    lay = build(FV_A).layout
    assert lay.groups[0] == KVPagesNeed(2, 24, 11, True, 40)
    assert lay.groups[1:3] == [StateNeed((10, 56)), StateNeed((2, 56))]
    assert lay.run_group[0] == (0, 1, 2) and lay.owners[0] == [(0, 0)] and lay.owners[2] == [(0, 2)]
    # the repeated lightning layers: one group each, three owners each
    g1, g2 = lay.run_group[1], lay.run_group[2]
    assert lay.groups[g1] == StateNeed((3, 20, 24)) and lay.owners[g1] == [1, 3, 5]
    assert lay.groups[g2] == StateNeed((2, 16, 48)) and lay.owners[g2] == [2, 4, 6]
    # keys and values of one size: no size of its own for the values
    assert KVPagesNeed(4, 16, 37) in lay.groups
    # keys and values of two sizes, the larger a size of the tensor-core kernels: rows of that size for both
    assert KVPagesNeed(2, 64, 5) in build(FV_B).layout.groups and KVPagesNeed(1, 64, 64) in build(FV_B).layout.groups
    # a convolution of one tap keeps an empty tail
    assert StateNeed((0, 128)) in build(FV_B).layout.groups
    assert all(isinstance(g, StateNeed) for g in build(FV_C).layout.groups)


def test_the_tensor_list_follows_the_configuration():
    names = {t.name: tuple(t.shape) for t in build(FV_A).tensor_specs()}
    assert names["embed"] == (203, 72) and names["final.norm.alpha"] == () and names["final.norm.b"] == (72,)
    assert names["l0.mix.left.q"] == (6 * 24, 72) and names["l0.mix.left.v"] == (2 * 40, 72)
    assert names["l0.mix.left.o"] == (72, 6 * 40) and names["l0.mix.left.q.norm"] == (24,)
    assert names["l0.mix.right.x"] == (5 + 2 * 10, 56) and names["l0.mix.right.conv"] == (56, 3)
    assert names["l0.mix.right.A_log"] == (56, 10) and names["l0.mix.left.out"] == (72,)
    assert names["l0.mlp.shared.sg"] == (1, 72) and names["l0.mlp.correction"] == (5,)
    assert names["l0.mlp.e4.down"] == (72, 24) and names["l0.hc2.mix"] == (3, 3) and names["l0.ls2"] == (72,)
    assert names["l1.mix.g"] == (3 * 24, 72) and names["l1.mlp.gate"] == (100, 72)
    assert "l2.norm2" not in names and "l2.hc2.in" not in names and "l2.ls1" in names
    assert "l3.mlp.shared.sg" not in names and "l3.mlp.shared.gate" not in names


@pytest.mark.parametrize("edit,what", [
    (lambda c: c["layers"][1].update(type="window"), "mixer type"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=4), "multiple"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["loop"].update(stop=7), "loop"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("mask"), "mask"),
    (lambda c: c["layers"][1]["mlp"].update(kind="glu"), "kind"),
])
def test_a_configuration_that_cannot_be_a_model_is_refused_with_the_reason(edit, what):
    cfg = copy.deepcopy(FV_A)
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        FevolornConfig.from_json(cfg)
    assert what in str(e.value)
