"""Munupel on the host: configuration reader, model spec, tensor list, cache layout and the
rescaled rotation's frequencies (no GPU)."""
import copy
import math

import pytest

import plain_munupel as pm
from munupel_util import MU_A, MU_B, MU_C
from rllm_b200.config.model_config import ConfigError
from rllm_b200.config.munupel_config import MunupelConfig
from rllm_b200.config.registry import resolve_architecture
from rllm_b200.models.decoder import DecoderModel
from rllm_b200.parts.rotary import rotary_frequencies
from rllm_b200.parts.spec import KVPagesNeed


def build(cfg):
    arch = resolve_architecture(cfg)
    return DecoderModel(arch.build_spec(arch.parse_config(cfg)))


def test_an_entry_that_uses_another_layers_tensors_is_a_second_run_with_its_own_cache():
    model = build(MU_A)
    assert [r.layer for r in model.spec.order] == [0, 1, 1, 2, 3, 2]
    assert [r.cache for r in model.spec.order] == list(range(6))
    lay = model.layout
    assert lay.run_group == [0, 1, 1, 2, 3, 2]
    assert lay.owners == [[0], [1, 2], [3, 5], [4]]
    names = {t.name for t in model.tensor_specs()}
    assert not any(n.startswith("l2.") or n.startswith("l5.") for n in names)
    # a chain of entries ends at the layer that has the tensors
    cfg = copy.deepcopy(MU_A)
    cfg["layers"].append(dict(copy.deepcopy(cfg["layers"][2]), weights_of=2))
    assert MunupelConfig.from_json(cfg).layers[6].weights_of == 1


def test_the_cache_layout_knows_windows_kept_tokens_and_chunks():
    lay = build(MU_A).layout
    assert lay.groups[0] == KVPagesNeed(2, 24, 11, True, 40, keep_first=3)
    assert lay.groups[1] == KVPagesNeed(4, 16, None, True, None, chunk=13)
    assert lay.groups[2] == KVPagesNeed(1, 40, 37, True, 24, keep_first=20)
    b = build(MU_B).layout.groups
    assert b[0] == KVPagesNeed(2, 64, 64, keep_first=1) and b[3] == KVPagesNeed(1, 16, None, True, 48, chunk=1)
    assert b[4] == KVPagesNeed(1, 16, 19)
    assert len(build(MU_C).layout.groups) == 3


def test_the_tensor_list_follows_the_configuration():
    names = {t.name: tuple(t.shape) for t in build(MU_A).tensor_specs()}
    assert names["embed"] == (211, 72) and names["head"] == (211, 72)
    assert names["final.norm"] == (72,) and names["final.norm.b"] == (72,)
    assert names["l0.norm1"] == (72,) and names["l0.norm1.b"] == (72,) and "l0.norm2" not in names
    assert names["l0.mix.q"] == (6 * 24, 72) and names["l0.mix.k"] == (2 * 24, 72) and names["l0.mix.v"] == (2 * 40, 72)
    assert names["l0.mix.o"] == (72, 6 * 40) and names["l0.mix.g"] == (6, 72) and names["l0.mix.sink"] == (6,)
    assert "l0.mix.q.b" not in names and "l0.mix.o.b" not in names
    assert names["l1.mix.g"] == (4 * 16, 72) and names["l1.mix.q.b"] == (64,) and names["l1.mix.v.b"] == (64,)
    assert names["l1.mix.o.b"] == (72,) and "l1.mix.sink" not in names and "l1.mlp.gate" not in names
    assert names["l4.mix.g"] == (3 * 28, 72) and names["l4.mix.k.b"] == (20,) and names["l4.mlp.down"] == (72, 40)
    assert names["l0.mlp.gate"] == (100, 72) and names["l0.mlp.up"] == (100, 72)


@pytest.mark.parametrize("dims,base,scaling", [
    (16, 300.0, (8.0, 64, 16.0, 2.0)), (8, 10000.0, (16.0, 8, 2.0, 0.5)), (64, 1e6, (4.0, 4096, 32.0, 1.0)),
    (2, 3.0, (2.0, 100, 1.0, 1.0)), (32, 10000.0, (1.0, 2048, 8.0, 4.0)), (48, 5e5, None)])
def test_the_rescaled_frequencies_match_the_plain_ones(dims, base, scaling):
    rot = {"dims": dims, "base": base}
    sc = None
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
        sc = dict(rot["scaling"], kind="yarn")
    want, mag = pm.rotation_frequencies(rot)
    got = rotary_frequencies(dims, base, sc)
    assert len(got) == dims // 2
    assert all(math.isclose(a, b, rel_tol=1e-12) for a, b in zip(got, want))
    from rllm_b200.parts.registry import build_part
    from rllm_b200.parts.spec import PartSpec
    part = build_part("position_encoding", PartSpec.of("rotary", head_dim=dims + 8, rotary_dim=dims, theta=base, scaling=sc))
    assert math.isclose(part.magnitude, mag, rel_tol=1e-12)
    if scaling is not None and scaling[0] > 1:
        # the fastest pair keeps its frequency where the ramp starts behind it, the slowest is divided by the factor
        assert got[-1] <= want[-1] and got[0] <= base ** 0


@pytest.mark.parametrize("edit,what", [
    (lambda c: c["layers"][1].update(type="attention_3"), "mixer type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=13), "even"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=26), "at most"),
    (lambda c: c["layers"][0]["mixer"].pop("mask"), "mask"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "positive"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].pop("slow"), "slow"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "kind"),
    (lambda c: c["layers"][2].update(weights_of=2), "no other layer"),
    (lambda c: c["layers"][2].update(weights_of=0), "other sizes"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.pop("width"), "width"),
])
def test_a_configuration_that_cannot_be_a_model_is_refused_with_the_reason(edit, what):
    cfg = copy.deepcopy(MU_A)
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        MunupelConfig.from_json(cfg)
    assert what in str(e.value)


def test_options_that_a_kind_does_not_have_are_not_read():
    """A cap on a windowed layer and kept tokens on a chunked one do not exist."""
    cfg = copy.deepcopy(MU_B)
    cfg["layers"][0]["mixer"]["softcap"] = 3.0
    cfg["layers"][1]["mixer"]["mask"]["keep_first"] = 5
    c = MunupelConfig.from_json(cfg)
    assert c.layers[0].mixer.softcap is None and c.layers[1].mixer.keep_first == 0
    assert c.layers[4].mixer.keep_first == 0 and c.layers[3].mixer.softcap is None
