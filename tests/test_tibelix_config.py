"""Tibelix on the host: configuration reader, model spec, tensor list and cache layout (no GPU)."""
import copy

import pytest

from tibelix_util import TB_A, TB_B, TB_C
from rllm_b200.config.model_config import ConfigError
from rllm_b200.config.registry import resolve_architecture
from rllm_b200.config.tibelix_config import TibelixConfig
from rllm_b200.models.decoder import DecoderModel
from rllm_b200.parts.spec import KVPagesNeed, StateNeed


def build(cfg):
    arch = resolve_architecture(cfg)
    return DecoderModel(arch.build_spec(arch.parse_config(cfg)))


def test_a_layer_that_reads_anothers_keys_uses_that_layers_cache_slot():
    model = build(TB_A)
    assert [r.layer for r in model.spec.order] == [0, 1, 2, 3, 4]
    assert [r.cache for r in model.spec.order] == [0, 1, 2, 1, 4]
    lay = model.layout
    assert lay.run_owner == [0, 1, 2, 1, 4]
    assert lay.groups[0] == StateNeed((3, 20 * 36 + 20 + 1))
    assert lay.groups[1] == KVPagesNeed(2, 24, None, True, 40)
    assert lay.groups[2] == KVPagesNeed(1, 44 + 12, None, values=False)
    assert lay.groups[3] == StateNeed((1, 12 * 8 + 12 + 1))
    assert lay.owners == [[0], [1], [2], [4]]
    b = build(TB_B)
    assert [r.cache for r in b.spec.order] == [0, 1, 2, 3, 0, 3]


def test_the_tensor_list_follows_the_configuration():
    names = {t.name: tuple(t.shape) for t in build(TB_A).tensor_specs()}
    assert names["embed"] == (211, 72) and names["final.norm"] == (72,) and "head" not in names
    for n in ("norm1", "norm1b", "norm2", "norm2b"):
        assert names["l0." + n] == (72,)
    assert "l2.norm2" not in names and "l2.norm2b" not in names and names["l2.norm1b"] == (72,)
    assert names["l0.mix.q"] == (60, 72) and names["l0.mix.v"] == (108, 72) and names["l0.mix.g"] == (108, 72)
    assert names["l0.mix.norm"] == (108,) and names["l0.mix.i"] == (3, 72) and names["l0.mix.f.b"] == (3,)
    assert names["l0.mlp.up"] == (100, 72) and names["l0.mlp.down"] == (72, 100) and "l0.mlp.gate" not in names
    assert names["l1.mix.q"] == (144, 72) and names["l1.mix.k"] == (48, 72) and names["l1.mix.v"] == (80, 72)
    assert names["l1.mix.g"] == (6, 72) and names["l1.mix.o"] == (72, 240) and "l1.mix.sink" not in names
    assert "l1.mix.q.norm" not in names
    assert names["l1.mlp.router"] == (6, 72) and names["l1.mlp.e5.gate"] == (24, 72) and "l1.mlp.e6.gate" not in names
    assert names["l1.mlp.shared.down"] == (72, 40)
    assert names["l2.mix.dq"] == (30, 72) and names["l2.mix.dkv"] == (56, 72) and names["l2.mix.uq"] == (96, 30)
    assert names["l2.mix.uk"] == (60, 44) and names["l2.mix.uv"] == (84, 44) and names["l2.mix.g"] == (84, 72)
    assert names["l2.mix.dkv.norm"] == (44,) and "l2.mix.sink" not in names
    assert "l3.mix.k" not in names and "l3.mix.v" not in names and names["l3.mix.q"] == (144, 72)
    assert names["l3.mix.g"] == (6, 72) and "l3.mlp.shared.gate" not in names and names["l3.mlp.e4.down"] == (72, 20)


def test_constants_reach_the_parts():
    model = build(TB_A)
    att, lat, ml = model.blocks[1].mixer, model.blocks[2].mixer, model.blocks[0].mixer
    assert att.q_temp == (0.7, 7) and att.scale == 0.3 and att.zero_sinks and att.gate == "head"
    assert att.qk_eps == 1e-5 and not att.qk_weights and att.slope_exp == 8.0 and not att.shares_kv
    assert model.blocks[3].mixer.shares_kv and model.blocks[3].mixer.q_temp == (0.2, 3)
    assert lat.position.interleaved and lat.rot_dims == 8 and lat.magnitude > 1.0 and lat.gate == "element"
    assert ml.cap == 6.0 and model.blocks[4].mixer.cap == 2.5
    ffn = model.blocks[1].ffn
    assert (ffn.groups, ffn.keep, ffn.renormalise, ffn.top) == (3, 2, True, 3) and ffn.shared is not None
    assert model.blocks[3].ffn.groups == 0 and model.blocks[3].ffn.shared is None
    assert all(n.unit_offset for b in model.blocks for n in b.norms) and model.final_norm.unit_offset
    assert build(TB_B).blocks[0].mixer.q_temp is None and build(TB_B).blocks[1].mixer.cap == 0.0
    assert build(TB_C).blocks[0].ffn.top == 4


@pytest.mark.parametrize("edit,what", [
    (lambda c: c["layers"][1].__setitem__("type", "attention_9"), "mixer type"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 4), "multiple"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_from", 2), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_from", 3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("dim", 32), "other head counts"),
    (lambda c: c["layers"][2]["mixer"]["rot"].__setitem__("dims", 14), "rot.dims"),
    (lambda c: c["layers"][2]["mixer"].__delitem__("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].__setitem__("count", 4), "groups"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].__setitem__("keep", 1), "groups"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 7), "top"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "sparse"), "kind"),
    (lambda c: c["norm"].__delitem__("eps"), "eps"),
    (lambda c: c.__delitem__("vocab"), "vocab"),
])
def test_what_cannot_be_a_model_is_refused_with_the_reason(edit, what):
    cfg = copy.deepcopy(TB_A)
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        TibelixConfig.from_json(cfg)
    assert what in str(e.value)


def test_a_chain_of_readers_is_refused_and_optional_keys_may_be_absent():
    cfg = copy.deepcopy(TB_B)
    cfg["layers"][5]["mixer"]["kv_from"] = 4          # layer 4 reads layer 0 itself
    with pytest.raises(ConfigError):
        TibelixConfig.from_json(cfg)
    c = TibelixConfig.from_json(TB_B)
    assert c.layers[0].mixer.q_temp is None and c.layers[1].mixer.gate_cap == 0.0
    assert c.layers[2].mixer.rot_scaling is None and c.layers[1].mlp.shared_ff == 64 and c.layers[3].mlp.groups == (4, 4)
