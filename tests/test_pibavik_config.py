"""Reading a Pibavik config.json: what is accepted, what is refused, what the lowering makes of it (no GPU)."""
import copy

import pytest

from infero_b200.config.pibavik import DISTANCE_SLOPE_EXP, PibavikConfig
from infero_b200.config.qwen2 import ConfigError
from infero_b200.registry import resolve_architecture
from pibavik_fixtures import CONFIGS


def _spec(cfg):
    return PibavikConfig.from_dict(cfg).to_model_spec()


def test_the_registry_knows_the_name():
    assert resolve_architecture({"architecture": "Pibavik"}).name == "Pibavik"


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_every_fixture_reads_and_lowers(name):
    cfg = CONFIGS[name]
    spec = _spec(cfg)
    assert spec.vocab_size == cfg["vocab"] and spec.hidden == cfg["width"] and len(spec.blocks) == len(cfg["layers"])
    assert spec.embed_scale == (cfg.get("embedding") or {}).get("scale", 1.0)
    for L, b in zip(cfg["layers"], spec.blocks):
        assert b.kind == "prenorm" and b.mixer_norm.eps == cfg["norm"]["eps"]
        assert (b.ffn is None) == (L["mlp"] is None)
        if b.ffn is not None:
            assert b.ffn.kind == "moe_scored" and b.ffn.weight_input and not b.ffn.route_renorm and b.ffn.route_score == "sigmoid"
            assert (b.ffn.experts, b.ffn.top, b.ffn.intermediate) == (L["mlp"]["router"]["experts"], L["mlp"]["router"]["top"], L["mlp"]["expert"]["ff"])
            assert b.ffn.shared_intermediate == (L["mlp"].get("shared") or {}).get("ff", 0)


def test_the_mixers_of_a_layer_list():
    spec = _spec(CONFIGS["A"])
    par, att, lat, borrow, _ = [b.mixer for b in spec.blocks]
    left, right = par.branches
    assert par.kind == "parallel" and par.branch_scales == (0.7, 1.2)
    assert left.kind == "normed_attention" and left.qk_norm_kind == "head" and left.out_gate and left.window == 24
    assert left.position.rotary_dim == 32 and left.position.theta == 5000.0 and left.distance_slope_exp == 0 and not left.sink
    assert dict(left.names)["q_norm"] == "mix.left.q.norm" and dict(right.names)["a_log"] == "mix.right.A_log"
    assert right.kind == "ssd" and (right.num_heads, right.value_dim, right.state_dim, right.rec_groups, right.conv_taps,
                                    right.norm_groups) == (4, 32, 32, 2, 4, 2)
    assert att.kind == "normed_attention" and att.distance_slope_exp == DISTANCE_SLOPE_EXP and att.position is None
    assert att.qk_norm_kind == "" and not att.qkv_bias and not att.out_gate
    assert lat.kind == "latent_attention" and (lat.latent_dim, lat.q_latent_dim, lat.rot_dim) == (64, 48, 0)
    assert borrow.borrows_cache and borrow.window == 50


def test_a_borrowed_cache_is_a_schedule_entry_and_keeps_the_longest_window():
    spec = _spec(CONFIGS["A"])
    assert [(e.block, e.cache, e.write_cache) for e in spec.schedule] == [(0, 0, True), (1, 1, True), (2, 2, True), (3, 1, False), (4, 4, True)]
    assert spec.blocks[1].mixer.keep_window == 50 and spec.blocks[3].mixer.keep_window == 50
    assert spec.blocks[1].mixer.window == 33
    from infero_b200.models.decoder import DecoderModel
    m = DecoderModel(spec)
    assert m.kv_specs[1].window == 50 and m.kv_specs[0].window == 24 and m.kv_specs[2].window is None
    assert m.kv_specs[2].head_dim == 64 and m.kv_specs[2].value_dim == 0
    assert set(m.state_specs) == {0, 4}
    assert m.state_specs[0].shape == ((4 - 1) * (4 * 32 + 2 * 2 * 32) + 4 * 32 * 32,)


def test_a_left_mixer_without_mask_or_rotation_and_defaults():
    spec = _spec(CONFIGS["C"])
    left = spec.blocks[1].mixer.branches[0]
    assert left.window is None and left.position is None and spec.embed_scale == 1.0
    assert spec.blocks[1].ffn is None and spec.blocks[1].ffn_norm is None


def _bad(path, value, name="A"):
    cfg = copy.deepcopy(CONFIGS[name])
    at = cfg
    for k in path[:-1]:
        at = at[k]
    if value is _DROP:
        at.pop(path[-1])
    else:
        at[path[-1]] = value
    return cfg


_DROP = object()


@pytest.mark.parametrize("path,value", [
    (("vocab",), 0), (("width",), "x"), (("norm",), {}), (("layers",), []),
    (("layers", 0, "type"), "conv"), (("layers", 0, "mixer"), None),
    (("layers", 1, "mixer", "heads"), 3),                       # not a multiple of the kv heads
    (("layers", 1, "mixer", "scale"), _DROP),
    (("layers", 1, "mixer", "mask"), {"size": 0}),
    (("layers", 3, "mixer", "kv_from"), 3),                     # itself
    (("layers", 3, "mixer", "kv_from"), 2),                     # a layer of another kind
    (("layers", 3, "mixer", "dim"), 32),                        # sizes differ from the owner's
    (("layers", 0, "mixer", "left", "rot"), {"base": 100.0, "dims": 7}),
    (("layers", 0, "mixer", "left", "rot"), {"dims": 16}),      # rotated coordinates without a base
    (("layers", 0, "mixer", "right", "groups"), 3),
    (("layers", 0, "mixer", "right", "norm_groups"), 5),
    (("layers", 0, "mixer", "right", "conv"), 17),
    (("layers", 0, "mixer", "right"), _DROP),
    (("layers", 2, "mixer", "q_rank"), _DROP),
    (("layers", 0, "mlp", "kind"), "dense"),
    (("layers", 0, "mlp", "router", "top"), 7),
    (("layers", 0, "mlp", "expert"), _DROP),
])
def test_refusals(path, value):
    with pytest.raises(ConfigError):
        PibavikConfig.from_dict(_bad(path, value))


def test_the_written_config_reads_back():
    cfg = PibavikConfig.from_dict(CONFIGS["B"])
    again = PibavikConfig.from_dict(cfg.to_json_dict())
    assert again.layers == cfg.layers and again.vocab == cfg.vocab and again.embed_scale == cfg.embed_scale
