"""Reading a Banelix config.json: keys, refusals, lowering to parts and the frequency tables (CPU)."""
import copy
import math

import numpy as np
import pytest

import plain_banelix as PB
from banelix_fixtures import CONFIGS
from infero_b200.config import ConfigError
from infero_b200.config.banelix import BanelixConfig, DECAY_SLOPE
from infero_b200.config.spec import PositionSpec
from infero_b200.models.decoder import DecoderModel
from infero_b200.registry import resolve_architecture


def _spec(raw):
    return BanelixConfig.from_dict(raw).to_model_spec()


def test_the_registry_knows_the_name():
    assert resolve_architecture(CONFIGS["A"]).name == "Banelix"


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_every_size_and_constant_comes_from_the_dictionary(name):
    raw = CONFIGS[name]
    s = _spec(raw)
    assert (s.vocab_size, s.hidden, s.embed_scale) == (raw["vocab"], raw["width"], raw["embedding"]["scale"])
    assert len(s.blocks) == len(raw["layers"]) == len(s.schedule)
    for b, L in zip(s.blocks, raw["layers"]):
        assert b.kind == "prenorm" and b.residual_scale == raw.get("residual_mult", 1.0)
        assert b.mixer_norm.eps == raw["norm"]["eps"]
        assert (b.ffn is None) == (L["mlp"] is None)
        if L["mlp"]:
            assert (b.ffn.kind, b.ffn.intermediate) == ("swiglu", L["mlp"]["ff"])
        m = L["mixer"]
        if L["type"] == "attention":
            x = b.mixer
            assert x.kind == "normed_attention" and x.sink and x.qk_norm_kind == "projection" and not x.value_from_key
            assert (x.num_heads, x.num_kv_heads, x.head_dim, x.v_dim, x.scale, x.window) == (
                m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"], m["mask"]["size"])
            assert x.borrows_cache == ("kv_from" in m)
        else:
            x = b.mixer
            assert x.kind == "parallel" and x.branch_scales == (m["left_scale"], m["right_scale"])
            left, right = x.branches
            assert left.kind == "normed_attention" and left.value_from_key and left.out_gate and not left.sink
            assert left.qk_norm_kind == "head_unit" and left.window is None
            assert (right.kind, right.rec_width, right.rec_blocks, right.conv_taps, right.rec_slope) == (
                "rglru", m["right"]["width"], m["right"]["blocks"], m["right"]["conv"], DECAY_SLOPE)


def test_a_borrowing_layer_reads_the_owners_slot_and_the_cache_keeps_the_longest_window():
    s = _spec(CONFIGS["A"])
    assert (s.schedule[2].cache, s.schedule[2].write_cache) == (s.schedule[0].cache, False)
    assert s.blocks[0].mixer.window == 24 and s.blocks[2].mixer.window == 41
    assert s.blocks[0].mixer.keep_window == s.blocks[2].mixer.keep_window == 41
    model = DecoderModel(s)
    assert model.kv_specs[s.schedule[0].cache].window == 41
    names = {d.name for d in model.declare()}
    assert "l2.mix.q" in names and "l2.mix.q.norm" in names and "l2.mix.q.b" in names
    assert not any(n.startswith("l2.mix.k") or n.startswith("l2.mix.v") for n in names)
    assert {"l1.mix.left.q.b", "l1.mix.left.g", "l1.mix.right.ra.b", "l1.mix.right.conv", "l1.mix.right.lam"} <= names
    assert "l1.mix.left.v" not in names
    assert model.state_specs[s.schedule[1].cache].shape == (4, 64)


def _bad(edit):
    raw = copy.deepcopy(CONFIGS["A"])
    edit(raw)
    return raw


@pytest.mark.parametrize("edit", [
    lambda r: r["layers"][0].update(type="conv"),
    lambda r: r["layers"][0]["mixer"].update(heads=3),
    lambda r: r["layers"][0]["mixer"]["rot"].update(dims=7),
    lambda r: r["layers"][0]["mixer"]["rot"].update(dims=66),
    lambda r: r["layers"][2]["mixer"].update(kv_from=2),
    lambda r: r["layers"][2]["mixer"].update(kv_heads=1),
    lambda r: r["layers"][1]["mixer"]["right"].update(blocks=3),
    lambda r: r["layers"][1]["mixer"]["right"].update(conv=0),
    lambda r: r["layers"][1]["mixer"]["left"].update(vdim=32),
    lambda r: r["layers"][1]["mlp"].update(kind="moe"),
    lambda r: r.update(vocab=0),
    lambda r: r["norm"].pop("eps"),
    lambda r: r.update(layers=[]),
])
def test_refusals(edit):
    with pytest.raises(ConfigError):
        BanelixConfig.from_dict(_bad(edit))


def test_what_a_config_leaves_out_does_not_exist():
    raw = copy.deepcopy(CONFIGS["A"])
    raw["layers"][0]["mixer"].pop("mask")                 # no mask: all earlier tokens
    raw["layers"][1]["mixer"].pop("left_scale")           # a scale of one
    raw["layers"][3]["mixer"]["left"].pop("rot")          # no rotation
    raw["layers"][2]["mixer"]["rot"].update(base=7.0)     # the reader's own queries turn as its own table says
    cfg = BanelixConfig.from_dict(raw)
    assert cfg.layers[0].attention.window is None and cfg.layers[1].left_scale == 1.0 and cfg.layers[3].attention.rot.dims == 0
    spec = cfg.to_model_spec()
    assert spec.blocks[0].mixer.window is None and spec.blocks[0].mixer.keep_window is None      # the borrowed cache keeps all
    assert spec.blocks[2].mixer.window == 41 and spec.blocks[3].mixer.branches[0].position is None
    raw = copy.deepcopy(CONFIGS["A"])
    raw["layers"][2]["mixer"].update(kv_from=1, heads=4, kv_heads=2)     # the keys and values of a parallel layer's attention
    spec = BanelixConfig.from_dict(raw).to_model_spec()
    assert spec.schedule[2].cache == 1 and not spec.schedule[2].write_cache


@pytest.mark.parametrize("dims,base,sc", [(32, 120000.0, (6.0, 1.0, 4.0, 2048)), (16, 900.0, (4.0, 1.0, 3.0, 48)),
                                          (64, 10000.0, (8.0, 1.0, 4.0, 64)), (8, 50.0, (2.0, 0.5, 2.0, 16)), (6, 9.0, None)])
def test_frequencies_scaled_by_bands_of_the_wavelength(dims, base, sc):
    from infero_b200.parts.rope import RopeNeox
    rope = RopeNeox(PositionSpec("rope_neox", base, dims, bands=sc))
    want, amp = PB.frequencies_by_wavelength(dims, base, dict(zip(("factor", "low", "high", "original"), sc)) if sc else None)
    assert rope.amplitude == amp == 1.0
    got = rope.inv_freq64("cpu").numpy()
    assert np.allclose(got, want.numpy(), rtol=1e-14, atol=0)
    if sc and dims >= 16:
        plainf = np.array(PB.base_frequencies(dims, base))
        ratio = got / plainf
        assert ratio.max() == 1.0 and abs(ratio.min() - 1.0 / sc[0]) < 1e-12     # both ends of the scaling are there
        if dims == 32:
            assert ((ratio > 1.0 / sc[0] + 1e-9) & (ratio < 1.0 - 1e-9)).any()   # and the blend between them


@pytest.mark.parametrize("dims,base,sc", [(64, 70000.0, (2.5, 256, 32.0, 1.0)), (64, 5000.0, (4.0, 32, 8.0, 1.0)), (6, 9.0, (3.0, 12, 6.0, 1.0))])
def test_frequencies_scaled_by_a_ramp_over_the_pair_index(dims, base, sc):
    from infero_b200.parts.rope import RopeNeox
    rope = RopeNeox(PositionSpec("rope_neox", base, dims, yarn=sc))
    want, amp = PB.frequencies_by_ramp(dims, base, dict(zip(("factor", "original", "fast", "slow"), sc)))
    assert np.allclose(rope.inv_freq64("cpu").numpy(), want.numpy(), rtol=1e-14, atol=0)
    assert math.isclose(rope.amplitude, amp) and amp > 1.0
