"""Typed configuration of the Banelix decoder, read from its own config.json keys.

config.json: ``architecture`` "Banelix", ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` (the embedding is
multiplied by it), ``residual_mult`` (what every sublayer's result is multiplied by as it enters the residual stream)
and ``layers``, one entry per layer: ``type``, ``mixer`` and ``mlp`` (null, or {``kind`` "dense", ``ff``}: a SwiGLU).
Layer i's tensors start with ``l<i>.``.

``type`` "attention": windowed grouped-query attention.  ``mixer``: ``heads``, ``kv_heads``, ``dim``, ``vdim``,
``scale``, ``mask.size`` (a query sees itself and the size - 1 tokens before it), ``rot`` = {``base``, ``dims``,
optionally ``scaling`` = {``factor``, ``original``, ``fast``, ``slow``}: the ramp over the pair index with its
amplitude}, optionally ``kv_from``: j (no key or value tensors; the layer reads layer j's cache).  q, k and v have
biases; q and k are RMS-normed over their whole projection with a weight before the rotation; the softmax has a sink.

``type`` "parallel": two mixers side by side on the same input, ``mixer.left`` and ``mixer.right``, added up with
``left_scale`` and ``right_scale``.  Left: causal grouped-query attention over all keys (``heads``, ``kv_heads``,
``dim``, ``vdim`` = ``dim``, ``scale``, ``rot`` with optional ``scaling`` = {``factor``, ``low``, ``high``,
``original``}: by bands of the wavelength) whose values are the keys as projected, with q and k biases, unit RMS per
head behind the rotation and a sigmoid gate per head on the result.  Right: a gated linear recurrence (``width``
channels, ``blocks`` blocks of gate matrices, ``conv`` taps).

Lowering: blocks "prenorm" with ``residual_scale``; mixers "normed_attention", "rglru" and "parallel"; a layer with
``kv_from`` becomes a schedule entry that reads the other layer's cache slot without writing it, and the cache keeps
the largest window of its readers.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .gositar import _number
from .qwen2 import ConfigError
from .spec import (BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry)
from .vufizen import _pos_int

DECAY_SLOPE = 8.0          # log a = -DECAY_SLOPE * r * softplus(lam); fixed by the design


@dataclass(frozen=True)
class BanelixRot:
    base: float
    dims: int
    scaling: Optional[Tuple[float, float, float, float]] = None     # attention: (factor, original, fast, slow);
                                                                    # left: (factor, low, high, original)


@dataclass(frozen=True)
class BanelixAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: BanelixRot
    window: Optional[int] = None      # None: all keys (the left mixer)
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class BanelixRecurrent:
    width: int
    blocks: int
    conv: int


@dataclass(frozen=True)
class BanelixLayer:
    type: str                         # "attention" | "parallel"
    attention: BanelixAttention       # the mixer itself, or the left one
    recurrent: Optional[BanelixRecurrent] = None
    left_scale: float = 1.0
    right_scale: float = 1.0
    ff: int = 0                       # 0: no feed-forward


def _rot(m: Dict[str, Any], where: str, dim: int, keys: Tuple[str, ...]) -> BanelixRot:
    rot = m.get("rot")
    if rot is None:                                   # no rotation at all
        return BanelixRot(10000.0, 0, None)
    if not isinstance(rot, dict):
        raise ConfigError(f"config.json: {where}.rot is not an object")
    dims = rot.get("dims", dim)
    if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > dim:
        raise ConfigError(f"config.json: {where}.rot.dims {dims!r} must be even and at most dim {dim}")
    base = _number(rot, "base", where + ".rot") if dims else 10000.0
    sc = rot.get("scaling")
    scaling = None
    if sc is not None and dims:
        scaling = tuple(_number(sc, k, where + ".rot.scaling") for k in keys)
        if base == 1.0:
            raise ConfigError(f"config.json: {where}.rot.scaling needs a base other than 1")
    return BanelixRot(base, dims, scaling)


def _attention(m: Dict[str, Any], where: str, windowed: bool) -> BanelixAttention:
    heads, kv = _pos_int(m, "heads", where), _pos_int(m, "kv_heads", where)
    dim, vdim = _pos_int(m, "dim", where), _pos_int(m, "vdim", where)
    if heads % kv:
        raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {kv} kv_heads")
    window, src = None, None
    if windowed:
        if m.get("mask") is not None:                 # no mask key: every earlier token is seen
            window = _pos_int(m["mask"], "size", where + ".mask")
        rot = _rot(m, where, dim, ("factor", "original", "fast", "slow"))
        if m.get("kv_from") is not None:
            src = m["kv_from"]
            if isinstance(src, bool) or not isinstance(src, int) or src < 0:
                raise ConfigError(f"config.json: {where}.kv_from {src!r} must be a layer's index")
    else:
        rot = _rot(m, where, dim, ("factor", "low", "high", "original"))
        if rot.scaling is not None and rot.scaling[1] == rot.scaling[2]:
            raise ConfigError(f"config.json: {where}.rot.scaling: low and high must differ")
        if vdim != dim:
            raise ConfigError(f"config.json: {where}: the values are the keys, so vdim {vdim} must equal dim {dim}")
    return BanelixAttention(heads, kv, dim, vdim, _number(m, "scale", where), rot, window, src)


@dataclass(frozen=True)
class BanelixConfig:
    vocab: int
    width: int
    eps: float
    embed_scale: float
    residual_mult: float
    layers: Tuple[BanelixLayer, ...]
    raw: Tuple[Tuple[str, Any], ...] = ()
    max_positions: int = 1 << 20

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "BanelixConfig":
        vocab, width = _pos_int(raw, "vocab", "config"), _pos_int(raw, "width", "config")
        eps = _number(raw.get("norm") or {}, "eps", "norm")
        embed_scale = _number(raw.get("embedding") or {"scale": 1.0}, "scale", "embedding", positive=False)
        mult = _number(raw, "residual_mult", "config", positive=False) if raw.get("residual_mult") is not None else 1.0
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(entries):
            where = f"layers[{i}]"
            m = L.get("mixer") if isinstance(L, dict) else None
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: {where}.mixer is missing")
            ff = 0
            ml = L.get("mlp")
            if ml is not None:
                if ml.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind {ml.get('kind')!r} is not 'dense'")
                ff = _pos_int(ml, "ff", where + ".mlp")
            if L.get("type") == "attention":
                layers.append(BanelixLayer("attention", _attention(m, where + ".mixer", True), ff=ff))
            elif L.get("type") == "parallel":
                left, right = m.get("left"), m.get("right")
                if not isinstance(left, dict) or not isinstance(right, dict):
                    raise ConfigError(f"config.json: {where}.mixer needs 'left' and 'right'")
                wr = where + ".mixer.right"
                rec = BanelixRecurrent(_pos_int(right, "width", wr), _pos_int(right, "blocks", wr), _pos_int(right, "conv", wr))
                if rec.width % rec.blocks:
                    raise ConfigError(f"config.json: {wr}: {rec.width} channels do not split into {rec.blocks} blocks")
                if rec.conv > 16:
                    raise ConfigError(f"config.json: {wr}: {rec.conv} taps, at most 16")
                layers.append(BanelixLayer("parallel", _attention(left, where + ".mixer.left", False), rec,
                                           _number(m, "left_scale", where + ".mixer", positive=False) if m.get("left_scale") is not None else 1.0,
                                           _number(m, "right_scale", where + ".mixer", positive=False) if m.get("right_scale") is not None else 1.0,
                                           ff))
            else:
                raise ConfigError(f"config.json: {where}.type {L.get('type')!r} is neither 'attention' nor 'parallel'")
        for i, L in enumerate(layers):
            a = L.attention
            if a.kv_from is None:
                continue
            where = f"layers[{i}].mixer.kv_from"
            if a.kv_from >= len(layers) or a.kv_from >= i:
                raise ConfigError(f"config.json: {where} {a.kv_from} must name an earlier layer")
            src = layers[a.kv_from]
            b = src.attention
            if b.kv_from is not None:
                raise ConfigError(f"config.json: {where}: layer {a.kv_from} has no keys and values of its own")
            if (b.kv_heads, b.dim, b.vdim) != (a.kv_heads, a.dim, a.vdim):
                raise ConfigError(f"config.json: {where}: layer {a.kv_from}'s key/value heads and sizes differ")
        return cls(vocab, width, eps, embed_scale, mult, tuple(layers), raw=tuple(raw.items()),
                   max_positions=int(raw.get("max_positions", 1 << 20)))

    def to_json_dict(self) -> Dict[str, Any]:
        keep = ("architecture", "vocab", "width", "norm", "embedding", "residual_mult", "layers", "max_positions")
        return {k: v for k, v in self.raw if k in keep}

    # ---- lowering to parts ---------------------------------------------------------------------
    def to_model_spec(self) -> ModelSpec:
        d = self.width
        norm = NormSpec(kind="rmsnorm", dim=d, eps=self.eps)
        # the cache of a layer keeps the largest window of the layers that read it
        keep = {i: L.attention.window for i, L in enumerate(self.layers) if L.attention.kv_from is None}
        for L in self.layers:
            if L.attention.kv_from is not None:
                mine, theirs = L.attention.window, keep[L.attention.kv_from]
                keep[L.attention.kv_from] = None if mine is None or theirs is None else max(mine, theirs)
        blocks, schedule = [], []
        for i, L in enumerate(self.layers):
            a = L.attention
            if L.type == "attention":
                pos = PositionSpec("rope_neox", a.rot.base, a.rot.dims, yarn=a.rot.scaling) if a.rot.dims else None
                src = i if a.kv_from is None else a.kv_from
                mixer = MixerSpec(kind="normed_attention", hidden=d, num_heads=a.heads, num_kv_heads=a.kv_heads,
                                  head_dim=a.dim, value_dim=a.vdim, qkv_bias=True, scale=a.scale, window=a.window,
                                  keep_window=keep[src], position=pos, qk_norm_kind="projection", sink=True,
                                  borrows_cache=a.kv_from is not None, norm_eps=self.eps, weight_suffix="")
                schedule.append(ScheduleEntry(block=i, cache=src, write_cache=a.kv_from is None))
            else:
                pos = PositionSpec("rope_neox", a.rot.base, a.rot.dims, bands=a.rot.scaling) if a.rot.dims else None
                rename = lambda table, side: tuple((r, leaf.replace("mix.", f"mix.{side}.", 1)) for r, leaf in table)   # noqa: E731
                from .spec import NORMED_ATTENTION_NAMES, RGLRU_NAMES
                left = MixerSpec(kind="normed_attention", hidden=d, num_heads=a.heads, num_kv_heads=a.kv_heads,
                                 head_dim=a.dim, value_dim=a.dim, qkv_bias=True, scale=a.scale, position=pos,
                                 qk_norm_kind="head_unit", value_from_key=True, out_gate=True, norm_eps=self.eps,
                                 names=rename(NORMED_ATTENTION_NAMES, "left"), weight_suffix="")
                r = L.recurrent
                right = MixerSpec(kind="rglru", hidden=d, rec_width=r.width, rec_blocks=r.blocks, rec_slope=DECAY_SLOPE,
                                  conv_taps=r.conv, names=rename(RGLRU_NAMES, "right"), weight_suffix="")
                mixer = MixerSpec(kind="parallel", hidden=d, branches=(left, right),
                                  branch_scales=(L.left_scale, L.right_scale), weight_suffix="")
                schedule.append(ScheduleEntry(block=i, cache=i))
            ffn = None
            if L.ff:
                ffn = FeedForwardSpec(kind="swiglu", hidden=d, intermediate=L.ff, weight_suffix="",
                                      names=(("gate", "mlp.gate"), ("up", "mlp.up"), ("down", "mlp.down")))
            blocks.append(BlockSpec(kind="prenorm", prefix=f"l{i}", mixer=mixer, ffn=ffn, mixer_norm=norm,
                                    ffn_norm=norm if ffn is not None else None, mixer_norm_name="norm1",
                                    ffn_norm_name="norm2", residual_scale=self.residual_mult))
        return ModelSpec(architecture="Banelix", vocab_size=self.vocab, hidden=d, blocks=tuple(blocks),
                         schedule=tuple(schedule), final_norm=norm, tie_embeddings=False, embed_name="embed",
                         final_norm_name="final.norm", head_name="head", max_positions=self.max_positions,
                         embed_scale=self.embed_scale)
