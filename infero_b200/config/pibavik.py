"""Typed configuration of the Pibavik decoder, read from its own config.json keys.

config.json: ``architecture`` "Pibavik", ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` (the embedding is
multiplied by it) and ``layers``, one entry per layer: ``type``, ``mixer`` and ``mlp`` (null, or a mixture of
experts {``kind`` "moe", ``expert.ff``, ``router.experts``, ``router.top``, optionally ``shared.ff``}).  Layer i's
tensors start with ``l<i>.``.  Every layer is a pre-norm layer with RMS norms.

``type`` "attention": grouped-query attention without biases and without rotation (``heads``, ``kv_heads``, ``dim``,
``vdim``, ``scale``, ``mask.size``: a query sees itself and the size - 1 tokens before it).  Positions enter as a
distance bias: head h's score loses 2^(-8 (h + 1) / heads) times the distance to the key.  With ``kv_from``: j the
layer has no key or value tensors and reads layer j's cache with its own queries, window and scale.

``type`` "latent_attention": causal attention over all keys whose keys and values are made from one cached latent
of ``kv_rank`` numbers per token (RMS-normed with a weight) and whose queries go through a normed latent of
``q_rank`` numbers; ``heads``, ``dim``, ``vdim``, ``scale``; no rotated part.

``type`` "parallel": two mixers side by side on the same input, ``mixer.left`` and ``mixer.right``, added up with
``left_scale`` and ``right_scale``.  Left: windowed grouped-query attention whose query and key heads are RMS-normed
with a weight shared by the heads, then rotated on their first ``rot.dims`` coordinates (``rot.base``), with a
sigmoid gate per head on the result.  Right: a state-space recurrence (``heads``, ``vdim``, ``state``, ``groups``,
``conv`` taps, ``norm_groups``).

The feed-forward's experts are down(relu(up x)^2); scores are the sigmoid of the router's logits, the ``top`` largest
are chosen, not renormalised, and multiply what the expert reads.

Lowering: blocks "prenorm"; mixers "normed_attention" (with a distance bias, or with the per-head norm, rotation and
gate), "latent_attention", "ssd" and "parallel"; feed-forward "moe_scored"; a layer with ``kv_from`` becomes a
schedule entry that reads the other layer's cache slot without writing it, and the cache keeps the largest window of
its readers.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .gositar import _number
from .qwen2 import ConfigError
from .spec import (BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry,
                   LATENT_ATTENTION_NAMES, NORMED_ATTENTION_NAMES, SSD_NAMES)
from .vufizen import _pos_int

DISTANCE_SLOPE_EXP = 8.0         # head h's slope is 2^(-DISTANCE_SLOPE_EXP (h + 1) / heads); fixed by the design
MAX_TAPS = 16


@dataclass(frozen=True)
class PibavikAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int] = None      # None: every earlier token is seen
    kv_from: Optional[int] = None
    rot_base: float = 10000.0         # the left mixer only
    rot_dims: int = 0


@dataclass(frozen=True)
class PibavikLatent:
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float


@dataclass(frozen=True)
class PibavikStateSpace:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclass(frozen=True)
class PibavikMlp:
    experts: int
    top: int
    ff: int
    shared_ff: int = 0                # 0: no shared expert


@dataclass(frozen=True)
class PibavikLayer:
    type: str                         # "attention" | "latent_attention" | "parallel"
    attention: Optional[PibavikAttention] = None      # the mixer itself, or the left one
    latent: Optional[PibavikLatent] = None
    state_space: Optional[PibavikStateSpace] = None
    left_scale: float = 1.0
    right_scale: float = 1.0
    mlp: Optional[PibavikMlp] = None


def _window(m: Dict[str, Any], where: str) -> Optional[int]:
    if m.get("mask") is None:
        return None
    if not isinstance(m["mask"], dict):
        raise ConfigError(f"config.json: {where}.mask is not an object")
    return _pos_int(m["mask"], "size", where + ".mask")


def _attention(m: Dict[str, Any], where: str, left: bool) -> PibavikAttention:
    heads, kv = _pos_int(m, "heads", where), _pos_int(m, "kv_heads", where)
    dim, vdim = _pos_int(m, "dim", where), _pos_int(m, "vdim", where)
    if heads % kv:
        raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {kv} kv_heads")
    src, base, dims = None, 10000.0, 0
    if left:
        rot = m.get("rot")
        if rot is not None:
            if not isinstance(rot, dict):
                raise ConfigError(f"config.json: {where}.rot is not an object")
            dims = rot.get("dims", dim)
            if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > dim:
                raise ConfigError(f"config.json: {where}.rot.dims {dims!r} must be even and at most dim {dim}")
            if dims:
                base = _number(rot, "base", where + ".rot")
    elif m.get("kv_from") is not None:
        src = m["kv_from"]
        if isinstance(src, bool) or not isinstance(src, int) or src < 0:
            raise ConfigError(f"config.json: {where}.kv_from {src!r} must be a layer's index")
    return PibavikAttention(heads, kv, dim, vdim, _number(m, "scale", where), _window(m, where), src, base, dims)


def _latent(m: Dict[str, Any], where: str) -> PibavikLatent:
    return PibavikLatent(_pos_int(m, "heads", where), _pos_int(m, "dim", where), _pos_int(m, "vdim", where),
                         _pos_int(m, "kv_rank", where), _pos_int(m, "q_rank", where), _number(m, "scale", where))


def _state_space(m: Dict[str, Any], where: str) -> PibavikStateSpace:
    s = PibavikStateSpace(_pos_int(m, "heads", where), _pos_int(m, "vdim", where), _pos_int(m, "state", where),
                          _pos_int(m, "groups", where), _pos_int(m, "conv", where), _pos_int(m, "norm_groups", where))
    if s.heads % s.groups:
        raise ConfigError(f"config.json: {where}: {s.heads} heads do not split into {s.groups} groups")
    if (s.heads * s.vdim) % s.norm_groups:
        raise ConfigError(f"config.json: {where}: {s.heads * s.vdim} channels do not split into {s.norm_groups} norm groups")
    if s.conv > MAX_TAPS:
        raise ConfigError(f"config.json: {where}: {s.conv} taps, at most {MAX_TAPS}")
    return s


def _mlp(ml: Any, where: str) -> Optional[PibavikMlp]:
    if ml is None:
        return None
    if not isinstance(ml, dict) or ml.get("kind") != "moe":
        raise ConfigError(f"config.json: {where}.kind {ml.get('kind') if isinstance(ml, dict) else ml!r} is not 'moe'")
    router, expert = ml.get("router"), ml.get("expert")
    if not isinstance(router, dict) or not isinstance(expert, dict):
        raise ConfigError(f"config.json: {where} needs 'router' and 'expert'")
    experts, top = _pos_int(router, "experts", where + ".router"), _pos_int(router, "top", where + ".router")
    if top > experts:
        raise ConfigError(f"config.json: {where}.router: top {top} of {experts} experts")
    shared = ml.get("shared")
    shared_ff = _pos_int(shared, "ff", where + ".shared") if isinstance(shared, dict) else 0
    return PibavikMlp(experts, top, _pos_int(expert, "ff", where + ".expert"), shared_ff)


@dataclass(frozen=True)
class PibavikConfig:
    vocab: int
    width: int
    eps: float
    embed_scale: float
    layers: Tuple[PibavikLayer, ...]
    raw: Tuple[Tuple[str, Any], ...] = ()
    max_positions: int = 1 << 20

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "PibavikConfig":
        vocab, width = _pos_int(raw, "vocab", "config"), _pos_int(raw, "width", "config")
        eps = _number(raw.get("norm") or {}, "eps", "norm")
        embed_scale = _number(raw.get("embedding") or {"scale": 1.0}, "scale", "embedding", positive=False)
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(entries):
            where = f"layers[{i}]"
            m = L.get("mixer") if isinstance(L, dict) else None
            if not isinstance(m, dict):
                raise ConfigError(f"config.json: {where}.mixer is missing")
            mlp = _mlp(L.get("mlp"), where + ".mlp")
            kind = L.get("type")
            if kind == "attention":
                layers.append(PibavikLayer("attention", attention=_attention(m, where + ".mixer", False), mlp=mlp))
            elif kind == "latent_attention":
                layers.append(PibavikLayer("latent_attention", latent=_latent(m, where + ".mixer"), mlp=mlp))
            elif kind == "parallel":
                left, right = m.get("left"), m.get("right")
                if not isinstance(left, dict) or not isinstance(right, dict):
                    raise ConfigError(f"config.json: {where}.mixer needs 'left' and 'right'")
                scale = lambda k: _number(m, k, where + ".mixer", positive=False) if m.get(k) is not None else 1.0   # noqa: E731
                layers.append(PibavikLayer("parallel", attention=_attention(left, where + ".mixer.left", True),
                                           state_space=_state_space(right, where + ".mixer.right"),
                                           left_scale=scale("left_scale"), right_scale=scale("right_scale"), mlp=mlp))
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is none of 'attention', 'latent_attention', 'parallel'")
        for i, L in enumerate(layers):
            a = L.attention
            if L.type != "attention" or a.kv_from is None:
                continue
            where = f"layers[{i}].mixer.kv_from"
            if a.kv_from >= i:
                raise ConfigError(f"config.json: {where} {a.kv_from} must name an earlier layer")
            src = layers[a.kv_from]
            b = src.attention
            if src.type != "attention" or b.kv_from is not None:
                raise ConfigError(f"config.json: {where}: layer {a.kv_from} has no keys and values of this kind")
            if (b.kv_heads, b.dim, b.vdim) != (a.kv_heads, a.dim, a.vdim):
                raise ConfigError(f"config.json: {where}: layer {a.kv_from}'s key/value heads and sizes differ")
        return cls(vocab, width, eps, embed_scale, tuple(layers), raw=tuple(raw.items()),
                   max_positions=int(raw.get("max_positions", 1 << 20)))

    def to_json_dict(self) -> Dict[str, Any]:
        keep = ("architecture", "vocab", "width", "norm", "embedding", "layers", "max_positions")
        return {k: v for k, v in self.raw if k in keep}

    # ---- lowering to parts ---------------------------------------------------------------------
    def to_model_spec(self) -> ModelSpec:
        d = self.width
        norm = NormSpec(kind="rmsnorm", dim=d, eps=self.eps)
        # the cache of a layer keeps the largest window of the layers that read it
        keep = {i: L.attention.window for i, L in enumerate(self.layers) if L.type == "attention" and L.attention.kv_from is None}
        for L in self.layers:
            if L.type == "attention" and L.attention.kv_from is not None:
                mine, theirs = L.attention.window, keep[L.attention.kv_from]
                keep[L.attention.kv_from] = None if mine is None or theirs is None else max(mine, theirs)
        rename = lambda table, side: tuple((r, leaf.replace("mix.", f"mix.{side}.", 1)) for r, leaf in table)   # noqa: E731
        blocks, schedule = [], []
        for i, L in enumerate(self.layers):
            a = L.attention
            if L.type == "attention":
                src = i if a.kv_from is None else a.kv_from
                mixer = MixerSpec(kind="normed_attention", hidden=d, num_heads=a.heads, num_kv_heads=a.kv_heads,
                                  head_dim=a.dim, value_dim=a.vdim, scale=a.scale, window=a.window, keep_window=keep[src],
                                  distance_slope_exp=DISTANCE_SLOPE_EXP, borrows_cache=a.kv_from is not None,
                                  norm_eps=self.eps, weight_suffix="")
                schedule.append(ScheduleEntry(block=i, cache=src, write_cache=a.kv_from is None))
            elif L.type == "latent_attention":
                t = L.latent
                mixer = MixerSpec(kind="latent_attention", hidden=d, num_heads=t.heads, head_dim=t.dim, value_dim=t.vdim,
                                  latent_dim=t.kv_rank, q_latent_dim=t.q_rank, rot_dim=0, scale=t.scale, norm_eps=self.eps,
                                  names=LATENT_ATTENTION_NAMES, weight_suffix="")
                schedule.append(ScheduleEntry(block=i, cache=i))
            else:
                pos = PositionSpec("rope_neox", a.rot_base, a.rot_dims) if a.rot_dims else None
                left = MixerSpec(kind="normed_attention", hidden=d, num_heads=a.heads, num_kv_heads=a.kv_heads,
                                 head_dim=a.dim, value_dim=a.vdim, scale=a.scale, window=a.window, position=pos,
                                 qk_norm_kind="head", out_gate=True, norm_eps=self.eps,
                                 names=rename(NORMED_ATTENTION_NAMES, "left"), weight_suffix="")
                r = L.state_space
                right = MixerSpec(kind="ssd", hidden=d, num_heads=r.heads, value_dim=r.vdim, state_dim=r.state,
                                  rec_groups=r.groups, norm_groups=r.norm_groups, conv_taps=r.conv, norm_eps=self.eps,
                                  names=rename(SSD_NAMES, "right"), weight_suffix="")
                mixer = MixerSpec(kind="parallel", hidden=d, branches=(left, right),
                                  branch_scales=(L.left_scale, L.right_scale), weight_suffix="")
                schedule.append(ScheduleEntry(block=i, cache=i))
            ffn = None
            if L.mlp is not None:
                ffn = FeedForwardSpec(kind="moe_scored", hidden=d, intermediate=L.mlp.ff, experts=L.mlp.experts,
                                      top=L.mlp.top, shared_intermediate=L.mlp.shared_ff, activation="relu2",
                                      route_score="sigmoid", route_renorm=False, weight_input=True, weight_suffix="")
            blocks.append(BlockSpec(kind="prenorm", prefix=f"l{i}", mixer=mixer, ffn=ffn, mixer_norm=norm,
                                    ffn_norm=norm if ffn is not None else None, mixer_norm_name="norm1",
                                    ffn_norm_name="norm2"))
        return ModelSpec(architecture="Pibavik", vocab_size=self.vocab, hidden=d, blocks=tuple(blocks),
                         schedule=tuple(schedule), final_norm=norm, tie_embeddings=False, embed_name="embed",
                         final_norm_name="final.norm", head_name="head", max_positions=self.max_positions,
                         embed_scale=self.embed_scale)
