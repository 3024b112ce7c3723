"""Architecture-neutral description of a decoder: what the parts are, layer by layer.

An architecture's own configuration (for instance ``Qwen2Config``) is read from its
``config.json`` keys and then lowered to a ``ModelSpec``.  Everything below the
architecture module works from the ``ModelSpec`` alone: parts are chosen by the ``kind``
string of their spec, sizes and constants travel inside the spec, and no part knows
which model it sits in.

The reference keeps one flat ``Config`` for every architecture
(crates/model/src/config.rs:41-110) and reads the block kind off the tensors that are
present (crates/model/src/weights.rs:810).  Here the block kind is explicit data.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple


def _name_map(given, defaults) -> dict:
    known = dict(defaults)
    out = dict(known)
    for k, v in given:
        if k not in known and k not in ("qkv", "gate_up"):
            raise ValueError(f"unknown tensor role '{k}' (known: {sorted(known)})")
        out[k] = v
    return out


# Leaf names (under the block's prefix) of the tensors the built-in parts bind, as the Hugging Face
# checkpoints of the Llama / Qwen2 family store them (crates/model/src/weights.rs:3165-3205,
# :2970-3004).  An architecture that stores the same arithmetic under other names passes its own in
# ``names``; "qkv" (one [q; k; v] stacked tensor) or "gate_up" (one [gate; up] stacked tensor) may
# stand for the separate ones.
ATTENTION_NAMES = (("q", "self_attn.q_proj"), ("k", "self_attn.k_proj"), ("v", "self_attn.v_proj"),
                   ("o", "self_attn.o_proj"))
SWIGLU_NAMES = (("gate", "mlp.gate_proj"), ("up", "mlp.up_proj"), ("down", "mlp.down_proj"))
# Mixers and feed-forwards with more tensors than those: the roles they know, with default leaf names.
DIFF_ATTENTION_NAMES = (("q", "mix.q"), ("k", "mix.k"), ("v", "mix.v"), ("o", "mix.o"),
                        ("q_conv", "mix.q.conv"), ("k_conv", "mix.k.conv"), ("v_conv", "mix.v.conv"),
                        ("q_norm", "mix.q.norm"), ("k_norm", "mix.k.norm"),
                        ("lq1", "mix.lq1"), ("lk1", "mix.lk1"), ("lq2", "mix.lq2"), ("lk2", "mix.lk2"))
HGRN2_NAMES = (("q", "mix.q"), ("f", "mix.f"), ("f_bias", "mix.f.b"), ("lower", "mix.lower"), ("v", "mix.v"),
               ("out_norm", "mix.norm"), ("o", "mix.o"))
MOE_NAMES = (("expert", "mlp.e{}"), ("gate", "gate"), ("up", "up"), ("down", "down"), ("router", "mlp.router"),
             ("shared", "mlp.shared"), ("shared_gate", "mlp.shared.sg"))
LATENT_ATTENTION_NAMES = (("q", "mix.q"), ("down", "mix.dkv"), ("latent_norm", "mix.dkv.norm"), ("up_k", "mix.uk"),
                          ("up_v", "mix.uv"), ("gate", "mix.g"), ("o", "mix.o"),
                          ("q_down", "mix.dq"), ("q_norm", "mix.dq.norm"), ("q_up", "mix.uq"))
RELU2_NAMES = (("up", "mlp.up"), ("down", "mlp.down"))
MOE_GROUPED_NAMES = (("expert", "mlp.e{}"), ("gate", "gate"), ("up", "up"), ("down", "down"), ("router", "mlp.router"),
                     ("correction", "mlp.correction"), ("shared", "mlp.shared"))
NORMED_ATTENTION_NAMES = (("q", "mix.q"), ("k", "mix.k"), ("v", "mix.v"), ("o", "mix.o"), ("gate", "mix.g"),
                          ("q_bias", "mix.q.b"), ("k_bias", "mix.k.b"), ("v_bias", "mix.v.b"),
                          ("q_norm", "mix.q.norm"), ("k_norm", "mix.k.norm"))
RGLRU_NAMES = (("y", "mix.y"), ("y_bias", "mix.y.b"), ("x", "mix.x"), ("x_bias", "mix.x.b"), ("conv", "mix.conv"),
               ("conv_bias", "mix.conv.b"), ("ra", "mix.ra"), ("ra_bias", "mix.ra.b"), ("ri", "mix.ri"),
               ("ri_bias", "mix.ri.b"), ("lam", "mix.lam"), ("o", "mix.o"))
SSD_NAMES = (("in", "mix.in"), ("conv", "mix.conv"), ("conv_bias", "mix.conv.b"), ("dt_bias", "mix.dt_bias"),
             ("a_log", "mix.A_log"), ("skip", "mix.D"), ("out_norm", "mix.norm"), ("o", "mix.o"))
MOE_SCORED_NAMES = (("expert", "mlp.e{}"), ("up", "up"), ("down", "down"), ("router", "mlp.router"), ("shared", "mlp.shared"))
MIXER_NAMES = {"diff_attention": DIFF_ATTENTION_NAMES, "hgrn2": HGRN2_NAMES, "latent_attention": LATENT_ATTENTION_NAMES,
               "normed_attention": NORMED_ATTENTION_NAMES, "rglru": RGLRU_NAMES, "parallel": (), "ssd": SSD_NAMES}
FEED_FORWARD_NAMES = {"moe_swiglu": MOE_NAMES, "relu2": RELU2_NAMES, "moe_grouped": MOE_GROUPED_NAMES,
                      "moe_scored": MOE_SCORED_NAMES}


@dataclass(frozen=True)
class PositionSpec:
    """Rotary position encoding applied to queries and keys inside a mixer.

    kind "rope_neox": pairs (i, i + rotary_dim/2), angle = pos * theta^(-2i/rotary_dim)
    (crates/kernels/src/cu/ops.cu:488-523, crates/kernels/src/cpu/mod.rs:275-314).
    kind "rope_interleaved": the same angles on adjacent pairs (2i, 2i + 1).

    ``yarn`` = (factor, original, fast, slow) stretches the long waves for contexts beyond the ``original`` length:
    with n(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta) the pair index whose wave makes t turns over the
    original length, lo = max(floor(n(fast)), 0), hi = min(ceil(n(slow)), rotary_dim - 1) and
    ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i's frequency is f_i (1 - ramp_i) + f_i / factor * ramp_i,
    and cos and sin are multiplied by 0.1 ln(factor) + 1.

    ``bands`` = (factor, low, high, original) scales by bands of the wavelength l = 2 pi / f instead: waves shorter than
    original / high keep their frequency, waves longer than original / low get it divided by ``factor``, and in between
    f becomes (1 - s) f / factor + s f with s = (original / l - low) / (high - low); the amplitude stays 1.
    """
    kind: str
    theta: float
    rotary_dim: int
    yarn: Optional[Tuple[float, float, float, float]] = None
    bands: Optional[Tuple[float, float, float, float]] = None


@dataclass(frozen=True)
class NormSpec:
    """kind "rmsnorm": x * rsqrt(mean(x^2) + eps) * w (crates/kernels/src/cu/ops.cu:44-62).
    kind "rmsnorm_scalar": the same with w a single stored number for all coordinates.
    kind "layernorm": (x - mean(x)) * rsqrt(mean((x - mean(x))^2) + eps) * w, no bias."""
    kind: str
    dim: int
    eps: float


@dataclass(frozen=True)
class MixerSpec:
    """Token mixer of one block.

    kind "gqa_attention": grouped-query attention over the paged cache.  ``window`` is
    None for all keys, or W so that key j is visible from query p iff j <= p and
    p - j < W.

    kind "diff_attention": every head has two attention maps of width ``head_dim`` over the same values
    of width ``value_dim``; their results a1, a2 combine to a1 - lambda a2 with one lambda per layer,
    exp(lq1 . lk1) - exp(lq2 . lk2) + ``diff``, followed by a weightless RMS norm over the value width and
    the factor 1 - ``diff``.  ``conv_taps`` > 0 puts a causal convolution over time on every channel of
    q, k and v right behind the projection; ``qk_norm`` an RMS norm (shared weight over ``head_dim``) on
    every map of every query and key head before the rotation.

    kind "hgrn2": a gated linear recurrence with a ``head_dim`` x ``value_dim`` state per head whose
    forget gate (bounded below by a stored vector) also scales what is written; the result of a head is
    RMS-normed over ``value_dim`` with a shared weight.  ``norm_eps`` is the eps of the norms inside a mixer.

    kind "latent_attention": keys and values of all heads are made from one cached row per token: the input
    product gives ``latent_dim`` numbers (RMS-normed with a weight: the latent c) and ``rot_dim`` more (a rotated key
    part shared by all heads); head n's key is [Wuk_n c | that part] (``head_dim`` + ``rot_dim`` wide, like its
    query), its value Wuv_n c (``value_dim`` wide).  ``position`` turns the ``rot_dim`` parts of queries and keys
    (its ``rotary_dim`` <= ``rot_dim``; ``rot_dim`` 0: no rotated part at all).  ``out_gate``: head n's result is
    multiplied by sigmoid of the n-th row of one more product of the mixer's input.  Causal softmax over all keys,
    ``scale`` as given.  ``q_latent_dim`` > 0: the queries go through a latent of their own, q = Wuq rms(Wdq h) w.

    kind "normed_attention": grouped-query attention whose queries and keys are normed.  ``qk_norm_kind``
    "projection": an RMS norm with a weight over the whole query projection (all heads at once) and over the whole key
    projection, before the rotation; "head_unit": every head of q and k divided by its root mean square (no weight)
    after the rotation; "head": an RMS norm over every head of q and of k with a weight of ``head_dim`` numbers shared by
    the heads (one for q, one for k), before the rotation; "": none.  ``distance_slope_exp`` = b > 0: head h's score
    loses s_h (i - j) for a key j seen from position i, with s_h = 2^(-b (h + 1) / H).  ``value_from_key``: there is no value projection, a key's value is the key as it
    was projected (before norm and rotation).  ``sink``: the softmax's denominator has one more term exp(0) without a
    value.  ``out_gate`` as above.  ``borrows_cache``: the layer has no key or value tensors at all and reads the cache
    another schedule entry writes (its ``ScheduleEntry.write_cache`` is False).  ``keep_window``: how many keys the
    cache keeps (the largest window of the layers that read it; None where any reads all keys); ``window`` is what
    this layer's own mask lets it see.  q, k and v have biases where ``qkv_bias`` says so.

    kind "rglru": a gated linear recurrence over ``rec_width`` channels: a gate branch y = gelu_tanh(Wy h + b) and a
    recurrent branch u = conv(Wx h + b) (a causal convolution of ``conv_taps`` taps per channel, with a bias); per
    block of rec_width / ``rec_blocks`` channels r = sigmoid(Ra u + b), i = sigmoid(Ri u + b);
    a = exp(-``rec_slope`` r softplus(lam)); S <- a S + sqrt(1 - a^2) i u; result Wo (S * y).

    kind "ssd": a selective state-space recurrence with a scalar decay per head (the state-space-duality form).  One
    input product gives [z | x | B | C | dt] with x and z ``num_heads`` * ``value_dim`` wide, B and C ``rec_groups`` *
    ``state_dim`` wide and one dt per head; x, B and C pass a causal convolution of ``conv_taps`` taps per channel (with a
    bias) and silu; dt = softplus(dt + dt_bias); per head S <- exp(-exp(A_log) dt) S + dt B x^T (S ``state_dim`` x
    ``value_dim``), y = S^T C + D x; y silu(z) is RMS-normed in ``norm_groups`` equal parts, times a weight, and goes
    through the output product.

    kind "parallel": the mixers of ``branches`` read the same input side by side; the result is the sum of their
    results times ``branch_scales``.  Branch b's tensors carry the leaf names of its own spec.
    """
    kind: str
    hidden: int
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    qkv_bias: bool = False
    out_bias: bool = False
    scale: float = 0.0
    window: Optional[int] = None
    position: Optional[PositionSpec] = None
    value_dim: int = 0                # width of a head's value; 0: head_dim
    conv_taps: int = 0
    qk_norm: bool = False
    norm_eps: float = 1e-6
    diff: float = 0.0
    rot_dim: int = 0                  # latent attention: width of the rotated part of a query / key
    latent_dim: int = 0               # latent attention: width of the cached latent
    out_gate: bool = False            # a sigmoid gate per head on the result
    qk_norm_kind: str = ""            # normed attention: "", "projection" or "head_unit"
    value_from_key: bool = False
    sink: bool = False
    borrows_cache: bool = False
    keep_window: Optional[int] = None
    distance_slope_exp: float = 0.0   # > 0: a distance bias with slopes 2^(-this (h + 1) / H) is taken off the scores
    q_latent_dim: int = 0             # latent attention: width of the queries' own latent; 0: a direct query product
    state_dim: int = 0                # ssd: rows of a head's state
    rec_groups: int = 1               # ssd: groups of heads that share B and C
    norm_groups: int = 1              # ssd: equal parts the gated result is normed in
    rec_width: int = 0
    rec_blocks: int = 1
    rec_slope: float = 8.0
    branches: Tuple["MixerSpec", ...] = ()
    branch_scales: Tuple[float, ...] = ()
    # free-form extras for mixers defined outside the framework
    extra: Tuple[Tuple[str, object], ...] = ()
    # role -> leaf name under the block's prefix (see ATTENTION_NAMES); roles not given keep the default
    names: Tuple[Tuple[str, str], ...] = ()
    weight_suffix: str = ".weight"    # what follows a matrix's leaf name in the checkpoint

    def get(self, key, default=None):
        for k, v in self.extra:
            if k == key:
                return v
        return default

    def tensor_names(self) -> dict:
        return _name_map(self.names, MIXER_NAMES.get(self.kind, ATTENTION_NAMES))

    @property
    def v_dim(self) -> int:
        return self.value_dim or self.head_dim


@dataclass(frozen=True)
class FeedForwardSpec:
    """kind "swiglu": down(silu(gate(x)) * up(x)) (crates/model/src/lib.rs:7391-7451).

    kind "moe_swiglu": ``experts`` SwiGLU experts of width ``intermediate`` of which every token uses the
    ``top`` with the largest router logits, weighted by the softmax over those logits alone; with
    ``shared_intermediate`` > 0 a SwiGLU expert of that width runs for every token and is added, times
    sigmoid(w . x) of a stored vector w.

    kind "relu2": down(relu(up(x))^2).

    kind "moe_grouped": experts of the gated form down(glu(gate(x), up(x))) with ``activation`` "glu_clamped"
    (g' = min(g, ``limit``), u' = clamp(u, -limit, limit), g' sigmoid(``act_alpha`` g') (u' + 1)) or "swiglu".  Routing:
    s = softmax of the router's logits over all experts; experts are picked by s + a stored per-expert correction
    (``route_correction``), among the ``route_keep`` best of ``route_groups`` groups of neighbouring experts (a
    group's score: its largest pick score); weights are s of the ``top`` picked over their sum.  With
    ``shared_intermediate`` > 0 an expert of that width (limit ``shared_limit``) runs for every token and is added.

    kind "moe_scored": experts of the ungated form down(act(up(x))) with ``activation`` "relu2".  Every expert's score is
    ``route_score`` of its router logit ("sigmoid"); the ``top`` largest are chosen (the lowest index wins a tie); the
    weights are the chosen scores, divided by their sum only where ``route_renorm`` says so; with ``weight_input`` the
    weight multiplies what the expert reads (the result is sum_c expert_c(w_c x)), else what it returns.  With
    ``shared_intermediate`` > 0 an expert of the same form and that width runs for every token and is added."""
    kind: str
    hidden: int
    intermediate: int
    experts: int = 0
    top: int = 0
    shared_intermediate: int = 0
    activation: str = "swiglu"
    limit: float = 0.0
    act_alpha: float = 1.0
    shared_limit: float = 0.0
    route_groups: int = 1
    route_keep: int = 1
    route_correction: bool = False
    route_score: str = "softmax"
    route_renorm: bool = True
    weight_input: bool = False
    extra: Tuple[Tuple[str, object], ...] = ()
    names: Tuple[Tuple[str, str], ...] = ()          # role -> leaf name (see SWIGLU_NAMES)
    weight_suffix: str = ".weight"

    def tensor_names(self) -> dict:
        return _name_map(self.names, FEED_FORWARD_NAMES.get(self.kind, SWIGLU_NAMES))


@dataclass(frozen=True)
class BlockSpec:
    """One layer: its parts and the tensor-name prefix its weights live under.

    kind "prenorm": x += mixer(norm1(x)); x += ffn(norm2(x)).
    kind "gated_postnorm": the sublayers read x itself and the norm sits on their result:
    x += norm1(mixer(x) * sigmoid(G1 x + b1)); x += norm2(ffn(x) * sigmoid(G2 x + b2)); the gates are
    there where ``mixer_gate_name`` / ``ffn_gate_name`` are given (bias: that name + ``gate_bias_suffix``),
    and ``ffn`` may be None (a layer with a mixer only).
    With ``residual_scale`` = m the sublayers' results enter the residual stream times m:
    x += m mixer(norm1(x)); x += m ffn(norm2(x)).
    kind "hyper_prenorm": the residual is ``streams`` vectors per token.  Sublayer q (1: mixer, 2: feed-forward) has
    three small tensors under ``hyper_names[q-1]``: ``.in`` [S], ``.mix`` [S, S] (from, to), ``.out`` [S];
    u = sum_s in[s] x_s; y = sublayer(norm_q(u)); x_r <- sum_s mix[s, r] x_s + out[r] y for all r at once.
    """
    kind: str
    prefix: str
    mixer: MixerSpec
    ffn: Optional[FeedForwardSpec]
    mixer_norm: NormSpec
    ffn_norm: Optional[NormSpec]
    # leaf names of the two norm weights under the prefix
    mixer_norm_name: str = "input_layernorm.weight"
    ffn_norm_name: str = "post_attention_layernorm.weight"
    mixer_gate_name: Optional[str] = None
    ffn_gate_name: Optional[str] = None
    gate_bias_suffix: str = ".b"
    streams: int = 0
    hyper_names: Tuple[str, str] = ("hc1", "hc2")
    residual_scale: float = 1.0


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a block.

    ``block`` indexes ``ModelSpec.blocks`` (a block may be named more than once).
    ``cache`` is the cache slot this execution reads; ``write_cache`` says whether it
    appends this step's keys and values there (False lets a layer read the cache another
    execution filled).
    """
    block: int
    cache: int
    write_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden: int
    blocks: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: NormSpec
    tie_embeddings: bool
    embed_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm.weight"
    head_name: str = "lm_head.weight"
    max_positions: int = 4096
    eos_token_ids: Tuple[int, ...] = ()
    embed_scale: float = 1.0
    logit_scale: float = 1.0
    streams: int = 0                  # > 0: the residual is this many vectors per token, all equal to the embedding at
                                      # the start and added up in front of the final norm (blocks of kind "hyper_prenorm")

    def num_cache_slots(self) -> int:
        return 1 + max((e.cache for e in self.schedule), default=-1)
