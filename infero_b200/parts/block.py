"""Arrangement of the parts in one layer."""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config.spec import BlockSpec
from ..registry import part_class
from .base import Part, TensorDecl


class PreNormBlock(Part):
    """x += mixer(norm1(x)); x += ffn(norm2(x))  (crates/metal/examples/qwen2_f16.rs:863-935).

    The adds are done by the norm that follows: ``forward`` receives the delta the layer
    before left pending and returns its own feed-forward delta the same way, so each
    residual add shares one pass over x with a normalisation.
    """

    def __init__(self, spec: BlockSpec):
        self.spec = spec
        p = spec.prefix
        self.mixer_norm = part_class("norm", spec.mixer_norm.kind)(spec.mixer_norm, f"{p}.{spec.mixer_norm_name}")
        self.mixer = part_class("mixer", spec.mixer.kind)(spec.mixer, p)
        self.ffn = self.ffn_norm = None      # a layer may have a mixer only
        if spec.ffn is not None:
            self.ffn_norm = part_class("norm", spec.ffn_norm.kind)(spec.ffn_norm, f"{p}.{spec.ffn_norm_name}")
            self.ffn = part_class("feed_forward", spec.ffn.kind)(spec.ffn, p)
        self._native = None                  # the native launcher of this block, made at first use

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None]

    def declare(self) -> List[TensorDecl]:
        out: List[TensorDecl] = []
        for part in self.parts():
            out += part.declare()
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for part in self.parts():
            part.bind(tensors)

    def _native_for(self, ctx):
        """This block's native launcher if the step ``ctx`` goes that way, else None."""
        native = self._native
        if native is None:
            from .native_block import NativeBlock
            native = self._native = NativeBlock(self)
        return native if native.wants(ctx) else None

    def forward(self, ctx, x, delta, slot):
        from .. import kernels as K
        m = float(getattr(self.spec, "residual_scale", 1.0))
        native = None if (m != 1.0 or isinstance(delta, K.Scaled)) else self._native_for(ctx)
        if native is not None:
            # the package's own parts in a bf16 step: the whole layer in one native call (same kernels,
            # same arguments, same order as below)
            out = native.run(ctx, x, delta, slot)
            if out is not None:
                return out
        if hasattr(delta, "as_partials"):
            delta = delta.as_partials()
        h = self.mixer_norm.forward(ctx, x, delta)
        a = self.mixer.forward(ctx, h, slot)
        if m != 1.0:
            a = K.Scaled(a, m)               # the norm that adds it multiplies as it adds
        if self.ffn is None:
            return a
        h = self.ffn_norm.forward(ctx, x, a)
        f = self.ffn.forward(ctx, h)
        return K.Scaled(f, m) if m != 1.0 else f


class GatedPostNormBlock(Part):
    """The sublayers read the residual stream itself; the norm sits on their result, behind a gate:

        x += norm1(mixer(x) * sigmoid(G1 x + b1));   x += norm2(ffn(x) * sigmoid(G2 x + b2))

    with norms of kind "rmsnorm_scalar" (one stored number).  A gate is there where the spec names it, and the
    feed-forward half where the spec has one.  x is float32; on the bf16 path the kernel that adds a
    sublayer's normed result also leaves the new x in bf16 for the next sublayer's products, and the first
    block of a run converts x once.  The block adds what a block before left pending and leaves nothing
    pending itself."""

    def __init__(self, spec: BlockSpec):
        from .linear import Linear  # noqa: F401
        self.spec = spec
        p = spec.prefix
        self.mixer_norm = part_class("norm", spec.mixer_norm.kind)(spec.mixer_norm, f"{p}.{spec.mixer_norm_name}")
        self.mixer = part_class("mixer", spec.mixer.kind)(spec.mixer, p)
        self.ffn = self.ffn_norm = None
        if spec.ffn is not None:
            self.ffn_norm = part_class("norm", spec.ffn_norm.kind)(spec.ffn_norm, f"{p}.{spec.ffn_norm_name}")
            self.ffn = part_class("feed_forward", spec.ffn.kind)(spec.ffn, p)
        for n in (self.mixer_norm, self.ffn_norm):
            if n is not None and not hasattr(n, "scalar"):
                raise ValueError("a gated post-norm block takes norms with a single stored number")
        self.gates = [None, None]            # Linear of each half's gate, or "stacked": the gate's rows ride on the
        self.gate_bias = [None, None]        # sublayer's own input product (parts with ``append_rows``)

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None]

    def _gate_names(self):
        s = self.spec
        return [s.mixer_gate_name, s.ffn_gate_name if self.ffn is not None else None]

    def declare(self) -> List[TensorDecl]:
        out: List[TensorDecl] = []
        for part in self.parts():
            out += part.declare()
        d = self.spec.mixer.hidden
        for name in self._gate_names():
            if name:
                out += [TensorDecl(f"{self.spec.prefix}.{name}", (d, d)),
                        TensorDecl(f"{self.spec.prefix}.{name}{self.spec.gate_bias_suffix}", (d,), role="bias")]
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        from .linear import Linear
        for part in self.parts():
            part.bind(tensors)
        for i, name in enumerate(self._gate_names()):
            if name:
                full = f"{self.spec.prefix}.{name}"
                part = self.mixer if i == 0 else self.ffn
                if hasattr(part, "append_rows"):
                    part.append_rows(tensors[full])
                    self.gates[i] = "stacked"
                else:
                    self.gates[i] = Linear(tensors[full], None, full)
                self.gate_bias[i] = tensors[full + self.spec.gate_bias_suffix].float().contiguous()

    def _input(self, ctx, x):
        """x in the type the products take: x itself in 32-bit, else its bf16 copy (left by the block before
        if that was of this kind, made here otherwise)."""
        if ctx.act_dtype == torch.float32:
            return x
        from ..kernels import layer_ops as L
        left = getattr(ctx, "_resid_act", None)
        if left is not None and left[0] == getattr(ctx, "schedule_index", -2) - 1 and left[1].shape == x.shape:
            return left[1]
        h = torch.empty(x.shape, dtype=ctx.act_dtype, device=x.device)
        L.cast_rows(x, h)
        return h

    def _half(self, ctx, x, h, y, i, norm):
        from ..kernels import layer_ops as L
        if self.gates[i] == "stacked":
            g = ctx.extra_product                # left by the sublayer that just ran
        else:
            g = self.gates[i].forward(h, out_dtype=torch.float32) if self.gates[i] is not None else None
        h_next = torch.empty(x.shape, dtype=ctx.act_dtype, device=x.device) if ctx.act_dtype != torch.float32 else None
        L.gated_scalar_norm_add(x, y, g, self.gate_bias[i], norm.scalar, norm.spec.eps, h_next)
        return x if h_next is None else h_next

    def forward(self, ctx, x, delta, slot):
        from .. import kernels as K
        if delta is not None:
            if hasattr(delta, "as_partials"):
                delta = delta.as_partials()
            if isinstance(delta, K.Partials):
                delta = delta.materialize(torch.float32)
            K.residual_add(x, delta.contiguous())
            ctx._resid_act = None
        h = self._input(ctx, x)
        y = self.mixer.forward(ctx, h, slot)
        h = self._half(ctx, x, h, y, 0, self.mixer_norm)
        if self.ffn is not None:
            y = self.ffn.forward(ctx, h)
            h = self._half(ctx, x, h, y, 1, self.ffn_norm)
        ctx._resid_act = (getattr(ctx, "schedule_index", -2), h)
        return None


class HyperPreNormBlock(Part):
    """A pre-norm layer whose residual is S streams per token (x float32 [T, S, d]).  For each sublayer (mixer, then
    feed-forward if there is one) with its small tensors ``in`` [S], ``mix`` [S, S] (from, to) and ``out`` [S]:

        u = sum_s in[s] x_s;   y = sublayer(norm(u));   x_r <- sum_s mix[s, r] x_s + out[r] y   (all r from the old x)

    with norms of kind "layernorm".  One kernel per sublayer does the update for the sublayer before and the weighted
    sum and norm for the next one (``hyper_step``); the update of a layer's last sublayer is left pending and done by
    the next block of this kind in its first pass, or by the model in front of the final norm (``pending`` /
    ``flush``).  The small tensors are float32 on both precisions."""

    def __init__(self, spec: BlockSpec):
        self.spec = spec
        p = spec.prefix
        self.S = int(spec.streams)
        if self.S < 1:
            raise ValueError("a hyper-connection block needs at least one stream")
        self.mixer_norm = part_class("norm", spec.mixer_norm.kind)(spec.mixer_norm, f"{p}.{spec.mixer_norm_name}")
        self.mixer = part_class("mixer", spec.mixer.kind)(spec.mixer, p)
        self.ffn = self.ffn_norm = None
        if spec.ffn is not None:
            self.ffn_norm = part_class("norm", spec.ffn_norm.kind)(spec.ffn_norm, f"{p}.{spec.ffn_norm_name}")
            self.ffn = part_class("feed_forward", spec.ffn.kind)(spec.ffn, p)
        for n in (self.mixer_norm, self.ffn_norm):
            if n is not None and n.spec.kind != "layernorm":
                raise ValueError("a hyper-connection block takes layer norms")
        self.hc = [None, None]               # per sublayer: (in, mix, out), float32

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None]

    def _hc_names(self):
        p, names = self.spec.prefix, self.spec.hyper_names
        return [f"{p}.{names[0]}"] + ([f"{p}.{names[1]}"] if self.ffn is not None else [])

    def declare(self) -> List[TensorDecl]:
        out: List[TensorDecl] = []
        for part in self.parts():
            out += part.declare()
        S = self.S
        for n in self._hc_names():
            out += [TensorDecl(f"{n}.in", (S,), role="bias", init="ones"), TensorDecl(f"{n}.out", (S,), role="bias", init="ones"),
                    TensorDecl(f"{n}.mix", (S, S), role="bias", init="eye")]
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for part in self.parts():
            part.bind(tensors)
        for i, n in enumerate(self._hc_names()):
            self.hc[i] = tuple(tensors[f"{n}.{leaf}"].float().contiguous() for leaf in ("in", "mix", "out"))

    @staticmethod
    def _as_f32(y):
        """A sublayer's result as the stream kernel takes it: float32, or a product left as partial sums without a bias
        (the kernel adds them up in its own pass)."""
        from .. import kernels as K
        if hasattr(y, "as_partials"):
            y = y.as_partials()
        if isinstance(y, K.Partials):
            return y if y.bias is None else y.materialize(torch.float32)
        return y if y.dtype == torch.float32 else y.float()

    def forward(self, ctx, x, delta, slot):
        from ..kernels import layer_ops as L
        T, S, d = x.shape
        assert S == self.S, f"the model keeps {S} streams, this block {self.S}"
        pend = delta                          # (y, mix, out) of the sublayer that ran last, or None
        eps = self.mixer_norm.spec.eps
        h = torch.empty((T, d), dtype=ctx.act_dtype, device=x.device)
        w_in, mix, w_out = self.hc[0]
        L.hyper_step(x, *(pend if pend is not None else (None, None, None)), w_in, self.mixer_norm.weight, eps, h)
        y = self._as_f32(self.mixer.forward(ctx, h, slot))
        if self.ffn is None:
            return (y, mix, w_out)
        w_in2, mix2, w_out2 = self.hc[1]
        h = torch.empty((T, d), dtype=ctx.act_dtype, device=x.device)
        L.hyper_step(x, y, mix, w_out, w_in2, self.ffn_norm.weight, self.ffn_norm.spec.eps, h)
        y = self._as_f32(self.ffn.forward(ctx, h))
        return (y, mix2, w_out2)

    @staticmethod
    def flush(x, pending) -> None:
        """Apply a pending update to the streams."""
        from ..kernels import layer_ops as L
        if pending is not None:
            L.hyper_step(x, pending[0], pending[1], pending[2], None, None, 0.0, None)
