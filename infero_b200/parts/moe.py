"""Mixture-of-experts feed-forward with SwiGLU experts and an optional shared expert."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels as K
from ..config.spec import FeedForwardSpec
from ..kernels import layer_ops as L
from .base import FeedForward, TensorDecl
from .linear import Linear
from .mlp import SwiGluMlp


class MoeSwiGlu(FeedForward):
    """z = Wr h in 32-bit; the ``top`` experts with the largest logits, weights = softmax over those logits
    alone; delta = sum_c w_c * down_e(silu(gate_e h) * up_e h).  A shared expert of the same form (width
    ``shared_intermediate``) runs for every token and is added times sigmoid(w_sg . h).

    The experts' matrices are stacked when the weights are bound: gate and up as [E, 2 ff, d] with rows
    alternating gate_j, up_j (the layout of the package's SwiGLU products), down as [E, d, ff]."""

    def __init__(self, spec: FeedForwardSpec, prefix: str):
        self.spec, self.prefix = spec, prefix
        self.E, self.top, self.ff = int(spec.experts), int(spec.top), int(spec.intermediate)
        self.names = spec.tensor_names()
        self.shared: Optional[SwiGluMlp] = None
        if spec.shared_intermediate > 0:
            sh = self.names["shared"]
            sub = FeedForwardSpec(kind="swiglu", hidden=spec.hidden, intermediate=spec.shared_intermediate,
                                  names=tuple((r, f"{sh}.{self.names[r]}") for r in ("gate", "up", "down")),
                                  weight_suffix=spec.weight_suffix)
            self.shared = SwiGluMlp(sub, prefix)

    def _expert(self, e: int, role: str) -> str:
        return f"{self.prefix}.{self.names['expert'].format(e)}.{self.names[role]}{self.spec.weight_suffix}"

    def _n(self, role: str) -> str:
        return f"{self.prefix}.{self.names[role]}{self.spec.weight_suffix}"

    def declare(self) -> List[TensorDecl]:
        d, ff = self.spec.hidden, self.ff
        out: List[TensorDecl] = []
        for e in range(self.E):
            out += [TensorDecl(self._expert(e, "gate"), (ff, d)), TensorDecl(self._expert(e, "up"), (ff, d)),
                    TensorDecl(self._expert(e, "down"), (d, ff))]
        out.append(TensorDecl(self._n("router"), (self.E, d)))
        if self.shared is not None:
            out += self.shared.declare()
            out.append(TensorDecl(self._n("shared_gate"), (1, d)))
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        g = torch.stack([tensors[self._expert(e, "gate")] for e in range(self.E)])
        u = torch.stack([tensors[self._expert(e, "up")] for e in range(self.E)])
        self.gate_up = torch.stack([g, u], dim=2).reshape(self.E, 2 * self.ff, self.spec.hidden).contiguous()
        self.down = torch.stack([tensors[self._expert(e, "down")] for e in range(self.E)]).contiguous()
        # one product gives the router's logits, the logit of the shared expert's gate and whatever rows the block
        # stacks behind (``append_rows``)
        rows = [tensors[self._n("router")]]
        if self.shared is not None:
            self.shared.bind(tensors)
            rows.append(tensors[self._n("shared_gate")].reshape(1, -1))
        self._route_rows = torch.cat(rows, dim=0)
        self.route = Linear(self._route_rows, None, f"{self.prefix}.route")
        self.extra = None

    def append_rows(self, weight: torch.Tensor) -> None:
        """Stack more rows of the layer's input product behind the router's; their result is left in
        ``ctx.extra_product`` (float32 [T, rows]) by ``forward``."""
        at = self._route_rows.shape[0]
        self.route = Linear(torch.cat([self._route_rows, weight], dim=0), None, f"{self.prefix}.route")
        self.extra = (at, weight.shape[0])

    def forward(self, ctx, h):
        T, d = h.shape
        z = self.route.forward(h, out_dtype=torch.float32)
        idx, w, gate = L.moe_select(z, self.E, self.top, self.E if self.shared is not None else -1)
        ctx.extra_product = z[:, self.extra[0]:self.extra[0] + self.extra[1]] if self.extra else None
        shared = None
        if self.shared is not None:
            shared = self.shared.forward(ctx, h)
            if isinstance(shared, K.Partials):
                shared = shared.materialize(torch.float32)
            elif shared.dtype != torch.float32:
                shared = shared.float()
        y = torch.empty((T, d), dtype=torch.float32, device=h.device)
        from ..kernels import moe as M
        M.experts(h, self.gate_up, self.down, idx, w, shared, gate, y)
        return y


class GroupedMoe(FeedForward):
    """Experts of the gated form down(glu(gate h, up h)) (the spec's ``activation``, ``limit``, ``act_alpha``), routed
    by a softmax over all experts: z = Wr h in 32-bit, s = softmax(z); the ``top`` experts with the largest
    s + correction are picked among the ``route_keep`` best of ``route_groups`` groups of neighbouring experts;
    delta = sum_c s_c / (sum of the picked s + 1e-20) * expert_c(h).  A shared expert of the same form
    (``shared_intermediate``, ``shared_limit``) runs for every token and is added as it is.

    The experts' matrices are stacked as in ``MoeSwiGlu`` ([E, 2 ff, d] with rows alternating gate_j, up_j; [E, d, ff])
    and run through the same three expert kernels."""

    def __init__(self, spec: FeedForwardSpec, prefix: str):
        from .mlp import GluMlp
        self.spec, self.prefix = spec, prefix
        self.E, self.top, self.ff = int(spec.experts), int(spec.top), int(spec.intermediate)
        self.names = spec.tensor_names()
        self.act = None if spec.activation == "swiglu" else (spec.activation, float(spec.limit), float(spec.act_alpha))
        self.shared: Optional[SwiGluMlp] = None
        if spec.shared_intermediate > 0:
            sh = self.names["shared"]
            sub = FeedForwardSpec(kind="glu", hidden=spec.hidden, intermediate=spec.shared_intermediate,
                                  activation=spec.activation, limit=spec.shared_limit, act_alpha=spec.act_alpha,
                                  names=tuple((r, f"{sh}.{self.names[r]}") for r in ("gate", "up", "down")),
                                  weight_suffix=spec.weight_suffix)
            self.shared = GluMlp(sub, prefix)

    _expert = MoeSwiGlu._expert
    _n = MoeSwiGlu._n

    def declare(self) -> List[TensorDecl]:
        d, ff = self.spec.hidden, self.ff
        out: List[TensorDecl] = []
        for e in range(self.E):
            out += [TensorDecl(self._expert(e, "gate"), (ff, d)), TensorDecl(self._expert(e, "up"), (ff, d)),
                    TensorDecl(self._expert(e, "down"), (d, ff))]
        out.append(TensorDecl(self._n("router"), (self.E, d)))
        if self.spec.route_correction:
            out.append(TensorDecl(f"{self.prefix}.{self.names['correction']}", (self.E,), role="bias"))
        if self.shared is not None:
            out += self.shared.declare()
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        g = torch.stack([tensors[self._expert(e, "gate")] for e in range(self.E)])
        u = torch.stack([tensors[self._expert(e, "up")] for e in range(self.E)])
        self.gate_up = torch.stack([g, u], dim=2).reshape(self.E, 2 * self.ff, self.spec.hidden).contiguous()
        self.down = torch.stack([tensors[self._expert(e, "down")] for e in range(self.E)]).contiguous()
        self.route = Linear(tensors[self._n("router")], None, f"{self.prefix}.route")
        self.correction = None
        if self.spec.route_correction:
            self.correction = tensors[f"{self.prefix}.{self.names['correction']}"].float().contiguous()
        if self.shared is not None:
            self.shared.bind(tensors)

    def forward(self, ctx, h):
        T, d = h.shape
        z = self.route.forward(h, out_dtype=torch.float32)
        idx, w = L.moe_select_grouped(z, self.correction, self.E, self.top, self.spec.route_groups, self.spec.route_keep)
        shared = None
        if self.shared is not None:
            shared = self.shared.forward(ctx, h)
            if isinstance(shared, K.Partials):
                shared = shared.materialize(torch.float32)
            elif shared.dtype != torch.float32:
                shared = shared.float()
        y = torch.empty((T, d), dtype=torch.float32, device=h.device)
        from ..kernels import moe as M
        M.experts(h, self.gate_up, self.down, idx, w, shared, None, y, self.act)
        return y


class ScoredMoe(FeedForward):
    """Ungated experts down(act(up h)) (``activation`` "relu2") chosen by scores: z = Wr h in 32-bit, s = sigmoid(z)
    (``route_score``); the ``top`` largest scores are chosen; the weights are those scores, over their sum only with
    ``route_renorm``.  With ``weight_input`` the weight multiplies what the expert reads, delta = sum_c expert_c(w_c h),
    else its result.  A shared expert of the same form (``shared_intermediate``) runs for every token and is added.

    The experts' matrices are stacked when the weights are bound: up [E, ff, d], down [E, d, ff]."""

    def __init__(self, spec: FeedForwardSpec, prefix: str):
        from .mlp import Relu2Mlp
        if spec.activation != "relu2":
            raise ValueError(f"ungated experts with activation '{spec.activation}': only 'relu2' has kernels")
        if spec.route_score != "sigmoid":
            raise ValueError(f"scores '{spec.route_score}' of the router's logits: only 'sigmoid' has a kernel")
        self.spec, self.prefix = spec, prefix
        self.E, self.top, self.ff = int(spec.experts), int(spec.top), int(spec.intermediate)
        self.names = spec.tensor_names()
        self.shared = None
        if spec.shared_intermediate > 0:
            sh = self.names["shared"]
            sub = FeedForwardSpec(kind="relu2", hidden=spec.hidden, intermediate=spec.shared_intermediate,
                                  names=tuple((r, f"{sh}.{self.names[r]}") for r in ("up", "down")),
                                  weight_suffix=spec.weight_suffix)
            self.shared = Relu2Mlp(sub, prefix)

    _expert = MoeSwiGlu._expert
    _n = MoeSwiGlu._n

    def declare(self) -> List[TensorDecl]:
        d, ff = self.spec.hidden, self.ff
        out: List[TensorDecl] = []
        for e in range(self.E):
            out += [TensorDecl(self._expert(e, "up"), (ff, d)), TensorDecl(self._expert(e, "down"), (d, ff))]
        out.append(TensorDecl(self._n("router"), (self.E, d)))
        if self.shared is not None:
            out += self.shared.declare()
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.up = torch.stack([tensors[self._expert(e, "up")] for e in range(self.E)]).contiguous()
        self.down = torch.stack([tensors[self._expert(e, "down")] for e in range(self.E)]).contiguous()
        self.route = Linear(tensors[self._n("router")], None, f"{self.prefix}.route")
        if self.shared is not None:
            self.shared.bind(tensors)

    def forward(self, ctx, h):
        T, d = h.shape
        # few rows: the router's product and the shared expert's last product stay split-K partial sums, which the
        # selection and the experts' last kernel add up themselves
        z = self.route.forward(h, out_dtype=torch.float32, defer=True)
        idx, w = L.moe_select_scored(z, self.E, self.top, renorm=bool(self.spec.route_renorm))
        shared = None
        if self.shared is not None:
            shared = self.shared.forward(ctx, h)
            if not isinstance(shared, K.Partials) and shared.dtype != torch.float32:
                shared = shared.float()
        y = torch.empty((T, d), dtype=torch.float32, device=h.device)
        from ..kernels import moe as M
        M.plain_experts(h, self.up, self.down, idx, w, bool(self.spec.weight_input), shared, y)
        return y
