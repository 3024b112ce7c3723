"""A gated linear recurrence over channels (the recurrent block of Griffin)."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.spec import MixerSpec
from ..kernels import layer_ops as L
from .base import Mixer, StateSpec, TensorDecl
from .linear import Linear


class RgLruMixer(Mixer):
    """Two branches of ``rec_width`` = C channels from one stacked input product [y | x] (32-bit, biases added):
    the gate branch gelu_tanh(y) and the recurrent branch u = conv(x), a causal convolution of ``conv_taps`` taps per
    channel with a bias.  Per block of C / ``rec_blocks`` channels r = sigmoid(Ra u + b) and i = sigmoid(Ri u + b);
    a = exp(-``rec_slope`` r softplus(lam)); S <- a S + sqrt(1 - a^2) i u; the output product takes S * gelu_tanh(y).

    The request's state slot is float32 [taps, C]: the convolution's last taps - 1 inputs, then S; zero when the
    request starts.  Convolution, gates, decay and state are 32-bit on both precisions.  The three stages
    (``input_rows``, ``core``, ``output_weight``) can be used separately, see ``NormedAttention``."""

    def __init__(self, spec: MixerSpec, prefix: str):
        self.spec, self.prefix = spec, prefix
        self.C, self.blocks, self.taps = int(spec.rec_width), int(spec.rec_blocks), int(spec.conv_taps)
        if self.C <= 0 or self.blocks <= 0 or self.C % self.blocks:
            raise ValueError(f"{self.C} channels do not split into {self.blocks} blocks")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"{self.taps} taps outside 1..16")
        self.names = spec.tensor_names()
        self.n_rows = 2 * self.C
        self.inp: Linear = None
        self.out: Linear = None

    def _n(self, role: str, matrix: bool = True) -> str:
        return f"{self.prefix}.{self.names[role]}" + (self.spec.weight_suffix if matrix else "")

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.taps, self.C), torch.float32)

    def declare(self) -> List[TensorDecl]:
        C, d, bs = self.C, self.spec.hidden, self.C // self.blocks
        return [TensorDecl(self._n("y"), (C, d)), TensorDecl(self._n("y_bias", False), (C,), role="bias"),
                TensorDecl(self._n("x"), (C, d)), TensorDecl(self._n("x_bias", False), (C,), role="bias"),
                TensorDecl(self._n("conv", False), (C, self.taps), role="bias", init="conv"),
                TensorDecl(self._n("conv_bias", False), (C,), role="bias"),
                TensorDecl(self._n("ra", False), (self.blocks, bs, bs), role="gate_matrix"),
                TensorDecl(self._n("ra_bias", False), (self.blocks, bs), role="bias"),
                TensorDecl(self._n("ri", False), (self.blocks, bs, bs), role="gate_matrix"),
                TensorDecl(self._n("ri_bias", False), (self.blocks, bs), role="bias"),
                TensorDecl(self._n("lam", False), (C,), role="bias"),
                TensorDecl(self._n("o"), (self.spec.hidden, C))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        wy, wx = tensors[self._n("y")], tensors[self._n("x")]
        if wy.dtype != wx.dtype:
            wy, wx = wy.float(), wx.float()
        self._rows = torch.cat([wy, wx], dim=0).contiguous()
        f32 = lambda r: tensors[self._n(r, False)].float().contiguous()          # noqa: E731
        self._bias = torch.cat([f32("y_bias"), f32("x_bias")]).contiguous()
        self.inp = Linear(self._rows, self._bias, f"{self.prefix}.yx")
        self.conv_w, self.conv_b = f32("conv"), f32("conv_bias")
        self.conv_wt = self.conv_w.t().contiguous()          # tap-major, as the convolution kernel reads it
        ra, ri = tensors[self._n("ra", False)], tensors[self._n("ri", False)]
        if ra.dtype != ri.dtype:
            ra, ri = ra.float(), ri.float()
        self.w_gates = torch.cat([ra, ri], dim=1).contiguous()         # [blocks, 2 bs, bs]: per block Ra's rows, then Ri's
        self.ra_b, self.ri_b = f32("ra_bias").reshape(-1), f32("ri_bias").reshape(-1)
        self.lam = f32("lam")
        self._out_w = tensors[self._n("o")]
        self.out = Linear(self._out_w, None, self._n("o"))

    def input_rows(self):
        return self._rows, self._bias

    def output_weight(self) -> torch.Tensor:
        return self._out_w

    @property
    def out_width(self) -> int:
        return self.C

    def core(self, ctx, proj: torch.Tensor, off: int, slot, out: torch.Tensor, scale: float = 1.0) -> None:
        q_lens = getattr(ctx, "h_q_len", None)
        longest = int(getattr(ctx, "max_q_len", 0)) or (int(q_lens.max()) if q_lens is not None and len(q_lens) else int(proj.shape[0]))
        L.rglru(proj, off, off + self.C, self.conv_w, self.conv_b, self.w_gates, self.ra_b, self.ri_b, self.lam,
                float(self.spec.rec_slope), ctx.state(slot.cache), ctx.tok_entry, ctx.entry_q_start, ctx.entry_q_len,
                ctx.entry_slot, ctx.n_entries, out, scale, max_q_len=longest,
                tensor_cores=ctx.act_dtype == torch.bfloat16, conv_wt=self.conv_wt)

    def forward(self, ctx, h, slot):
        proj = self.inp.forward(h, out_dtype=torch.float32)
        act = torch.empty((h.shape[0], self.C), dtype=h.dtype, device=h.device)
        self.core(ctx, proj, 0, slot, act)
        return self.out.forward(act, defer=True, residual=True, out_dtype=torch.float32)
