"""A selective state-space recurrence with a scalar decay per head (the state-space-duality form of Mamba-2)."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.spec import MixerSpec
from ..kernels import layer_ops as L
from .base import Mixer, StateSpec, TensorDecl
from .linear import Linear


class SsdMixer(Mixer):
    """One input product gives [z | x | B | C | dt] in 32-bit: z and x are ``num_heads`` * ``value_dim`` wide, B and C
    ``rec_groups`` * ``state_dim`` wide, dt has one number per head.  x, B and C pass a causal convolution of
    ``conv_taps`` taps per channel (with a bias) and silu; dt = softplus(dt + dt_bias); head h (group
    h // (heads / groups)) keeps S [state_dim, value_dim]:  S <- exp(-exp(A_log_h) dt) S + dt B x^T,  y = S^T C + D_h x.
    y * silu(z) is RMS-normed in ``norm_groups`` equal parts, times a weight, and goes through the output product.

    The request's state slot is a float32 vector: the convolution's last taps - 1 inputs, then S; zero when the request
    starts.  Convolution, step sizes, decays, the state and the norm are 32-bit on both precisions.  The three stages
    (``input_rows``, ``core``, ``output_weight``) can be used separately, see ``NormedAttention``."""

    def __init__(self, spec: MixerSpec, prefix: str):
        self.spec, self.prefix = spec, prefix
        self.Hn, self.P, self.N = int(spec.num_heads), int(spec.v_dim), int(spec.state_dim)
        self.G, self.parts, self.taps = int(spec.rec_groups), int(spec.norm_groups), int(spec.conv_taps)
        if min(self.Hn, self.P, self.N, self.G, self.parts) <= 0:
            raise ValueError("a state-space mixer needs heads, value_dim, state_dim, groups and norm groups")
        if self.Hn % self.G or (self.Hn * self.P) % self.parts:
            raise ValueError(f"{self.Hn} heads of {self.P} do not split into {self.G} groups / {self.parts} norm groups")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"{self.taps} taps outside 1..16")
        if self.N > 256:
            raise ValueError(f"a state of {self.N} rows, at most 256")
        self.inner = self.Hn * self.P
        self.CH = self.inner + 2 * self.G * self.N
        self.n_rows = 2 * self.inner + 2 * self.G * self.N + self.Hn
        self.names = spec.tensor_names()
        self.inp: Linear = None
        self.out: Linear = None

    def _n(self, role: str, matrix: bool = True) -> str:
        return f"{self.prefix}.{self.names[role]}" + (self.spec.weight_suffix if matrix else "")

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((L.ssd_state_floats(self.Hn, self.N, self.P, self.G, self.taps),), torch.float32)

    def declare(self) -> List[TensorDecl]:
        d = self.spec.hidden
        return [TensorDecl(self._n("in"), (self.n_rows, d)),
                TensorDecl(self._n("conv", False), (self.CH, self.taps), role="bias", init="conv"),
                TensorDecl(self._n("conv_bias", False), (self.CH,), role="bias"),
                TensorDecl(self._n("dt_bias", False), (self.Hn,), role="bias"),
                TensorDecl(self._n("a_log", False), (self.Hn,), role="bias"),
                TensorDecl(self._n("skip", False), (self.Hn,), role="bias"),
                TensorDecl(self._n("out_norm", False), (self.inner,), role="norm", init="ones"),
                TensorDecl(self._n("o"), (d, self.inner))]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        f32 = lambda r: tensors[self._n(r, False)].float().contiguous()          # noqa: E731
        self._rows = tensors[self._n("in")]
        self.inp = Linear(self._rows, None, self._n("in"))
        self.conv_w, self.conv_b = f32("conv"), f32("conv_bias")
        self.dt_bias, self.a_log, self.skip, self.norm_w = f32("dt_bias"), f32("a_log"), f32("skip"), f32("out_norm")
        self._out_w = tensors[self._n("o")]
        self.out = Linear(self._out_w, None, self._n("o"))

    def input_rows(self):
        return self._rows, None

    def output_weight(self) -> torch.Tensor:
        return self._out_w

    @property
    def out_width(self) -> int:
        return self.inner

    def core(self, ctx, proj: torch.Tensor, off: int, slot, out: torch.Tensor, scale: float = 1.0) -> None:
        q_lens = getattr(ctx, "h_q_len", None)
        longest = int(getattr(ctx, "max_q_len", 0)) or (int(q_lens.max()) if q_lens is not None and len(q_lens) else int(proj.shape[0]))
        L.ssd(proj, off, off + self.inner, off + self.inner + self.CH, self.conv_w, self.conv_b, self.dt_bias, self.a_log,
              self.skip, self.norm_w, float(self.spec.norm_eps), self.parts, ctx.state(slot.cache), ctx.tok_entry,
              ctx.entry_q_start, ctx.entry_q_len, ctx.entry_slot, ctx.n_entries, out, self.Hn, self.G, self.N, self.P,
              scale, max_q_len=longest)

    def forward(self, ctx, h, slot):
        proj = self.inp.forward(h, out_dtype=torch.float32)
        act = torch.empty((h.shape[0], self.inner), dtype=h.dtype, device=h.device)
        self.core(ctx, proj, 0, slot, act)
        return self.out.forward(act, defer=True, residual=True, out_dtype=torch.float32)
