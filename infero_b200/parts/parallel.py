"""Several mixers side by side on the same input."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.spec import MixerSpec
from ..registry import part_class
from .base import KvCacheSpec, Mixer, StateSpec, TensorDecl
from .linear import Linear


class ParallelMixer(Mixer):
    """result = sum_b scale_b * mixer_b(h).  The branches are mixers that expose their three stages (``input_rows``,
    ``core``, ``output_weight``): their input rows are stacked into one product of h, each branch's ``core`` writes
    its activations, already times scale_b, into its own columns of one array, and one output product over the
    output weights laid side by side along the contraction adds the branches up:

        [a_1 s_1 | a_2 s_2 | ...] [W_1 | W_2 | ...]^T  =  sum_b s_b W_b a_b.

    At most one branch may keep paged keys and values and at most one a state; both live in this mixer's cache slot."""

    def __init__(self, spec: MixerSpec, prefix: str):
        if not spec.branches or len(spec.branches) != len(spec.branch_scales):
            raise ValueError("a parallel mixer needs branches and one scale per branch")
        self.spec, self.prefix = spec, prefix
        self.branches = [part_class("mixer", b.kind)(b, prefix) for b in spec.branches]
        for b in self.branches:
            if not all(hasattr(b, a) for a in ("input_rows", "core", "output_weight", "out_width")):
                raise ValueError(f"mixer {type(b).__name__} cannot run as a branch: it does not expose its stages")
        if sum(b.cache_spec() is not None for b in self.branches) > 1 or sum(b.state_spec() is not None for b in self.branches) > 1:
            raise ValueError("at most one branch with paged keys and values and one with a state")
        self.scales = [float(s) for s in spec.branch_scales]
        self.inp: Linear = None
        self.out: Linear = None

    def cache_spec(self) -> Optional[KvCacheSpec]:
        return next((c for c in (b.cache_spec() for b in self.branches) if c is not None), None)

    def state_spec(self) -> Optional[StateSpec]:
        return next((s for s in (b.state_spec() for b in self.branches) if s is not None), None)

    def declare(self) -> List[TensorDecl]:
        return [d for b in self.branches for d in b.declare()]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        rows, biases, outs = [], [], []
        for b in self.branches:
            b.bind(tensors)
            w, bias = b.input_rows()
            rows.append(w)
            biases.append(bias)
            outs.append(b.output_weight())
        if len({w.dtype for w in rows}) > 1:
            rows = [w.float() for w in rows]
        if len({w.dtype for w in outs}) > 1:
            outs = [w.float() for w in outs]
        bias = None
        if any(b is not None for b in biases):
            bias = torch.cat([b if b is not None else torch.zeros(w.shape[0], dtype=torch.float32, device=w.device)
                              for b, w in zip(biases, rows)]).contiguous()
        self.inp = Linear(torch.cat(rows, dim=0).contiguous(), bias, f"{self.prefix}.mix.in")
        self.out = Linear(torch.cat(outs, dim=1).contiguous(), None, f"{self.prefix}.mix.out")
        self.row_offsets, self.col_offsets, r, c = [], [], 0, 0
        for b, w in zip(self.branches, rows):
            self.row_offsets.append(r)
            self.col_offsets.append(c)
            r += w.shape[0]
            c += b.out_width
        self.act_width = c
        for b in self.branches:                 # the branches' own products are not used; drop what only they held
            b.inp = b.out = None

    def forward(self, ctx, h, slot):
        proj = self.inp.forward(h, out_dtype=torch.float32)
        act = torch.empty((h.shape[0], self.act_width), dtype=h.dtype, device=h.device)
        for b, r, c, s in zip(self.branches, self.row_offsets, self.col_offsets, self.scales):
            b.core(ctx, proj, r, slot, act[:, c:c + b.out_width], s)
        return self.out.forward(act, defer=True, residual=True, out_dtype=torch.float32)
