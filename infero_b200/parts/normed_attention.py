"""Grouped-query attention over the paged cache with normed queries and keys."""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .. import kernels as K
from ..config.spec import MixerSpec
from ..kernels import layer_ops as L
from ..registry import part_class
from .base import KvCacheSpec, Mixer, TensorDecl
from .linear import Linear


class NormedAttention(Mixer):
    """H query heads over G key/value heads (query head h reads kv head h // (H/G)), keys ``head_dim`` wide, values
    ``value_dim`` wide.  One stacked input product gives [q | k | v | gate] (those the layer has) in 32-bit, biases
    added; ``qk_prepare`` norms and rotates q and k (``qk_norm_kind`` "projection": weighted RMS over the whole
    projection before the rotation; "head_unit": unit RMS per head after it; "head": RMS per head with a weight shared
    by the heads, before the rotation) and appends keys and values to the cache; then attention (causal, optionally
    windowed, optionally with a sink in the softmax's denominator, optionally with a distance bias: head h's score
    loses 2^(-b (h + 1) / H) times the distance to the key, b = ``distance_slope_exp``), an optional sigmoid gate per
    head, and the output product.

    ``value_from_key``: no value projection; the cached value of a token is its key as projected.  ``borrows_cache``:
    no key or value tensors at all; the layer reads the cache of the schedule entry it is pointed at.

    A mixer that runs several mixers side by side (``ParallelMixer``) uses the three stages separately:
    ``input_rows`` (what to stack into a common input product), ``core`` (from product rows to the activations the
    output product takes, times a constant) and ``output_weight``."""

    NORM_MODES = {"": 0, "projection": 1, "head_unit": 2, "head": 3}

    def __init__(self, spec: MixerSpec, prefix: str):
        if spec.num_kv_heads <= 0 or spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} heads are not a multiple of {spec.num_kv_heads} kv heads")
        if spec.qk_norm_kind not in self.NORM_MODES:
            raise ValueError(f"unknown norm of queries and keys '{spec.qk_norm_kind}'")
        self.spec, self.prefix = spec, prefix
        self.H, self.G, self.D, self.V = spec.num_heads, spec.num_kv_heads, spec.head_dim, spec.v_dim
        if spec.value_from_key and self.V != self.D:
            raise ValueError("values taken from the keys are as wide as the keys")
        self.own_kv = not spec.borrows_cache
        self.own_v = self.own_kv and not spec.value_from_key
        self.names = spec.tensor_names()
        self.rope = None
        if spec.position is not None and spec.position.rotary_dim > 0:
            self.rope = part_class("position", spec.position.kind)(spec.position)
            if getattr(self.rope, "pairing", None) == "adjacent" or not hasattr(self.rope, "inv_freq64"):
                raise ValueError(f"this mixer turns pairs (i, i + dims/2) from a frequency table; position kind "
                                 f"'{spec.position.kind}' does otherwise")
        # columns of the stacked product
        self.q_off = 0
        self.k_off = self.H * self.D if self.own_kv else -1
        self.v_off = self.H * self.D + self.G * self.D if self.own_v else -1
        self.g_off = self.H * self.D + (self.G * self.D if self.own_kv else 0) + (self.G * self.V if self.own_v else 0)
        self.n_rows = self.g_off + (self.H if spec.out_gate else 0)
        self.inp: Linear = None
        self.out: Linear = None

    def _n(self, role: str, matrix: bool = True) -> str:
        return f"{self.prefix}.{self.names[role]}" + (self.spec.weight_suffix if matrix else "")

    def _roles(self) -> List[Tuple[str, int]]:
        r = [("q", self.H * self.D)]
        if self.own_kv:
            r.append(("k", self.G * self.D))
        if self.own_v:
            r.append(("v", self.G * self.V))
        return r

    def cache_spec(self) -> Optional[KvCacheSpec]:
        s = self.spec
        keep = s.keep_window if s.keep_window is not None else s.window
        return KvCacheSpec(self.G, self.D, keep, v_head_dim=self.V)

    def declare(self) -> List[TensorDecl]:
        s, d = self.spec, self.spec.hidden
        out = [TensorDecl(self._n(r), (n, d)) for r, n in self._roles()]
        if s.qkv_bias:
            out += [TensorDecl(self._n(r + "_bias", False), (n,), role="bias") for r, n in self._roles()]
        if s.qk_norm_kind == "projection":
            out += [TensorDecl(self._n(r + "_norm", False), (n,), role="norm", init="ones") for r, n in self._roles() if r != "v"]
        if s.qk_norm_kind == "head":
            out += [TensorDecl(self._n(r + "_norm", False), (self.D,), role="norm", init="ones") for r, _ in self._roles() if r != "v"]
        if s.out_gate:
            out.append(TensorDecl(self._n("gate"), (self.H, d)))
        out.append(TensorDecl(self._n("o"), (d, self.H * self.V)))
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        ws = [tensors[self._n(r)] for r, _ in self._roles()]
        if s.out_gate:
            ws.append(tensors[self._n("gate")])
        if len({w.dtype for w in ws}) > 1:
            ws = [w.float() for w in ws]
        self._rows = torch.cat(ws, dim=0).contiguous()
        self._bias = None
        if s.qkv_bias:
            bs = [tensors[self._n(r + "_bias", False)].float() for r, _ in self._roles()]
            if s.out_gate:
                bs.append(torch.zeros(self.H, dtype=torch.float32, device=bs[0].device))
            self._bias = torch.cat(bs).contiguous()
        self.inp = Linear(self._rows, self._bias, f"{self.prefix}.qkv")
        self._out_w = tensors[self._n("o")]
        self.out = Linear(self._out_w, None, self._n("o"))
        self.q_norm = self.k_norm = None
        if s.qk_norm_kind in ("projection", "head"):
            self.q_norm = tensors[self._n("q_norm", False)].float().contiguous()
            self.k_norm = tensors[self._n("k_norm", False)].float().contiguous() if self.own_kv else None
        self.slopes = None
        if s.distance_slope_exp > 0:
            self.slopes = torch.tensor([2.0 ** (-float(s.distance_slope_exp) * (h + 1) / self.H) for h in range(self.H)],
                                       dtype=torch.float32, device=self._out_w.device)

    # ---- the three stages -------------------------------------------------------------------------------------------
    def input_rows(self):
        """(weight [rows, d], bias [rows] float32 or None) of this mixer's share of an input product."""
        return self._rows, self._bias

    def output_weight(self) -> torch.Tensor:
        return self._out_w

    @property
    def out_width(self) -> int:
        return self.H * self.V

    def core(self, ctx, proj: torch.Tensor, off: int, slot, out: torch.Tensor, scale: float = 1.0) -> None:
        """``proj`` float32 [T, >= off + rows]: this mixer's product rows start at column ``off``.  ``out`` [T, H*V] in the
        step's element type (a column slice allowed) receives the heads' results, gated, times ``scale``."""
        s = self.spec
        H, G, D, V = self.H, self.G, self.D, self.V
        T = proj.shape[0]
        dev = proj.device
        kv = ctx.kv_cache(slot.cache)
        table = ctx.block_table(kv.group)
        write = bool(slot.write_cache) and self.own_kv
        if self.own_kv != bool(slot.write_cache):
            raise ValueError("a layer with keys and values of its own writes its cache slot; one without reads another's")
        freq = self.rope.inv_freq64(dev) if self.rope is not None else None
        amp = float(getattr(self.rope, "amplitude", 1.0)) if self.rope is not None else 1.0
        q = torch.empty((T, H * D), dtype=ctx.act_dtype, device=dev)
        L.qk_prepare(proj, off + self.q_off, off + self.k_off if self.own_kv else -1, off + self.v_off if self.own_v else -1,
                     self.NORM_MODES[s.qk_norm_kind], self.q_norm, self.k_norm, s.norm_eps, freq, amp, ctx.positions,
                     ctx.tok_entry, table, kv.page_size, q, kv.k, kv.v, H, G, D, V, write_cache=write)
        direct = not s.out_gate and scale == 1.0
        attn = out if direct else torch.empty((T, H * V), dtype=ctx.act_dtype, device=dev)
        from ..kernels import attention as A
        A.paged_attention_ex(ctx, q, attn, kv, table, H, G, D, V, s.window, s.scale, s.sink, slopes=self.slopes)
        if not direct:
            gate = proj[:, off + self.g_off:off + self.g_off + H] if s.out_gate else None
            L.head_gate(attn, gate, out, H, V, scale)

    def forward(self, ctx, h, slot):
        proj = self.inp.forward(h, out_dtype=torch.float32)
        act = torch.empty((h.shape[0], self.H * self.V), dtype=h.dtype, device=h.device)
        self.core(ctx, proj, 0, slot, act)
        return self.out.forward(act, defer=True, residual=True, out_dtype=torch.float32)
