"""Latent attention over the paged cache: one small cached row per token makes the keys and values of all heads."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.spec import MixerSpec
from ..registry import part_class
from .base import KvCacheSpec, Mixer, TensorDecl
from .linear import Linear


class LatentAttention(Mixer):
    """H heads; a query head is [D plain | R rotated] wide.  The input product also gives C + R numbers per token:
    the first C, RMS-normed with a weight, are the latent c, the last R a rotated key part shared by all heads.
    Head n's key is [Wuk_n c | rotated part] and its value Wuv_n c (V wide); causal softmax of q . k * scale; with
    ``out_gate`` head n's result is multiplied by sigmoid((Wg h)_n); heads side by side, output product.

    The cache holds the row [c | rotated part] only (one kv head of width C + R, no separate values), and the
    up-projections are carried to the query side: (Wuk_n^T q_plain,n) . c gives the same score as q_plain,n . (Wuk_n c),
    and Wuv_n applied to the softmax-weighted sum of latents the same result as the sum of values.  A step is

        stacked product [q; down; gate]  ->  prepare (norm, rotation, cache append, head-major queries)
        ->  per-head product with Wuk^T  ->  attention over latent rows  ->  per-head product with Wuv
        ->  finish (gate, heads side by side)  ->  output product.

    Rotation: the position part's table (with any stretching of the frequencies and its amplitude) and pairing; R may
    be 0 (no rotated part: positions enter through the causal mask alone).

    ``q_latent_dim`` = Q > 0: the queries have a latent of their own.  The stacked product gives [dq | down (| gate)], the
    first Q columns are RMS-normed with a weight (32-bit) and a second product with Wuq [H (D + R), Q] gives the queries."""

    def __init__(self, spec: MixerSpec, prefix: str):
        self.spec, self.prefix = spec, prefix
        self.H, self.D, self.R, self.V, self.C = spec.num_heads, spec.head_dim, spec.rot_dim, spec.v_dim, spec.latent_dim
        self.Q = int(spec.q_latent_dim)
        if min(self.H, self.D, self.V, self.C) <= 0 or self.R < 0 or self.Q < 0:
            raise ValueError("latent attention needs heads, head_dim, value_dim and latent_dim")
        if spec.window:
            raise ValueError("latent attention keeps every key")
        self.names = spec.tensor_names()
        self.rope, self.pairing, self.amp = None, "half", 1.0
        if spec.position is not None and spec.position.rotary_dim > 0:
            if spec.position.rotary_dim > self.R:
                raise ValueError(f"{spec.position.rotary_dim} rotated coordinates in a part of {self.R}")
            self.rope = part_class("position", spec.position.kind)(spec.position)
            if not hasattr(self.rope, "inv_freq64"):
                raise ValueError(f"latent attention needs a rotary table; position kind '{spec.position.kind}' has none")
            self.pairing = getattr(self.rope, "pairing", "half")
            self.amp = float(getattr(self.rope, "amplitude", 1.0))
        self.qkv: Linear = None
        self.out: Linear = None

    def _n(self, role: str) -> str:
        leaf = self.names[role]
        return f"{self.prefix}.{leaf}" + ("" if role in ("latent_norm", "q_norm") else self.spec.weight_suffix)

    def cache_spec(self) -> Optional[KvCacheSpec]:
        return KvCacheSpec(1, self.C + self.R, None, v_head_dim=0)        # the values are the first C columns of a key row

    def declare(self) -> List[TensorDecl]:
        d, H, D, R, V, C = self.spec.hidden, self.H, self.D, self.R, self.V, self.C
        if self.Q:
            q = [TensorDecl(self._n("q_down"), (self.Q, d)), TensorDecl(self._n("q_norm"), (self.Q,), role="norm", init="ones"),
                 TensorDecl(self._n("q_up"), (H * (D + R), self.Q))]
        else:
            q = [TensorDecl(self._n("q"), (H * (D + R), d))]
        out = q + [TensorDecl(self._n("down"), (C + R, d)),
               TensorDecl(self._n("latent_norm"), (C,), role="norm", init="ones"),
               TensorDecl(self._n("up_k"), (H * D, C)), TensorDecl(self._n("up_v"), (H * V, C)),
               TensorDecl(self._n("o"), (d, H * V))]
        if self.spec.out_gate:
            out.append(TensorDecl(self._n("gate"), (H, d)))
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        H, D, R, V, C = self.H, self.D, self.R, self.V, self.C
        rows = [tensors[self._n("q_down" if self.Q else "q")], tensors[self._n("down")]]
        if self.spec.out_gate:
            rows.append(tensors[self._n("gate")])
        if len({t.dtype for t in rows}) > 1:
            rows = [t.float() for t in rows]
        self.qkv = Linear(torch.cat(rows, dim=0), None, f"{self.prefix}.q_down")
        nq = self.Q or H * (D + R)
        self.q_off, self.kv_off, self.gate_off = 0, nq, nq + C + R
        self.q_norm = self.q_up = None
        if self.Q:
            self.q_norm = tensors[self._n("q_norm")].float().contiguous()
            self.q_up = Linear(tensors[self._n("q_up")], None, self._n("q_up"))
        self.latent_norm = tensors[self._n("latent_norm")].float().contiguous()
        # [H, C, D]: head n's rows of Wuk, transposed, so that the product with the plain query parts is a @ w^T
        self.up_k_t = tensors[self._n("up_k")].view(H, D, C).transpose(1, 2).contiguous()
        self.up_v = tensors[self._n("up_v")].view(H, V, C).contiguous()
        self.out = Linear(tensors[self._n("o")], None, self._n("o"))

    def forward(self, ctx, h, slot):
        from ..kernels import latent_attention as A
        H, D, R, V, C = self.H, self.D, self.R, self.V, self.C
        T, dev = h.shape[0], h.device
        proj = self.qkv.forward(h, out_dtype=torch.float32)             # [T, H (D + R) + C + R (+ H)], never rounded
        kv = ctx.kv_cache(slot.cache)
        table = ctx.block_table(kv.group)
        # whole 128-row tiles per head where the grouped tensor-core product runs
        rows = -(-T // A.TILE) * A.TILE if (h.dtype == torch.bfloat16 and D % 8 == 0 and C % 8 == 0) else T
        q_plain = torch.empty((H, rows, D), dtype=h.dtype, device=dev)
        q_rot = torch.empty((H, rows, R), dtype=torch.float32, device=dev)
        freq = self.rope.inv_freq64(dev) if self.rope is not None else None
        q_src = None
        if self.Q:
            from ..kernels import layer_ops as L
            cq = torch.empty((T, self.Q), dtype=h.dtype, device=dev)
            L.gated_group_norm(proj[:, :self.Q], None, self.q_norm, self.spec.norm_eps, 1, cq)
            q_src = self.q_up.forward(cq, out_dtype=torch.float32)
        A.prepare(proj, self.q_off, self.kv_off, self.latent_norm, self.spec.norm_eps, freq, self.pairing, self.amp,
                  ctx.positions, ctx.tok_entry, table, kv.k, kv.page_size, q_plain, q_rot, T, H, D, R, C,
                  write_cache=slot.write_cache, q_src=q_src)
        q_lat = torch.empty((H, rows, C), dtype=torch.float32, device=dev)
        A.per_head_product(q_plain, self.up_k_t, q_lat, T)
        o_lat = torch.empty((H, rows, C), dtype=h.dtype, device=dev)
        A.attention(ctx, q_lat, q_rot, o_lat, kv, table, T, H, C, R, self.spec.scale)
        val = torch.empty((H, rows, V), dtype=torch.float32, device=dev)
        A.per_head_product(o_lat, self.up_v, val, T)
        attn = torch.empty((T, H * V), dtype=h.dtype, device=dev)
        gate = proj[:, self.gate_off:self.gate_off + H] if self.spec.out_gate else None
        A.finish(val, gate, attn, T, H, V)
        return self.out.forward(attn, defer=True, residual=True)
