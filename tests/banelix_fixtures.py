"""Small Banelix configurations, random model folders and plain logits for the tests."""
from __future__ import annotations

import functools
import os
import random
import tempfile
from typing import Dict, List

import numpy as np
import torch

import plain_banelix as PB
import plain_qwen2

_TMP = tempfile.mkdtemp(prefix="infero_b200_banelix_")
# Largest |engine - plain| over a row of logits, relative to the request's largest |logit|.
TOL = {"float32": 3e-5, "bfloat16": 0.12}


def _left(heads, kv, dim, scale, dims=None, base=10000.0, bands=None):
    rot = {"base": base, "dims": dim if dims is None else dims}
    if bands:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), bands))
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale, "rot": rot}


def _par(left, width, blocks, conv, ls=0.7, rs=1.1):
    return {"left": left, "right": {"width": width, "blocks": blocks, "conv": conv}, "left_scale": ls, "right_scale": rs}


def _att(heads, kv, dim, vdim, scale, window, dims=None, base=5000.0, ramp=None, kv_from=None):
    rot = {"base": base, "dims": dim if dims is None else dims}
    if ramp:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), ramp))
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window}, "rot": rot}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


# A: sizes the tensor-core kernels take (heads of 64, widths in multiples of 64); a layer that borrows keys and values and
#    looks further back than their owner does; both kinds of frequency scaling inside a short prompt
A = {"architecture": "Banelix", "vocab": 211, "width": 128, "norm": {"eps": 2e-5}, "embedding": {"scale": 3.0},
     "residual_mult": 0.5, "layers": [
         _layer("attention", _att(4, 2, 64, 64, 0.2, 24, ramp=(4.0, 32, 8.0, 1.0)), 192),
         _layer("parallel", _par(_left(4, 2, 64, 0.15, dims=16, base=900.0, bands=(4.0, 1.0, 3.0, 48)), 64, 2, 4), 192),
         _layer("attention", _att(2, 2, 64, 64, 0.2, 41, ramp=(4.0, 32, 8.0, 1.0), kv_from=0), 0),
         _layer("parallel", _par(_left(2, 1, 64, 0.15, base=900.0), 128, 1, 3, ls=1.0, rs=0.4), 128)]}
# B: odd sizes that no tensor-core kernel takes; values wider and narrower than keys; three blocks; two taps; no
#    residual_mult key; the first layer is a parallel one
B = {"architecture": "Banelix", "vocab": 97, "width": 36, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "layers": [
    _layer("parallel", _par(_left(3, 3, 10, 0.4, dims=4, base=77.0), 30, 3, 2), 20),
    _layer("attention", _att(6, 2, 6, 10, 0.5, 7, base=40.0), 0),
    _layer("attention", _att(2, 1, 12, 5, 0.3, 19, dims=6, base=9.0, ramp=(3.0, 12, 6.0, 1.0)), 24),
    _layer("attention", _att(4, 2, 6, 10, 0.5, 5, base=40.0, kv_from=1), 12)]}
# C: values that make mechanisms vanish: one head, one block, one tap (no convolution tail), a window of one (a token
#    sees itself only) and a window longer than any prompt, no rotated coordinates, scales of 1
C = {"architecture": "Banelix", "vocab": 61, "width": 40, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
     "residual_mult": 1.0, "layers": [
         _layer("attention", _att(1, 1, 8, 8, 0.35, 1), 16),
         _layer("parallel", _par(_left(1, 1, 16, 0.3, dims=0), 24, 1, 1, ls=1.0, rs=1.0), 0),
         _layer("attention", _att(5, 5, 8, 4, 0.35, 4096, dims=2), 48)]}
# D: heads of 128 and a long window for the bf16 kernels; four taps; borrowed keys with the same window
D = {"architecture": "Banelix", "vocab": 301, "width": 256, "norm": {"eps": 1e-6}, "embedding": {"scale": 8.0},
     "residual_mult": 0.4, "layers": [
         _layer("parallel", _par(_left(4, 2, 128, 0.09, dims=64, bands=(8.0, 1.0, 4.0, 64)), 256, 4, 4, ls=0.8, rs=1.2), 256),
         _layer("attention", _att(4, 1, 128, 128, 0.09, 100, ramp=(2.0, 64, 16.0, 1.0)), 256),
         _layer("attention", _att(4, 1, 128, 128, 0.09, 100, ramp=(2.0, 64, 16.0, 1.0), kv_from=1), 256)]}
CONFIGS = {"A": A, "B": B, "C": C, "D": D}


@functools.lru_cache(maxsize=None)
def model_dir(name: str, seed: int = 5, store: str = "bfloat16", sharp: float = 2.5) -> str:
    """A random model folder.  Random projections give an almost flat softmax, which hides a wrong key, so the query
    projections are multiplied by ``sharp``; and a random decay forgets within a few tokens, which hides a lost state,
    so the decay's parameter is moved to where a state lasts for dozens of tokens."""
    from safetensors.torch import load_file, save_file
    from infero_b200.loading import write_random_model_dir
    d = os.path.join(_TMP, f"{name}_{seed}_{store}_{sharp}")
    write_random_model_dir(d, CONFIGS[name], seed=seed, dtype=store, std=0.15, norm_std=0.1)
    p = os.path.join(d, "model.safetensors")
    w = load_file(p)
    for k in list(w):
        if k.endswith(".q"):
            w[k] = (w[k].float() * sharp).to(w[k].dtype)
        if k.endswith(".lam"):
            w[k] = (w[k].float() - 3.5).to(w[k].dtype)
        if k.endswith(".ra") or k.endswith(".ri"):
            w[k] = (w[k].float() * 3.0).to(w[k].dtype)
    save_file(w, p, metadata={"format": "pt"})
    return d


@functools.lru_cache(maxsize=None)
def plain_model(mdir: str):
    return plain_qwen2.read_model(mdir, torch.float64)


def plain_logits(mdir: str, reqs: Dict[str, List[int]]) -> Dict[str, np.ndarray]:
    cfg, w = plain_model(mdir)
    return {rid: PB.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}


def make_requests(name: str, lengths, seed: int = 0) -> Dict[str, List[int]]:
    rng = random.Random(seed)
    V = CONFIGS[name]["vocab"]
    return {f"r{i}": [rng.randrange(V) for _ in range(n)] for i, n in enumerate(lengths)}
