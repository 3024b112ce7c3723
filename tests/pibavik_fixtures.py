"""Small Pibavik configurations, random model folders and plain logits for the tests."""
from __future__ import annotations

import copy
import functools
import os
import random
import tempfile
from typing import Dict, List

import numpy as np
import torch

import plain_pibavik as PP
import plain_qwen2

_TMP = tempfile.mkdtemp(prefix="infero_b200_pibavik_")
# Largest |engine - plain| over a row of logits, relative to the request's largest |logit|.
TOL = {"float32": 3e-5, "bfloat16": 0.12}


def _left(heads, kv, dim, vdim, scale, window=None, dims=None, base=10000.0):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if dims is None or dims > 0:
        m["rot"] = {"base": base, "dims": dim if dims is None else dims}
    return m


def _right(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def _par(left, right, ls=0.7, rs=1.2):
    return {"left": left, "right": right, "left_scale": ls, "right_scale": rs}


def _att(heads, kv, dim, vdim, scale, window, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _lat(heads, dim, vdim, kv_rank, q_rank, scale):
    return {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale}


def _moe(experts, top, ff, shared=0):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def _layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


# A: sizes the tensor-core kernels take (heads of 64, a latent of 64); a layer that borrows keys and values and looks
#    further back than their owner does; two experts of six per token
A = {"architecture": "Pibavik", "vocab": 211, "width": 128, "norm": {"eps": 2e-5}, "embedding": {"scale": 3.0}, "layers": [
    _layer("parallel", _par(_left(4, 2, 64, 64, 0.2, window=24, dims=32, base=5000.0), _right(4, 32, 32, 2, 4, 2)), _moe(6, 2, 64, 32)),
    _layer("attention", _att(4, 2, 64, 64, 0.2, 33), _moe(6, 2, 64, 32)),
    _layer("latent_attention", _lat(4, 32, 32, 64, 48, 0.25), _moe(6, 2, 64)),
    _layer("attention", _att(8, 2, 64, 64, 0.15, 50, kv_from=1), None),
    _layer("parallel", _par(_left(2, 1, 64, 64, 0.2, window=40, base=300.0), _right(2, 64, 16, 1, 3, 1), ls=1.0, rs=0.5), _moe(6, 2, 64, 32))]}
# B: odd sizes that no tensor-core kernel takes; values wider and narrower than keys; two taps; every expert chosen; the
#    first layer is a parallel one; a layer without feed-forward
B = {"architecture": "Pibavik", "vocab": 97, "width": 36, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.5}, "layers": [
    _layer("parallel", _par(_left(3, 3, 10, 6, 0.4, window=7, dims=4, base=77.0), _right(3, 10, 5, 1, 2, 3)), _moe(5, 5, 20)),
    _layer("latent_attention", _lat(2, 6, 10, 12, 7, 0.5), None),
    _layer("attention", _att(6, 2, 6, 10, 0.5, 5), _moe(3, 1, 12, 24)),
    _layer("attention", _att(2, 1, 12, 5, 0.3, 19), _moe(5, 5, 20)),
    _layer("attention", _att(4, 2, 6, 10, 0.5, 11, kv_from=2), _moe(5, 2, 20, 8))]}
# C: values that make mechanisms vanish: one head, one expert of one, one tap (no convolution tail), a window of one (a
#    token sees itself only) and a window longer than any prompt, a left mixer that sees every token, no rotated
#    coordinates, scales of 1, no embedding scale, as many groups as heads, one norm group
C = {"architecture": "Pibavik", "vocab": 61, "width": 40, "norm": {"eps": 1e-5}, "layers": [
    _layer("attention", _att(1, 1, 8, 8, 0.35, 1), _moe(1, 1, 16)),
    _layer("parallel", _par(_left(1, 1, 16, 16, 0.3, dims=0), _right(2, 12, 8, 2, 1, 1), ls=1.0, rs=1.0), None),
    _layer("latent_attention", _lat(1, 8, 8, 8, 8, 0.3), _moe(4, 1, 16, 16)),
    _layer("attention", _att(5, 5, 8, 4, 0.35, 4096), _moe(4, 3, 24))]}
# D: heads of 128 and a long window for the bf16 kernels; a latent of 128; a state of 128 rows; four taps; borrowed keys
#    with the same window; every expert chosen (a near tie between experts may fall either way in bf16)
D = {"architecture": "Pibavik", "vocab": 301, "width": 256, "norm": {"eps": 1e-6}, "embedding": {"scale": 8.0}, "layers": [
    _layer("parallel", _par(_left(4, 2, 128, 128, 0.09, window=100, dims=64), _right(4, 64, 128, 2, 4, 2), ls=0.8, rs=1.1), _moe(4, 4, 128, 128)),
    _layer("attention", _att(4, 1, 128, 128, 0.09, 100), _moe(4, 4, 128, 128)),
    _layer("latent_attention", _lat(4, 64, 64, 128, 96, 0.12), _moe(4, 4, 128)),
    _layer("attention", _att(4, 1, 128, 128, 0.09, 100, kv_from=1), _moe(4, 4, 128, 128))]}
CONFIGS = {"A": A, "B": B, "C": C, "D": D}


def all_experts(cfg: dict) -> dict:
    """The configuration with every expert chosen for every token."""
    out = copy.deepcopy(cfg)
    for L in out["layers"]:
        if L["mlp"]:
            L["mlp"]["router"]["top"] = L["mlp"]["router"]["experts"]
    return out


CONFIGS["A_all"] = all_experts(A)
CONFIGS["B_all"] = all_experts(B)


@functools.lru_cache(maxsize=None)
def model_dir(name: str, seed: int = 5, store: str = "bfloat16", sharp: float = 1.25) -> str:
    """A random model folder.  Random projections give an almost flat softmax, which hides a wrong key, so the query
    projections are multiplied by ``sharp``; and random step sizes forget within a few tokens, which hides a lost
    state, so the step's bias is moved to where a state lasts for dozens of tokens."""
    from safetensors.torch import load_file, save_file
    from infero_b200.loading import write_random_model_dir
    d = os.path.join(_TMP, f"{name}_{seed}_{store}_{sharp}")
    write_random_model_dir(d, CONFIGS[name], seed=seed, dtype=store, std=0.15, norm_std=0.1)
    p = os.path.join(d, "model.safetensors")
    w = load_file(p)
    for k in list(w):
        if k.endswith(".q") or k.endswith(".uq"):
            w[k] = (w[k].float() * (1.0 if name == "D" else sharp)).to(w[k].dtype)     # D: wide heads are sharp enough
        if k.endswith(".dt_bias"):
            w[k] = (w[k].float() - 2.5).to(w[k].dtype)
        if k.endswith(".router"):
            w[k] = (w[k].float() * 4.0).to(w[k].dtype)
    save_file(w, p, metadata={"format": "pt"})
    return d


@functools.lru_cache(maxsize=None)
def plain_model(mdir: str):
    return plain_qwen2.read_model(mdir, torch.float64)


def plain_logits(mdir: str, reqs: Dict[str, List[int]]) -> Dict[str, np.ndarray]:
    cfg, w = plain_model(mdir)
    return {rid: PP.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}


def make_requests(name: str, lengths, seed: int = 0) -> Dict[str, List[int]]:
    rng = random.Random(seed)
    V = CONFIGS[name]["vocab"]
    return {f"r{i}": [rng.randrange(V) for _ in range(n)] for i, n in enumerate(lengths)}
