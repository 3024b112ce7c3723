"""A plain, slow statement of the Pibavik decoder on whole sequences, one function per mechanism, in
64-bit torch on the CPU.  It is what the engine's kernels, cache and scheduler are held to; it shares
nothing with the package.

Notation: x [T, d] is one sequence (positions 0..T-1); matrices are stored [out, in] and applied as
y = x @ W.T; ``w`` maps tensor names to 64-bit tensors; ``cfg`` is the config.json dictionary.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


# ---- small pieces ------------------------------------------------------------------------------------
def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis, times ``weight`` (None: no weight)."""
    y = x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0.0)


def visible(T: int, window: Optional[int]):
    """[T, T] bool: query i (row) sees key j (column) iff 0 <= i - j (< window)."""
    i = torch.arange(T).unsqueeze(1)
    j = torch.arange(T).unsqueeze(0)
    ok = j <= i
    if window is not None:
        ok = ok & (i - j < window)
    return ok


def softmax_attention(q, k, v, scale: float, window: Optional[int], slopes=None):
    """q [T, H, D], k [T, G, D], v [T, G, V] -> [T, H, V].  Query head h reads key/value head h // (H / G);
    score = q . k * scale - slopes[h] * (i - j) where ``slopes`` is given."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    kk = k.repeat_interleave(rep, dim=1)
    vv = v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale
    if slopes is not None:
        dist = (torch.arange(T).unsqueeze(1) - torch.arange(T).unsqueeze(0)).to(q.dtype)
        s = s - slopes.view(H, 1, 1) * dist
    s = s.masked_fill(~visible(T, window), float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hij,jhv->ihv", p, vv)


# ---- mixer "attention": distance bias, window, optionally another layer's keys and values --------------
def distance_slopes(H: int, dtype=torch.float64):
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=dtype)


def biased_keys_values(h, w, p: str, m: dict):
    T = h.shape[0]
    G, D, V = int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    return (h @ w[p + ".k"].T).view(T, G, D), (h @ w[p + ".v"].T).view(T, G, V)


def biased_attention(h, w, p: str, m: dict, kv):
    T = h.shape[0]
    H, D = int(m["heads"]), int(m["dim"])
    q = (h @ w[p + ".q"].T).view(T, H, D)
    k, v = kv
    a = softmax_attention(q, k, v, float(m["scale"]), int(m["mask"]["size"]), distance_slopes(H, h.dtype))
    return a.reshape(T, -1) @ w[p + ".o"].T


# ---- mixer "latent_attention" --------------------------------------------------------------------------
def latent_attention(h, w, p: str, m: dict, eps: float):
    T = h.shape[0]
    H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    cq = rms_norm(h @ w[p + ".dq"].T, w[p + ".dq.norm"], eps)
    q = (cq @ w[p + ".uq"].T).view(T, H, D)
    c = rms_norm(h @ w[p + ".dkv"].T, w[p + ".dkv.norm"], eps)
    k = (c @ w[p + ".uk"].T).view(T, H, D)
    v = (c @ w[p + ".uv"].T).view(T, H, V)
    a = softmax_attention(q, k, v, float(m["scale"]), None)
    return a.reshape(T, -1) @ w[p + ".o"].T


# ---- mixer "parallel": gated, normed, partly rotated window attention beside a state-space recurrence --
def rotate_half(x, base: float, dims: int):
    """x [T, n, D]: coordinate i < dims/2 turns with coordinate i + dims/2 by position * base^(-2i/dims)."""
    if dims == 0:
        return x
    T = x.shape[0]
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    ang = torch.arange(T, dtype=x.dtype).unsqueeze(1) * f.unsqueeze(0)          # [T, half]
    c, s = torch.cos(ang).unsqueeze(1), torch.sin(ang).unsqueeze(1)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def left_attention(h, w, p: str, m: dict, eps: float):
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = rms_norm((h @ w[p + ".q"].T).view(T, H, D), w[p + ".q.norm"], eps)
    k = rms_norm((h @ w[p + ".k"].T).view(T, G, D), w[p + ".k.norm"], eps)
    v = (h @ w[p + ".v"].T).view(T, G, V)
    rot = m.get("rot") or {}
    dims = int(rot.get("dims", 0))
    if dims:
        q, k = rotate_half(q, float(rot["base"]), dims), rotate_half(k, float(rot["base"]), dims)
    window = int(m["mask"]["size"]) if m.get("mask") else None
    a = softmax_attention(q, k, v, float(m["scale"]), window)
    a = a * torch.sigmoid(h @ w[p + ".g"].T).unsqueeze(-1)
    return a.reshape(T, -1) @ w[p + ".o"].T


def causal_conv(x, taps_w, bias):
    """x [T, C], taps_w [C, K] (the last column multiplies the current token), zeros before the sequence."""
    T, C = x.shape
    K = taps_w.shape[1]
    pad = torch.cat([torch.zeros(K - 1, C, dtype=x.dtype), x], dim=0)
    out = bias.unsqueeze(0).expand(T, C).clone()
    for j in range(K):
        out = out + pad[j:j + T] * taps_w[:, j]
    return out


def state_space(x, B, C, dt, A_log, D):
    """x [T, heads, P], B and C [T, groups, N], dt [T, heads] (already positive).  Per head a state S [N, P]:
    S <- exp(-exp(A_log) dt) S + dt B x^T;  y = S^T C + D x."""
    T, Hn, P = x.shape
    Gn, N = B.shape[1], B.shape[2]
    per = Hn // Gn
    S = torch.zeros(Hn, N, P, dtype=x.dtype)
    rate = torch.exp(A_log)
    ys = []
    for t in range(T):
        Bt = B[t].repeat_interleave(per, dim=0)          # [heads, N]
        Ct = C[t].repeat_interleave(per, dim=0)
        decay = torch.exp(-rate * dt[t])                 # [heads]
        S = decay.view(Hn, 1, 1) * S + dt[t].view(Hn, 1, 1) * Bt.unsqueeze(2) * x[t].unsqueeze(1)
        ys.append(torch.einsum("hnp,hn->hp", S, Ct) + D.view(Hn, 1) * x[t])
    return torch.stack(ys)


def grouped_rms_norm(y, weight, parts: int, eps: float):
    T, n = y.shape
    z = rms_norm(y.view(T, parts, n // parts), None, eps).reshape(T, n)
    return z * weight


def right_state_space(h, w, p: str, m: dict, eps: float):
    T = h.shape[0]
    Hn, P, N, Gn = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    inner = Hn * P
    proj = h @ w[p + ".in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * Gn * N], proj[:, 2 * inner + 2 * Gn * N:]
    xbc = silu(causal_conv(xbc, w[p + ".conv"], w[p + ".conv.b"]))
    x = xbc[:, :inner].view(T, Hn, P)
    B = xbc[:, inner:inner + Gn * N].view(T, Gn, N)
    C = xbc[:, inner + Gn * N:].view(T, Gn, N)
    dt = softplus(dt + w[p + ".dt_bias"])
    y = state_space(x, B, C, dt, w[p + ".A_log"], w[p + ".D"]).reshape(T, inner)
    y = grouped_rms_norm(y * silu(z), w[p + ".norm"], int(m["norm_groups"]), eps)
    return y @ w[p + ".o"].T


def parallel_mixer(h, w, p: str, m: dict, eps: float):
    return float(m["left_scale"]) * left_attention(h, w, p + ".left", m["left"], eps) \
        + float(m["right_scale"]) * right_state_space(h, w, p + ".right", m["right"], eps)


# ---- feed-forward -------------------------------------------------------------------------------------
def relu2_expert(h, w, p: str):
    return torch.relu(h @ w[p + ".up"].T).pow(2) @ w[p + ".down"].T


def routed_experts(h, w, p: str, ml: dict):
    """Scores sigmoid(Wr h); the ``top`` largest are chosen (the lowest index wins a tie); a chosen expert's score
    multiplies what the expert reads; a shared expert is added."""
    E, top = int(ml["router"]["experts"]), int(ml["router"]["top"])
    s = torch.sigmoid(h @ w[p + ".router"].T)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(E), key=lambda e: (-float(s[t, e]), e))[:top]
        for e in order:
            out[t] = out[t] + relu2_expert((s[t, e] * h[t]).unsqueeze(0), w, f"{p}.e{e}")[0]
    if ml.get("shared"):
        out = out + relu2_expert(h, w, p + ".shared")
    return out


# ---- the model ----------------------------------------------------------------------------------------
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], residuals: Optional[list] = None):
    """Logits [T, vocab] of one sequence; ``residuals`` collects the residual stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    kept = {}                                       # layer -> its keys and values, for layers that borrow them
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}", L["mixer"]
        h = rms_norm(x, w[p + ".norm1"], eps)
        if L["type"] == "parallel":
            y = parallel_mixer(h, w, p + ".mix", m, eps)
        elif L["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = biased_keys_values(h, w, p + ".mix", m)
            y = biased_attention(h, w, p + ".mix", m, kept[i if src is None else int(src)])
        elif L["type"] == "latent_attention":
            y = latent_attention(h, w, p + ".mix", m, eps)
        else:
            raise ValueError(L["type"])
        x = x + y
        if L.get("mlp") is not None:
            x = x + routed_experts(rms_norm(x, w[p + ".norm2"], eps), w, p + ".mlp", L["mlp"])
        if residuals is not None:
            residuals.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
