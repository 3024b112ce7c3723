"""A plain, slow statement of the Banelix decoder on whole sequences, one function per mechanism, in
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


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z.pow(3))))


def silu(z):
    return z * torch.sigmoid(z)


# ---- rotary positions --------------------------------------------------------------------------------
def base_frequencies(dims: int, base: float) -> List[float]:
    return [base ** (-2.0 * i / dims) for i in range(dims // 2)]


def frequencies_by_wavelength(dims: int, base: float, sc: Optional[dict]):
    """Scaling by bands of the wavelength l = 2 pi / f (record {factor, low, high, original}): short waves
    (l < original / high) stay, long waves (l > original / low) are divided by ``factor``, in between the two are
    blended with s = (original / l - low) / (high - low).  Amplitude 1."""
    f = base_frequencies(dims, base)
    if sc:
        factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        out = []
        for v in f:
            wave = 2.0 * math.pi / v
            if wave < orig / high:
                out.append(v)
            elif wave > orig / low:
                out.append(v / factor)
            else:
                s = (orig / wave - low) / (high - low)
                out.append((1.0 - s) * v / factor + s * v)
        f = out
    return torch.tensor(f, dtype=torch.float64), 1.0


def frequencies_by_ramp(dims: int, base: float, sc: Optional[dict]):
    """Scaling by a ramp over the pair index (record {factor, original, fast, slow}); cos and sin grow by
    0.1 ln(factor) + 1."""
    f = base_frequencies(dims, base)
    if not sc:
        return torch.tensor(f, dtype=torch.float64), 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def index_of(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(index_of(float(sc["slow"]))), dims - 1)
    out = []
    for i, v in enumerate(f):
        ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
        out.append(v / factor * ramp + v * (1.0 - ramp))
    return torch.tensor(out, dtype=torch.float64), 0.1 * math.log(factor) + 1.0


def rotate_half(x, positions, freqs, amp: float):
    """x [T, n, D]: coordinate i < len(freqs) turns with coordinate i + len(freqs); the rest stays."""
    half = freqs.numel()
    if half == 0:
        return x.clone()
    ang = positions.to(torch.float64).unsqueeze(-1) * freqs
    c, s = (torch.cos(ang) * amp).unsqueeze(1), (torch.sin(ang) * amp).unsqueeze(1)
    out = x.clone()
    a, b = x[..., :half], x[..., half:2 * half]
    out[..., :half] = a * c - b * s
    out[..., half:2 * half] = b * c + a * s
    return out


# ---- attention over a whole sequence -----------------------------------------------------------------
def attend(q, k, v, scale: float, window: Optional[int], sink: bool):
    """q [T, H, D], k [T, G, D], v [T, G, V] -> [T, H * V].  Query i sees key j with j <= i and, with a window W,
    i - j < W.  ``sink``: the softmax's denominator has one more term exp(0) that carries no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    idx = torch.arange(T)
    seen = idx[None, :] <= idx[:, None]
    if window:
        seen &= (idx[:, None] - idx[None, :]) < window
    outs = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~seen, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        if sink:
            m = torch.clamp(m, min=0.0)
        e = torch.exp(s - m)
        den = e.sum(dim=-1, keepdim=True)
        if sink:
            den = den + torch.exp(-m)
        outs.append((e / den) @ v[:, g])
    return torch.cat(outs, dim=-1)


# ---- the windowed attention mixer --------------------------------------------------------------------
def window_keys_values(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float):
    """Keys (normed over the whole projection with a weight, then rotated) and values of a layer that has them."""
    T = h.shape[0]
    G, D, V = m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    freqs, amp = frequencies_by_ramp(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    k = h @ w[p + ".k"].T + w[p + ".k.b"]
    k = rms_norm(k, w[p + ".k.norm"], eps).view(T, G, D)
    k = rotate_half(k, pos, freqs, amp)
    v = (h @ w[p + ".v"].T + w[p + ".v.b"]).view(T, G, V)
    return k, v


def window_attention(h, w, p: str, m: dict, eps: float, kv):
    """``kv``: this layer's own keys and values, or those of the layer it borrows them from."""
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    pos = torch.arange(T)
    freqs, amp = frequencies_by_ramp(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    q = h @ w[p + ".q"].T + w[p + ".q.b"]
    q = rms_norm(q, w[p + ".q.norm"], eps).view(T, H, D)
    q = rotate_half(q, pos, freqs, amp)
    a = attend(q, kv[0], kv[1], float(m["scale"]), int(m["mask"]["size"]), sink=True)
    return a @ w[p + ".o"].T


# ---- the two mixers that run side by side ------------------------------------------------------------
def left_attention(h, w, p: str, m: dict, eps: float):
    """Causal attention whose values are the keys as projected; rotation on the first coordinates, unit RMS per head
    behind it; a sigmoid gate per head on the result."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    pos = torch.arange(T)
    freqs, amp = frequencies_by_wavelength(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    q = (h @ w[p + ".q"].T + w[p + ".q.b"]).view(T, H, D)
    k = (h @ w[p + ".k"].T + w[p + ".k.b"]).view(T, G, D)
    v = k.clone()
    q = rms_norm(rotate_half(q, pos, freqs, amp), None, eps)
    k = rms_norm(rotate_half(k, pos, freqs, amp), None, eps)
    a = attend(q, k, v, float(m["scale"]), None, sink=False).view(T, H, D)
    gate = torch.sigmoid(h @ w[p + ".g"].T)                            # [T, H]
    return (a * gate.unsqueeze(-1)).reshape(T, H * D) @ w[p + ".o"].T


def causal_conv(x, taps_w, bias):
    """x [T, C]; taps_w [C, taps], the last column multiplies the token itself; zeros before the sequence."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], dim=0)
    out = torch.zeros_like(x)
    for j in range(taps):
        out = out + padded[j:j + T] * taps_w[:, j]
    return out + bias


def gated_recurrence(u, w, p: str, blocks: int):
    """S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t from S = 0, with log a_t = -8 r_t softplus(lam) and the gates r, i
    sigmoids of block-diagonal products of u."""
    T, C = u.shape
    bs = C // blocks
    ub = u.view(T, blocks, bs)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + ".ra"]) + w[p + ".ra.b"]).reshape(T, C)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + ".ri"]) + w[p + ".ri.b"]).reshape(T, C)
    log_a = -8.0 * r * torch.nn.functional.softplus(w[p + ".lam"])
    a = torch.exp(log_a)
    gain = torch.sqrt(1.0 - a * a)
    S = torch.zeros(C, dtype=u.dtype)
    out = []
    for t in range(T):
        S = a[t] * S + gain[t] * i[t] * u[t]
        out.append(S)
    return torch.stack(out)


def right_recurrent(h, w, p: str, m: dict):
    y = gelu_tanh(h @ w[p + ".y"].T + w[p + ".y.b"])
    u = causal_conv(h @ w[p + ".x"].T + w[p + ".x.b"], w[p + ".conv"], w[p + ".conv.b"])
    S = gated_recurrence(u, w, p, int(m["blocks"]))
    return (S * y) @ w[p + ".o"].T


def parallel_mixer(h, w, p: str, m: dict, eps: float):
    return float(m["left_scale"]) * left_attention(h, w, p + ".left", m["left"], eps) \
        + float(m["right_scale"]) * right_recurrent(h, w, p + ".right", m["right"])


# ---- feed-forward -------------------------------------------------------------------------------------
def dense_mlp(h, w, p: str):
    return (silu(h @ w[p + ".gate"].T) * (h @ w[p + ".up"].T)) @ w[p + ".down"].T


# ---- the model ----------------------------------------------------------------------------------------
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], residuals: Optional[list] = None):
    """Logits [T, vocab] of one sequence; ``residuals`` collects the residual stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    mult = float(cfg.get("residual_mult", 1.0))
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)] * float(cfg["embedding"]["scale"])
    kept = {}                                       # layer -> its keys and values, for layers that borrow them
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}", L["mixer"]
        h = rms_norm(x, w[p + ".norm1"], eps)
        if L["type"] == "parallel":
            y = parallel_mixer(h, w, p + ".mix", m, eps)
        elif L["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = window_keys_values(h, w, p + ".mix", m, eps)
            y = window_attention(h, w, p + ".mix", m, eps, kept[i if src is None else int(src)])
        else:
            raise ValueError(L["type"])
        x = x + mult * y
        if L.get("mlp") is not None:
            x = x + mult * dense_mlp(rms_norm(x, w[p + ".norm2"], eps), w, p + ".mlp")
        if residuals is not None:
            residuals.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
