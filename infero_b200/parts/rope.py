"""Rotary position encoding, NeoX pairing."""
from __future__ import annotations

import numpy as np
import torch

from ..config.spec import PositionSpec
from .base import PositionEncoding


def yarn_stretch(inv, theta: float, dims: int, factor: float, original: float, fast: float, slow: float):
    """Frequencies stretched for contexts beyond ``original`` tokens, and the amplitude that goes with them.
    n(t) = dims * ln(original / (2 pi t)) / (2 ln theta) is the pair index whose wave makes t turns over the original
    length; pairs below lo = floor(n(fast)) keep their frequency, pairs above hi = ceil(n(slow)) get it divided by
    ``factor``, a linear ramp in between.  64-bit on the host."""
    import math

    def index_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo = max(math.floor(index_of(fast)), 0)
    hi = min(math.ceil(index_of(slow)), dims - 1)
    ramp = np.clip((np.arange(inv.shape[0], dtype=np.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return inv / factor * ramp + inv * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def band_scale(inv, factor: float, low: float, high: float, original: float):
    """Frequencies scaled by bands of the wavelength l = 2 pi / f: waves shorter than original / high stay, waves longer
    than original / low are divided by ``factor``, in between f becomes (1 - s) f / factor + s f with
    s = (original / l - low) / (high - low).  64-bit on the host."""
    import math
    out = np.array(inv, dtype=np.float64)
    for i, f in enumerate(inv):
        wave = 2.0 * math.pi / f
        if wave < original / high:
            continue
        if wave > original / low:
            out[i] = f / factor
        else:
            s = (original / wave - low) / (high - low)
            out[i] = (1.0 - s) * f / factor + s * f
    return out


class RopeNeox(PositionEncoding):
    """inv_freq[i] = theta^(-2i / rotary_dim), i < rotary_dim/2; angle = pos * inv_freq[i]
    (crates/kernels/src/cu/ops.cu:488-523).  The table is made on the host in 64-bit and
    rounded once to 32-bit; the kernel multiplies by the position and takes sincosf."""

    def __init__(self, spec: PositionSpec):
        self.spec = spec
        if spec.rotary_dim % 2:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be even")
        half = spec.rotary_dim // 2
        inv = np.float64(spec.theta) ** (-2.0 * np.arange(half, dtype=np.float64) / spec.rotary_dim)
        # what cos and sin are multiplied by (1 unless the frequencies are stretched); kernels that take an
        # amplitude ask for it, mixers whose kernels have none refuse a table that needs one
        self.amplitude = 1.0
        if getattr(spec, "yarn", None):
            inv, self.amplitude = yarn_stretch(inv, spec.theta, spec.rotary_dim, *spec.yarn)
        if getattr(spec, "bands", None):
            inv = band_scale(inv, *spec.bands)
        self._inv_host = torch.from_numpy(inv.astype(np.float32))
        self._inv_host64 = torch.from_numpy(np.ascontiguousarray(inv, dtype=np.float64))
        self._inv_dev = {}

    def inv_freq(self, device) -> torch.Tensor:
        key = str(device)
        if key not in self._inv_dev:
            self._inv_dev[key] = self._inv_host.to(device)
        return self._inv_dev[key]

    def inv_freq64(self, device) -> torch.Tensor:
        """The table as it was made, in 64-bit, for kernels that form the angle in 64-bit."""
        key = ("f64", str(device))
        if key not in self._inv_dev:
            self._inv_dev[key] = self._inv_host64.to(device)
        return self._inv_dev[key]


class RopeInterleaved(RopeNeox):
    """The same angles on adjacent pairs: dimension 2i turns with dimension 2i + 1.  Mixers whose kernels
    take the pairing as a parameter ask ``pairing``; the table is the one of the base class."""
    pairing = "adjacent"
