"""Position encodings that act on query and key heads.

``rope_half``: Llama's rotate-half RoPE over the whole head, unscaled.  The
cos/sin table is built once in float32 on the host from the reference's formula
(crates/nnis-model/src/runtime.rs:1166-1184): inv_f = 1 / theta^(2j/d),
angle = position * inv_f.  ``none`` leaves heads as they are.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch

from .base import POSITIONS, PositionEncoding

# one table per (head_dim, theta, max_positions, device): every layer of a model asks
# for the same one
_TABLES: Dict[tuple, Tuple[torch.Tensor, torch.Tensor]] = {}


class RotaryHalf(PositionEncoding):
    """params: head_dim, theta, max_positions.  The tables are made when first asked
    for (listing a model's tensor names needs none)."""

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.key = (int(params["head_dim"]), float(params["theta"]), int(params["max_positions"]),
                    str(torch.device(device)))

    def rotary_tables(self) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        if self.key not in _TABLES:
            d, theta, positions, _ = self.key
            half = d // 2
            exponent = (2 * torch.arange(half, dtype=torch.float32)) / float(d)
            inv_freq = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32), exponent)
            angle = torch.arange(positions, dtype=torch.float32)[:, None] * inv_freq[None, :]
            _TABLES[self.key] = (torch.cos(angle).to(self.device).contiguous(),
                                 torch.sin(angle).to(self.device).contiguous())
        return _TABLES[self.key]


class RotaryFrequencies(PositionEncoding):
    """Rotation of the first ``dims`` of a vector by angles position * f_i,
    f_i = base^(-2i/dims), i = 0 .. dims/2 - 1, with the angle and its cosine and sine
    computed in float32 inside the kernels from a table of the ``dims / 2`` frequencies:
    no table of positions, so no bound on them.  params: dims, base, and optionally
    ``pairing`` ("half": value i turns with value i + dims/2, the rule; "neighbours":
    value 2i with value 2i + 1; the mixer's kernel has to know the pairing it is given)
    and ``scaling`` {factor, low, high, original}: frequencies whose wavelength 2 pi / f
    exceeds original / low are divided by ``factor``, those with a wavelength below
    original / high stay, and between the two the frequency is (1 - s) f / factor + s f
    with s = (original / wavelength - low) / (high - low).  A second form of ``scaling``,
    {ramp: "index", factor, original, fast, slow}, blends by the INDEX of a frequency: with
    at(t) = dims * ln(original / (2 pi t)) / (2 ln base), the index whose wavelength makes t turns
    over ``original`` positions, lo = max(floor(at(fast)), 0), hi = min(ceil(at(slow)), dims - 1) and
    r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), the frequency is r_i f_i / factor +
    (1 - r_i) f_i, and every cosine and sine is multiplied by ``magnitude`` = 0.1 ln(factor) + 1
    (a mixer's kernel has to apply it; 1.0 for every other form).  Mixers whose kernels take
    frequencies (latent attention, retention, attention with a sink, differential attention) ask
    for ``frequencies()``."""

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.dims = int(params["dims"])
        self.base = float(params["base"])
        self.pairing = params.get("pairing", "half")
        self.scaling = params.get("scaling")
        if self.dims < 0 or self.dims % 2:
            raise ValueError(f"rotation: dims={self.dims} must be even")
        if self.pairing not in ("half", "neighbours"):
            raise ValueError(f"rotation: pairing {self.pairing!r} is not known (half, neighbours)")
        self.by_index = self.scaling is not None and self.scaling.get("ramp") == "index"
        self.magnitude = 1.0
        if self.by_index:
            sc = self.scaling
            if not all(float(sc[k]) > 0 for k in ("factor", "original", "fast", "slow")) or self.base <= 1.0:
                raise ValueError("rotation: the ramp over indices needs positive factor, original, fast, slow "
                                 "and a base above 1")
            self.magnitude = 0.1 * math.log(float(sc["factor"])) + 1.0
        elif self.scaling is not None:
            sc = self.scaling
            if not all(float(sc[k]) > 0 for k in ("factor", "low", "high", "original")) \
                    or float(sc["high"]) == float(sc["low"]):
                raise ValueError("rotation: scaling needs positive factor, low, high, original and low != high")
        self._freq: Optional[torch.Tensor] = None

    def _ramped(self, freq: torch.Tensor) -> torch.Tensor:
        sc = self.scaling
        factor, original = float(sc["factor"]), float(sc["original"])

        def at(turns: float) -> float:
            return self.dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))
        lo = max(math.floor(at(float(sc["fast"]))), 0)
        hi = min(math.ceil(at(float(sc["slow"]))), self.dims - 1)
        f = freq.to(torch.float64)
        ramp = torch.clamp((torch.arange(f.numel(), dtype=torch.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return (f / factor * ramp + f * (1.0 - ramp)).to(torch.float32)

    def _scaled(self, freq: torch.Tensor) -> torch.Tensor:
        sc = self.scaling
        factor, low, high, original = (float(sc[k]) for k in ("factor", "low", "high", "original"))
        f = freq.to(torch.float64)
        wavelength = 2.0 * math.pi / f
        s = (original / wavelength - low) / (high - low)
        between = (1.0 - s) * f / factor + s * f
        out = torch.where(wavelength < original / high, f, torch.where(wavelength > original / low, f / factor, between))
        return out.to(torch.float32)

    def frequencies(self) -> torch.Tensor:
        if self._freq is None:
            half = self.dims // 2
            exponent = -(2 * torch.arange(half, dtype=torch.float64)) / float(max(self.dims, 1))
            freq = torch.pow(torch.tensor(self.base, dtype=torch.float64), exponent)
            if self.scaling is not None and half:
                freq = self._ramped(freq) if self.by_index else self._scaled(freq.to(torch.float32))
            freq = freq.to(torch.float32)
            # (one spare entry so that dims == 0 still has an address)
            self._freq = torch.cat([freq, torch.zeros(1)]).to(self.device).contiguous()
        return self._freq


class NoPosition(PositionEncoding):
    def rotary_tables(self):
        return None


POSITIONS.register("rope_half", RotaryHalf)
POSITIONS.register("rope_frequencies", RotaryFrequencies)
POSITIONS.register("none", NoPosition)
