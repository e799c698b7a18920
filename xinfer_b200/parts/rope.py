"""Rotary position encoding.  ``inv_freq_j = 1 / theta^(2j / rotary_dim)`` computed in float64
and rounded to float32, angle = position * inv_freq in float32, cos/sin tables in float32
(src/models/layers/rotary_emb.rs:42-62; the reference then rounds the tables to the model dtype,
qwen3.rs:221-231 - here they stay float32 in both precisions).  The tables are applied by the
attention kernel that also norms q/k and writes the cache."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from .. import kernels
from ..config.plan import RopeSpec, YarnScaling
from .base import PositionEncoding, register_position_encoding


@dataclass
class RotaryTables:
    cos: torch.Tensor  # [max_positions, rotary_dim / 2] float32
    sin: torch.Tensor
    rotary_dim: int
    interleaved: bool


_TABLE_CACHE = {}


def inv_frequencies(theta: float, rotary_dim: int, scaling=None, rounded_once: bool = False) -> np.ndarray:
    """``rounded_once``: formed in float64 and rounded to float32 at the end (the table path without scaling
    keeps the reference's order: the power rounded to float32, then its reciprocal)."""
    j = np.arange(0, rotary_dim, 2, dtype=np.float64)
    if scaling is None and not rounded_once:
        return (np.float32(1.0) / np.power(np.float64(theta), j / np.float64(rotary_dim)).astype(np.float32)).astype(np.float32)
    # long wavelengths turn more slowly (``RopeScaling``); formed in float64, rounded once to float32
    f = np.power(np.float64(theta), -j / np.float64(rotary_dim))
    if scaling is None:
        return f.astype(np.float32)
    if isinstance(scaling, YarnScaling):
        # pairs that make many turns within the original length keep their frequency, pairs that make few are
        # slowed by the factor, with a linear ramp over the pair index between the two
        def pair_at(turns: float) -> float:
            return rotary_dim * np.log(scaling.original / (2.0 * np.pi * turns)) / (2.0 * np.log(np.float64(theta)))
        lo = max(np.floor(pair_at(scaling.fast)), 0.0)
        hi = min(np.ceil(pair_at(scaling.slow)), rotary_dim - 1.0)
        ramp = np.clip((j / 2.0 - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return (f / scaling.factor * ramp + f * (1.0 - ramp)).astype(np.float32)
    wavelength = 2.0 * np.pi / f
    s = (scaling.original / wavelength - scaling.low) / (scaling.high - scaling.low)
    blended = (1.0 - s) * f / scaling.factor + s * f
    f = np.where(wavelength < scaling.original / scaling.high, f,
                 np.where(wavelength > scaling.original / scaling.low, f / scaling.factor, blended))
    return f.astype(np.float32)


class Rope(PositionEncoding):
    kind = "rope"
    graph_safe = True

    def __init__(self, spec: RopeSpec, prefix: str, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        if spec.rotary_dim % 2 or spec.rotary_dim > spec.head_dim or spec.rotary_dim <= 0:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be even and at most head_dim {spec.head_dim}")
        if spec.layout not in ("neox", "interleaved"):
            raise ValueError(f"unknown rotary layout '{spec.layout}'")
        self._tables = None
        self._inv = None

    def frequencies(self) -> torch.Tensor:
        """float32 ``[rotary_dim / 2]`` on the device: what a kernel that forms its angles itself multiplies
        a position by."""
        if self._inv is None:
            s = self.spec
            key = ("inv", str(self.device), s.theta, s.rotary_dim, s.scaling)
            if key not in _TABLE_CACHE:
                _TABLE_CACHE[key] = torch.from_numpy(inv_frequencies(s.theta, s.rotary_dim, s.scaling, True)).to(self.device)
            self._inv = _TABLE_CACHE[key]
        return self._inv

    def rotary(self) -> RotaryTables:
        if not self.spec.tables:
            raise ValueError("this rotary encoding keeps no tables (its spec says tables=False); use frequencies()")
        if self._tables is None:
            s = self.spec
            key = (str(self.device), s.theta, s.rotary_dim, s.max_positions, s.scaling, s.magnitude)
            if key not in _TABLE_CACHE:  # layers with the same constants share one table
                half = s.rotary_dim // 2
                inv = torch.from_numpy(inv_frequencies(s.theta, s.rotary_dim, s.scaling)).to(self.device)
                cos = torch.empty((s.max_positions, half), dtype=torch.float32, device=self.device)
                sin = torch.empty_like(cos)
                kernels.rope_table(cos, sin, inv)
                if s.magnitude != 1.0:
                    cos.mul_(s.magnitude)
                    sin.mul_(s.magnitude)
                _TABLE_CACHE[key] = (cos, sin)
            cos, sin = _TABLE_CACHE[key]
            self._tables = RotaryTables(cos, sin, s.rotary_dim, s.layout == "interleaved")
        return self._tables


register_position_encoding("rope", Rope)
