"""Position encodings as tables that the attention kernels read by position.

Rotary: inv_freq[j] = theta^(-2j/rd), angle = pos * inv_freq[j] in float
(qwen_triton/modules/rotary.py:14-26).  The table keeps float cos and sin; the reference rounds
them to the model dtype before use, this library does not.
"""
from __future__ import annotations

import torch

from .base import Runtime, register_position


@register_position("rope")
class RotaryTable:
    def __init__(self, params, runtime: Runtime) -> None:
        self.theta = float(params["theta"])
        self.rotary_dim = int(params["rotary_dim"])
        # which elements turn together: (i, i + rotary_dim / 2) as in the reference (kernels/rope.py:59-69), or
        # neighbours (2i, 2i + 1) with pairing = "interleaved"
        pairing = params.get("pairing", "half")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"rotary pairing {pairing!r} is neither 'half' nor 'interleaved'")
        self.interleaved = pairing == "interleaved"
        if self.rotary_dim % 2 or self.rotary_dim <= 0 or self.rotary_dim > int(params["head_dim"]):
            raise ValueError(f"rotary_dim={self.rotary_dim} must be even and within head_dim={params['head_dim']}")
        # "float64": frequencies and angles are formed in float64 and only cos and sin are rounded to float, so that an
        # angle of thousands of radians is not off by its float rounding; the default forms them in float as the
        # reference does
        self.angles = str(params.get("angles", "float32"))
        if self.angles not in ("float32", "float64"):
            raise ValueError(f"rotary angles in {self.angles!r} (float32 or float64)")
        self.runtime = runtime

    def key(self) -> tuple:
        return ("rope", self.theta, self.rotary_dim, self.angles)          # the table does not depend on the pairing

    def table(self, max_positions: int) -> torch.Tensor:
        """float32 [max_positions, rotary_dim]: cos in the first half of each row, sin in the second."""
        work = torch.float64 if self.angles == "float64" else torch.float32
        exponent = torch.arange(0, self.rotary_dim, 2, dtype=work) / self.rotary_dim
        inv_freq = 1.0 / (self.theta ** exponent)
        angles = torch.arange(max_positions, dtype=work)[:, None] * inv_freq[None, :]
        return torch.cat((angles.cos(), angles.sin()), dim=-1).to(torch.float32).contiguous().to(self.runtime.device)


@register_position("rope_yarn")
class YarnRotaryTable:
    """Rotary angles whose slow pairs are stretched (YaRN): with f_i = theta^(-2i/rd) and, for a pair that turns t times
    within ``original`` positions, where(t) = rd ln(original / (2 pi t)) / (2 ln theta), the pairs below lo =
    max(floor(where(fast)), 0) keep f_i, those above hi = min(ceil(where(slow)), rd - 1) turn at f_i / factor, and those
    between blend the two by ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1).  cos and sin are multiplied by
    ``magnitude`` (default 0.1 ln(factor) + 1).  Frequencies and angles are formed in float64, cos and sin rounded once
    to float.  Parameters: ``theta``, ``rotary_dim``, ``head_dim``, ``factor``, ``original``, ``fast``, ``slow``."""

    interleaved = False

    def __init__(self, params, runtime: Runtime) -> None:
        import math
        self.theta = float(params["theta"])
        self.rotary_dim = int(params["rotary_dim"])
        if self.rotary_dim % 2 or self.rotary_dim <= 0 or self.rotary_dim > int(params["head_dim"]):
            raise ValueError(f"rotary_dim={self.rotary_dim} must be even and within head_dim={params['head_dim']}")
        self.factor, self.original = float(params["factor"]), float(params["original"])
        self.fast, self.slow = float(params["fast"]), float(params["slow"])
        if self.factor <= 0 or self.original <= 0 or self.fast <= 0 or self.slow <= 0 or self.theta <= 1:
            raise ValueError("YaRN scaling needs positive factor, original, fast and slow, and theta above 1")
        self.magnitude = float(params["magnitude"]) if params.get("magnitude") is not None else 0.1 * math.log(self.factor) + 1.0
        self.runtime = runtime

    def key(self) -> tuple:
        return ("rope_yarn", self.theta, self.rotary_dim, self.factor, self.original, self.fast, self.slow, self.magnitude)

    def frequencies(self) -> torch.Tensor:
        import math
        half = self.rotary_dim // 2
        plain = self.theta ** (-torch.arange(half, dtype=torch.float64) * 2.0 / self.rotary_dim)
        where = lambda turns: self.rotary_dim * math.log(self.original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))
        lo = max(math.floor(where(self.fast)), 0)
        hi = min(math.ceil(where(self.slow)), self.rotary_dim - 1)
        ramp = ((torch.arange(half, dtype=torch.float64) - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        return plain / self.factor * ramp + plain * (1.0 - ramp)

    def table(self, max_positions: int) -> torch.Tensor:
        """float32 [max_positions, rotary_dim]: cos in the first half of each row, sin in the second, both times the magnitude."""
        angles = torch.arange(max_positions, dtype=torch.float64)[:, None] * self.frequencies()[None, :]
        return (torch.cat((angles.cos(), angles.sin()), dim=-1) * self.magnitude).to(torch.float32).contiguous().to(self.runtime.device)


@register_position("rope_wavelength")
class WavelengthRotaryTable:
    """Rotary angles whose frequencies are stretched by wavelength: with f_i = theta^(-2i/rd) and wavelength l_i = 2 pi / f_i,
    a pair with l_i < original / high keeps f_i, one with l_i > original / low turns at f_i / factor, and the pairs between
    blend the two, (1 - s) f_i / factor + s f_i with s = (original / l_i - low) / (high - low).  Without ``factor`` the
    rotation is plain.  Frequencies and angles are formed in float64, cos and sin rounded once to float.  Parameters:
    ``theta``, ``rotary_dim``, ``head_dim``, and optionally ``factor``, ``low``, ``high``, ``original``."""

    interleaved = False

    def __init__(self, params, runtime: Runtime) -> None:
        self.theta = float(params["theta"])
        self.rotary_dim = int(params["rotary_dim"])
        if self.rotary_dim % 2 or self.rotary_dim <= 0 or self.rotary_dim > int(params["head_dim"]):
            raise ValueError(f"rotary_dim={self.rotary_dim} must be even and within head_dim={params['head_dim']}")
        self.scaling = None
        if params.get("factor") is not None:
            self.scaling = tuple(float(params[key]) for key in ("factor", "low", "high", "original"))
            factor, low, high, original = self.scaling
            if factor <= 0 or original <= 0 or low <= 0 or high <= low:
                raise ValueError("stretched rotation needs positive factor, original and low, and high above low")
        self.runtime = runtime

    def key(self) -> tuple:
        return ("rope_wavelength", self.theta, self.rotary_dim, self.scaling)

    def frequencies(self) -> torch.Tensor:
        import math
        plain = self.theta ** (-torch.arange(self.rotary_dim // 2, dtype=torch.float64) * 2.0 / self.rotary_dim)
        if self.scaling is None:
            return plain
        factor, low, high, original = self.scaling
        wavelength = 2.0 * math.pi / plain
        blend = ((original / wavelength - low) / (high - low))
        mixed = (1.0 - blend) * plain / factor + blend * plain
        return torch.where(wavelength < original / high, plain, torch.where(wavelength > original / low, plain / factor, mixed))

    def table(self, max_positions: int) -> torch.Tensor:
        """float32 [max_positions, rotary_dim]: cos in the first half of each row, sin in the second."""
        angles = torch.arange(max_positions, dtype=torch.float64)[:, None] * self.frequencies()[None, :]
        return torch.cat((angles.cos(), angles.sin()), dim=-1).to(torch.float32).contiguous().to(self.runtime.device)


@register_position("none")
class NoPosition:
    def __init__(self, params, runtime: Runtime) -> None:
        self.runtime = runtime

    def key(self) -> tuple:
        return ("none",)

    def table(self, max_positions: int):
        return None
