"""Rotary position encoding (NeoX half-split form)."""
from __future__ import annotations

import torch

from .base import PositionEncoding
from .registry import POSITION_ENCODINGS


@POSITION_ENCODINGS.register("rotary")
class RotaryPosition(PositionEncoding):
    """inv_freq[i] = theta ** (-2i / R), i = 0 .. R/2 - 1, built in float32 exactly as the reference does
    (utils/layers.py:147,157) with R = ``rotary_dim``; angle = position * inv_freq is formed in the kernel that
    rotates Q and K.  Parameters: ``head_dim``, ``theta``; optional ``rotary_dim`` (default head_dim: the whole
    head rotates, as in the reference), ``pairing`` ("halves", the reference's NeoX form, or "interleaved") and
    ``attention_factor`` (1: the default schedule; mixers may refuse anything else)."""

    KNOWN_PARAMS = ("head_dim", "theta", "rotary_dim", "pairing", "attention_factor")

    def __init__(self, params, weights, runtime):
        super().__init__(params, weights, runtime)
        head_dim, theta = int(params["head_dim"]), float(params["theta"])
        rotary_dim = int(params.get("rotary_dim") or head_dim)
        if rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
            raise ValueError(f"rotary encoding needs an even rotary_dim of at most head_dim {head_dim}, got {rotary_dim}")
        dim_indices = torch.arange(0, rotary_dim, 2, dtype=torch.long)
        inverse = 1.0 / (theta ** (dim_indices.to(torch.float32) / rotary_dim))
        self.head_dim, self.rotary_dim = head_dim, rotary_dim
        self.pairing = params.get("pairing") or "halves"
        self.attention_factor = float(params.get("attention_factor") or 1.0)
        self.inv_freq = inverse.to(torch.float32).to(runtime.device).contiguous()


@POSITION_ENCODINGS.register("stretched_rotary")
class StretchedRotaryPosition(PositionEncoding):
    """Rotary frequencies stretched for contexts longer than the ``original`` one (the YaRN scheme of Peng et al.,
    "YaRN: Efficient Context Window Extension of Large Language Models"): pairs that turn fast keep their frequency,
    pairs that turn slowly have it divided by ``factor``, with a linear ramp between.

        f_i  = theta ** (-2i / R),  i < R / 2
        d(t) = R ln(original / (2 pi t)) / (2 ln theta)        the pair that makes t turns over the original context
        lo   = max(floor(d(fast)), 0),  hi = min(ceil(d(slow)), R - 1)
        r_i  = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
        inv_freq_i = f_i / factor * r_i + f_i * (1 - r_i)

    and cos and sin are multiplied by ``attention_factor`` = 0.1 ln(factor) + 1 (``magnitude_slope`` in place of 0.1,
    when given).  Parameters: ``head_dim``, ``theta``, ``rotary_dim`` (default head_dim), ``factor``, ``original``,
    ``fast``, ``slow``; optional ``pairing`` and ``magnitude_slope``.  The table is made in float64 and held in float32;
    the angle position * inv_freq is formed in the kernel that rotates Q and K."""

    KNOWN_PARAMS = ("head_dim", "theta", "rotary_dim", "factor", "original", "fast", "slow", "pairing", "magnitude_slope")

    def __init__(self, params, weights, runtime):
        import math

        super().__init__(params, weights, runtime)
        head_dim, theta = int(params["head_dim"]), float(params["theta"])
        rotary_dim = int(params.get("rotary_dim") or head_dim)
        if rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
            raise ValueError(f"rotary encoding needs an even rotary_dim of at most head_dim {head_dim}, got {rotary_dim}")
        factor, original = float(params["factor"]), float(params["original"])
        if factor <= 0 or original <= 0 or theta <= 1:
            raise ValueError(f"stretched rotary needs factor > 0, original > 0 and theta > 1, got {factor}, {original}, {theta}")

        def pair_of(turns: float) -> float:
            return rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

        low = max(math.floor(pair_of(float(params["fast"]))), 0)
        high = min(math.ceil(pair_of(float(params["slow"]))), rotary_dim - 1)
        table = []
        for i in range(rotary_dim // 2):
            plain = theta ** (-2.0 * i / rotary_dim)
            ramp = min(max((i - low) / max(high - low, 0.001), 0.0), 1.0)
            table.append(plain / factor * ramp + plain * (1.0 - ramp))
        self.head_dim, self.rotary_dim = head_dim, rotary_dim
        self.pairing = params.get("pairing") or "halves"
        slope = params.get("magnitude_slope")
        self.attention_factor = (0.1 if slope is None else float(slope)) * math.log(factor) + 1.0
        self.inv_freq = torch.tensor(table, dtype=torch.float64).to(torch.float32).to(runtime.device).contiguous()


@POSITION_ENCODINGS.register("banded_rotary")
class BandedRotaryPosition(PositionEncoding):
    """Rotary frequencies scaled band by band of their wavelength (the long-context scheme of the Llama 3.1 models):
    with f_i = theta ** (-2i / R) and the wavelength l_i = 2 pi / f_i,

        l_i < original / high:   f_i              pairs that turn fast stay as they are
        l_i > original / low:    f_i / factor     pairs that turn slowly are slowed down further
        between:                 (1 - s) f_i / factor + s f_i,   s = (original / l_i - low) / (high - low)

    Parameters: ``head_dim``, ``theta``, ``rotary_dim`` (default head_dim), ``factor``, ``low``, ``high``, ``original``;
    optional ``pairing``.  The table is made in float64 and held in float32; the angle position * inv_freq is formed in
    the kernel that rotates Q and K."""

    KNOWN_PARAMS = ("head_dim", "theta", "rotary_dim", "factor", "low", "high", "original", "pairing")

    def __init__(self, params, weights, runtime):
        import math

        super().__init__(params, weights, runtime)
        head_dim, theta = int(params["head_dim"]), float(params["theta"])
        rotary_dim = int(params.get("rotary_dim") or head_dim)
        if rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
            raise ValueError(f"rotary encoding needs an even rotary_dim of at most head_dim {head_dim}, got {rotary_dim}")
        factor, original = float(params["factor"]), float(params["original"])
        low, high = float(params["low"]), float(params["high"])
        if factor <= 0 or original <= 0 or not 0 < low < high:
            raise ValueError(f"banded rotary needs factor > 0, original > 0 and 0 < low < high, got {factor}, {original}, {low}, {high}")
        table = []
        for i in range(rotary_dim // 2):
            plain = theta ** (-2.0 * i / rotary_dim)
            wavelength = 2.0 * math.pi / plain
            if wavelength < original / high:
                table.append(plain)
            elif wavelength > original / low:
                table.append(plain / factor)
            else:
                ramp = (original / wavelength - low) / (high - low)
                table.append((1.0 - ramp) * plain / factor + ramp * plain)
        self.head_dim, self.rotary_dim = head_dim, rotary_dim
        self.pairing = params.get("pairing") or "halves"
        self.attention_factor = 1.0
        self.inv_freq = torch.tensor(table, dtype=torch.float64).to(torch.float32).to(runtime.device).contiguous()
