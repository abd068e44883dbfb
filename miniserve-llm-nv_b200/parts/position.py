"""Position encodings applied to queries and keys inside the attention mixer.

``rope``: rotation by ``position * theta^(-2j/rotary_dim)`` (miniserve/model/rope.py:24-52),
half-split pairing ``(j, j + rotary_dim/2)`` by default, interleaved pairing ``(2j, 2j+1)`` or
a rotary size below the head size as options.  Angles, cosines and sines are float32 and are
computed once per step for all layers that share the same encoding.  With ``scaling`` the
frequencies are stretched the YaRN way (see :func:`scaled_frequencies`) and cosines and sines get a
common magnitude.
``none``: no position encoding.

A position part either offers ``fused_args(ctx)``, the arguments of the fused
norm+rotation+append kernel, or returns None there and implements ``apply(q, k, ctx)``, which the
mixer calls on the projected heads before they are appended.
"""

from __future__ import annotations

import math
from typing import Mapping, Optional

import torch

from .. import kernels
from .base import Part, register_position
from .context import StepContext


def scaled_frequencies(dims: int, theta: float, factor: float, original: float, fast: float, slow: float) -> tuple[list, float]:
    """YaRN: the frequencies ``f_i = theta^(-2i/dims)`` of a rotation over ``dims`` entries, stretched for contexts
    ``factor`` times longer than the ``original`` one, and the magnitude that multiplies cosines and sines.

    A pair that turns ``t`` times within ``original`` positions has the (fractional) index
    ``pair(t) = dims ln(original / (2 pi t)) / (2 ln theta)``.  Pairs up to ``lo = max(floor(pair(fast)), 0)`` keep their
    frequency, pairs from ``hi = min(ceil(pair(slow)), dims - 1)`` on are slowed down by ``factor``, and between the
    two the share ``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)`` of the frequency is slowed down:
    ``f_i / factor * ramp_i + f_i (1 - ramp_i)``.  The magnitude is ``0.1 ln(factor) + 1``.  Computed in double
    precision here, rounded to float32 once by the caller."""
    def pair(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo = max(math.floor(pair(fast)), 0)
    hi = min(math.ceil(pair(slow)), dims - 1)
    frequencies = []
    for i in range(dims // 2):
        f = theta ** (-2.0 * i / dims)
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        frequencies.append(f / factor * ramp + f * (1.0 - ramp))
    return frequencies, 0.1 * math.log(factor) + 1.0


@register_position("rope")
class RotaryPosition(Part):
    def __init__(self, *, head_dim: int, theta: float, rotary_dim: Optional[int] = None,
                 interleaved: bool = False, scaling: Optional[Mapping[str, float]] = None,
                 frequencies: str = "float32") -> None:
        self.head_dim = head_dim
        self.theta = float(theta)
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        self.interleaved = bool(interleaved)
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= head_dim:
            raise ValueError(f"rotary size {self.rotary_dim} must be even and within the head size {head_dim}")
        # ``scaling``: the mapping {factor, original, fast, slow} of :func:`scaled_frequencies`, or None
        self.scaling = None if not scaling else tuple(float(scaling[key]) for key in ("factor", "original", "fast", "slow"))
        # "float32": the frequencies come from float32 arithmetic (rope.py:24-25); "float64": theta^(-2i/dims) is
        # computed in double precision and rounded to float32 once
        if frequencies not in ("float32", "float64"):
            raise ValueError(f"frequencies are computed in 'float32' or 'float64', not {frequencies!r}")
        self.frequencies = frequencies
        self.magnitude = 1.0
        self._inv_freq: Optional[torch.Tensor] = None

    def inv_freq(self, device) -> torch.Tensor:
        """``1 / theta ** (arange(0, rotary_dim, 2) / rotary_dim)`` in float32 (rope.py:24-25), or the scaled frequencies."""
        if self._inv_freq is None or self._inv_freq.device != torch.device(device):
            if self.scaling is not None:
                frequencies, self.magnitude = scaled_frequencies(self.rotary_dim, self.theta, *self.scaling)
                self._inv_freq = torch.tensor(frequencies, dtype=torch.float64).to(torch.float32).to(device)
            elif self.frequencies == "float64":
                exact = [self.theta ** (-2.0 * i / self.rotary_dim) for i in range(self.rotary_dim // 2)]
                self._inv_freq = torch.tensor(exact, dtype=torch.float64).to(torch.float32).to(device)
            else:
                exponents = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
                self._inv_freq = (1.0 / (self.theta ** exponents)).to(device)
        return self._inv_freq

    def tables(self, ctx: StepContext) -> torch.Tensor:
        """float32 ``[N, rotary_dim/2, 2]`` of (cos, sin) times the magnitude, shared through the step's memo."""
        key = ("rope", self.theta, self.rotary_dim, self.scaling, self.frequencies)
        table = ctx.memo.get(key)
        if table is None:
            table = torch.empty((ctx.n_tokens, self.rotary_dim // 2, 2), dtype=torch.float32, device=ctx.device)
            inv_freq = self.inv_freq(ctx.device)
            kernels.rope_table(ctx.positions, inv_freq, table, self.magnitude)
            ctx.memo[key] = table
        return table

    def fused_args(self, ctx: StepContext):
        return self.tables(ctx), self.rotary_dim, self.interleaved


@register_position("none")
class NoPosition(Part):
    def __init__(self, **_ignored) -> None:
        pass

    def fused_args(self, ctx: StepContext):
        return None, 0, False
