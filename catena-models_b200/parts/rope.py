"""Rotary position encoding with per-frequency factors.

rate[i] = theta^(-2i/head_dim) / factor[i], both steps in float32 as the reference does them
(the power on the host, src/catena.rs:185-204; the division in the kernel,
src/catena/lfm3.hex:726-734); the kernel forms angle = float(position) * rate[i] and rotates
the halves of the head against each other (src/catena/lfm3.hex:706-746).  `factors_name` is
the tensor of per-frequency divisors, or None for factor 1 (sliding layers ignore the factors
and use a base of their own).
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import Position, register_part


class Rotary(Position):
    prompt_capturable = True
    fused_decode_ok = True
    supports_append = True

    def __init__(self, head_dim, theta, factors_name=None):
        self.head_dim, self.theta, self.factors_name = head_dim, float(theta), factors_name
        self._rate = None

    def tensor_specs(self):
        if self.factors_name is None:
            return []
        return [TensorSpec(self.factors_name, (self.head_dim // 2,), "rope_factors")]

    def bind(self, tensors, rt):
        half = self.head_dim // 2
        exponent = (2 * torch.arange(half, dtype=torch.float32)) / torch.tensor(float(self.head_dim), dtype=torch.float32)
        freq = torch.pow(torch.tensor(self.theta, dtype=torch.float32), -exponent)
        if self.factors_name is not None:
            freq = freq / tensors[self.factors_name].to("cpu", torch.float32)
        self._rate = freq.to(rt.device).contiguous()

    def rate_table(self):
        return self._rate


class PartialYarnRotary(Position):
    """Rotation of the leading `dims` channels of a vector, channel i against channel i + dims/2, with rates
    rescaled for a longer context than the one trained on (YaRN): with f_i = theta^(-2i/dims), turn(t) =
    dims ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(turn(fast)), 0), hi = min(ceil(turn(slow)),
    dims - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns at
    f_i / factor * ramp_i + f_i (1 - ramp_i), and sine and cosine are multiplied by `magnitude` = 0.1 ln(factor)
    + 1.  Without `factor` the rates are the plain f_i and the magnitude is 1.  The rates are formed in double
    precision on the host and kept as float32; the kernel forms angle = float(position) * rate."""
    prompt_capturable = True
    supports_append = True

    def __init__(self, dims, theta, factor=None, original=None, fast=None, slow=None):
        import math

        if dims % 2:
            raise ValueError(f"{dims} turned channels: an even number is needed")
        self.dims, self.theta = dims, float(theta)
        half = dims // 2
        rates = [self.theta ** (-2.0 * i / dims) for i in range(half)]
        self.magnitude = 1.0
        if factor is not None:
            turn = lambda t: dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(self.theta))
            lo, hi = max(math.floor(turn(fast)), 0), min(math.ceil(turn(slow)), dims - 1)
            ramp = [min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(half)]
            rates = [f / factor * r + f * (1.0 - r) for f, r in zip(rates, ramp)]
            self.magnitude = 0.1 * math.log(factor) + 1.0
        self.rates = rates
        self._rate = None

    def bind(self, tensors, rt):
        self._rate = torch.tensor(self.rates, dtype=torch.float64).to(torch.float32).to(rt.device).contiguous()

    def rate_table(self):
        return self._rate


class PairedRotary(Position):
    """Rotation of the leading `dims` channels of a vector, channel 2i against channel 2i + 1 (the interleaved layout),
    pair i at the rate f_i = theta^(-2i/dims); the other channels pass unchanged.  With `factor` the rates are rescaled for
    a longer context than the one trained on, by the same rule as `PartialYarnRotary` (turn(t) = dims ln(original /
    (2 pi t)) / (2 ln theta), lo = max(floor(turn(fast)), 0), hi = min(ceil(turn(slow)), dims - 1), ramp_i = clamp((i - lo)
    / max(hi - lo, 0.001), 0, 1), rate f_i / factor * ramp_i + f_i (1 - ramp_i)), and sine and cosine are multiplied by
    `magnitude` = 0.1 ln(factor) + 1.  The rates are formed in double precision on the host and kept as float32; the
    kernel forms angle = float(position) * rate."""
    prompt_capturable = True
    supports_append = True
    pairing = "interleaved"

    def __init__(self, dims, theta, factor=None, original=None, fast=None, slow=None):
        import math

        if dims % 2 or dims < 2:
            raise ValueError(f"{dims} turned channels: an even number is needed")
        self.dims, self.theta = dims, float(theta)
        self.rates = [self.theta ** (-2.0 * i / dims) for i in range(dims // 2)]
        self.magnitude = 1.0
        if factor is not None:
            turn = lambda t: dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(self.theta))
            lo, hi = max(math.floor(turn(fast)), 0), min(math.ceil(turn(slow)), dims - 1)
            ramp = [min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(dims // 2)]
            self.rates = [f / factor * r + f * (1.0 - r) for f, r in zip(self.rates, ramp)]
            self.magnitude = 0.1 * math.log(factor) + 1.0
        self._rate = None

    def bind(self, tensors, rt):
        self._rate = torch.tensor(self.rates, dtype=torch.float64).to(torch.float32).to(rt.device).contiguous()

    def rate_table(self):
        return self._rate


class NoPosition(Position):
    """No position encoding: the head vectors are left unrotated."""
    prompt_capturable = True
    fused_decode_ok = True
    supports_append = True


register_part("position", "rotary", Rotary)
register_part("position", "none", NoPosition)
register_part("position", "paired_rotary", PairedRotary)
register_part("position", "partial_yarn_rotary", PartialYarnRotary)
