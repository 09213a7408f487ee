"""Rotary position encoding: the frequencies a mixer's fused kernel rotates with.

inv_freq_i = theta^(-2i/rot_dim), angle = position * inv_freq_i, pairs (d, d + head_dim/2)
(pico_vllm/model.py:80-90, 116-123): ``pairing = "half"``, the only pairing the kernels have; a
position part may name another (``"interleaved"``: pairs (2i, 2i+1)) and the kernels then refuse it
with a KernelError instead of rotating wrongly.  The reference looks angles up in a table of cos/sin that
ends up in bfloat16 (pico_vllm/run_single.py:13); here the kernel computes them in float32
from the position.  ``rot_dim`` below ``head_dim`` rotates only the first rot_dim/2 pairs;
:class:`NoPosition` rotates nothing.
"""
from __future__ import annotations

import math

import torch

from ..errors import ConfigError
from .base import Part
from .registry import register


@register("position", "rotary")
class Rotary(Part):
    pairing = "half"

    def __init__(self, head_dim: int, theta: float, rot_dim: int = None, pairing: str = "half"):
        self.head_dim, self.theta, self.pairing = head_dim, theta, pairing
        self.rot_dim = head_dim if rot_dim is None else rot_dim
        if self.rot_dim % 2 or self.rot_dim > head_dim:
            raise ConfigError(f"rotary: rot_dim {self.rot_dim} must be even and at most head_dim {head_dim}")
        self.inv_freq = None

    def frequencies(self) -> torch.Tensor:
        # the same float32 expression as the reference (pico_vllm/model.py:80-82)
        return 1.0 / (self.theta ** (torch.arange(0, self.rot_dim, 2).float() / self.rot_dim))

    def materialize(self, device, dtype):
        self.inv_freq = self.frequencies().to(device)


@register("position", "yarn_rotary")
class YarnRotary(Part):
    """Rotary encoding on the first ``rot_dim`` dimensions of a head, dimension i paired with i + rot_dim/2, with
    frequencies stretched for contexts beyond the ``original`` length (YaRN: Peng, Quesnelle, Fan, Shippole, "YaRN:
    Efficient Context Window Extension of Large Language Models"):

        f_i = theta^(-2i/rot_dim);   turns(i) = how often dimension i goes round within ``original`` positions
        dimensions with more than ``fast`` turns keep f_i, those with fewer than ``slow`` get f_i / factor, and between
        the two dimension numbers lo = floor(dim(fast)), hi = ceil(dim(slow)), dim(t) = rot_dim ln(original / (2 pi t))
        / (2 ln theta), the share of f_i / factor grows linearly:  ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1).
        cos and sin are multiplied by ``mult`` = 0.1 ln(factor) + 1.

    ``factor`` None: plain frequencies and mult 1.  ``pairing`` is "rot_half": the pairs lie inside the rotated
    dimensions (the same as "half" when rot_dim == head_dim)."""
    pairing = "rot_half"

    def __init__(self, head_dim: int, theta: float, rot_dim: int = None, factor: float = None, original: int = 0,
                 fast: float = 32.0, slow: float = 1.0):
        self.head_dim, self.theta = head_dim, float(theta)
        self.rot_dim = head_dim if rot_dim is None else rot_dim
        if self.rot_dim % 2 or not 0 <= self.rot_dim <= head_dim:
            raise ConfigError(f"yarn_rotary: rot_dim {self.rot_dim} must be even and at most head_dim {head_dim}")
        if factor is not None and (factor <= 0 or original <= 0 or fast <= 0 or slow <= 0):
            raise ConfigError("yarn_rotary: factor, original, fast and slow must be positive")
        self.factor, self.original, self.fast, self.slow = factor, original, fast, slow
        self.mult = 1.0 if factor is None else 0.1 * math.log(factor) + 1.0
        self.inv_freq = None

    def frequencies(self) -> torch.Tensor:
        n = self.rot_dim
        i = torch.arange(n // 2, dtype=torch.float64)
        f = self.theta ** (-2.0 * i / n) if n else i
        if self.factor is not None and n:
            def dim_of(turns):
                return n * math.log(self.original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))
            lo = max(math.floor(dim_of(self.fast)), 0)
            hi = min(math.ceil(dim_of(self.slow)), n - 1)
            ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
            f = f / self.factor * ramp + f * (1.0 - ramp)
        return f.to(torch.float32)

    def materialize(self, device, dtype):
        self.inv_freq = self.frequencies().to(device)


@register("position", "none")
class NoPosition(Part):
    pairing = "half"

    def __init__(self, head_dim: int = 0, **_):
        self.head_dim, self.rot_dim = head_dim, 0
        self.inv_freq = None

    def materialize(self, device, dtype):
        self.inv_freq = torch.zeros(0, dtype=torch.float32, device=device)
