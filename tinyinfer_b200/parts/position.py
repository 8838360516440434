"""Position encodings. The rotary part owns the float32 inverse frequencies
inv_freq[j] = theta ** (-2j / rotary_dim) (tinyinfer/layers/rotary_embedding.py:38-48 of the
reference, which also keeps them in float32 under a bfloat16 model, :51-70); the rotation itself
happens inside the mixer's fused norm + rotation + cache-append kernel."""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding, register_position


class RotaryEncoding(PositionEncoding):
    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        if spec.rotary_dim <= 0 or spec.rotary_dim % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {spec.rotary_dim}")
        blend = getattr(spec, "blend", None)
        self.factor = 1.0
        if getattr(spec, "exact_frequencies", False) or blend is not None:
            exponent = torch.arange(0, spec.rotary_dim, 2, dtype=torch.float64) / spec.rotary_dim
            freq = float(spec.theta) ** -exponent
            if blend is not None:
                freq, self.factor = blended(freq, spec.rotary_dim, float(spec.theta), blend)
            self.inv_freq = freq.to(torch.float32).to(device)
        else:
            exponent = torch.arange(0, spec.rotary_dim, 2, dtype=torch.float32) / spec.rotary_dim
            self.inv_freq = (1.0 / (spec.theta ** exponent)).to(device)
        self.rotary_dim = spec.rotary_dim
        self.interleaved = bool(getattr(spec, "interleaved", False))

    def rotation(self):
        from .. import ops
        return ops.Rotation(self.rotary_dim, inv_freq=self.inv_freq, interleaved=self.interleaved, factor=self.factor)


def blended(freq: torch.Tensor, rotary_dim: int, theta: float, blend):
    """(frequencies, factor on cosines and sines) of a ``FrequencyBlend``: pairs that turn fewer than ``slow`` times
    over the original length are slowed down ``factor`` times, those that turn more than ``fast`` times stay, the
    pairs between are blended linearly in the pair index. Float64 in, float64 out."""
    if not blend.factor > 0 or blend.original <= 0 or not blend.fast > 0 or not blend.slow > 0 or theta <= 1.0:
        raise ValueError("a frequency blend needs a positive factor, original length and turn counts, and theta > 1")

    def pair(turns: float) -> float:
        return rotary_dim * math.log(blend.original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo = max(math.floor(pair(blend.fast)), 0)
    hi = min(math.ceil(pair(blend.slow)), rotary_dim - 1)
    j = torch.arange(rotary_dim // 2, dtype=torch.float64)
    ramp = torch.clamp((j - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return freq / blend.factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(blend.factor) + 1.0


class NoPosition(PositionEncoding):
    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.inv_freq = None
        self.rotary_dim = 0


register_position("rope", RotaryEncoding)
register_position("none", NoPosition)
