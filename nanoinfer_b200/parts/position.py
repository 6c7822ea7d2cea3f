"""Position encodings.  A mixer asks its encoding for the constants its kernel needs."""
from __future__ import annotations

import math

import numpy as np
import torch

from ..config.model_config import ConfigError
from ..config.registry import register_part
from .base import Part


def rope_inverse_frequencies(rotary_dim: int, theta: float, scaling) -> np.ndarray:
    """FP32 inverse frequencies of the rotary pairs, with the optional llama3 rescaling.

    freq_i = 1 / theta^(2i / rotary_dim); with scaling, by wavelength 2*pi/freq:
    >= original/low_freq_factor: freq / factor;  > original/high_freq_factor: blend
    (1 - s) * freq / factor + s * freq with s = (original / wavelen - low) / (high - low);
    else unchanged.  All in FP32, as src/op/kernels/cpu/rope_kernel.cpp:117-139 and
    src/op/kernels/cuda/rope_kernel.cu:95-132 compute them.
    """
    f32 = np.float32
    half = rotary_dim // 2
    freqs = np.empty(half, dtype=np.float32)
    for p in range(half):
        freq = f32(1.0) / np.power(f32(theta), f32(p * 2) / f32(rotary_dim), dtype=np.float32)
        if scaling is not None:
            orig = f32(scaling.original_max_position_embeddings)
            low, high = f32(scaling.low_freq_factor), f32(scaling.high_freq_factor)
            factor = f32(scaling.factor)
            wavelen = f32(2.0) * f32(math.pi) / freq
            if wavelen >= orig / low:
                freq = freq / factor
            elif wavelen > orig / high:
                smooth = (orig / wavelen - low) / (high - low)
                freq = (f32(1.0) - smooth) * freq / factor + smooth * freq
        freqs[p] = freq
    return freqs


class RotaryEncoding(Part):
    """Rotary encoding: holds inv_freq [rotary_dim/2] FP32 on the device and the pairing.

    What a mixer reads from ANY position encoding: ``rotary_dim`` (0: nothing is rotated), ``inv_freq``,
    ``interleaved``, and ``head_slopes`` - None, or float32 [num_heads] on the device: the encoding adds
    slope[h] * (key position - query position) to the scaled attention scores of head h (then the mixer
    uses the plain attention kernel, which takes such a bias, in either precision)."""
    head_slopes = None

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        super().__init__(spec, hidden_size, weights, rt)
        if spec.rotary_dim <= 0 or spec.rotary_dim % 2:
            raise ConfigError(f"rotary_dim {spec.rotary_dim} must be positive and even")
        if spec.pairing not in ("half", "interleaved"):
            raise ConfigError(f"rope pairing '{spec.pairing}' must be 'half' or 'interleaved'")
        if spec.scaling is not None and spec.scaling.rope_type != "llama3":
            raise ConfigError(f"rope scaling '{spec.scaling.rope_type}' is not supported")
        self.rotary_dim = spec.rotary_dim
        self.interleaved = spec.pairing == "interleaved"
        self.inv_freq = torch.from_numpy(
            rope_inverse_frequencies(spec.rotary_dim, spec.theta, spec.scaling)).to(rt.device)


class NoEncoding(Part):
    """No position encoding: queries and keys are used as projected."""
    head_slopes = None

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        super().__init__(spec, hidden_size, weights, rt)
        self.rotary_dim = 0
        self.interleaved = False
        self.inv_freq = torch.zeros(1, dtype=torch.float32, device=rt.device)


register_part("position", "rope", RotaryEncoding, replace=True)
register_part("position", "none", NoEncoding, replace=True)
