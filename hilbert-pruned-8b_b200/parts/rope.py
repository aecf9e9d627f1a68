"""Rotary position encoding with optional llama3 or YaRN frequency scaling.

``inv_freq[i] = 1 / theta^(2i/rot)`` in 32-bit, then the llama3 rule per frequency: long
wavelengths divided by ``factor``, short ones kept, the band between interpolated
(cleanroom-transformer/src/model.c:450-469).  At position p the pair ``(i, i + rot/2)`` of
each head is rotated by ``inv_freq[i] * float(p)`` (cpu_backend.c:87-98).  The table of
frequencies is made once on the host; cosines and sines of a step's positions are made
once per step on the device and shared by every layer that uses the same parameters.

YaRN (``yarn = {factor, original, fast, slow}``): with ``dim(t) = rot ln(original / (2 pi t)) /
(2 ln theta)``, ``lo = max(floor(dim(fast)), 0)``, ``hi = min(ceil(dim(slow)), rot - 1)`` and
``ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)`` the frequency of pair i is
``f_i / factor * ramp_i + f_i (1 - ramp_i)``: fast pairs keep their frequency, slow ones are
stretched, the band between is blended.  Cosines and sines are all multiplied by
``0.1 ln(factor) + 1``.

Linear scaling (``linear = factor``): every frequency is divided by the factor (positions are stretched alike for all
pairs); evaluated in 64-bit and rounded once to 32-bit.
"""
from __future__ import annotations

import numpy as np
import torch

from .base import POSITION_ENCODINGS, PositionEncoding


def rotary_inv_freq(rotary_dim: int, theta: float, llama3=None) -> np.ndarray:
    f32 = np.float32
    k = np.arange(rotary_dim // 2, dtype=np.float32)
    expo = (f32(2.0) * k) / f32(rotary_dim)
    freq = (f32(1.0) / np.power(f32(theta), expo, dtype=np.float32)).astype(np.float32)
    if llama3 is not None:
        factor = f32(llama3["factor"])
        low = f32(llama3["low_freq_factor"])
        high = f32(llama3["high_freq_factor"])
        orig = f32(llama3["original_max_position_embeddings"])
        pi = f32(3.14159265358979323846)
        out = np.empty_like(freq)
        for i, f in enumerate(freq):
            wavelen = f32(2.0) * pi / f
            low_wavelen = orig / low
            high_wavelen = orig / high
            scaled = f / factor if wavelen > low_wavelen else f
            if not (wavelen < high_wavelen) and not (wavelen > low_wavelen):
                smooth = (orig / wavelen - low) / (high - low)
                scaled = (f32(1.0) - smooth) * scaled / factor + smooth * scaled
            out[i] = f32(scaled)
        freq = out
    return freq.astype(np.float32)


def yarn_inv_freq(rotary_dim: int, theta: float, yarn) -> np.ndarray:
    """The YaRN frequencies (``yarn`` None: the unscaled ones), evaluated in 64-bit and rounded
    once to 32-bit."""
    import math
    i = np.arange(rotary_dim // 2, dtype=np.float64)
    f = np.power(float(theta), -2.0 * i / rotary_dim)
    if yarn is None:
        return f.astype(np.float32)
    factor, orig = float(yarn["factor"]), float(yarn["original"])

    def dim_of(turns: float) -> float:
        return rotary_dim * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(float(theta)))

    lo = max(math.floor(dim_of(float(yarn["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(yarn["slow"]))), rotary_dim - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return (f / factor * ramp + f * (1.0 - ramp)).astype(np.float32)


def yarn_amplitude(yarn) -> float:
    import math
    return 0.1 * math.log(float(yarn["factor"])) + 1.0


@POSITION_ENCODINGS.register("rotary")
class RotaryEmbedding(PositionEncoding):
    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        self.head_dim = int(spec.params["head_dim"])
        self.rotary_dim = int(spec.params["rotary_dim"])
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary: rotary_dim {self.rotary_dim} does not fit head_dim {self.head_dim}")
        yarn = spec.get("yarn")
        if yarn is not None and spec.get("llama3") is not None:
            raise ValueError("rotary: llama3 and yarn scaling exclude each other")
        linear = spec.get("linear")
        if linear is not None and (yarn is not None or spec.get("llama3") is not None):
            raise ValueError("rotary: one kind of frequency scaling at a time")
        if linear is not None:
            if not float(linear) > 0.0:
                raise ValueError("rotary: the linear scaling factor must be positive")
            i = np.arange(self.rotary_dim // 2, dtype=np.float64)
            self.inv_freq_host = (np.power(float(spec.params["theta"]), -2.0 * i / self.rotary_dim) / float(linear)).astype(np.float32)
        elif yarn is not None or spec.get("frequencies_in_64_bit"):
            self.inv_freq_host = yarn_inv_freq(self.rotary_dim, float(spec.params["theta"]), yarn)
        else:
            self.inv_freq_host = rotary_inv_freq(self.rotary_dim, float(spec.params["theta"]), spec.get("llama3"))
        self.amplitude = yarn_amplitude(yarn) if yarn is not None else 1.0
        self._inv_freq = None
        self._key = "rope:" + repr(spec)

    @property
    def inv_freq(self) -> torch.Tensor:
        if self._inv_freq is None:
            self._inv_freq = torch.from_numpy(self.inv_freq_host.copy()).to(self.ctx.device)
        return self._inv_freq

    def prepare(self, step) -> None:
        if self._key in step.shared:
            return
        half = self.rotary_dim // 2
        table = self.ctx.workspace.buffer(self._key, (self.ctx.max_step_tokens, half, 2), torch.float32)
        table = table[: step.num_tokens]
        self.ctx.ops.rope_table(step.positions, self.inv_freq, table, self.amplitude)
        step.shared[self._key] = table

    def rotation_table(self, step):
        """``([tokens, rot/2, 2] cosines and sines of this step's positions, rot)``."""
        self.prepare(step)
        return step.shared[self._key], self.rotary_dim
