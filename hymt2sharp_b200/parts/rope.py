"""Rotate-half (NeoX) rotary position encoding with an optional dynamic-NTK base.

frequencies f_i = 1 / base^(i / half), i in [0, half), half = rope_dim / 2
(src/HyMT2Sharp/Ops.cs:175-177); angle = position * f_i as a float32 product;
pairs (i, i + half); dims from rope_dim on are left as they are
(src/HyMT2Sharp/Ops.cs:159-164).  The base is theta, or theta * alpha^(d/(d-2))
for alpha > 0 (src/HyMT2Sharp/ModelConfig.cs:31-34), and arrives here already
computed.  The table of frequencies is built once on the host and handed to the
kernel that rotates q and k while it appends k and v to the cache.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .base import RotaryEpilogue, register_part


_TABLES: dict = {}   # (device, the frequencies' bytes) -> their tensor on the device


class NeoXRotary:
    def __init__(self, head_dim: int, rope_dim: int, base: float):
        if rope_dim % 2 or rope_dim > head_dim or rope_dim < 0:
            raise ValueError(f"rope_dim {rope_dim} must be even and at most head_dim {head_dim}")
        self.head_dim, self.rope_dim, self.base = int(head_dim), int(rope_dim), float(base)
        half = self.rope_dim // 2
        freq = np.empty(half, dtype=np.float32)
        base32 = np.float32(self.base)
        for i in range(half):
            expo = np.float32(i) / np.float32(half)
            freq[i] = np.float32(1.0) / np.float32(math.pow(float(base32), float(expo)))
        self._host = freq
        self.inv_freq = None

    def tensors(self):
        return {}

    def load(self, weights, device, dtype):
        # layers with the same frequencies share one tensor on the device: what a step works out from a table
        # (the angles of its tokens) then serves all of them
        key = (str(torch.device(device)), self._host.tobytes())
        if key not in _TABLES:
            _TABLES[key] = torch.from_numpy(self._host).to(device)
        self.inv_freq = _TABLES[key]

    def kernel_epilogue(self, ctx) -> RotaryEpilogue:
        """Rotate-half pairs by a table of frequencies: exactly what the appending kernels do on the way."""
        return RotaryEpilogue(self.inv_freq if self.rope_dim else None, self.rope_dim)

    def apply(self, qkv, ctx, heads, kv_heads, head_dim):
        raise NotImplementedError("NeoXRotary is applied by the fused rotation kernel")


register_part("position", "neox_rope", NeoXRotary)


class YarnInterleavedRotary:
    """Rotary encoding on neighbouring pairs with YaRN frequency scaling.

    Of a vector's first `dims` entries, (2i, 2i+1) are a pair that turns by position * f_i, with
    f_i = base^(-2i/dims).  With `scaling` = (factor, original, fast, slow): a pair index is mapped to
    where a wavelength of `original / turns` positions falls, dim(turns) = dims * ln(original / (2 pi turns)) /
    (2 ln base); lo = max(floor(dim(fast)), 0), hi = min(ceil(dim(slow)), dims - 1), ramp_i = clamp((i - lo) /
    max(hi - lo, 0.001), 0, 1); the frequency becomes f_i / factor * ramp_i + f_i * (1 - ramp_i), and cosine and sine
    are multiplied by 0.1 * ln(factor) + 1 (the `amplitude` of the epilogue).
    The table is computed on the host in float64 and rounded to float32 once; the angle is the float32 product
    position * f_i in the kernels.
    """

    def __init__(self, dims: int, base: float, scaling: dict | None = None):
        if dims % 2 or dims < 0:
            raise ValueError(f"{dims} rotated entries: the number must be even")
        self.dims, self.base, self.scaling = int(dims), float(base), dict(scaling) if scaling else None
        half = self.dims // 2
        f = np.array([self.base ** (-2.0 * i / self.dims) for i in range(half)], dtype=np.float64)
        self.amplitude = 1.0
        if self.scaling:
            factor, original = float(self.scaling["factor"]), float(self.scaling["original"])
            fast, slow = float(self.scaling["fast"]), float(self.scaling["slow"])

            def dim_of(turns: float) -> float:
                return self.dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))

            lo = max(math.floor(dim_of(fast)), 0)
            hi = min(math.ceil(dim_of(slow)), self.dims - 1)
            ramp = np.clip((np.arange(half, dtype=np.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            f = f / factor * ramp + f * (1.0 - ramp)
            self.amplitude = 0.1 * math.log(factor) + 1.0
        self._host = f.astype(np.float32)
        self.inv_freq = None

    def tensors(self):
        return {}

    def load(self, weights, device, dtype):
        key = (str(torch.device(device)), self._host.tobytes())
        if key not in _TABLES:
            _TABLES[key] = torch.from_numpy(self._host).to(device)
        self.inv_freq = _TABLES[key]

    def kernel_epilogue(self, ctx) -> RotaryEpilogue:
        return RotaryEpilogue(self.inv_freq if self.dims else None, self.dims, pairing="interleaved", amplitude=self.amplitude)

    def apply(self, qkv, ctx, heads, kv_heads, head_dim):
        raise NotImplementedError("YarnInterleavedRotary is applied by the kernels that take an interleaved epilogue")


register_part("position", "yarn_interleaved", YarnInterleavedRotary)


class WavelengthScaledRotary:
    """Rotate-half rotary encoding whose frequencies are scaled by their wavelength (the long-context rule of Llama 3.1).

    Of a head's first `dims` entries, (i, i + dims/2) are a pair that turns by position * f_i, f_i = base^(-2i/dims).
    With `scaling` = (factor, low, high, original): a frequency whose wavelength l = 2 pi / f is shorter than original / high
    stays; one longer than original / low becomes f / factor; between the two, with s = (original / l - low) / (high - low),
    it becomes (1 - s) f / factor + s f.  The table is computed on the host in float64 and rounded to float32 once; the angle is
    the float32 product position * f_i in the kernels, which take the table as the rotate-half epilogue.
    """

    def __init__(self, dims: int, base: float, scaling: dict | None = None):
        if dims % 2 or dims < 0:
            raise ValueError(f"{dims} rotated entries: the number must be even")
        self.dims, self.base, self.scaling = int(dims), float(base), dict(scaling) if scaling else None
        f = [self.base ** (-2.0 * i / self.dims) for i in range(self.dims // 2)]
        if self.scaling:
            factor, low, high, original = (float(self.scaling[k]) for k in ("factor", "low", "high", "original"))
            short, long = original / high, original / low
            for i, fi in enumerate(f):
                wavelength = 2.0 * math.pi / fi
                if wavelength > long:
                    f[i] = fi / factor
                elif wavelength >= short:
                    s = (original / wavelength - low) / (high - low)
                    f[i] = (1.0 - s) * fi / factor + s * fi
        self._host = np.asarray(f, dtype=np.float64).astype(np.float32)
        self.inv_freq = None

    def tensors(self):
        return {}

    def load(self, weights, device, dtype):
        key = (str(torch.device(device)), self._host.tobytes())
        if key not in _TABLES:
            _TABLES[key] = torch.from_numpy(self._host).to(device)
        self.inv_freq = _TABLES[key]

    def kernel_epilogue(self, ctx) -> RotaryEpilogue:
        return RotaryEpilogue(self.inv_freq if self.dims else None, self.dims)

    def apply(self, qkv, ctx, heads, kv_heads, head_dim):
        raise NotImplementedError("WavelengthScaledRotary is applied by the kernels that take a rotate-half epilogue")


register_part("position", "wavelength_scaled_rope", WavelengthScaledRotary)
