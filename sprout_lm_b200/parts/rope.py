"""Rotary position encoding with half-split pairs (d, d + head_dim/2), angle =
position / theta**(2d / head_dim) (src/qwen.ts:81-92).

The angles are computed in float64 on the host for every position up to ``max_positions``
and kept as float32 cosine and sine tables; the kernel that rotates q and k reads them.
"""
from __future__ import annotations

import numpy as np
import torch

from .base import Part, register_part


@register_part("position", "rope_half_split")
class HalfSplitRotary(Part):
    def __init__(self, prefix: str, head_dim: int, theta: float, max_positions: int):
        if head_dim % 2:
            raise ValueError("rotary position encoding needs an even head_dim")
        if theta <= 0 or max_positions <= 0:
            raise ValueError("rotary position encoding needs positive theta and max_positions")
        self.head_dim, self.theta, self.max_positions = int(head_dim), float(theta), int(max_positions)

    def angles(self) -> np.ndarray:
        d = np.arange(self.head_dim // 2, dtype=np.float64)
        inv = self.theta ** (2.0 * d / self.head_dim)
        return np.arange(self.max_positions, dtype=np.float64)[:, None] / inv[None, :]

    interleaved = False          # pairs (d, d + head_dim / 2)

    def rotary_tables(self, runtime):
        """The tables depend on (head_dim, theta, max_positions) alone: all layers of a model share
        one copy on the device."""
        def build():
            angle = self.angles()
            cos = torch.from_numpy(np.cos(angle).astype(np.float32)).to(runtime.device)
            sin = torch.from_numpy(np.sin(angle).astype(np.float32)).to(runtime.device)
            return cos.contiguous(), sin.contiguous()
        shared = getattr(runtime, "shared", None)
        return shared(("rope_half_split", self.head_dim, self.theta, self.max_positions), build) if shared else build()


@register_part("position", "none")
class NoPosition(Part):
    """No position encoding: q and k are used as projected."""

    def __init__(self, prefix: str = "", **_):
        pass

    def rotary_tables(self, runtime):
        return None


def yarn_frequencies(dims: int, theta: float, factor: float, original: float, fast: float, slow: float) -> np.ndarray:
    """Frequencies of a rotation over ``dims`` elements whose slow pairs are stretched by ``factor``:
    with f_i = theta**(-2i/dims) and pair(t) = dims * ln(original / (2 pi t)) / (2 ln theta), the pairs
    below lo = max(floor(pair(fast)), 0) keep f_i, those above hi = min(ceil(pair(slow)), dims - 1)
    get f_i / factor, and between them the two are mixed linearly (float64)."""
    i = np.arange(dims // 2, dtype=np.float64)
    f = theta ** (-2.0 * i / dims)

    def pair(turns: float) -> float:
        return dims * np.log(original / (2.0 * np.pi * turns)) / (2.0 * np.log(theta))
    lo = max(int(np.floor(pair(fast))), 0)
    hi = min(int(np.ceil(pair(slow))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp)


class _Rotary(Part):
    """Tables of a rotation over the first ``dims`` elements of a vector: cos and sin of
    position * f_i, times ``magnitude``; float64 on the host, float32 [max_positions, dims / 2] on the
    device, one copy per distinct set of constants."""
    interleaved = False

    def __init__(self, prefix: str, dims: int, theta: float, max_positions: int, scaling: dict | None = None):
        if dims <= 0 or dims % 2:
            raise ValueError("rotary position encoding needs an even, positive number of elements")
        if theta <= 1 or max_positions <= 0:
            raise ValueError("rotary position encoding needs a base above 1 and positive max_positions")
        self.dims, self.theta, self.max_positions = int(dims), float(theta), int(max_positions)
        self.scaling = None
        if scaling is not None:
            self.scaling = tuple(float(scaling[key]) for key in ("factor", "original", "fast", "slow"))
            if self.scaling[0] <= 0 or self.scaling[1] <= 0 or self.scaling[2] <= 0 or self.scaling[3] <= 0:
                raise ValueError("rotary scaling needs positive factor, original, fast and slow")

    def frequencies(self) -> np.ndarray:
        if self.scaling is None:
            return self.theta ** (-2.0 * np.arange(self.dims // 2, dtype=np.float64) / self.dims)
        return yarn_frequencies(self.dims, self.theta, *self.scaling)

    @property
    def magnitude(self) -> float:
        return 1.0 if self.scaling is None else 0.1 * float(np.log(self.scaling[0])) + 1.0

    def rotary_tables(self, runtime):
        def build():
            angle = np.arange(self.max_positions, dtype=np.float64)[:, None] * self.frequencies()[None, :]
            cos = torch.from_numpy((np.cos(angle) * self.magnitude).astype(np.float32)).to(runtime.device)
            sin = torch.from_numpy((np.sin(angle) * self.magnitude).astype(np.float32)).to(runtime.device)
            return cos.contiguous(), sin.contiguous()
        key = ("rotary", self.dims, self.theta, self.max_positions, self.scaling)
        shared = getattr(runtime, "shared", None)
        return shared(key, build) if shared else build()


@register_part("position", "rope_interleaved")
class InterleavedRotary(_Rotary):
    """Pairs (2i, 2i + 1), angle = position * theta**(-2i / dims)."""
    interleaved = True


@register_part("position", "rope_yarn")
class ScaledHalfSplitRotary(_Rotary):
    """Pairs (i, i + dims / 2); with ``scaling`` (factor, original, fast, slow) the frequencies are those of
    ``yarn_frequencies`` and cos and sin are multiplied by 0.1 ln(factor) + 1."""
    interleaved = False


@register_part("position", "rope_linear")
class LinearScaledRotary(Part):
    """Pairs (i, i + dims / 2) over the first ``dims`` elements, angle = position * theta**(-2i / dims) / factor
    (``factor`` 1: no scaling).  Tables as the other rotations keep them: float64 on the host, float32 on the device,
    one copy per set of constants."""
    interleaved = False

    def __init__(self, prefix: str, dims: int, theta: float, max_positions: int, factor: float = 1.0):
        if dims <= 0 or dims % 2:
            raise ValueError("rotary position encoding needs an even, positive number of elements")
        if theta <= 0 or max_positions <= 0 or factor <= 0:
            raise ValueError("rotary position encoding needs positive theta, max_positions and factor")
        self.dims, self.theta, self.max_positions, self.factor = int(dims), float(theta), int(max_positions), float(factor)

    def frequencies(self) -> np.ndarray:
        return self.theta ** (-2.0 * np.arange(self.dims // 2, dtype=np.float64) / self.dims) / self.factor

    def rotary_tables(self, runtime):
        def build():
            angle = np.arange(self.max_positions, dtype=np.float64)[:, None] * self.frequencies()[None, :]
            cos = torch.from_numpy(np.cos(angle).astype(np.float32)).to(runtime.device)
            sin = torch.from_numpy(np.sin(angle).astype(np.float32)).to(runtime.device)
            return cos.contiguous(), sin.contiguous()
        key = ("rope_linear", self.dims, self.theta, self.max_positions, self.factor)
        shared = getattr(runtime, "shared", None)
        return shared(key, build) if shared else build()
