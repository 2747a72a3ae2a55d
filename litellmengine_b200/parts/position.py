"""Position encodings.  A position part owns how queries and keys are encoded by position.

Two ways to be one:
  * `rotation(batch)` returns a `Rotation` (the tables of a half-split rotation) or None (nothing
    is done to q and k): the attention mixer's fused kernel then normalises, rotates and writes
    the cache in one pass.
  * no `rotation` method, but `apply(q, k, batch) -> (q, k)`: float32 [T, heads, head_dim]
    tensors (k is None for a mixer without keys of its own) after the per-head norms, returned
    encoded.  The mixer runs the norms, this method, and the cache write as separate kernels,
    so an encoding of any kind needs no change to the mixer or to its kernels.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..config.specs import PositionSpec
from .registry import register_position


@dataclass
class Rotation:
    """What the fused kernel rotates by: pairs (i, i + rotary_dim/2) of a head by the angle
    float(position) * inv_freq[i]; `angles` is the step's table of their sines and cosines
    (float32 [T, rotary_dim/2, 2]) or None, in which case the kernel computes them."""
    inv_freq: torch.Tensor
    rotary_dim: int
    angles: Optional[torch.Tensor] = None


@register_position("none")
class NoPosition:
    def __init__(self, spec: PositionSpec, head_dim: int, device):
        pass

    def rotation(self, batch) -> Optional[Rotation]:
        return None


@register_position("sinusoid_added")
class AddedSinusoid:
    """A model's `embedding_position`: the vector with entry 2i = sin(p * theta^(-2i/width)) and entry
    2i+1 = cos of the same angle is added to the embedding of the token at position p, in 32-bit, inside
    the embedding kernel.  The frequencies are tabulated once in double precision, so that the angle is
    exact to a float's last bit at any position.  `embed` returns the float32 stream; in a 16-bit run
    mode the same rows in the compute dtype are left in `batch.tables["stream_copy"]` for a first layer
    whose sublayers read the stream itself."""

    def __init__(self, spec: PositionSpec, width: int, device):
        if not spec.theta > 0:
            raise ValueError("the sinusoid's base must be positive")
        i = torch.arange((width + 1) // 2, dtype=torch.float64)
        self.inv_freq = torch.pow(torch.tensor(float(spec.theta), dtype=torch.float64), -2.0 * i / width).to(device)

    def embed(self, batch, table: torch.Tensor, compute_dtype: torch.dtype) -> torch.Tensor:
        from ..csrc import ops
        narrow = None if compute_dtype == torch.float32 else compute_dtype
        h, copy = ops.embedding_sinusoid(batch.token_ids, table, batch.positions, self.inv_freq, batch.status,
                                         feedback=getattr(batch, "feedback", None), copy_dtype=narrow)
        if copy is not None and getattr(batch, "tables", None) is not None:
            batch.tables["stream_copy"] = (h, copy)
        return h


@register_position("rope")
class RotaryPosition:
    """Half-split rotation: inv_freq[i] = powf(theta, -(2 i) / rotary_dim) with theta and the
    exponent held as float32, as the reference computes per call (src/layers/rotary.cu:81-83).
    The table is made once, as the correctly rounded float32 power (the power taken in double
    precision of the float32 operands, then rounded): an inv_freq that is one unit in the last
    place off turns into an angle error of position * 6e-8, which is what separates one powf
    from another at long contexts.  The angle float(pos) * inv_freq[i] and its sine and cosine
    are computed in 32-bit inside the kernel (src/layers/rotary.cu:101-105)."""

    def __init__(self, spec: PositionSpec, head_dim: int, device):
        rd = spec.rotary_dim or head_dim
        if rd <= 0 or rd % 2 != 0 or rd > head_dim:
            raise ValueError(f"rotary_dim {rd} must be even and at most head_dim {head_dim}")
        if not spec.theta > 0:
            raise ValueError("rope theta must be positive")
        self.rotary_dim = rd
        i = torch.arange(rd // 2, dtype=torch.float32)
        expo = -(2.0 * i) / torch.tensor(float(rd), dtype=torch.float32)            # float32 quotient
        theta32 = torch.tensor(spec.theta, dtype=torch.float32)
        inv = torch.pow(theta32.double(), expo.double()).to(torch.float32)
        self.inv_freq = inv.to(device).contiguous()
        self._key = ("rope", float(spec.theta), rd)
        self._table_ok = rd == head_dim and head_dim in (64, 128)      # what the kernel that reads the table takes

    def rotation(self, batch) -> Rotation:
        return Rotation(self.inv_freq, self.rotary_dim, self.angles(batch))

    def angles(self, batch):
        """The step's table of sines and cosines, made by the first layer that asks and shared by
        all layers with the same theta and rotary_dim; None for steps of few tokens, whose kernels
        compute their own before they wait for the projection."""
        from ..csrc import ops
        tables = getattr(batch, "tables", None)
        if (tables is None or not self._table_ok or batch.num_tokens < ops.ROPE_TABLE_MIN_TOKENS
                or not self.inv_freq.is_cuda):
            return None
        if self._key not in tables:
            tables[self._key] = ops.rope_angles(batch.positions, self.inv_freq)
        return tables[self._key]


@register_position("rope_pairs")
class PairRotation:
    """Rotation of neighbouring pairs: entries 2i and 2i + 1 of the first `rotary_dim` entries of a head turn by the
    angle float(position) * freq[i]; (a, b) becomes (a cos - b sin, b cos + a sin) * magnitude.  freq[i] =
    theta^(-2i/rotary_dim), stretched by `scaling` = (factor, original, fast, slow) where the spec has one: pairs
    whose wavelength is long against the original context are slowed by `factor`, short ones stay, with a linear
    ramp over the pair index between the two (see `PositionSpec`).  The table is made once, in double precision, and
    rounded to float32; angle, sine and cosine are 32-bit inside the kernels that rotate.  A mixer reads `freq`,
    `rotary_dim`, `magnitude` and `pairs` and hands them to its kernel."""

    pairs = True

    def __init__(self, spec: PositionSpec, head_dim: int, device):
        import math
        rd = spec.rotary_dim or head_dim
        if rd <= 0 or rd % 2 or rd > head_dim:
            raise ValueError(f"rotary_dim {rd} must be even and at most {head_dim}")
        if not spec.theta > 1.0:
            raise ValueError("the rotation's base must exceed 1")
        p = dict(spec.params)
        base = float(spec.theta)
        freq = [base ** (-2.0 * i / rd) for i in range(rd // 2)]
        if p.get("scaling") is not None:
            factor, original, fast, slow = (float(v) for v in p["scaling"])
            pair = lambda turns: rd * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
            lo, hi = max(math.floor(pair(fast)), 0), min(math.ceil(pair(slow)), rd - 1)
            for i in range(rd // 2):
                ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
                freq[i] = freq[i] / factor * ramp + freq[i] * (1.0 - ramp)
        self.rotary_dim = rd
        self.magnitude = float(p.get("magnitude", 1.0))
        self.freq = torch.tensor(freq, dtype=torch.float64).to(torch.float32).to(device).contiguous()

    def kernel_args(self):
        """(freq, dims, magnitude, pairs) as the rotating kernels take them."""
        return (self.freq, self.rotary_dim, self.magnitude, self.pairs)
