"""Normalisation parts."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.specs import NormSpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .registry import register_norm


@register_norm("rmsnorm")
class RMSNorm:
    """out = v * rsqrt(mean(v^2) + eps) * weight with v = x (+ delta), everything in 32-bit
    (src/layers/rms_norm.cu:77-93).  The weight multiplies directly (no 1 + w)."""

    accepts_partials = True    # `delta` may be an ops.PartialSum: the kernel adds the k-splits as it reads
    center = False             # what a kernel that applies this norm itself needs to know beside weight and eps

    def __init__(self, spec: NormSpec, size: int):
        self.eps = float(spec.eps)
        self.size = size
        self.name = getattr(spec, "weight_name", "weight")     # '' when the tensor is named like the norm itself
        self.weight: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        return {self.name: ParamSpec((self.size,), role="scale", init=("one_plus_normal", 0.01))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.name].contiguous()

    def add_normed(self, h: torch.Tensor, y, copy_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
        """h += norm(y) * weight in place (the norm of a sublayer's OUTPUT joined with the residual add);
        returns the new h in `copy_dtype` if one is asked for."""
        return ops.rmsnorm_add(h, y, self.weight, self.eps, copy_dtype)

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype, delta: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None, write_sum: bool = False) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps, out_dtype, delta=delta, rows=rows, write_sum=write_sum)


@register_norm("layernorm")
class LayerNorm:
    """out = (v - mean(v)) * rsqrt(mean((v - mean(v))^2) + eps) * weight with v = x (+ delta), a weight and no
    bias, everything in 32-bit.  The kernel is the one that serves models with several residual streams, run on
    one stream with unit coefficients."""

    accepts_partials = True
    center = True

    def __init__(self, spec: NormSpec, size: int):
        self.eps = float(spec.eps)
        self.size = size
        self.name = getattr(spec, "weight_name", "weight")
        self.weight: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        return {self.name: ParamSpec((self.size,), role="scale", init=("one_plus_normal", 0.01))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.name].contiguous()

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype, delta=None, rows: Optional[torch.Tensor] = None,
                write_sum: bool = False) -> torch.Tensor:
        if isinstance(delta, ops.PartialSum) and delta.rounds_to is not None:
            delta = ops.as_tensor(delta)
        return ops.stream_norm(x, delta, None, None, None, self.weight, self.eps, True, out_dtype, rows=rows,
                               write_back=write_sum)


class PendingNormed:
    """A sublayer's output that has not joined the residual stream yet, with the norm it passes on its way there
    (None: it joins as it is).  The kernel that norms the next sublayer's input applies both on the way."""

    def __init__(self, y, norm=None):
        self.y, self.norm = y, norm


@register_norm("tanh")
class TanhNorm:
    """out = tanh(alpha * v) * weight + bias with v = x (+ what is pending), elementwise, everything in 32-bit: a norm
    that computes no mean and no variance (the spec's eps is not used).  `alpha` is one learned number.  Tensors:
    the weight under the norm's own name (or `weight_name`), `alpha` [] and `b` [size] beside it.  `delta` may be a
    `PendingNormed`: a sublayer's output and the norm of this kind that it passes before the residual add, which
    the same kernel applies; with `write_sum` (or always for a `PendingNormed`) the sum is written back into x."""

    accepts_partials = True
    center = False

    def __init__(self, spec: NormSpec, size: int):
        self.eps = float(spec.eps)
        self.size = size
        self.name = getattr(spec, "weight_name", "weight")
        self.weight = self.alpha = self.bias = None

    def parameters(self) -> Dict[str, ParamSpec]:
        return {self.name: ParamSpec((self.size,), role="scale", init=("one_plus_normal", 0.05)),
                "alpha": ParamSpec((), role="scale", init=("one_plus_normal", 0.1)),
                "b": ParamSpec((self.size,), role="scale", init=("normal", 0.05))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.name].contiguous()
        self.alpha = tensors["alpha"].reshape(1).contiguous()
        self.bias = tensors["b"].contiguous()

    def triple(self):
        return (self.alpha, self.weight, self.bias)

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype, delta=None, rows: Optional[torch.Tensor] = None,
                write_sum: bool = False) -> torch.Tensor:
        post = None
        if isinstance(delta, PendingNormed):
            post = delta.norm.triple() if delta.norm is not None else None
            delta = delta.y
        if isinstance(delta, ops.PartialSum) and delta.rounds_to is not None:
            delta = ops.as_tensor(delta)             # k-splits of a product that is not 32-bit: their sum is rounded first
        return ops.tanh_norm(x, delta, post, self.triple(), out_dtype, rows=rows)

    def add_normed(self, h: torch.Tensor, y) -> None:
        """h += norm(y) in place, nothing returned: the norm on a sublayer's output with nothing behind it."""
        ops.tanh_norm(h, y, self.triple(), None)
