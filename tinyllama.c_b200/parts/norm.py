"""RMSNorm over the 32-bit residual stream.

o = x * 1/sqrt(mean(x^2) + eps) * w  (CodeClaper/tinyllama.c cpu_op.c:44-64, applied per
row at cpu_op.c:526-533).  The reference fixes eps at 1e-6 (def.h:10); here it is a
parameter.  Statistics are 32-bit; the output takes the activation type.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from .base import LayerCache, Part, StateRequest, StepInfo, WeightSpec, register_norm, to_vec


@register_norm("rmsnorm")
class RMSNorm(Part):
    def __init__(self, width: int, eps: float, weight_name: str, offset: float = 0.0):
        """offset: what is added to the stored weight (1.0 for a weight stored as its distance from one)."""
        self.width, self.eps, self.weight_name, self.offset = int(width), float(eps), weight_name, float(offset)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.weight_name, (self.width,), "ones" if self.offset == 0.0 else "near_zero")]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        self.weight = to_vec(tensors[self.weight_name], device)
        if self.offset != 0.0:
            self.weight = (self.weight + self.offset).contiguous()        # in 32 bits

    def forward(self, x32: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        ops.rmsnorm(x32, self.weight, self.eps, out, rows)
        return out

    def add_normed(self, parts: Optional[torch.Tensor], residual: torch.Tensor, extra: Optional[torch.Tensor] = None,
                   gate: Optional[torch.Tensor] = None, copy: Optional[torch.Tensor] = None) -> None:
        """As a sublayer's output norm: residual += norm(y) with y = the sum of parts [T, (n,) D] (+ sigmoid(gate[t]) *
        extra[t], gate being a logit per row).  copy [T, D]: receives the new residual rows in its own type (what the
        next sublayer reads where it has no norm in front)."""
        ops.rmsnorm_add(parts, self.weight, self.eps, residual, extra, gate, gate_sigmoid=True, copy=copy)


@register_norm("layernorm")
class LayerNorm(Part):
    """Layer norm with a weight and no bias: (x - mean(x)) / sqrt(var(x) + eps) * w, var the mean of the squared deviations.
    Statistics are 32-bit.  Two layer norms of one width and eps applied to the SAME rows (a layer whose mixer and
    feed-forward each norm the layer's input) share the statistics: forward_pair writes both results in one pass."""

    def __init__(self, width: int, eps: float, weight_name: str):
        self.width, self.eps, self.weight_name = int(width), float(eps), weight_name
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.weight_name, (self.width,), "ones")]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        self.weight = to_vec(tensors[self.weight_name], device)

    def forward(self, x32: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        ops.layernorm(x32, self.weight, self.eps, out, rows)
        return out

    def pairs_with(self, other) -> bool:
        return type(other) is LayerNorm and other.width == self.width and other.eps == self.eps

    def forward_pair(self, x32: torch.Tensor, out: torch.Tensor, other: "LayerNorm", out_other: torch.Tensor) -> None:
        """out = this norm of x32, out_other = `other`'s norm of the same rows (pairs_with(other) must hold)."""
        ops.layernorm(x32, self.weight, self.eps, out, None, other.weight, out_other)


@register_norm("rmsnorm_shift")
class RMSNormShift(RMSNorm):
    """RMSNorm followed by a token shift: with n[t] the normed row, the result is n[t] + (n[t-1] - n[t]) * mix, mix a
    learned vector [D] and n[t-1] the normed row of the sequence's previous token (zeros before the first).  The last
    normed row of a sequence is kept per sequence (32-bit) between steps."""

    def __init__(self, width: int, eps: float, weight_name: str, mix_name: str, offset: float = 0.0,
                 cache_key: str = "shift"):
        super().__init__(width, eps, weight_name, offset)
        self.mix_name, self.cache_key = mix_name, cache_key
        self.mix: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return super().weight_specs() + [WeightSpec(self.mix_name, (self.width,), "unit_interval")]

    def cache_requests(self) -> list:
        return [StateRequest(self.cache_key, (self.width,))]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        super().bind(tensors, dtype, device)
        self.mix = to_vec(tensors[self.mix_name], device)

    def forward(self, x32, out, rows=None):
        raise ValueError("rmsnorm_shift: a norm with a token shift needs the step and the cache (forward_step)")

    def forward_step(self, x32: torch.Tensor, out: torch.Tensor, step: StepInfo, cache: LayerCache) -> torch.Tensor:
        if not cache.writes:
            raise ValueError("rmsnorm_shift: the kept row would advance twice in a step on another entry's cache")
        ops.rmsnorm_shift(x32, self.weight, self.mix, self.eps, cache.state[self.cache_key], step, out)
        return out


@register_norm("none")
class NoNorm(Part):
    """No norm: the sublayer reads the residual stream itself.  forward() hands the stream over in the activation type
    (bfloat16 products want bfloat16 inputs); a mixer that says `reads_stream = True` is given the 32-bit rows instead."""
    identity = True

    def __init__(self, width: int):
        self.width = int(width)

    def forward(self, x32: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if rows is not None:
            raise ValueError("norm 'none' copies whole steps; it serves no row selection")
        ops.convert(x32, out)
        return out


@register_norm("rmsnorm_mean")
class RMSNormMean(Part):
    """How a layer joins several mixers that run side by side: every mixer's result is RMS-normed by itself with a weight
    of its own, and the results are averaged: y = scale * sum_i rmsnorm(y_i) * w_i (scale 1/n unless given).  Where the
    layer has a mixer output norm, residual += out_norm(y) in the same kernel."""

    def __init__(self, width: int, eps: float, weight_names, scale: Optional[float] = None):
        self.width, self.eps, self.weight_names = int(width), float(eps), tuple(weight_names)
        if not (1 <= len(self.weight_names) <= 8):
            raise ValueError(f"rmsnorm_mean: {len(self.weight_names)} summands (1..8)")
        self.scale = float(scale) if scale is not None else 1.0 / len(self.weight_names)
        self.weights: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(n, (self.width,), "ones") for n in self.weight_names]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        self.weights = torch.stack([to_vec(tensors[n], device) for n in self.weight_names]).contiguous()

    def add_joined(self, parts: torch.Tensor, residual: torch.Tensor, out_norm: Optional[RMSNorm] = None,
                   copy: Optional[torch.Tensor] = None) -> None:
        """parts float32 [T, n, D]: the mixers' results side by side.  copy [T, D]: receives the new residual rows in its
        own type."""
        if out_norm is not None and type(out_norm) is not RMSNorm:
            raise ValueError("rmsnorm_mean: the norm after the join must be a plain RMS norm")
        ops.rmsnorm_mean_add(parts, self.weights, self.eps, self.scale, residual,
                             None if out_norm is None else out_norm.weight, 0.0 if out_norm is None else out_norm.eps, copy=copy)
