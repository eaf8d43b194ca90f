"""Position encodings of the attention mixer.

Rotary, split-half ("NEOX") form: for pair i of the first r dims of a head,
theta_i = 1/base^(2i/r), angle = position * theta_i, (a, b) = (x[i], x[i + r/2]) ->
(a cos - b sin, a sin + b cos); dims past r are copied (CodeClaper/tinyllama.c
cpu_op.c:637-651).  The reference recomputes powf/cosf/sinf per element; here the
inverse frequencies are a table built once in 64-bit and rounded to 32-bit, and the
angle is the 32-bit product with the integer position.  A rotation is described to the
mixer by its table: the kernels that store keys and values (and single-token attention)
rotate by themselves.  "none" rotates nothing.  Any other encoding of positions in q and k
is a Position part with a transform() of its own (see parts/base.py).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .base import Position, register_position


@register_position("rope_neox")
class RotaryNeox(Position):
    layout = "split_half"          # which dimensions form a pair: (i, i + r/2)

    def __init__(self, head_dim: int, theta: float, rope_dim: Optional[int] = None, scaling: Optional[dict] = None):
        """scaling: how the frequencies f_i = theta^(-2i/r) are stretched for sequences longer than `original` positions.
        kind "bands": with the wave's length l = 2 pi / f, f is kept where l < original / high, divided by factor where
        l > original / low, and blended between, (1 - s) f / factor + s f with s = (original / l - low) / (high - low).
        kind "ramp": with x(t) = r ln(original / (2 pi t)) / (2 ln theta) the (real) pair index whose wave makes t turns over
        `original` positions, lo = max(floor(x(fast)), 0), hi = min(ceil(x(slow)), r - 1) and ramp_i = clamp((i - lo) /
        max(hi - lo, 0.001), 0, 1): f_i / factor * ramp_i + f_i (1 - ramp_i), and every cosine and sine is multiplied by
        0.1 ln(factor) + 1 (`amplitude`; a mixer that rotates by itself asks for it)."""
        self.head_dim = int(head_dim)
        self.scaling = dict(scaling) if scaling else None
        self.amplitude = 1.0
        if self.scaling is not None:
            kind = self.scaling.get("kind")
            need = {"bands": ("factor", "low", "high", "original"), "ramp": ("factor", "fast", "slow", "original")}.get(kind)
            if need is None or any(not isinstance(self.scaling.get(k), (int, float)) or isinstance(self.scaling.get(k), bool)
                                   for k in need):
                raise ValueError(f"rotation scaling {scaling!r}: kind 'bands' (factor, low, high, original) or 'ramp' "
                                 f"(factor, fast, slow, original), all numbers")
            if self.scaling["factor"] <= 0 or self.scaling["original"] <= 0 or (kind == "bands" and self.scaling["high"] == self.scaling["low"]):
                raise ValueError(f"rotation scaling {scaling!r}: factor and original must be positive, high and low differ")
        self.rope_dim = int(rope_dim) if rope_dim else self.head_dim      # falcon_h1.c:265
        if self.rope_dim % 2 or self.rope_dim > self.head_dim:
            raise ValueError(f"rotary width {self.rope_dim} must be even and at most head_dim {self.head_dim}")
        self.theta = float(theta)
        self.inv_freq: Optional[torch.Tensor] = None

    def bind(self, tensors, dtype, device) -> None:
        i = torch.arange(self.rope_dim // 2, dtype=torch.float64)
        inv = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float64), 2.0 * i / self.rope_dim)
        sc = self.scaling
        if sc is not None and sc["kind"] == "bands":
            wave = 2.0 * math.pi / inv
            s = ((sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"]))
            blend = (1.0 - s) * inv / sc["factor"] + s * inv
            inv = torch.where(wave < sc["original"] / sc["high"], inv, torch.where(wave > sc["original"] / sc["low"], inv / sc["factor"], blend))
        elif sc is not None:
            at = lambda turns: self.rope_dim * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))
            lo, hi = max(math.floor(at(sc["fast"])), 0), min(math.ceil(at(sc["slow"])), self.rope_dim - 1)
            ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            inv = inv / sc["factor"] * ramp + inv * (1.0 - ramp)
            self.amplitude = 0.1 * math.log(sc["factor"]) + 1.0
        self.inv_freq = inv.to(torch.float32).to(device).contiguous()

    def rotation_table(self) -> torch.Tensor:
        """The inverse frequencies (float32 [rope_dim/2]) for the kernels, which rotate by themselves."""
        return self.inv_freq


@register_position("rope_interleaved")
class RotaryInterleaved(RotaryNeox):
    """The same angles with neighbours as pairs: dimensions (2i, 2i+1) of the first rope_dim turn by position *
    theta^(-2i/rope_dim); (u, v) -> (u cos - v sin, v cos + u sin).  Only mixers whose kernels rotate this way take it."""
    layout = "interleaved"


@register_position("none")
class NoPosition(RotaryNeox):
    """No position encoding: queries and keys are stored as projected."""

    def __init__(self, head_dim: int):
        super().__init__(head_dim, 10000.0, head_dim)

    def bind(self, tensors, dtype, device) -> None:
        self.inv_freq = torch.zeros(0, dtype=torch.float32, device=device)
