"""Gated delta-rule mixer: a recurrence whose state is a matrix per head that every token corrects towards its own
(key, value) pair.

Three projections of the mixer's input h give queries and keys (G heads of dk values each) and values (H heads of dv;
value head i reads query/key head i // (H / G)).  All three are smoothed along the sequence, channel by channel, by a
depthwise filter of `taps` weights that ends at the current token (weights [channels, taps], newest tap last; the
sequence is preceded by zeros), then go through SiLU.  Queries and keys are then scaled to unit length per head,
x * rsqrt(sum(x^2) + l2_eps), the query further by q_scale (dk ** -0.5 unless given).  Per head the
write strength b = sigmoid(W_b h) and the decay a = exp(-exp(A_log) * softplus(W_a h + dt_bias)); the state M [dk, dv] is
decayed, asked what it would return for the new key (the prediction p), corrected by the write w, and read with the query:

    M <- a M;    p = M^T k;    w = b (v - p);    M <- M + k w^T;    r = M^T q

(the read-out comes last: it already contains what this token wrote).  Each head's r gets an RMS norm across its dv
values with one weight vector [dv] common to all heads, is gated by silu(W_g h), and W_o maps the heads' results back.
M [H, dk, dv] and the last taps - 1 inputs of the convolution are kept per sequence between steps (32-bit; a sequence
at position 0 starts from zeros); everything between the projections and the output projection is 32-bit.

The six projections of h are one product.  The convolution (with the decay beside it: dt = softplus(W_a h + dt_bias),
a = exp(dt * -exp(A_log))) is the kernel that serves every short convolution of the library.

Options.  decay="channel": a factor per head AND key channel, a [H, dk] = exp(-exp(A_log_h) * softplus(W_a2 (W_a1 h) +
dt_bias)) with a low-rank pair of matrices and dt_bias of H * dk values; the state's rows are decayed each by its own
factor, M <- diag(a) M.  gate_rank: the gate's projection is a low-rank pair as well, W_g2 (W_g1 h).  gate="sigmoid":
the read-out is gated by sigmoid(.) instead of silu(.).  The ranks are no keys of a configuration: the stored matrices
give them (shapes_from).  The first matrices of both pairs are stacked with the other projections of h; the hidden rows
are rounded to the activation type and the two second products follow (dt_bias in the epilogue of the decay's).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ... import ops
from ..base import LayerCache, Part, StateRequest, StepInfo, WeightSpec, register_mixer, scratch_buf, to_vec
from ..linear import StackedLinear


@register_mixer("delta")
class DeltaMixer(Part):
    def __init__(self, hidden: int, n_heads: int, n_qk_heads: int, key_dim: int, v_dim: int, conv_taps: int, eps: float,
                 names: Dict[str, str], l2_eps: float = 1e-6, q_scale: Optional[float] = None, cache_key: str = "delta",
                 decay: str = "head", gate: str = "silu", low_rank_gate: bool = False, decay_rank: Optional[int] = None,
                 gate_rank: Optional[int] = None):
        """names: tensor names of q, k, v (their convolutions are these names + '.conv'), b, a, A_log, dt_bias, norm, g, o;
        with decay "channel" a1 and a2 instead of a, with low_rank_gate g1 and g2 instead of g.  eps: of the output norm.
        decay_rank, gate_rank: the hidden widths of the low-rank pairs for a model that is yet to be written (a stored
        model's matrices give them)."""
        if decay not in ("head", "channel") or gate not in ("silu", "sigmoid"):
            raise ValueError(f"delta: decay '{decay}' (head or channel), gate '{gate}' (silu or sigmoid)")
        self.decay_kind, self.gate_kind, self.low_rank_gate = decay, gate, bool(low_rank_gate)
        self.decay_rank = int(decay_rank) if decay_rank else None
        self.gate_rank = int(gate_rank) if gate_rank else None
        self.hidden, self.H, self.G, self.dk, self.dv, self.K = (int(hidden), int(n_heads), int(n_qk_heads), int(key_dim),
                                                                 int(v_dim), int(conv_taps))
        if self.H % self.G:
            raise ValueError(f"delta: {self.H} heads are not a multiple of {self.G} query/key heads")
        if not (1 <= self.dk <= ops.MAX_DELTA_KEY_DIM):
            raise ValueError(f"delta: keys of {self.dk} values are outside what the kernel is built for (1..{ops.MAX_DELTA_KEY_DIM})")
        if not (1 <= self.K <= ops.MAX_CONV_TAPS):
            raise ValueError(f"delta: {self.K} convolution taps are outside what the kernels are built for (1..{ops.MAX_CONV_TAPS})")
        if self.H > ops.MAX_HEADS:
            raise ValueError(f"delta: {self.H} heads exceed the kernels' limit of {ops.MAX_HEADS}")
        self.eps, self.l2_eps = float(eps), float(l2_eps)
        self.q_scale = float(q_scale) if q_scale is not None else self.dk ** -0.5
        self.names, self.cache_key = dict(names), cache_key
        n = self.names
        self.Cd = 2 * self.G * self.dk + self.H * self.dv          # channels of the convolution: q | k | v
        self.o = StackedLinear(self.H * self.dv)
        self.o.add(n["o"], hidden)
        self.dtype = None
        self._lay_out()

    def _lay_out(self) -> None:
        """The stacked projection of h (its widths depend on the ranks of the low-rank pairs)."""
        n, hidden = self.names, self.hidden
        default = max(8, hidden // 16)
        self.ra = (self.decay_rank or default) if self.decay_kind == "channel" else 0
        self.rg = (self.gate_rank or default) if self.low_rank_gate else 0
        self.proj = StackedLinear(hidden)
        self.q_off = self.proj.add(n["q"], self.G * self.dk)
        self.k_off = self.proj.add(n["k"], self.G * self.dk)
        self.v_off = self.proj.add(n["v"], self.H * self.dv)
        self.b_off = self.proj.add(n["b"], self.H)
        # what comes last is what the second products read: the hidden rows of the low-rank pairs side by side
        self.a_off = self.proj.add(n["a1"], self.ra) if self.ra else self.proj.add(n["a"], self.H)
        self.g_off = self.proj.add(n["g1"], self.rg) if self.rg else self.proj.add(n["g"], self.H * self.dv)
        self.a2 = self.g2 = None
        if self.ra:
            self.a2 = StackedLinear(self.ra)
            self.a2.add(n["a2"], self.H * self.dk, n["dt_bias"])      # dt_bias joins in the product's epilogue
        if self.rg:
            self.g2 = StackedLinear(self.rg)
            self.g2.add(n["g2"], self.H * self.dv)

    def shapes_from(self, shapes: Dict[str, tuple]) -> None:
        """The hidden widths of the low-rank pairs are no keys of the configuration: the stored matrices give them."""
        n = self.names
        if self.decay_kind == "channel" and n["a1"] in shapes:
            self.decay_rank = int(shapes[n["a1"]][0])
        if self.low_rank_gate and n["g1"] in shapes:
            self.gate_rank = int(shapes[n["g1"]][0])
        self._lay_out()

    def weight_specs(self) -> List[WeightSpec]:
        n = self.names
        specs = self.proj.weight_specs() + self.o.weight_specs() + [
            WeightSpec(n["q"] + ".conv", (self.G * self.dk, self.K), "conv"), WeightSpec(n["k"] + ".conv", (self.G * self.dk, self.K), "conv"),
            WeightSpec(n["v"] + ".conv", (self.H * self.dv, self.K), "conv"), WeightSpec(n["A_log"], (self.H,), "a_log"),
            WeightSpec(n["norm"], (self.dv,), "ones")]
        if self.a2 is not None:
            specs += [WeightSpec(n["a2"], (self.H * self.dk, self.ra)), WeightSpec(n["dt_bias"], (self.H * self.dk,), "dt_bias")]
        else:
            specs.append(WeightSpec(n["dt_bias"], (self.H,), "dt_bias"))
        if self.g2 is not None:
            specs += self.g2.weight_specs()
        return specs

    def cache_requests(self) -> list:
        return [StateRequest(self.cache_key + ".conv", (self.K - 1, self.Cd)),
                StateRequest(self.cache_key + ".state", (self.H, self.dk, self.dv))]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        n = self.names
        self.dtype = dtype
        self.proj.bind(tensors, dtype, device)
        self.o.bind(tensors, dtype, device)
        self.conv_w = to_vec(torch.cat([tensors[n[x] + ".conv"].to(torch.float32).reshape(-1, self.K) for x in ("q", "k", "v")], dim=0),
                             device)
        self.A = (-torch.exp(tensors[n["A_log"]].to(torch.float32))).to(device).contiguous()      # decay = exp(dt * A)
        self.dt_bias = to_vec(tensors[n["dt_bias"]], device)
        for second in (self.a2, self.g2):
            if second is not None:
                second.bind(tensors, dtype, device)
        self._none = torch.zeros(0, dtype=torch.float32, device=device)
        self.norm_w = to_vec(tensors[n["norm"]], device).repeat(self.H).contiguous()              # one weight for every head

    def forward(self, normed: torch.Tensor, step: StepInfo, cache: LayerCache, residual: torch.Tensor,
                accumulate: bool = True) -> None:
        if not (cache.writes and cache.kv_writes):
            raise ValueError("delta: a recurrent mixer cannot run on another layer's cache without storing "
                             "(its window and state would advance twice in one step)")
        T, dev, f32 = step.n_rows, normed.device, torch.float32
        new = lambda tag, shape, dt: scratch_buf(f"delta.{self.cache_key}.{tag}", shape, dt, dev)
        proj = new("proj", (T, self.proj.out_features), f32)
        self.proj.forward(normed, proj)
        qkv = new("qkv", (T, self.Cd), f32)
        fresh = len(step.host_start) == step.n_seqs and not any(step.host_start)
        channel = self.decay_kind == "channel"
        if channel:            # the convolution alone; the decays come from the second product of their pair
            none = self._none.view(T, 0) if T else self._none
            ops.mamba_conv(proj, self.q_off, self.a_off, self.conv_w, None, self._none, self._none, cache.state[self.cache_key + ".conv"],
                           step.cu_seqlens, step.row_seq, step.slots, step.start_pos, qkv, none, none, step.max_new == 1, False, fresh)
        else:
            dt, decay = new("dt", (T, self.H), f32), new("decay", (T, self.H), f32)
            ops.mamba_conv(proj, self.q_off, self.a_off, self.conv_w, None, self.dt_bias, self.A, cache.state[self.cache_key + ".conv"],
                           step.cu_seqlens, step.row_seq, step.slots, step.start_pos, qkv, dt, decay, step.max_new == 1, False, fresh)
        gate = proj[:, self.g_off:self.g_off + self.H * self.dv]
        if self.ra or self.rg:
            # the hidden rows of the low-rank pairs, side by side at the end of the projection, in the activation type
            hidden = new("hidden", (T, self.ra + self.rg), self.dtype)
            first = self.a_off if self.ra else self.g_off
            ops.convert(proj[:, first:first + self.ra + self.rg], hidden)
            if self.ra:
                decay = new("decay", (T, self.H * self.dk), f32)
                self.a2.forward(hidden[:, :self.ra], decay)
            if self.rg:
                gate = new("gate", (T, self.H * self.dv), f32)
                self.g2.forward(hidden[:, self.ra:], gate)
        beta = new("beta", (T, self.H), f32)
        ops.delta_prepare(qkv, self.q_off, self.k_off, self.G, self.dk, self.l2_eps, self.q_scale, proj, self.b_off, self.H, beta,
                          decay if channel else None, self.A if channel else None)
        y = new("y", (T, self.H * self.dv), f32)
        ops.delta_rule(qkv, self.q_off, self.k_off, self.v_off, beta, decay, cache.state[self.cache_key + ".state"], step, y,
                       self.H, self.G, self.dk, self.dv, per_channel=channel)
        gated = new("gated", (T, self.H * self.dv), self.dtype)
        ops.gated_rmsnorm(y, gate, self.norm_w, self.eps, self.H, True, gated, gate=self.gate_kind)
        self.o.forward(gated, residual, accumulate=accumulate)
