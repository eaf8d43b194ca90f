"""Dense gated feed-forward.

d = W_down (act(W_gate x) * (W_up x)), act = SiLU (SwiGLU; CodeClaper/tinyllama.c
falcon_h1.c:382-395) or another registered activation.  The gate and up projections are
stacked into one product.  The multiplier on the gate's pre-activation, the one on the
output, the biases, the choice of activation and of tensor names have no counterpart in
the reference.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from .base import Part, PartSpec, WeightSpec, act_empty, register_feed_forward, scratch_buf
from .linear import StackedLinear


@register_feed_forward("swiglu")
class SwiGLU(Part):
    def __init__(self, hidden: int, intermediate: int, prefix: str, bias: bool = False, gate_scale: float = 1.0,
                 down_scale: float = 1.0, act: str = "silu", names: Optional[Dict[str, str]] = None, limit: float = 0.0,
                 alpha: float = 1.0):
        """act: "silu", "gelu_tanh", or "swish_clamped": with g = min(W_gate h, limit) and u = W_up h held within +-limit,
        g * sigmoid(alpha g) * (u + 1) (the product and the activation are then two kernels).  names: tensor names of gate, up, down after the prefix (default: the
        gate_proj.weight / up_proj.weight / down_proj.weight of the architecture's checkpoints; biases, where asked
        for, are those names with .bias for .weight)."""
        self.hidden, self.F = int(hidden), int(intermediate)
        if act not in ops.DENSE_ACTS:
            raise ValueError(f"feed-forward: unknown activation '{act}'; known: {sorted(ops.DENSE_ACTS)}")
        if act == "swish_clamped" and not limit > 0:
            raise ValueError(f"feed-forward: the clamped activation needs a positive limit, got {limit!r}")
        self.act, self.limit, self.alpha = act, float(limit), float(alpha)
        nm = dict(gate="gate_proj.weight", up="up_proj.weight", down="down_proj.weight")
        nm.update(names or {})
        w = lambda n: prefix + nm[n]
        b = (lambda n: prefix + (nm[n][:-len(".weight")] if nm[n].endswith(".weight") else nm[n]) + ".bias") if bias \
            else (lambda n: None)
        self.gate_up = StackedLinear(hidden)
        self.gate_up.add(w("gate"), self.F, b("gate"), 1.0, gate_scale)
        self.gate_up.add(w("up"), self.F, b("up"))
        self.down = StackedLinear(self.F)
        self.down.add(w("down"), hidden, b("down"), 1.0, down_scale)

    def weight_specs(self) -> List[WeightSpec]:
        return self.gate_up.weight_specs() + self.down.weight_specs()

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        self.gate_up.bind(tensors, dtype, device)
        self.down.bind(tensors, dtype, device)
        # Rows regrouped as 8 gate rows followed by their 8 up rows, so that the product's epilogue
        # has a feature's gate and up side by side and writes silu(gate) * up directly.
        self.interleaved = self.F % 8 == 0 and self.act in ops.GLU_ACTS
        if self.interleaved:
            F = self.F
            idx = torch.arange(2 * F, device=self.gate_up.weight.device).reshape(2, F // 8, 8).permute(1, 0, 2).reshape(-1)
            self.gate_up.weight = self.gate_up.weight[idx].contiguous()
            if self.gate_up.colscale is not None:
                self.gate_up.colscale = self.gate_up.colscale[idx].contiguous()
            if self.gate_up.colbias is not None:
                self.gate_up.colbias = self.gate_up.colbias[idx].contiguous()

    def forward(self, normed: torch.Tensor, residual: torch.Tensor, accumulate: bool = True) -> None:
        """Adds the result into `residual` (float32 [T, D]), or overwrites it with accumulate False."""
        T = normed.shape[0]
        act = scratch_buf("swiglu.act", (T, self.F), normed.dtype, normed.device)
        if self.interleaved:
            ops.linear_swiglu(normed, self.gate_up.weight, act, self.gate_up.colscale, self.gate_up.colbias, self.act)
        else:
            gu = scratch_buf("swiglu.gate_up", (T, 2 * self.F), torch.float32, normed.device)
            self.gate_up.forward(normed, gu)
            ops.glu(gu, act, self.act, interleaved=self.interleaved, limit=self.limit, alpha=self.alpha)
        self.down.forward(act, residual, accumulate=accumulate)



@register_feed_forward("mlp")
class DenseFeedForward(Part):
    """A feed-forward without a gate: d = W_down act(W_up x), act the square of max(., 0) ("relu_squared").  Two products
    with the activation between them (32-bit in, activation type out)."""

    def __init__(self, hidden: int, intermediate: int, names: Dict[str, str], act: str = "relu_squared"):
        """names: tensor names of up and down."""
        if act not in ("relu_squared",):
            raise ValueError(f"feed-forward: unknown activation '{act}' of a feed-forward without a gate; known: ['relu_squared']")
        self.hidden, self.F, self.act = int(hidden), int(intermediate), act
        self.up = StackedLinear(hidden)
        self.up.add(names["up"], self.F)
        self.down = StackedLinear(self.F)
        self.down.add(names["down"], hidden)

    def weight_specs(self) -> List[WeightSpec]:
        return self.up.weight_specs() + self.down.weight_specs()

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        self.up.bind(tensors, dtype, device)
        self.down.bind(tensors, dtype, device)

    def forward(self, normed: torch.Tensor, residual: torch.Tensor, accumulate: bool = True) -> None:
        """Adds the result into `residual` (float32 [T, D]), or overwrites it with accumulate False."""
        T = normed.shape[0]
        u = scratch_buf("mlp.up", (T, self.F), torch.float32, normed.device)
        self.up.forward(normed, u)
        act = scratch_buf("mlp.act", (T, self.F), normed.dtype, normed.device)
        ops.convert(u, act, self.act)
        self.down.forward(act, residual, accumulate=accumulate)

    def forward_parts(self, normed: torch.Tensor):
        """(the result as one term float32 [T, 1, D], None, None), for a block that runs this feed-forward beside its mixers
        and adds its terms afterwards (add_parts)."""
        out = scratch_buf("mlp.out", (normed.shape[0], 1, self.hidden), torch.float32, normed.device)
        self.forward(normed, out[:, 0], accumulate=False)
        return out, None, None

    def add_parts(self, terms, residual: torch.Tensor, accumulate: bool = True) -> None:
        ops.rmsnorm_add(terms[0], None, 0.0, residual, None, None, gate_sigmoid=True, accumulate=accumulate)


@register_feed_forward("moe")
class MoEFeedForward(Part):
    """Mixture of experts.  By default, with a sigmoid router:

    Router scores s = sigmoid(W_router h), the logits as 32-bit sums; a token is routed to its `top` highest-scoring experts, and
    its weights are those scores unchanged (they need not sum to one).  An expert is fed the token scaled by its weight: the result
    is sum_e expert_e(s_e h), every expert a gated feed-forward W_down (silu(W_gate x) * (W_up x)) without biases.
    Gate and up are linear, so the weight is applied to their 32-bit results.  An optional shared expert (a
    feed-forward part of its own) runs on every token and is added times sigmoid(w_sg . h), one number per token; its
    gate is computed with the router, as one more row of the router's matrix.

    The experts' weights are stacked [E, 2F, D] and [E, D, F]; rows are sorted by expert on the device, and every
    (token, choice) pair's result gets a row of its own, which the norm that follows (or `forward`) adds in the order
    of the token's choices: a token's result does not depend on what else is in the batch.

    Other routers and experts, by constructor arguments: a bias on the router's logits (router_bias_name); weights that are
    a softmax restricted to the picked logits (weights="softmax"); the weight applied to what the expert returns instead of
    to what it is fed (weight_on="output": sum_e s_e expert_e(h); the down product is linear, so the weight multiplies the
    32-bit activation); the activation act="swish_clamped": with g = min(W_gate h, limit) and u = W_up h held within
    +-limit, g * sigmoid(alpha g) * (u + 1).  weights="softmax_all": the scores are the softmax over ALL router outputs, an
    expert is chosen by its score plus a learned correction (choice_bias_name) and weighted by the score alone, not
    renormalised.  n_identity > 0: the router has that many more outputs than there are experts; the last n_identity stand for
    experts that return their input (times the weight) and have no tensors.  act="relu_squared": experts without a gate,
    W_down max(W_up h, 0)^2 (expert_names gives up and down only; the weight goes on the output)."""

    def __init__(self, hidden: int, n_experts: int, top: int, expert_ff: int, router_name: str, expert_names: Dict[str, str],
                 shared: Optional[PartSpec] = None, shared_gate_name: Optional[str] = None, router_bias_name: Optional[str] = None,
                 weights: str = "sigmoid", weight_on: str = "input", act: str = "silu", limit: float = 0.0, alpha: float = 1.0,
                 choice_bias_name: Optional[str] = None, n_identity: int = 0, weights_sum_to: float = 0.0):
        """expert_names: patterns of gate, up, down with {e} for the expert's index.  weights_sum_to > 0 (weights
        "softmax_all"): a token's weights are the chosen scores divided by their sum (+ 1e-20) times this number."""
        self.weights_sum_to = float(weights_sum_to)
        if self.weights_sum_to < 0 or (self.weights_sum_to and weights != "softmax_all"):
            raise ValueError("moe: weights normed to a sum go with weights 'softmax_all' and a positive sum")
        if weights not in ops.ROUTE_WEIGHTS or weight_on not in ("input", "output") or act not in ops.MOE_ACTS:
            raise ValueError(f"moe: unknown weighting '{weights}', weight placement '{weight_on}' or activation '{act}'")
        if act == "swish_clamped" and not limit > 0:
            raise ValueError(f"moe: the clamped activation needs a positive limit, got {limit!r}")
        self.router_bias_name, self.weights, self.weight_on, self.act = router_bias_name, weights, weight_on, act
        self.limit, self.alpha = float(limit), float(alpha)
        self.hidden, self.E, self.top, self.F = int(hidden), int(n_experts), int(top), int(expert_ff)
        self.n_identity, self.choice_bias_name = int(n_identity), choice_bias_name
        self.n_out = self.E + self.n_identity              # router outputs
        self.gated = act not in ops.UNGATED_ACTS
        if not self.gated and weight_on != "output":
            raise ValueError("moe: an expert without a gate is not linear before its activation: the weight goes on its output")
        if self.n_identity < 0 or (choice_bias_name is not None and weights != "softmax_all") or (self.n_identity and shared is not None):
            raise ValueError("moe: identity outputs cannot be negative, a choice bias belongs to weights 'softmax_all', and identity "
                             "outputs do not go with a shared expert")
        if not (1 <= self.top <= self.n_out):
            raise ValueError(f"moe: {self.top} of {self.n_out} router outputs cannot be chosen")
        self.router_name, self.expert_names, self.shared_gate_name = router_name, dict(expert_names), shared_gate_name
        self.shared = shared.build() if shared is not None else None
        if (self.shared is None) != (shared_gate_name is None):
            raise ValueError("moe: a shared expert and its gate come together")
        self.dtype = None

    def weight_specs(self) -> List[WeightSpec]:
        specs = [WeightSpec(self.router_name, (self.n_out, self.hidden))]
        if self.router_bias_name:
            specs.append(WeightSpec(self.router_bias_name, (self.n_out,)))
        if self.choice_bias_name:
            specs.append(WeightSpec(self.choice_bias_name, (self.n_out,), "near_zero"))
        for e in range(self.E):
            n = {k: v.format(e=e) for k, v in self.expert_names.items()}
            if self.gated:
                specs.append(WeightSpec(n["gate"], (self.F, self.hidden)))
            specs += [WeightSpec(n["up"], (self.F, self.hidden)), WeightSpec(n["down"], (self.hidden, self.F))]
        if self.shared is not None:
            specs += self.shared.weight_specs() + [WeightSpec(self.shared_gate_name, (1, self.hidden))]
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        from .linear import matrix_dtype
        self.dtype = dtype
        # The router's logits are 32-bit sums.  A weight stored in bfloat16 times an input rounded to bfloat16 has an exact
        # 32-bit product, so the bfloat16 product with 32-bit accumulation IS the 32-bit result and a bfloat16 run keeps
        # such a router in bfloat16 (the tensor cores); a router stored in 32-bit, and every 32-bit run, multiplies in 32-bit.
        rows = [tensors[self.router_name]] + ([tensors[self.shared_gate_name]] if self.shared is not None else [])
        rdt = torch.bfloat16 if all(matrix_dtype(r.dtype, dtype) == torch.bfloat16 for r in rows) else torch.float32
        self.router = torch.cat([r.to(device=device, dtype=rdt) for r in rows], dim=0).contiguous()
        self.router_bias = None
        if self.router_bias_name:                # added to the 32-bit logits in the product's epilogue (nothing on the shared gate's)
            self.router_bias = torch.zeros(self.router.shape[0], dtype=torch.float32, device=device)
            self.router_bias[:self.n_out] = tensors[self.router_bias_name].to(device=device, dtype=torch.float32)
        self.choice_bias = tensors[self.choice_bias_name].to(device=device, dtype=torch.float32).contiguous() \
            if self.choice_bias_name else None
        names = [{k: v.format(e=e) for k, v in self.expert_names.items()} for e in range(self.E)]
        mdt = torch.bfloat16
        for n in names:
            for k in (("gate", "up", "down") if self.gated else ("up", "down")):
                if matrix_dtype(tensors[n[k]].dtype, dtype) == torch.float32:
                    mdt = torch.float32
        to = lambda t: t.to(device=device, dtype=mdt)
        if self.gated:
            self.w_gate_up = torch.stack([torch.cat([to(tensors[n["gate"]]), to(tensors[n["up"]])], dim=0) for n in names]).contiguous()
        else:                                    # [E, F, D]: one product an expert
            self.w_gate_up = torch.stack([to(tensors[n["up"]]) for n in names]).contiguous()
        self.w_down = torch.stack([to(tensors[n["down"]]) for n in names]).contiguous()
        if self.shared is not None:
            self.shared.bind(tensors, dtype, device)

    takes_stream = True        # forward(..., stream=x32): an expert that returns its input returns the 32-bit rows

    def forward_parts(self, normed: torch.Tensor, stream: Optional[torch.Tensor] = None):
        """(parts float32 [T, top, D], shared expert's output float32 [T, D] or None, its gate's logit float32 [T] or
        None): the result is sum_k parts[:, k] + sigmoid(logit) * shared.  stream: the 32-bit rows that `normed` is a
        copy of, where the layer has no norm in front of this part (identity experts then return those)."""
        T, dev = normed.shape[0], normed.device
        n_logits = self.router.shape[0]
        logits = scratch_buf("moe.logits", (T, n_logits), torch.float32, dev)
        ops.linear(normed, self.router, logits, None, self.router_bias)
        routing = ops.moe_route(logits, self.n_out, self.top, ops.moe_tile_rows(normed, self.w_gate_up, self.dtype, self.top, self.F),
                                self.weights, self.choice_bias, self.n_identity, self.weights_sum_to)
        act = scratch_buf("moe.act", (T * self.top, self.F), self.dtype, dev)
        parts = scratch_buf("moe.parts", (T, self.top, self.hidden), torch.float32, dev)
        ops.moe_experts(normed, self.w_gate_up, self.w_down, routing, self.top, act, parts, self.act, self.weight_on, self.limit,
                        self.alpha)
        if self.n_identity:
            ops.moe_identity(stream if stream is not None else normed, routing, self.top, self.E, parts)
        if self.shared is None:
            return parts, None, None
        shared_out = scratch_buf("moe.shared", (T, self.hidden), torch.float32, dev)
        self.shared.forward(normed, shared_out, accumulate=False)
        return parts, shared_out, logits[:, self.n_out]      # the gate's logit: whoever adds the terms takes its sigmoid

    def add_parts(self, terms, residual: torch.Tensor, accumulate: bool = True) -> None:
        """Adds what forward_parts returned into `residual` (a token's terms in the order of its choices).  A block that
        runs this feed-forward beside its mixers computes the terms on a stream of their own and adds them here."""
        parts, extra, gate = terms
        ops.rmsnorm_add(parts, None, 0.0, residual, extra, gate, gate_sigmoid=True, accumulate=accumulate)

    def forward(self, normed: torch.Tensor, residual: torch.Tensor, accumulate: bool = True,
                stream: Optional[torch.Tensor] = None) -> None:
        self.add_parts(self.forward_parts(normed, stream), residual, accumulate)
