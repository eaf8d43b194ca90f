"""Time mixing with a decaying matrix state per head (the "wkv" mixer).

With x the layer's input and x' the previous token's (zeros before the first), each of the five projections reads a mix
of its own, m_s = x + (x' - x) * mu_s for s in r, k, v, g, w.  r, k, v = W_r m_r, W_k m_k, W_v m_v (heads x dim),
gate = silu(W_g m_g), and a decay per head and key channel, w = exp(-exp(W_w2 tanh(W_w1 m_w) + w0)).  Per head, with the
state S [dim, dim] (rows: key channels):

    o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t            S_t = diag(w_t) S_(t-1) + k_t v_t^T

u a learned bonus that only the current token gets.  Every head's o is divided by its root mean square, the heads side by
side are multiplied by a weight and by the gate, then W_o.  The state and the previous token's input are kept per sequence
(32-bit, zero at position 0).  The mixer reads the residual stream itself in 32 bits (`reads_stream`): the mixes are formed
there and rounded once for the products.  The four products of equal shape run as one grouped product (one group per mix).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ... import ops
from ..base import LayerCache, Part, StateRequest, StepInfo, WeightSpec, register_mixer, scratch_buf, to_vec
from ..linear import StackedLinear, matrix_dtype


@register_mixer("wkv")
class WKVMixer(Part):
    reads_stream = True        # forward() takes the 32-bit input rows, not a copy in the activation type
    MIXES = ("r", "k", "v", "g", "w")
    TILED_FROM_ROWS = 256      # steps of this many rows run r, k, v, g as four products of the tiled kernel

    def __init__(self, hidden: int, n_heads: int, head_dim: int, eps: float, names: Dict[str, str], cache_key: str = "wkv",
                 decay_rank: Optional[int] = None):
        """names: tensor names of mu_r, mu_k, mu_v, mu_g, mu_w, r, k, v, g, w1, w2, w0, u, norm, o.  decay_rank: the width
        of the decay's hidden layer; a stored model's w1 gives it (shapes_from), a model that is yet to be written takes
        this number, or a sixteenth of the model width."""
        self.hidden, self.H, self.d, self.eps = int(hidden), int(n_heads), int(head_dim), float(eps)
        if not (1 <= self.d <= ops.MAX_WKV_HEAD_DIM):
            raise ValueError(f"wkv: heads of {head_dim} channels are outside what the kernel is built for (1..{ops.MAX_WKV_HEAD_DIM})")
        if self.H > ops.MAX_HEADS:
            raise ValueError(f"wkv: {n_heads} heads exceed the kernels' limit of {ops.MAX_HEADS}")
        self.names, self.cache_key = dict(names), cache_key
        self.decay_rank = int(decay_rank) if decay_rank else None
        self.o = StackedLinear(self.H * self.d)
        self.o.add(names["o"], hidden)
        self.dtype = None

    def shapes_from(self, shapes: Dict[str, tuple]) -> None:
        """The decay's hidden width is no key of the configuration: the stored tensor gives it."""
        if self.names["w1"] in shapes:
            self.decay_rank = int(shapes[self.names["w1"]][0])

    def weight_specs(self) -> List[WeightSpec]:
        n, HD, D = self.names, self.H * self.d, self.hidden
        R = self.decay_rank or max(8, D // 16)
        specs = [WeightSpec(n["mu_" + s], (D,), "unit_interval") for s in self.MIXES]
        specs += [WeightSpec(n[s], (HD, D)) for s in ("r", "k", "v", "g")]
        specs += [WeightSpec(n["w1"], (R, D)), WeightSpec(n["w2"], (HD, R)), WeightSpec(n["w0"], (HD,), "normal"),
                  WeightSpec(n["u"], (self.H, self.d), "normal"), WeightSpec(n["norm"], (HD,), "ones")]
        return specs + self.o.weight_specs()

    def cache_requests(self) -> list:
        return [StateRequest(self.cache_key + ".shift", (self.hidden,)),
                StateRequest(self.cache_key + ".state", (self.H, self.d, self.d))]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        n = self.names
        self.dtype = dtype
        self.o.bind(tensors, dtype, device)
        self.mu = torch.stack([to_vec(tensors[n["mu_" + s]], device) for s in self.MIXES]).contiguous()
        mats = [tensors[n[s]] for s in ("r", "k", "v", "g", "w1", "w2")]
        mdt = torch.float32 if any(matrix_dtype(m.dtype, dtype) == torch.float32 for m in mats) else torch.bfloat16
        self.act_dtype = mdt
        self.w_rkvg = torch.stack([tensors[n[s]].to(device=device, dtype=mdt) for s in ("r", "k", "v", "g")]).contiguous()
        self.w1 = tensors[n["w1"]].to(device=device, dtype=mdt).contiguous()
        self.w2 = tensors[n["w2"]].to(device=device, dtype=mdt).contiguous()
        self.decay_rank = int(self.w1.shape[0])
        self.w0 = to_vec(tensors[n["w0"]], device)
        self.u = to_vec(tensors[n["u"]], device)
        self.norm_w = to_vec(tensors[n["norm"]], device)

    def forward(self, x32: torch.Tensor, step: StepInfo, cache: LayerCache, residual: torch.Tensor, accumulate: bool = True) -> None:
        if not cache.writes:
            raise ValueError("wkv: a recurrent mixer cannot run on another layer's cache without storing "
                             "(its state would advance twice in one step)")
        if x32.dtype != torch.float32:
            raise ValueError("wkv: this mixer reads the 32-bit residual stream itself (a layer whose mixer norm is 'none')")
        T, dev, HD, D = step.n_rows, x32.device, self.H * self.d, self.hidden
        new = lambda tag, shape, dtype: scratch_buf(f"wkv.{self.cache_key}.{tag}", shape, dtype, dev)
        mixes = new("mixes", (T, 5, D), self.act_dtype)
        ops.shift_mix(x32, self.mu, cache.state[self.cache_key + ".shift"], step, mixes)
        flat = mixes.view(T, 5 * D)
        rkvg = new("rkvg", (T, 4 * HD), torch.float32)
        if T >= self.TILED_FROM_ROWS and self.act_dtype == torch.bfloat16:
            # prompts: each of r, k, v, g is a full-size product of its own mix, so each takes the tiled tensor-core kernel
            for i in range(4):
                ops.linear(flat[:, i * D:(i + 1) * D], self.w_rkvg[i], rkvg[:, i * HD:(i + 1) * HD])
        else:
            ops.linear_heads(flat, D, self.w_rkvg, rkvg, HD)                   # groups r, k, v, g: one launch for the four
        hidden = new("decay_hidden", (T, self.decay_rank), torch.float32)
        ops.linear(flat[:, 4 * D:], self.w1, hidden)
        hidden_act = new("decay_act", (T, self.decay_rank), self.act_dtype)
        ops.convert(hidden, hidden_act, "tanh")
        decay_log = new("decay_log", (T, HD), torch.float32)
        ops.linear(hidden_act, self.w2, decay_log, None, self.w0)
        o = new("o", (T, HD), torch.float32)
        ops.wkv_scan(rkvg, 0, HD, 2 * HD, decay_log, self.u, cache.state[self.cache_key + ".state"], step, self.H, self.d, o)
        gated = new("gated", (T, HD), self.dtype)
        # per head: o / rms(o) * weight, then the gate silu(g)
        ops.gated_rmsnorm(o, rkvg[:, 3 * HD:], self.norm_w, self.eps, self.H, True, gated)
        self.o.forward(gated, residual, accumulate=accumulate)
