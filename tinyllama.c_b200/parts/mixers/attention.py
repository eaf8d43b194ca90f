"""Grouped-query attention mixer over the paged key/value cache.

CodeClaper/tinyllama.c: q/k/v projections with optional biases (falcon_h1.c:315-330),
rotation of q and k (falcon_h1.c:332-333), K/V write-through and causal attention with
kv head h/(H/KV), scale 1/sqrt(head_dim) and an optional window (cpu_op.c:964-1064;
graph.c:1275), output projection (falcon_h1.c:338).  The multipliers on the input, the
keys and the output have no counterpart there; they fold into the projections.

Options beyond that, each a constructor argument: tensor names of one's own; a score scale other than
1/sqrt(head size); values of another size than the keys (the narrower of the two is padded with zero rows of
its projection, so that the kernels see one head size); a rotation of neighbouring pairs (2i, 2i+1); queries and
keys scaled to unit root mean square per head after the rotation (no weight); and an output gate, the
concatenated heads times the sigmoid of one more projection of the mixer's input.  A rotation of neighbours and
the norm run as one kernel on the 32-bit projection before keys and values are stored.  Further: biases under names of
one's own; values that ARE the keys as projected (no value projection: the key's rows serve twice in the stacked product, so
the cached value is the key before any norm or rotation); an RMS norm with a weight over the WHOLE query projection and the
whole key projection (all heads together) before the rotation; scores capped by tanh; a sink of score 0 in the softmax.
Further still: an RMS norm with a weight per HEAD of queries and keys before the rotation (one weight vector for all query
heads, one for all key heads); frequencies stretched for long sequences and cosines and sines of another amplitude (the
position part's business); a sink whose score is learned per head; a window that keeps the sequence's first keys visible;
and two score maps per head over the same values whose results are subtracted and normed (`maps=2`): the kernels then see
twice the heads, the queries regrouped so that a map's heads share the map's keys, and one kernel joins the pairs.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ... import ops
from ..base import KVRequest, LayerCache, Part, PartSpec, StepInfo, WeightSpec, act_empty, register_mixer, scratch_buf, to_vec
from ..linear import StackedLinear


@register_mixer("attention")
class AttentionMixer(Part):
    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int, prefix: str,
                 position: PartSpec, bias: bool = False, window: Optional[int] = None, in_scale: float = 1.0,
                 out_scale: float = 1.0, key_scale: float = 1.0, cache_key: str = "kv",
                 names: Optional[Dict[str, str]] = None, scale: Optional[float] = None, v_dim: Optional[int] = None,
                 qk_norm_eps: Optional[float] = None, gate: Optional[str] = None, values: str = "projection",
                 whole_norm: Optional[Dict[str, object]] = None, softcap: float = 0.0, sink: bool = False,
                 head_norm: Optional[Dict[str, object]] = None, sink_name: Optional[str] = None, keep_first: int = 0,
                 maps: int = 1, difference: Optional[Dict[str, object]] = None):
        """names: tensor names of q, k, v, o (and g, the gate's projection) after the prefix, where they are not the
        q_proj.weight ... of the architecture's checkpoints (biases then take no part).  scale: what scores are
        multiplied by (default head_dim ** -0.5).  v_dim: size of a value head (default head_dim).  qk_norm_eps: queries
        and keys are divided by sqrt(mean(x^2) + eps) per head after the rotation.  gate: "sigmoid" or "silu" of the
        projection named g multiplies the heads' results.  names may also give q_bias, k_bias, v_bias.  values "keys":
        v = the key projection (with its bias) as it is before norm and rotation; there is no v tensor.  whole_norm =
        dict(q=name, k=name, eps=...): q <- q / sqrt(mean(q^2) + eps) * w_q over all H * head_dim values at once, k
        likewise, before the rotation.  softcap > 0: score <- softcap * tanh(score / softcap) after the scale.  sink: the
        softmax's denominator is 1 + sum exp(score).  head_norm = dict(q=name, k=name, eps=...): every query head becomes
        x / sqrt(mean(x^2) + eps) * w_q over its head_dim values (w_q [head_dim] serves all heads), every key head likewise,
        before the rotation.  sink_name: a tensor [n_heads] of sink scores, exp(sink_h) joins head h's denominator as it is
        (not scaled).  keep_first (with a window): the first keep_first positions stay visible to every later query.
        maps = 2 with difference = dict(init=number, eps=..., lq1=, lk1=, lq2=, lk2= names of vectors [head_dim]): the q tensor
        has n_heads * 2 * head_dim rows and the k tensor n_kv_heads * 2 * head_dim, head by head as [map 1, map 2]; each map is
        an attention of its own over the head's values, and with lam = exp(lq1 . lk1) - exp(lq2 . lk2) + init the head's result
        is o = a1 - lam a2, o / sqrt(mean(o^2) + eps) * (1 - init)."""
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are not a multiple of {n_kv_heads} key/value heads")
        if not (1 <= int(head_dim) <= ops.MAX_HEAD_DIM):
            raise ValueError(f"attention: head size {head_dim} is outside what the kernels are built for "
                             f"(1..{ops.MAX_HEAD_DIM})")
        if int(n_heads) > ops.MAX_HEADS:
            raise ValueError(f"attention: {n_heads} heads exceed the kernels' limit of {ops.MAX_HEADS}")
        self.qk_dim, self.v_dim = int(head_dim), int(v_dim) if v_dim else int(head_dim)
        if not (1 <= self.v_dim <= ops.MAX_HEAD_DIM):
            raise ValueError(f"attention: value size {self.v_dim} is outside what the kernels are built for (1..{ops.MAX_HEAD_DIM})")
        # one head size for the kernels: the wider of keys and values; the other is padded with zeros
        # with two maps the kernels see twice the heads: map m of key/value head g is head g * maps + m of theirs, and the
        # queries are regrouped so that the per_group query heads of (g, m) follow one another
        self.maps, self.Hq, self.per_group = int(maps), int(n_heads), int(n_heads) // int(n_kv_heads)
        if self.maps not in (1, 2) or (self.maps == 2) != (difference is not None):
            raise ValueError("attention: one map, or two with the constants of their difference")
        self.hidden, self.H, self.KV, self.hd = int(hidden), self.maps * int(n_heads), self.maps * int(n_kv_heads), max(self.qk_dim, self.v_dim)
        self.window = int(window) if window else None
        self.cache_key = cache_key
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.qk_dim)
        self.qk_norm_eps = float(qk_norm_eps) if qk_norm_eps is not None else None
        if gate is not None and gate not in ops.GATES:
            raise ValueError(f"attention: unknown output gate '{gate}'; known: {sorted(ops.GATES)}")
        self.gate = gate
        self.position = position.build()
        layout = getattr(self.position, "layout", "split_half")
        if layout not in ("split_half", "interleaved"):
            raise ValueError(f"attention: the kernels of this mixer rotate split-half or neighbouring pairs; position part "
                             f"'{position.name}' pairs dimensions as '{layout}'")
        # neighbouring pairs and the norm after the rotation are one kernel on the projection; the kernels that store
        # keys and values (which rotate split-half pairs themselves) then rotate nothing
        self.head_norm = dict(head_norm) if head_norm else None
        if self.head_norm and not {"q", "k", "eps"} <= set(self.head_norm):
            raise ValueError("attention: a norm per head needs q, k (weight names) and eps")
        self.pre_transform = layout == "interleaved" or self.qk_norm_eps is not None or self.head_norm is not None \
            or getattr(self.position, "scaling", None) is not None
        if names is not None and bias:
            raise ValueError("attention: tensor names of one's own name their biases themselves (q_bias, k_bias, v_bias)")
        if values not in ("projection", "keys"):
            raise ValueError(f"attention: values '{values}' (projection or keys)")
        if values == "keys" and (self.v_dim != self.qk_dim or key_scale != 1.0):
            raise ValueError("attention: values that are the keys have the keys' size and no multiplier of their own")
        self.values, self.softcap, self.sink = values, float(softcap), bool(sink) or sink_name is not None
        self.sink_name, self.keep_first = sink_name, int(keep_first)
        if self.keep_first < 0 or (self.keep_first and not self.window):
            raise ValueError("attention: first keys that stay visible go with a window")
        self.difference = dict(difference) if difference else None
        if self.difference and (not {"init", "eps", "lq1", "lk1", "lq2", "lk2"} <= set(self.difference) or gate or sink_name
                                or values != "projection" or whole_norm):
            raise ValueError("attention: two maps need init, eps and the names lq1, lk1, lq2, lk2, and take no gate, learned "
                             "sink, whole-projection norm or keys as values")
        self.sink_values = None
        if self.softcap < 0:
            raise ValueError(f"attention: a score cap of {softcap}")
        self.whole_norm = dict(whole_norm) if whole_norm else None
        if self.whole_norm and (self.qk_dim != self.hd or not {"q", "k", "eps"} <= set(self.whole_norm)):
            raise ValueError("attention: a norm over the whole projection needs q, k (weight names) and eps, and unpadded heads")
        nm = dict(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", o="o_proj.weight")
        nm.update(names or {})
        if self.gate and "g" not in nm:
            raise ValueError("attention: an output gate needs the name of its projection ('g')")
        b = (lambda n: prefix + n + ".bias") if bias else (lambda n: prefix + nm[n[0] + "_bias"] if n[0] + "_bias" in nm else None)
        qk_heads = lambda n: (n, self.qk_dim, self.hd) if self.qk_dim != self.hd else None
        v_heads = lambda n: (n, self.v_dim, self.hd) if self.v_dim != self.hd else None
        q_rows = v_rows = None
        if self.maps > 1:
            M, r, d, G = self.maps, self.per_group, self.qk_dim, int(n_kv_heads)
            # stored q rows (head, map, dim) -> (key/value head, map, head within the group, dim)
            q_rows = (self.H * d, [((g * r + j) * M + m) * d + i for g in range(G) for m in range(M) for j in range(r) for i in range(d)])
            # the values of key/value head g once for every map
            v_rows = (G * self.v_dim, [g * self.v_dim + i for g in range(G) for m in range(M) for i in range(self.v_dim)])
        self.qkv = StackedLinear(hidden)
        self.q_off = self.qkv.add(prefix + nm["q"], self.H * self.hd, b("q_proj"), in_scale, heads=qk_heads(self.H), gather=q_rows)
        self.k_off = self.qkv.add(prefix + nm["k"], self.KV * self.hd, b("k_proj"), in_scale, key_scale, heads=qk_heads(self.KV))
        if values == "keys":          # the key's rows once more: what is cached as the value is the key as projected
            self.v_off = self.qkv.add(prefix + nm["k"], self.KV * self.hd, b("k_proj"), in_scale)
        else:
            self.v_off = self.qkv.add(prefix + nm["v"], self.KV * self.hd, b("v_proj"), in_scale, heads=v_heads(self.KV), gather=v_rows)
        self.g_off = self.qkv.add(prefix + nm["g"], self.H * self.hd, None, in_scale, heads=v_heads(self.H)) if self.gate else None
        self.o = StackedLinear(self.Hq * self.hd, in_heads=v_heads(self.Hq))
        self.o.add(prefix + nm["o"], hidden, b("o_proj"), 1.0, out_scale)
        self.dtype = None
        self.prefix = prefix
        self.q_norm_w = self.k_norm_w = None

    @property
    def single_token_launches(self) -> int:
        """Kernels that mix() launches in a one-token step: one where the fused kernel serves (a
        bfloat16 cache, a head size it is built for, a position part with a rotation table), else
        rotation + split keys + merge."""
        fused = self.dtype == torch.bfloat16 and self.position.rotation_table() is not None \
            and ops.library().tlc_attention_decode_fused_ok(self.H, self.KV, self.hd) \
            and not ops.DISABLE_FUSED_DECODE_ATTENTION
        return (1 if fused else 3) + int(self.pre_transform) + int(self.gate is not None) + int(self.whole_norm is not None) \
            + int(self.maps > 1)

    @property
    def _own_softmax(self) -> bool:
        """A capped score or a sink: served by the tcgen05 kernel of prompts, the fused kernel of single tokens, the warp kernels
        and the split-key kernels of single tokens."""
        return self.softcap > 0 or self.sink

    def weight_specs(self) -> List[WeightSpec]:
        specs, seen = [], set()
        for sp in self.qkv.weight_specs() + self.o.weight_specs() + self.position.weight_specs():
            if sp.name not in seen:               # (values that are the keys list the key's tensors twice)
                seen.add(sp.name)
                specs.append(sp)
        if self.whole_norm:
            specs += [WeightSpec(self.prefix + self.whole_norm["q"], (self.H * self.hd,), "ones"),
                      WeightSpec(self.prefix + self.whole_norm["k"], (self.KV * self.hd,), "ones")]
        if self.head_norm:
            specs += [WeightSpec(self.prefix + self.head_norm["q"], (self.qk_dim,), "ones"),
                      WeightSpec(self.prefix + self.head_norm["k"], (self.qk_dim,), "ones")]
        if self.sink_name:
            specs.append(WeightSpec(self.prefix + self.sink_name, (self.Hq,), "near_zero"))
        if self.difference:
            specs += [WeightSpec(self.prefix + self.difference[n], (self.qk_dim,), "near_zero") for n in ("lq1", "lk1", "lq2", "lk2")]
        return specs

    def cache_requests(self) -> list:
        return [KVRequest(self.cache_key, self.KV, self.hd, self.window, keep_first=self.keep_first if self.window else 0)]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        self.dtype = dtype
        self.qkv.bind(tensors, dtype, device)
        self.o.bind(tensors, dtype, device)
        self.position.bind(tensors, dtype, device)
        if self.whole_norm:
            self.q_norm_w = to_vec(tensors[self.prefix + self.whole_norm["q"]], device)
            self.k_norm_w = to_vec(tensors[self.prefix + self.whole_norm["k"]], device)
        self.q_head_w = self.k_head_w = None
        if self.head_norm:
            self.q_head_w = to_vec(tensors[self.prefix + self.head_norm["q"]], device)
            self.k_head_w = to_vec(tensors[self.prefix + self.head_norm["k"]], device)
        if self.sink_name:
            self.sink_values = to_vec(tensors[self.prefix + self.sink_name], device)
        if self.difference:
            vec = lambda n: tensors[self.prefix + self.difference[n]].to(device="cpu", dtype=torch.float32)
            init = float(self.difference["init"])
            self.lam = float(torch.exp((vec("lq1") * vec("lk1")).sum()) - torch.exp((vec("lq2") * vec("lk2")).sum())) + init
        self._no_rotation = torch.zeros(0, dtype=torch.float32, device=device)
        # arrival counters of the one-kernel attention of single-token steps: this mixer's own, so that no other
        # mixer, model or stream ever shares them; made here, outside any stream capture
        self._arrivals = ops.new_arrival_counters(device) if torch.device(device).type == "cuda" else None

    def input_projection(self) -> StackedLinear:
        """What this mixer computes from the normed input before anything else (a block may stack
        the input projections of its mixers into one product)."""
        return self.qkv

    def forward(self, normed: torch.Tensor, step: StepInfo, cache: LayerCache, residual: torch.Tensor) -> None:
        qkv = act_empty((step.n_rows, self.qkv.out_features), normed, torch.float32)
        self.qkv.forward(normed, qkv)
        self.forward_projected(qkv, step, cache, residual)

    def forward_projected(self, qkv: torch.Tensor, step: StepInfo, cache: LayerCache, residual: torch.Tensor) -> None:
        """qkv: this mixer's input projection, float32 [T, q|k|v] (rows may be strided)."""
        self.output(self.mix(qkv, step, cache), residual)

    def output_projection(self) -> StackedLinear:
        """What turns mix()'s result into this mixer's share of the residual stream (a block may run
        the output projections of its mixers as one product over their results side by side)."""
        return self.o

    mix_takes_max_blocks = True    # mix() can bound how many SMs its prompt kernel holds

    def mix(self, qkv: torch.Tensor, step: StepInfo, cache: LayerCache, out: Optional[torch.Tensor] = None,
            max_blocks: int = 0) -> torch.Tensor:
        """Everything between the input projection and the output projection: [T, H*hd], written
        to `out` (rows may be strided) where one is given.  max_blocks > 0: the attention kernel of a prompt
        holds at most that many SMs (a block that runs another mixer beside this one leaves it the rest)."""
        T = step.n_rows
        kv = cache.kv[self.cache_key]
        if self.whole_norm:           # over all heads at once, before any rotation (the value columns keep the projection)
            ops.qk_whole_norm(qkv, self.q_off, self.H * self.hd, self.q_norm_w, self.k_off, self.KV * self.hd, self.k_norm_w,
                              float(self.whole_norm["eps"]))
        table = self.position.rotation_table()
        if table is None:
            # not a rotation: the part changes q and k in place; what is stored below is its result
            self.position.transform(qkv, self.q_off, self.k_off, step, self.H, self.KV, self.hd)
            table = self._no_rotation
        if self.pre_transform:
            ops.qk_rotate_norm(qkv, self.q_off, self.k_off, self.H, self.KV, self.hd, self.qk_dim, table,
                               getattr(self.position, "layout", "split_half") == "interleaved", self.qk_norm_eps, step.positions,
                               self.q_head_w, self.k_head_w, float(self.head_norm["eps"]) if self.head_norm else 0.0,
                               float(getattr(self.position, "amplitude", 1.0)))
            table = self._no_rotation
        joined = out
        if self.maps > 1:             # the kernels write the maps' results; the join writes the heads'
            out = None
        if step.max_new == 1 and ops.attention_decode_fused_ok(qkv, self.dtype, self.H, self.KV, self.hd):
            # one token per sequence: rotation, store and attention in one kernel
            att = out if out is not None else scratch_buf(f"attention.{self.cache_key}.out", (T, self.H * self.hd), self.dtype, qkv.device)
            ops.attention_decode_fused(qkv, self.q_off, self.k_off, self.v_off, kv.k_pages, kv.v_pages, table,
                                       cache.writes, kv.block_table, step.positions, step.row_seq, step.slots, att,
                                       self.H, self.KV, self.hd, self.scale, self.window or 0,
                                       step.max_context, self._arrivals, self.softcap, self.sink, self.keep_first, self.sink_values)
            return self._joined(self._gated(att, qkv), joined)
        q = scratch_buf(f"attention.{self.cache_key}.q", (T, self.H * self.hd), self.dtype, qkv.device)
        ops.rope_kv_store(qkv, self.q_off, self.k_off, self.v_off, q, kv.k_pages, kv.v_pages, table, step.positions,
                          step.row_seq, step.slots, kv.block_table, self.H, self.KV, self.hd, cache.writes)
        att = out if out is not None else scratch_buf(f"attention.{self.cache_key}.out", (T, self.H * self.hd), self.dtype, qkv.device)
        ops.attention(q, kv.k_pages, kv.v_pages, kv.block_table, step.positions, step.row_seq, step.slots, att,
                      self.H, self.KV, self.hd, self.scale, self.window or 0,
                      step.max_context if step.max_new == 1 else 0, step.cu_seqlens, step.start_pos, step.max_context,
                      max_blocks, softcap=self.softcap, sink=self.sink, keep_first=self.keep_first, sink_values=self.sink_values)
        return self._joined(self._gated(att, qkv), joined)

    def _joined(self, att: torch.Tensor, out: Optional[torch.Tensor]) -> torch.Tensor:
        """With two maps a head: the pairs' difference, normed (one kernel); else the kernels' result as it is."""
        if self.maps == 1:
            return att
        if out is None:
            out = scratch_buf(f"attention.{self.cache_key}.joined", (att.shape[0], self.Hq * self.hd), self.dtype, att.device)
            if self.v_dim != self.hd:
                out.zero_()           # (what lies past a head's values meets zero columns of the output projection)
        ops.difference_join(att, self.hd, out, self.hd, self.Hq, self.per_group, self.v_dim, self.lam, float(self.difference["eps"]),
                            1.0 - float(self.difference["init"]))
        return out

    def _gated(self, att: torch.Tensor, qkv: torch.Tensor) -> torch.Tensor:
        if self.gate:
            ops.gate_mul(att, qkv[:, self.g_off:self.g_off + self.H * self.hd], self.gate)
        return att

    def output(self, att: torch.Tensor, residual: torch.Tensor) -> None:
        """Adds the output projection of `att` into the residual stream."""
        self.o.forward(att, residual, accumulate=True)
