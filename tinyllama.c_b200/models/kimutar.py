"""Kimutar: per layer a mixer and a feed-forward side by side, each on a layer norm of its own of the layer's input,

    x <- x + mixer(n1(x)) + ff(n2(x)),        n(x) = (x - mean(x)) / sqrt(var(x) + eps) * w

with three kinds of mixer.  'attention': grouped-query attention with TWO score maps per head over the same values (the q
and k tensors hold the maps head by head), an RMS norm with a weight per head and map on queries and keys, a split-half
rotation of the first dimensions with frequencies blended along a ramp over the pair index and enlarged cosines and sines,
and the maps joined as o = a1 - lambda a2, o / rms(o) * (1 - diff), lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff.
'attention_2': biases on q, k, v and the output, the same norm per head, a rotation of neighbouring pairs with frequencies
kept, divided or blended by their wave's length, a sliding window that keeps the sequence's first tokens visible, and a
learned sink per head in the softmax's denominator.  'channel_delta': the gated delta rule with a decay per head and key
channel from a low-rank pair of matrices, a sigmoid gate from another pair, and the read-out normed per head.  The
feed-forward is dense, W_down max(W_up h, 0)^2, or a mixture of gated experts (SiLU) whose router takes a softmax over all
experts, chooses by score plus a stored correction and weighs by the chosen scores normed to a given sum, beside a shared
expert times the sigmoid of one more projection.  A range of layers may repeat: every pass has caches of its own and begins
with a learned vector added to the stream.  The final norm is a layer norm; the head is a matrix of its own.  This file only
turns a KimutarConfig into data: one LayerSpec per layer, the run order, and the tensor names ('l<i>.' + norm1, norm2,
mix.*, mlp.*; 'embed'; 'loop.step'; 'final.norm'; 'head').
"""
from __future__ import annotations

from typing import List, Optional

from ..config.base import register_architecture
from ..config.kimutar import KimutarConfig
from ..parts.base import LayerRun, LayerSpec, PartSpec
from .model import Model

UNIT_EPS = 1e-6            # under the root when the delta rule's queries and keys are made unit vectors
LOOP_TABLE = "loop.step"   # [times, width]: row t joins the stream before pass t of the repeated range


def _norm(cfg: KimutarConfig, name: str) -> PartSpec:
    return PartSpec("norm", "layernorm", dict(width=cfg.width, eps=cfg.eps, weight_name=name))


def _position(m: dict, kind: str, scaling_kind: str) -> PartSpec:
    rot = m["rot"]
    if rot["dims"] == 0:
        return PartSpec("position", "none", dict(head_dim=m["dim"]))
    scaling = dict(rot["scaling"], kind=scaling_kind) if rot.get("scaling") is not None else None
    return PartSpec("position", kind, dict(head_dim=m["dim"], theta=rot["base"], rope_dim=rot["dims"], scaling=scaling))


def _mixer(cfg: KimutarConfig, i: int) -> PartSpec:
    layer, p = cfg.layers[i], f"l{i}.mix."
    m, kind = layer["mixer"], layer["type"]
    common = dict(hidden=cfg.width, n_heads=m["heads"], n_kv_heads=m["kv_heads"], prefix=p) if kind != "channel_delta" else {}
    if kind == "attention":
        return PartSpec("mixer", "attention", dict(
            common, head_dim=m["dim"], v_dim=m["vdim"], position=_position(m, "rope_neox", "ramp"), scale=m["scale"],
            names=dict(q="q", k="k", v="v", o="o"), head_norm=dict(q="q.norm", k="k.norm", eps=cfg.eps), maps=2,
            difference=dict(init=m["diff"], eps=cfg.eps, lq1="lq1", lk1="lk1", lq2="lq2", lk2="lk2")))
    if kind == "attention_2":
        mask = m.get("mask") or {}
        return PartSpec("mixer", "attention", dict(
            common, head_dim=m["dim"], v_dim=m["vdim"], position=_position(m, "rope_interleaved", "bands"), scale=m["scale"],
            names=dict(q="q", k="k", v="v", o="o", q_bias="q.b", k_bias="k.b", v_bias="v.b", o_bias="o.b"),
            head_norm=dict(q="q.norm", k="k.norm", eps=cfg.eps), sink_name="sink", window=mask.get("size"),
            keep_first=mask.get("keep_first", 0) if mask.get("size") else 0))
    names = {k: p + k for k in ("q", "k", "v", "b", "a1", "a2", "A_log", "dt_bias", "norm", "g1", "g2", "o")}
    return PartSpec("mixer", "delta", dict(
        hidden=cfg.width, n_heads=m["heads"], n_qk_heads=m["kv_heads"], key_dim=m["dim"], v_dim=m["vdim"], conv_taps=m["conv"],
        eps=cfg.eps, names=names, l2_eps=UNIT_EPS, decay="channel", gate="sigmoid", low_rank_gate=True,
        decay_rank=m.get("decay_rank"), gate_rank=m.get("gate_rank")))


def _feed_forward(cfg: KimutarConfig, i: int) -> Optional[PartSpec]:
    mlp, p = cfg.layers[i].get("mlp"), f"l{i}.mlp."
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("feed_forward", "mlp", dict(hidden=cfg.width, intermediate=mlp["ff"], names=dict(up=p + "up", down=p + "down"),
                                                    act="relu_squared"))
    router, shared = mlp["router"], mlp.get("shared")
    shared_part = None if shared is None else PartSpec("feed_forward", "swiglu", dict(
        hidden=cfg.width, intermediate=shared["ff"], prefix=p + "shared.", names=dict(gate="gate", up="up", down="down")))
    return PartSpec("feed_forward", "moe", dict(
        hidden=cfg.width, n_experts=router["experts"], top=router["top"], expert_ff=mlp["expert"]["ff"], router_name=p + "router",
        choice_bias_name=p + "correction", expert_names={k: p + "e{e}." + k for k in ("gate", "up", "down")},
        weights="softmax_all", weights_sum_to=router["scale"], weight_on="output", act="silu", shared=shared_part,
        shared_gate_name=None if shared is None else p + "shared.sg"))


def layer_specs(cfg: KimutarConfig) -> List[LayerSpec]:
    specs = []
    for i in range(len(cfg.layers)):
        ffn = _feed_forward(cfg, i)
        specs.append(LayerSpec(_norm(cfg, f"l{i}.norm1"), (_mixer(cfg, i),), _norm(cfg, f"l{i}.norm2") if ffn is not None else None, ffn,
                               parallel=True))
    return specs


def run_order(cfg: KimutarConfig) -> List[LayerRun]:
    """The layers in the order they run: the repeated range `times` times in a row, every entry with a cache of its own,
    every pass's first entry after row t of the loop's table."""
    n, loop = len(cfg.layers), cfg.loop
    if loop is None:
        return [LayerRun(i) for i in range(n)]
    order = [LayerRun(i) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [LayerRun(i, add=(LOOP_TABLE, t) if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return order + [LayerRun(i) for i in range(loop["stop"], n)]


def build(cfg: KimutarConfig) -> Model:
    tables = {LOOP_TABLE: cfg.loop["times"]} if cfg.loop is not None else None
    # a layer without a feed-forward has no use for the feed-forward's norm, stored or not; nor a model without a repeated
    # range for the table of its passes
    unused = [f"l{i}.norm2" for i, layer in enumerate(cfg.layers) if layer.get("mlp") is None] + ([LOOP_TABLE] if cfg.loop is None else [])
    return Model(cfg, layer_specs(cfg), run_order(cfg), _norm(cfg, "final.norm"), embed_name="embed", head_name="head",
                 vocab=cfg.vocab, hidden=cfg.width, row_tables=tables, unused_tensors=unused)


register_architecture("Kimutar", KimutarConfig, build)
