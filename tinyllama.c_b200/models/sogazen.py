"""Sogazen: per layer a mixer and a feed-forward that read the residual stream itself (no norm in front); the norm sits
on what they return,

    x <- x + norm1(mixer(x))        x <- x + norm2(ff(x))

with two kinds of mixer.  'parallel': an attention mixer and a Mamba2 mixer side by side on the same input, each result
RMS-normed over the model width with a weight of its own, the two averaged.  The attention has no value projection (a
key as projected, before its norm and rotation, is also the value), biases on q and k, an RMS norm over the whole query
and the whole key projection, a split-half rotation of the first dimensions of every head, scores capped by tanh, and a
softmax whose denominator has one more term of score 0.  'wkv': time mixing with a decaying matrix state per head.  The
feed-forward is dense, W_down(g sigmoid(1.702 g) (u + 1)) with g = min(W_gate h, limit) and u = W_up h held within +-limit,
or a mixture of experts without gates, W_down max(W_up h, 0)^2, whose router takes a softmax over all its outputs, chooses by
score plus a correction, weighs by the score alone, and whose last outputs stand for experts that return their input.  The
logits are capped by tanh.  This file only turns a SogazenConfig into data: one LayerSpec per layer and the tensor names
('l<i>.' + norm1, norm2, mix.*, mlp.*; 'embed'; 'head'; 'final.norm').
"""
from __future__ import annotations

from typing import List, Optional

from ..config.base import register_architecture
from ..config.sogazen import SogazenConfig
from ..parts.base import LayerSpec, PartSpec
from .model import Model

SWISH_ALPHA = 1.702        # the dense feed-forward's activation: g * sigmoid(SWISH_ALPHA * g) * (u + 1)


def _norm(cfg: SogazenConfig, name: str) -> PartSpec:
    return PartSpec("norm", "rmsnorm", dict(width=cfg.width, eps=cfg.eps, weight_name=name))


def _stream(cfg: SogazenConfig) -> PartSpec:
    return PartSpec("norm", "none", dict(width=cfg.width))          # the sublayer reads the stream itself


def _attention(cfg: SogazenConfig, m: dict, p: str) -> PartSpec:
    position = PartSpec("position", "rope_neox", dict(head_dim=m["dim"], theta=m["rot"]["base"], rope_dim=m["rot"]["dims"])) \
        if m["rot"]["dims"] > 0 else PartSpec("position", "none", dict(head_dim=m["dim"]))
    return PartSpec("mixer", "attention", dict(
        hidden=cfg.width, n_heads=m["heads"], n_kv_heads=m["kv_heads"], head_dim=m["dim"], v_dim=m["vdim"], prefix=p,
        position=position, names=dict(q="q", k="k", o="o", q_bias="q.b", k_bias="k.b"), values="keys", scale=m["scale"],
        whole_norm=dict(q="q.norm", k="k.norm", eps=cfg.eps), softcap=m["softcap"], sink=True))


def _mamba(cfg: SogazenConfig, m: dict, p: str) -> PartSpec:
    return PartSpec("mixer", "mamba2", dict(
        hidden=cfg.width, d_ssm=m["heads"] * m["vdim"], n_heads=m["heads"], d_head=m["vdim"], n_groups=m["groups"],
        d_state=m["state"], d_conv=m["conv"], prefix=p, eps=cfg.eps, conv_bias=True, norm_groups=m["norm_groups"],
        names=dict(in_proj="in", out_proj="o", conv="conv", conv_bias="conv.b", A_log="A_log", D="D", dt_bias="dt_bias",
                   norm="norm")))


def _wkv(cfg: SogazenConfig, m: dict, p: str) -> PartSpec:
    names = {k: p + k for k in ("r", "k", "v", "g", "w1", "w2", "w0", "u", "norm", "o")}
    names.update({"mu_" + s: p + "mu." + s for s in ("r", "k", "v", "g", "w")})
    return PartSpec("mixer", "wkv", dict(hidden=cfg.width, n_heads=m["heads"], head_dim=m["dim"], eps=cfg.eps, names=names,
                                         decay_rank=m.get("decay_rank")))


def _feed_forward(cfg: SogazenConfig, i: int) -> Optional[PartSpec]:
    mlp, p = cfg.layers[i].get("mlp"), f"l{i}.mlp."
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("feed_forward", "swiglu", dict(hidden=cfg.width, intermediate=mlp["ff"], prefix=p, act="swish_clamped",
                                                       limit=mlp["limit"], alpha=SWISH_ALPHA,
                                                       names=dict(gate="gate", up="up", down="down")))
    router = mlp["router"]
    return PartSpec("feed_forward", "moe", dict(
        hidden=cfg.width, n_experts=router["experts"], top=router["top"], expert_ff=mlp["expert"]["ff"],
        router_name=p + "router", choice_bias_name=p + "correction", n_identity=router.get("identity", 0),
        expert_names={k: p + "e{e}." + k for k in ("up", "down")}, weights="softmax_all", weight_on="output",
        act="relu_squared"))


def layer_specs(cfg: SogazenConfig) -> List[LayerSpec]:
    specs = []
    for i, layer in enumerate(cfg.layers):
        L, m = f"l{i}.", layer["mixer"]
        ffn = _feed_forward(cfg, i)
        if layer["type"] == "parallel":
            mixers = (_attention(cfg, m["left"], L + "mix.left."), _mamba(cfg, m["right"], L + "mix.right."))
            join = PartSpec("norm", "rmsnorm_mean", dict(width=cfg.width, eps=cfg.eps,
                                                        weight_names=(L + "mix.left.out", L + "mix.right.out")))
        else:
            mixers, join = (_wkv(cfg, m, L + "mix."),), None
        specs.append(LayerSpec(_stream(cfg), mixers, _stream(cfg) if ffn is not None else None, ffn,
                               mixer_out_norm=_norm(cfg, L + "norm1"),
                               ffn_out_norm=_norm(cfg, L + "norm2") if ffn is not None else None, mixer_join=join))
    return specs


def build(cfg: SogazenConfig) -> Model:
    return Model(cfg, layer_specs(cfg), None, _norm(cfg, "final.norm"), embed_name="embed", head_name="head", vocab=cfg.vocab,
                 hidden=cfg.width, logit_softcap=cfg.logit_softcap)


register_architecture("Sogazen", SogazenConfig, build)
