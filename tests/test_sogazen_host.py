"""Sogazen without a GPU: the configuration's checks, what the builder makes of a configuration (parts, tensor names and
shapes, cache needs, a size that only a stored tensor gives), and the plain implementation's mechanisms against
restatements of their own definitions."""
import copy

import numpy as np
import pytest

from tinyllama_c_b200.config import ConfigError, config_from_dict
from tinyllama_c_b200.config.base import lookup_architecture
from tinyllama_c_b200.parts.base import KVRequest, StateRequest

import configs
from plain import sogazen_plain as plain


def build(cfg: dict):
    c = config_from_dict(cfg)
    return lookup_architecture(c.architecture)[1](c)


def test_builder_names_shapes_and_cache_needs():
    m = build(configs.SOGAZEN_A)
    got = {s.name: tuple(s.shape) for s in m.weight_specs()}
    assert got["embed"] == (140, 48) and got["head"] == (140, 48) and got["final.norm"] == (48,)
    # wkv: 3 heads of 8, a decay layer of 5 values
    assert got["l0.mix.r"] == (24, 48) and got["l0.mix.mu.w"] == (48,) and got["l0.mix.w1"] == (5, 48) and got["l0.mix.w2"] == (24, 5)
    assert got["l0.mix.w0"] == (24,) and got["l0.mix.u"] == (3, 8) and got["l0.mix.norm"] == (24,) and got["l0.mix.o"] == (48, 24)
    # experts without gates; the router has one output more than there are experts
    assert got["l0.mlp.router"] == (4, 48) and got["l0.mlp.correction"] == (4,) and got["l0.mlp.e2.up"] == (20, 48)
    assert got["l0.mlp.e2.down"] == (48, 20) and "l0.mlp.e0.gate" not in got and "l0.mlp.e3.up" not in got
    # attention: no value projection, biases on q and k, norm weights over the whole projections
    assert got["l1.mix.left.q"] == (96, 48) and got["l1.mix.left.q.b"] == (96,) and got["l1.mix.left.k"] == (48, 48)
    assert got["l1.mix.left.k.b"] == (48,) and got["l1.mix.left.q.norm"] == (96,) and got["l1.mix.left.k.norm"] == (48,)
    assert got["l1.mix.left.o"] == (48, 96) and not any(n.startswith("l1.mix.left.v") for n in got)
    # Mamba2: z | x | B | C | dt rows, a two-dimensional convolution weight
    assert got["l1.mix.right.in"] == (48 + 48 + 8 + 8 + 3, 48) and got["l1.mix.right.conv"] == (64, 2) and got["l1.mix.right.conv.b"] == (64,)
    assert got["l1.mix.right.norm"] == (48,) and got["l1.mix.right.o"] == (48, 48) and got["l1.mix.right.A_log"] == (3,)
    assert got["l1.mix.left.out"] == (48,) and got["l1.mix.right.out"] == (48,) and got["l1.norm1"] == (48,) and got["l1.norm2"] == (48,)
    assert got["l1.mlp.gate"] == (40, 48) and got["l1.mlp.down"] == (48, 40)
    assert not any(n.startswith("l2.mlp") or n == "l2.norm2" for n in got)
    reqs = m.cache_requests()
    assert reqs[1][0] == KVRequest("kv", 2, 24, None)
    assert StateRequest("mamba.conv", (1, 64)) in reqs[1] and StateRequest("mamba.ssm", (3, 16, 8)) in reqs[1]
    assert reqs[0] == [StateRequest("wkv.shift", (48,)), StateRequest("wkv.state", (3, 8, 8))]
    # the sublayers read the stream itself; the parallel layers join their mixers' results
    assert all(getattr(b.mixer_norm, "identity", False) for b in m.layers)
    assert [b.mixer_join is not None for b in m.layers] == [False, True, True, False, True]
    assert m.logit_softcap == 8.0


def test_a_size_that_only_a_stored_tensor_gives():
    cfg = copy.deepcopy(configs.SOGAZEN_A)
    del cfg["layers"][0]["mixer"]["decay_rank"]
    m = build(cfg)
    m.adopt_shapes({"l0.mix.w1": (7, 48)})
    got = {s.name: tuple(s.shape) for s in m.weight_specs()}
    assert got["l0.mix.w1"] == (7, 48) and got["l0.mix.w2"] == (24, 7)


@pytest.mark.parametrize("edit,text", [
    (lambda c: c["layers"][1]["mixer"]["left"].update(vdim=16), "vdim"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=7), "rot"),
    (lambda c: c["layers"][1]["mixer"]["left"].pop("softcap"), "softcap"),
    (lambda c: c["layers"][1]["mixer"]["left"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(norm_groups=5), "norm_groups"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(groups=2), "groups"),
    (lambda c: c["layers"][1]["mixer"].pop("right"), "right"),
    (lambda c: c["layers"][0]["mixer"].pop("dim"), "dim"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "router"),
    (lambda c: c["layers"][0]["mlp"].pop("expert"), "expert"),
    (lambda c: c["layers"][1]["mlp"].pop("limit"), "limit"),
    (lambda c: c["layers"][0].update(type="attention"), "type"),
    (lambda c: c.pop("logit_softcap"), "logit_softcap"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_configuration_faults_are_named(edit, text):
    cfg = copy.deepcopy(configs.SOGAZEN_A)
    edit(cfg)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(cfg)


def test_plain_sink_cap_and_rotation():
    s = np.array([0.3, -1.0, 2.0])
    p = plain.sink_softmax(s)
    assert np.allclose(p, np.exp(s) / (1.0 + np.exp(s).sum())) and p.sum() < 1.0
    assert np.allclose(plain.sink_softmax(s - 50.0).sum(), np.exp(s - 50.0).sum() / (1.0 + np.exp(s - 50.0).sum()))
    assert np.allclose(plain.capped(np.array([1e-3, 100.0, -100.0]), 5.0), [1e-3, 5.0, -5.0], atol=1e-6)
    # a rotation keeps lengths, leaves the dimensions behind `dims` alone, and position 0 turns nothing
    g = np.random.default_rng(0)
    x = g.standard_normal((4, 2, 12))
    y = plain.rotate_halves(x, [0, 1, 7, 300], 100.0, 8)
    assert np.array_equal(y[0], x[0]) and np.array_equal(y[..., 8:], x[..., 8:])
    assert np.allclose((y[..., :8] ** 2).sum(-1), (x[..., :8] ** 2).sum(-1))
    # dimension i pairs with i + dims/2: a unit vector on dimension 0 stays within dimensions 0 and 4
    e = np.zeros((1, 1, 12)); e[..., 0] = 1.0
    r = plain.rotate_halves(e, [3], 100.0, 8)[0, 0]
    assert np.allclose(r[0], np.cos(3.0)) and np.allclose(r[4], np.sin(3.0)) and np.count_nonzero(np.abs(r) > 1e-12) == 2


def test_plain_recurrences_against_their_unrolled_sums():
    g = np.random.default_rng(1)
    # wkv with one head: o_t = sum_{s<t} (prod_{s<j<t} w_j) (r_t . k_s) v_s + (r_t . (u k_t)) v_t
    T, D, d = 6, 5, 4
    names = ["mu.r", "mu.k", "mu.v", "mu.g", "mu.w"]
    W = {"a." + n: g.uniform(0, 1, D) for n in names}
    W.update({"a." + n: g.standard_normal((d, D)) * 0.5 for n in ("r", "k", "v", "g")})
    W.update({"a.w1": g.standard_normal((3, D)), "a.w2": g.standard_normal((d, 3)), "a.w0": g.standard_normal(d) - 1.0,
              "a.u": g.standard_normal((1, d)), "a.norm": np.ones(d), "a.o": np.eye(d)})
    h = g.standard_normal((T, D))
    out = plain.wkv_mixer(h, W, "a.", dict(heads=1, dim=d), 1e-6)
    prev = np.concatenate([np.zeros((1, D)), h[:-1]])
    mix = lambda s: h + (prev - h) * W["a.mu." + s]
    r, k, v = mix("r") @ W["a.r"].T, mix("k") @ W["a.k"].T, mix("v") @ W["a.v"].T
    gate = plain.silu(mix("g") @ W["a.g"].T)
    w = np.exp(-np.exp(np.tanh(mix("w") @ W["a.w1"].T) @ W["a.w2"].T + W["a.w0"]))
    for t in range(T):
        o = (r[t] * W["a.u"][0] * k[t]).sum() * v[t]
        for s in range(t):
            decay = np.prod(w[s + 1:t], axis=0)
            o = o + (r[t] * decay * k[s]).sum() * v[s]
        want = o / np.sqrt((o * o).mean() + 1e-6) * gate[t]
        assert np.allclose(out[t], want)
    # the convolution's last tap is the current token's, and nothing comes before the start
    conv = plain.causal_conv(np.arange(12.0).reshape(6, 2), np.array([[1.0, 10.0], [0.0, 1.0]]), np.zeros(2))
    assert np.allclose(conv[:, 0], [0, 20, 42, 64, 86, 108]) and np.allclose(conv[:, 1], [1, 3, 5, 7, 9, 11])


def test_plain_routing_and_identity_outputs():
    g = np.random.default_rng(2)
    D = 6
    W = {"m.router": g.standard_normal((5, D)), "m.correction": np.array([0.0, 0.0, 5.0, 0.0, 5.0])}
    for e in range(3):
        W[f"m.e{e}.up"], W[f"m.e{e}.down"] = g.standard_normal((4, D)), g.standard_normal((D, 4))
    mlp = dict(router=dict(experts=3, top=2, identity=2), expert=dict(ff=4))
    h = g.standard_normal((9, D))
    chosen, weight = plain.route(h, W, "m.", mlp)
    assert (np.sort(chosen, axis=1) == [2, 4]).all()                 # the correction decides the choice ...
    z = h @ W["m.router"].T
    s = np.exp(z) / np.exp(z).sum(-1, keepdims=True)
    assert np.allclose(weight, np.take_along_axis(s, chosen, axis=1)) and (weight.sum(1) < 1.0).all()      # ... not the weight
    out = plain.expert_ff(h, W, "m.", mlp)
    want = s[:, [4]] * h + s[:, [2]] * ((np.maximum(h @ W["m.e2.up"].T, 0.0) ** 2) @ W["m.e2.down"].T)
    assert np.allclose(out, want)
    lim = 0.5
    Wd = {"f.gate": g.standard_normal((7, D)), "f.up": g.standard_normal((7, D)), "f.down": np.eye(7)}
    y = plain.dense_ff(h, Wd, "f.", dict(limit=lim))
    gg, u = np.minimum(h @ Wd["f.gate"].T, lim), np.clip(h @ Wd["f.up"].T, -lim, lim)
    assert np.allclose(y, gg / (1.0 + np.exp(-1.702 * gg)) * (u + 1.0)) and (h @ Wd["f.gate"].T).max() > lim
