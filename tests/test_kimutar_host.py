"""Kimutar without a GPU: the configuration's checks, what the builder makes of a configuration (parts, tensor names and
shapes, cache needs, the run order of a repeated range, sizes that only stored tensors give), the library's pieces that
need no kernel (stretched frequency tables, rows of a projection gathered and padded, pages that a window keeps), and the
plain implementation's mechanisms against restatements of their own definitions."""
import copy
import math

import numpy as np
import pytest
import torch

from tinyllama_c_b200.cache import Cache
from tinyllama_c_b200.config import ConfigError, config_from_dict
from tinyllama_c_b200.config.base import lookup_architecture
from tinyllama_c_b200.parts.base import KVRequest, LayerRun, StateRequest
from tinyllama_c_b200.parts.linear import StackedLinear
from tinyllama_c_b200.parts.position import RotaryInterleaved, RotaryNeox

import configs
from plain import kimutar_plain as plain


def build(cfg: dict):
    c = config_from_dict(cfg)
    return lookup_architecture(c.architecture)[1](c)


def test_builder_names_shapes_and_cache_needs():
    m = build(configs.KIMUTAR_A)
    got = {s.name: tuple(s.shape) for s in m.weight_specs()}
    assert got["embed"] == (150, 52) and got["head"] == (150, 52) and got["final.norm"] == (52,) and got["loop.step"] == (3, 52)
    # the delta rule: 2 query/key heads of 8 for 4 value heads of 12, two taps, low-rank pairs of 5 and 7
    assert got["l0.mix.q"] == (16, 52) and got["l0.mix.k.conv"] == (16, 2) and got["l0.mix.v"] == (48, 52) and got["l0.mix.v.conv"] == (48, 2)
    assert got["l0.mix.b"] == (4, 52) and got["l0.mix.A_log"] == (4,) and got["l0.mix.a1"] == (5, 52) and got["l0.mix.a2"] == (32, 5)
    assert got["l0.mix.dt_bias"] == (32,) and got["l0.mix.g1"] == (7, 52) and got["l0.mix.g2"] == (48, 7) and got["l0.mix.norm"] == (12,)
    assert got["l0.mix.o"] == (52, 48) and "l0.mix.a" not in got and "l0.mix.g" not in got
    # experts with gates, a correction, a shared expert with its gate
    assert got["l0.mlp.router"] == (4, 52) and got["l0.mlp.correction"] == (4,) and got["l0.mlp.e3.gate"] == (20, 52)
    assert got["l0.mlp.e3.down"] == (52, 20) and got["l0.mlp.shared.up"] == (16, 52) and got["l0.mlp.shared.sg"] == (1, 52)
    assert "l3.mlp.shared.up" not in got and got["l3.mlp.e1.up"] == (12, 52)
    # two maps: twice the query and key rows, values once, four vectors of the difference, no biases
    assert got["l1.mix.q"] == (4 * 2 * 24, 52) and got["l1.mix.k"] == (2 * 2 * 24, 52) and got["l1.mix.v"] == (2 * 16, 52)
    assert got["l1.mix.q.norm"] == (24,) and got["l1.mix.lk2"] == (24,) and got["l1.mix.o"] == (52, 64) and "l1.mix.q.b" not in got
    assert got["l1.mlp.up"] == (40, 52) and got["l1.mlp.down"] == (52, 40) and "l1.mlp.gate" not in got
    # the window layer: biases, a sink per head, values wider than keys
    assert got["l2.mix.q"] == (48, 52) and got["l2.mix.q.b"] == (48,) and got["l2.mix.v"] == (72, 52) and got["l2.mix.v.b"] == (72,)
    assert got["l2.mix.o"] == (52, 72) and got["l2.mix.o.b"] == (52,) and got["l2.mix.sink"] == (3,) and got["l2.mix.k.norm"] == (16,)
    assert got["l2.norm1"] == (52,) and "l2.norm2" not in got and not any(n.startswith("l2.mlp") for n in got)
    # the run order: layers 0 and 1 three times, each entry with a cache of its own, every pass after its row of the table
    assert m.schedule == [LayerRun(0, add=("loop.step", 0)), LayerRun(1), LayerRun(0, add=("loop.step", 1)), LayerRun(1),
                          LayerRun(0, add=("loop.step", 2)), LayerRun(1), LayerRun(2), LayerRun(3), LayerRun(4)]
    reqs = m.cache_requests()
    assert sorted(reqs) == list(range(9))
    assert reqs[0] == reqs[2] == [StateRequest("delta.conv", (1, 80)), StateRequest("delta.state", (4, 8, 12))]
    assert reqs[1] == reqs[5] == [KVRequest("kv", 4, 24, None)]              # two maps: twice the key/value heads, the wider size
    assert reqs[6] == [KVRequest("kv", 3, 24, 5, keep_first=2)] and reqs[7] == [KVRequest("kv", 1, 20, 70)]
    # both norms of a layer are applied to its input
    assert all(b.parallel_ffn == (b.ffn is not None) for b in m.layers) and m.layers[0].own_parallel_norm
    assert m.layers[0].mixer_norm.pairs_with(m.layers[0].ffn_norm)


def test_without_a_repeated_range_and_without_window_or_scaling():
    cfg = copy.deepcopy(configs.KIMUTAR_B)
    del cfg["loop"]
    m = build(cfg)
    assert m.schedule == [LayerRun(i) for i in range(5)] and "loop.step" not in {s.name for s in m.weight_specs()}
    assert m.cache_requests()[4] == [KVRequest("kv", 2, 64, None)]
    assert m.layers[4].mixers[0].position.scaling is None and m.layers[0].mixers[0].position.scaling["kind"] == "bands"
    assert m.layers[2].mixers[0].position.scaling["kind"] == "ramp"


def test_a_stored_norm_of_a_feed_forward_that_is_not_there_is_no_fault():
    from tinyllama_c_b200.weights.loader import WeightError, check_tensors, random_tensors
    m = build(configs.KIMUTAR_A)
    tensors = random_tensors(m, 1)
    check_tensors(m, dict(tensors, **{"l2.norm2": torch.ones(52)}))
    with pytest.raises(WeightError, match="l1.norm3"):
        check_tensors(m, dict(tensors, **{"l1.norm3": torch.ones(52)}))


def test_sizes_that_only_stored_tensors_give():
    cfg = copy.deepcopy(configs.KIMUTAR_A)
    del cfg["layers"][0]["mixer"]["decay_rank"], cfg["layers"][0]["mixer"]["gate_rank"]
    m = build(cfg)
    m.adopt_shapes({"l0.mix.a1": (9, 52), "l0.mix.g1": (3, 52)})
    got = {s.name: tuple(s.shape) for s in m.weight_specs()}
    assert got["l0.mix.a1"] == (9, 52) and got["l0.mix.a2"] == (32, 9) and got["l0.mix.g1"] == (3, 52) and got["l0.mix.g2"] == (48, 3)


@pytest.mark.parametrize("edit,text", [
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].pop("fast"), "scaling"),
    (lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].update(high=1.0), "high and low"),
    (lambda c: c["layers"][1]["mixer"].pop("diff"), "diff"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][2]["mixer"]["mask"].update(size=0), "mask"),
    (lambda c: c["layers"][2]["mixer"]["mask"].update(keep_first=-1), "mask"),
    (lambda c: c["layers"][0]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "router"),
    (lambda c: c["layers"][0]["mlp"]["router"].pop("scale"), "router"),
    (lambda c: c["layers"][0]["mlp"].pop("expert"), "expert"),
    (lambda c: c["layers"][0]["mlp"].update(shared=dict()), "shared"),
    (lambda c: c["layers"][1]["mlp"].pop("ff"), "ff"),
    (lambda c: c["layers"][1]["mlp"].update(kind="gated"), "kind"),
    (lambda c: c["layers"][0].update(type="delta"), "type"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(times=0), "loop"),
    (lambda c: c["loop"].update(start=2, stop=2), "loop"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.update(width=0), "width"),
])
def test_configuration_faults_are_named(edit, text):
    cfg = copy.deepcopy(configs.KIMUTAR_A)
    edit(cfg)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(cfg)


# ---- pieces of the library that need no kernel -------------------------------------------------------------------------------
@pytest.mark.parametrize("base,dims,sc", [(500000.0, 40, dict(factor=3.0, original=1024, fast=16.0, slow=2.0)),
                                          (100.0, 8, dict(factor=4.0, original=64, fast=8.0, slow=2.0)),
                                          (10000.0, 64, dict(factor=40.0, original=4096, fast=32.0, slow=1.0)),
                                          (50.0, 2, dict(factor=3.0, original=10, fast=1.0, slow=1.0))])
def test_frequencies_blended_along_a_ramp(base, dims, sc):
    part = RotaryNeox(dims + 8, base, dims, dict(sc, kind="ramp"))
    part.bind({}, torch.float32, "cpu")
    want, grow = plain.ramp_frequencies(base, dims, sc)
    assert np.array_equal(part.inv_freq.numpy(), want.astype(np.float32)) and part.amplitude == grow == 0.1 * math.log(sc["factor"]) + 1.0
    plain_f = plain.plain_frequencies(base, dims)
    assert np.all(want <= plain_f * (1 + 1e-12)) and np.all(want >= plain_f / sc["factor"] * (1 - 1e-12))


@pytest.mark.parametrize("base,dims,sc", [(300000.0, 80, dict(factor=6.0, low=1.0, high=3.0, original=1024)),
                                          (10000.0, 16, dict(factor=3.0, low=1.0, high=5.0, original=50)),
                                          (500000.0, 128, dict(factor=32.0, low=1.0, high=4.0, original=8192))])
def test_frequencies_kept_divided_or_blended_by_wave_length(base, dims, sc):
    part = RotaryInterleaved(dims, base, dims, dict(sc, kind="bands"))
    part.bind({}, torch.float32, "cpu")
    want = plain.band_frequencies(base, dims, sc)
    assert np.array_equal(part.inv_freq.numpy(), want.astype(np.float32)) and part.amplitude == 1.0
    f = plain.plain_frequencies(base, dims)
    wave = 2 * math.pi / f
    short, long_ = wave < sc["original"] / sc["high"], wave > sc["original"] / sc["low"]
    assert short.any() and long_.any() and (~short & ~long_).any()           # all three bands occur
    assert np.array_equal(want[short], f[short]) and np.allclose(want[long_], f[long_] / sc["factor"], rtol=1e-15)
    with pytest.raises(ValueError, match="scaling"):
        RotaryNeox(8, 100.0, 8, dict(kind="stretch", factor=2.0))


def test_rows_of_a_projection_gathered_and_padded_with_their_bias():
    g = torch.Generator().manual_seed(3)
    w, b = torch.randn(6, 5, generator=g), torch.randn(6, generator=g)
    lin = StackedLinear(5)
    lin.add("w", 3 * 4, "b", heads=(3, 2, 4), gather=(6, [4, 5, 0, 1, 0, 1]))     # three heads of two rows, padded to four
    lin.add("u", 2)
    assert [(s.name, tuple(s.shape)) for s in lin.weight_specs()] == [("w", (6, 5)), ("b", (6,)), ("u", (2, 5))]
    lin.bind({"w": w, "b": b, "u": torch.ones(2, 5)}, torch.float32, "cpu")
    rows = [4, 5, None, None, 0, 1, None, None, 0, 1, None, None]
    for i, r in enumerate(rows):
        assert torch.equal(lin.weight[i], w[r] if r is not None else torch.zeros(5))
        assert float(lin.colbias[i]) == (float(b[r]) if r is not None else 0.0)
    assert lin.out_features == 14 and torch.equal(lin.colbias[12:], torch.zeros(2))
    with pytest.raises(ValueError, match="gathered"):
        StackedLinear(5).add("w", 4, gather=(6, [0, 1, 2]))


def test_a_window_that_keeps_the_first_positions_keeps_their_pages():
    reqs = {0: [KVRequest("kv", 2, 8, 70, keep_first=65)], 1: [KVRequest("kv", 2, 8, 70, keep_first=3)], 2: [KVRequest("kv", 2, 8, 70)]}
    c = Cache(reqs, 64 * 24, 2, torch.float32, "cpu")
    assert len(c.kv_groups) == 3                                  # what is kept is part of what a group is
    s = c.acquire()
    c.reserve(s, 400)
    c.commit(s, 400)
    held = [g.pool.n_held for g in c.kv_groups]
    assert held == [2 + 2, 1 + 2, 2]                              # pages 5 and 6 hold positions 331..; the first two or one stay
    assert [p >= 0 for p in c.kv_groups[0].pages_of[s]] == [True, True, False, False, False, True, True]
    c.reserve(s, 1)
    c.commit(s, 1)
    c.check()
    c.release(s)
    assert [g.pool.n_held for g in c.kv_groups] == [0, 0, 0]


# ---- the plain mechanisms against their definitions -------------------------------------------------------------------------------
def test_plain_mask_and_sink():
    assert [j for j in range(12) if plain.visible(11, j, 4, 3)] == [0, 1, 2, 8, 9, 10, 11]
    assert [j for j in range(12) if plain.visible(5, j, 4, 3)] == [0, 1, 2, 3, 4, 5] and not plain.visible(3, 4)
    assert [j for j in range(12) if plain.visible(11, j, 4, 0)] == [8, 9, 10, 11] and plain.visible(11, 0)
    # one key of score 0 beside a sink of score s: the weight is 1 / (1 + e^s); a sink far below every score vanishes
    q, k, v = np.zeros((1, 4)), np.ones((1, 4)), np.full((1, 2), 6.0)
    for s in (-3.0, 0.0, 2.0):
        assert np.allclose(plain.attend(q, k, v, 1.0, sink=s), 6.0 / (1.0 + math.exp(s)))
    assert np.allclose(plain.attend(q, k, v, 1.0, sink=-800.0), 6.0) and np.allclose(plain.attend(q, k, v, 1.0), 6.0)
    # three keys, the loud one outside a window of 2 unless it is kept
    q, k, v = np.ones((4, 1)), np.array([[9.0], [0.0], [0.0], [0.0]]), np.array([[1.0], [0.0], [0.0], [0.0]])
    assert plain.attend(q, k, v, 1.0, 2, 0)[3, 0] == 0.0 and plain.attend(q, k, v, 1.0, 2, 1)[3, 0] > 0.99
    assert plain.attend(q, k, v, 1.0, 2, 0)[1, 0] > 0.99


def test_plain_rotations():
    x = np.arange(16, dtype=np.float64).reshape(1, 1, 16)
    f = np.array([0.5, 0.25])
    a = np.float32(3) * f.astype(np.float32)
    h = plain.rotate_halves(x, [3], f, 2.0)[0, 0]
    assert np.allclose(h[0], 2 * (0 * math.cos(a[0]) - 2 * math.sin(a[0]))) and np.allclose(h[3], 2 * (3 * math.cos(a[1]) + 1 * math.sin(a[1])))
    n = plain.rotate_neighbours(x, [3], f)[0, 0]
    assert np.allclose(n[2], 2 * math.cos(a[1]) - 3 * math.sin(a[1])) and np.allclose(n[1], 1 * math.cos(a[0]) + 0 * math.sin(a[0]))
    assert np.array_equal(h[4:], x[0, 0, 4:]) and np.array_equal(n[4:], x[0, 0, 4:])


def test_plain_delta_rule_against_its_unrolled_steps():
    g = np.random.default_rng(1)
    q, k, v = g.standard_normal((2, 3)), g.standard_normal((2, 3)), g.standard_normal((2, 2))
    beta, decay = np.array([0.5, 0.25]), g.random((2, 3))
    o = plain.delta_scan(q, k, v, beta, decay)
    S1 = np.outer(k[0], beta[0] * v[0])                                  # the state was zero: nothing to correct
    assert np.allclose(o[0], S1.T @ q[0])
    D = decay[1][:, None] * S1
    S2 = D + np.outer(k[1], beta[1] * (v[1] - D.T @ k[1]))
    assert np.allclose(o[1], S2.T @ q[1])
    # a decay of one in every channel and a write of full strength: asking with the same unit key returns the value
    k1 = np.array([[0.6, 0.8, 0.0]])
    assert np.allclose(plain.delta_scan(k1, k1, np.array([[2.0, -1.0]]), np.array([1.0]), np.ones((1, 3))), [[2.0, -1.0]])


def test_plain_routing_and_feed_forwards():
    z = np.array([0.0, 1.0, 0.9, -1.0])
    s = np.exp(z) / np.exp(z).sum()
    order, w = plain.route(z, np.zeros(4), 2, 3.0)
    assert order == [1, 2] and np.allclose(w, s[[1, 2]] / s[[1, 2]].sum() * 3.0) and np.isclose(w.sum(), 3.0)
    order, w2 = plain.route(z, np.array([0.0, 0.0, 0.0, 1.0]), 2, 3.0)      # the correction changes the choice, not the scores
    assert order == [3, 1] and np.allclose(w2, s[[3, 1]] / s[[3, 1]].sum() * 3.0)
    assert plain.route(np.zeros(3), np.zeros(3), 2, 1.0)[0] == [0, 1]        # ties: the lowest index first
    W = {"up": np.array([[1.0, 0.0], [0.0, -1.0]]), "down": np.array([[1.0, 1.0]])}
    assert np.allclose(plain.dense(np.array([[3.0, 2.0], [-1.0, -2.0]]), W, ""), [[9.0], [4.0]])
    x = np.array([0.5, -1.0])
    E = {"e.gate": np.eye(2), "e.up": 2 * np.eye(2), "e.down": np.ones((1, 2))}
    assert np.allclose(plain.gated_expert(x, E, "e."), (plain.silu(x) * 2 * x).sum())


def test_plain_run_order_and_layer_norm():
    cfg = dict(layers=[0, 1, 2, 3], loop=dict(start=1, stop=3, times=2))
    assert plain.run_order(cfg) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    assert plain.run_order(dict(layers=[0, 1])) == [(0, None), (1, None)]
    x = np.array([[1.0, 2.0, 3.0, 6.0]])
    n = plain.layer_norm(x, np.array([1.0, 1.0, 2.0, 1.0]), 0.0)
    assert np.allclose(n, (x - 3.0) / math.sqrt(3.5) * np.array([1.0, 1.0, 2.0, 1.0]))
