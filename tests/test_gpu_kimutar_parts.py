"""Each Kimutar mechanism alone on the GPU against its plain function (tests/plain/kimutar_plain.py), on inputs made so that
a fault shows: the layer norm alone and as a pair that shares its statistics; the weighted norm per head before a rotation
of either pairing, with enlarged cosines and sines, at positions up to 4,097; a sliding window that keeps the sequence's
first keys and a learned sink per head in all four attention kernels (the warp kernel, single tokens with the keys split,
prompts on tcgen05 with the keys whole and in ranges, single tokens in one kernel), with one loud key just inside and just
outside the window, the last kept key and the first one that is not, at page borders; the join of two attention maps; the
delta rule with a decay per key channel, a state that barely decays in most channels and is asked hundreds of tokens and
several steps later for what was written at token 3, in slots that held rubbish and a slot used again; routing over all
experts with a correction that changes the choice but not the weight and weights normed to a given sum; the dense
feed-forward without a gate; the sigmoid gate of a normed read-out.
"""
import math

import numpy as np
import pytest
import torch

from tinyllama_c_b200 import ops
from plain import ops_plain
from plain import kimutar_plain as plain
from test_gpu_kernels import TOL as KTOL, _paged_setup, _step_arrays, cmp, gen, rnd

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device="cuda")


class _Step:
    pass


# ---- layer norm ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("D", [5, 52, 64, 1000, 4098, 8200])
def test_layer_norm_alone_in_pairs_and_of_chosen_rows(dtype, D):
    """Rows with a mean far from zero (a norm that forgets to subtract it, or takes E[x^2] - mean^2, shows)."""
    g = np.random.default_rng(1)
    x = g.standard_normal((9, D)) * 2.0 + 30.0
    x = x.astype(np.float32).astype(np.float64)
    w1, w2 = 1 + 0.2 * g.standard_normal(D), 1 + 0.2 * g.standard_normal(D)
    tol = 2e-4 if dtype == "float32" else 1e-2      # (deviations of ~2 from values of ~30: seven bits of the 32-bit input are gone)
    out1, out2 = torch.empty((9, D), dtype=DT[dtype], device="cuda"), torch.empty((9, D), dtype=DT[dtype], device="cuda")
    ops.layernorm(dev(x), dev(w1), 1e-5, out1)
    want1, want2 = plain.layer_norm(x, w1, 1e-5), plain.layer_norm(x, w2, 1e-5)
    assert np.abs(out1.float().cpu().numpy() - want1).max() <= tol * np.abs(want1).max()
    ops.layernorm(dev(x), dev(w1), 1e-5, out1, None, dev(w2), out2)
    assert np.abs(out1.float().cpu().numpy() - want1).max() <= tol * np.abs(want1).max()
    assert np.abs(out2.float().cpu().numpy() - want2).max() <= tol * np.abs(want2).max()
    rows = [7, 0, 3]
    out3 = torch.empty((3, D), dtype=DT[dtype], device="cuda")
    ops.layernorm(dev(x), dev(w2), 1e-6, out3, dev(rows, torch.int32))
    want3 = plain.layer_norm(x[rows], w2, 1e-6)
    assert np.abs(out3.float().cpu().numpy() - want3).max() <= tol * np.abs(want3).max()


def test_a_learned_row_joins_every_row():
    g = np.random.default_rng(2)
    x, v = g.standard_normal((37, 52)).astype(np.float32), g.standard_normal(52).astype(np.float32)
    xd = dev(x)
    ops.add_row(xd, dev(v))
    assert np.array_equal(xd.cpu().numpy(), x + v[None, :])


# ---- the norm per head before the rotation ------------------------------------------------------------------------------------
@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("H,KV,stride,dim,rot", [(3, 2, 24, 16, 8), (4, 1, 64, 64, 64), (2, 2, 40, 40, 0), (5, 5, 96, 48, 24)])
def test_weighted_head_norm_then_rotation(H, KV, stride, dim, rot, interleaved):
    g = np.random.default_rng(3)
    T = 11
    pos = np.array([0, 1, 2, 63, 64, 65, 1000, 4095, 4096, 4097, 7], dtype=np.int32)
    width = (H + KV) * stride + 3
    x = (g.standard_normal((T, width)) * 3.0).astype(np.float32)
    qw, kw = 1 + 0.3 * g.standard_normal(dim), 1 + 0.3 * g.standard_normal(dim)
    freq = plain.plain_frequencies(777.0, rot) * g.uniform(0.3, 1.0, rot // 2) if rot else np.zeros(0)
    freq = freq.astype(np.float32).astype(np.float64)
    amp = 1.0693
    xd = dev(x)
    ops.qk_rotate_norm(xd, 2, 2 + H * stride, H, KV, stride, dim, dev(freq), interleaved, None, dev(pos, torch.int32),
                       dev(qw), dev(kw), 1e-5, amp)
    got = xd.cpu().numpy().astype(np.float64)
    want = x.astype(np.float64).copy()
    for off, n, w in ((2, H, qw), (2 + H * stride, KV, kw)):
        heads = x[:, off:off + n * stride].astype(np.float64).reshape(T, n, stride)[:, :, :dim]
        normed = plain.unit_rms(heads, 1e-5) * w
        if interleaved:
            turned = plain.rotate_neighbours(normed, pos, freq)
            # (the plain rotation of neighbours has no amplitude: apply it to the rotated dimensions)
            turned[..., :rot] = (turned[..., :rot] - 0.0) * amp
        else:
            turned = plain.rotate_halves(normed, pos, freq, amp)
        block = want[:, off:off + n * stride].reshape(T, n, stride)
        block[:, :, :dim] = turned
        want[:, off:off + n * stride] = block.reshape(T, n * stride)
    assert np.abs(got - want).max() <= 3e-5 * np.abs(want).max()
    assert np.array_equal(got[:, :2], x[:, :2].astype(np.float64)) and np.array_equal(got[:, -1], x[:, -1].astype(np.float64))


# ---- a window that keeps the first keys, and a sink per head: the four attention kernels -----------------------------------------
def _mark_keys(k_pages, table, slots, seq, marks):
    """Scales single cached keys of sequence `seq` (position -> factor) so that they stand out for every query."""
    for p, f in marks.items():
        k_pages[int(table[int(slots[seq]), p // 64]), :, p % 64, :] *= f


def _loud_positions(last, window, keep):
    """For a query at position `last`: the last key outside the window and the first inside it, the last kept key and the
    first that is not kept."""
    marks = {last - window: 6.0, last - window + 1: 5.0}
    if keep:
        marks[keep - 1] = 7.0
    if keep < last - window:
        marks[keep] = 8.0
    return {p: f for p, f in marks.items() if 0 <= p <= last}


WINDOWS = [(5, 2), (64, 1), (33, 3), (130, 70), (100, 64), (1, 1), (40, 0)]


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("window,keep", WINDOWS)
@pytest.mark.parametrize("H,KV,hd", [(6, 3, 24), (4, 1, 80), (9, 1, 64)])
def test_window_kept_keys_and_sink_of_any_rows_and_of_split_keys(dtype, H, KV, hd, window, keep):
    """The warp kernel on a step that mixes prompts (one continues at position 300) with single rows, and the split-key
    kernels of single-token steps (also with more key pieces than the longest row needs)."""
    g = gen(41)
    sink = rnd(g, H, scale=2.0)
    starts, lens = [0, 300, 63, 5], [270, 40, 2, 1]
    pos, row_seq, cu, _ = _step_arrays(starts, lens)
    slots, table, k_pages, v_pages = _paged_setup(g, 4, [s + n for s, n in zip(starts, lens)], KV, hd, DT[dtype])
    T = sum(lens)
    q = rnd(g, T, H * hd, dtype=DT[dtype])
    _mark_keys(k_pages, table, slots, 0, _loud_positions(269, window, keep))
    _mark_keys(k_pages, table, slots, 1, _loud_positions(339, window, keep))
    args = [q, k_pages, v_pages, table, pos, row_seq, slots, torch.empty(T, H * hd, dtype=DT[dtype]), H, KV, hd,
            1.0 / math.sqrt(hd), window, 0, None, None, 0, 0, 0, 0.0, False, keep, sink]
    cmp("attention", args, [7], tol_of=KTOL[DT[dtype]] * 2)
    if keep and window + keep < 200:                   # the kept keys show: the same call without them differs by far more
        kept = args[7].float().clone()
        ops_plain.attention(*args[:-2], 0, sink)
        assert (args[7].float() - kept).abs().max() > 0.1 * kept.abs().max()
    starts = [0, 269, 63, 700, 128]
    pos, row_seq, cu, _ = _step_arrays(starts, [1] * 5)
    slots, table, k_pages, v_pages = _paged_setup(g, 5, [s + 1 for s in starts], KV, hd, DT[dtype], n_slots=6)
    q = rnd(g, 5, H * hd, dtype=DT[dtype])
    _mark_keys(k_pages, table, slots, 1, _loud_positions(269, window, keep))
    _mark_keys(k_pages, table, slots, 3, _loud_positions(700, window, keep))
    for max_keys in (701, 1024):
        cmp("attention", [q, k_pages, v_pages, table, pos, row_seq, slots, torch.empty(5, H * hd, dtype=DT[dtype]), H, KV,
                          hd, 1.0 / math.sqrt(hd), window, max_keys, None, None, 0, 0, 0, 0.0, False, keep, sink], [7],
            tol_of=KTOL[DT[dtype]] * 2)


@pytest.mark.parametrize("key_ranges", [0, 3])
@pytest.mark.parametrize("window,keep", WINDOWS)
@pytest.mark.parametrize("H,KV,hd", [(8, 2, 128), (6, 1, 64), (3, 3, 64)])
def test_window_kept_keys_and_sink_of_prompts_on_tcgen05(H, KV, hd, window, keep, key_ranges):
    """Prompts that cross 128-row tiles, one that continues at position 2,100 (its kept keys lie many key tiles in front of
    its window), single rows; the keys whole and cut into ranges."""
    g = gen(42)
    sink = rnd(g, H, scale=2.0)
    starts, lens = [0, 2100, 0, 63, 0], [333, 129, 70, 2, 1]
    pos, row_seq, cu, start_pos = _step_arrays(starts, lens)
    totals = [s + n for s, n in zip(starts, lens)]
    slots, table, k_pages, v_pages = _paged_setup(g, 5, totals, KV, hd, torch.bfloat16, n_slots=7)
    T = sum(lens)
    q = rnd(g, T, H * hd, dtype=torch.bfloat16)
    marks = {}
    for last in (127, 128, 200, 332):
        marks.update(_loud_positions(last, window, keep))
    _mark_keys(k_pages, table, slots, 0, marks)
    marks = {}
    for last in (2100, 2163, 2228):
        marks.update(_loud_positions(last, window, keep))
    _mark_keys(k_pages, table, slots, 1, marks)
    args = [q, k_pages, v_pages, table, pos, row_seq, slots, torch.empty(T, H * hd, dtype=torch.bfloat16), H, KV, hd,
            1.0 / math.sqrt(hd), window, 0, cu, start_pos, max(totals), 0, key_ranges, 0.0, False, keep, sink]
    cmp("attention", args, [7], tol_of=KTOL[torch.bfloat16] * 2.5)
    torch.cuda.synchronize()
    ops.check_errors()
    if keep and key_ranges == 0:
        kept = args[7].float().clone()
        ops_plain.attention(*args[:-2], 0, sink)
        assert (args[7].float() - kept).abs().max() > 0.1 * kept.abs().max()


@pytest.mark.parametrize("window,keep", WINDOWS)
@pytest.mark.parametrize("H,KV,hd,rope", [(8, 2, 128, 64), (6, 1, 64, 64), (6, 3, 64, 0), (2, 2, 256, 128)])
def test_window_kept_keys_and_sink_of_single_tokens_in_one_kernel(H, KV, hd, rope, window, keep):
    """Rotation, store of the new row and attention in one launch: the keys in one piece a block, in several pieces that
    another block merges, and pieces of two rounds."""
    g = gen(43)
    sink = rnd(g, H, scale=2.0)
    starts = [0, 200, 63, 3300, 127, 128]
    B = len(starts)
    pos, row_seq, cu, _ = _step_arrays(starts, [1] * B)
    slots, table, k_pages, v_pages = _paged_setup(g, B, [s + 1 for s in starts], KV, hd, torch.bfloat16, n_slots=7)
    _mark_keys(k_pages, table, slots, 3, _loud_positions(3300, window, keep))
    _mark_keys(k_pages, table, slots, 1, _loud_positions(200, window, keep))
    qkv = rnd(g, B, (H + 2 * KV) * hd)
    inv = (1.0 / torch.pow(torch.tensor(1e4, dtype=torch.float64),
                           torch.arange(rope // 2, dtype=torch.float64) * 2 / max(rope, 1))).float()
    scale = 1.3 / math.sqrt(hd)
    k_ref, v_ref = k_pages.clone(), v_pages.clone()
    q_ref = torch.empty(B, H * hd, dtype=torch.bfloat16)
    ops_plain.rope_kv_store(qkv, 0, H * hd, (H + KV) * hd, q_ref, k_ref, v_ref, inv, pos, row_seq, slots, table, H, KV, hd, True)
    out_ref = torch.empty(B, H * hd, dtype=torch.bfloat16)
    ops_plain.attention(q_ref, k_ref, v_ref, table, pos, row_seq, slots, out_ref, H, KV, hd, scale, window, 0, None, None, 0, 0, 0,
                        0.0, False, keep, sink)
    counters = ops.new_arrival_counters("cuda")
    try:
        for max_keys, passes in ((3301, 0), (4096, 2), (3301, 1000)):
            ops.attention_decode_fused_passes(passes)
            out = torch.empty(B, H * hd, dtype=torch.bfloat16, device="cuda")
            ops.attention_decode_fused(qkv.cuda(), 0, H * hd, (H + KV) * hd, k_pages.cuda(), v_pages.cuda(), inv.cuda(), True, table.cuda(),
                                       pos.cuda(), row_seq.cuda(), slots.cuda(), out, H, KV, hd, scale, window, max_keys, counters, 0.0,
                                       False, keep, sink.cuda())
            torch.cuda.synchronize()
            ops.check_errors()
            ref = out_ref.double()
            err = (ref - out.cpu().double()).abs().max()
            assert err <= KTOL[torch.bfloat16] * 2.5 * ref.abs().max(), f"max_keys {max_keys}, passes {passes}: {err}"
    finally:
        ops.attention_decode_fused_passes(0)


def test_a_sink_of_its_own_score_shows():
    """One key of score 0 and a sink of score s: the output is the value times 1 / (1 + e^s)."""
    for s in (-2.0, 0.0, 3.0):
        k_pages, v_pages = torch.zeros(1, 1, 64, 8), torch.ones(1, 1, 64, 8)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32)
        out = torch.empty(1, 8, device="cuda")
        ops.attention(torch.ones(1, 8).cuda(), k_pages.cuda(), v_pages.cuda(), i32([[0]]).cuda(), i32([0]).cuda(), i32([0]).cuda(),
                      i32([0]).cuda(), out, 1, 1, 8, 0.5, sink_values=torch.tensor([s]).cuda())
        assert abs(float(out[0, 0]) - 1.0 / (1.0 + math.exp(s))) < 1e-6


# ---- the join of two maps ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("H,per_group,hd,vd", [(4, 2, 24, 16), (2, 2, 64, 64), (6, 1, 96, 96), (3, 3, 40, 8)])
def test_difference_of_two_maps_normed(dtype, H, per_group, hd, vd):
    g = np.random.default_rng(5)
    T, lam, eps, scale = 13, 0.37, 1e-5, 0.7
    maps = g.standard_normal((T, 2 * H, hd))
    maps = plain.bf16_round(maps) if dtype == "bfloat16" else maps.astype(np.float32).astype(np.float64)
    out = torch.full((T, H * hd), 9.0, dtype=DT[dtype], device="cuda")
    ops.difference_join(dev(maps.reshape(T, -1), DT[dtype]), hd, out, hd, H, per_group, vd, lam, eps, scale)
    got = out.float().cpu().numpy().reshape(T, H, hd)
    for h in range(H):
        grp, j = divmod(h, per_group)
        a1, a2 = maps[:, 2 * grp * per_group + j, :vd], maps[:, (2 * grp + 1) * per_group + j, :vd]
        want = plain.unit_rms(a1 - lam * a2, eps) * scale
        tol = 2e-5 if dtype == "float32" else 8e-3
        assert np.abs(got[:, h, :vd] - want).max() <= tol * np.abs(want).max(), f"head {h}"
        assert np.all(got[:, h, vd:] == 9.0)          # what lies past a head's values is not touched


# ---- the delta rule with a decay per key channel ---------------------------------------------------------------------------------
@pytest.mark.parametrize("split", [0, 8, 16])
@pytest.mark.parametrize("H,G,dk,dv", [(2, 1, 8, 8), (4, 2, 40, 12), (2, 2, 64, 64), (3, 3, 100, 33), (2, 1, 256, 16), (1, 1, 130, 70),
                                       (2, 1, 128, 128)])
def test_delta_rule_with_a_decay_per_channel(H, G, dk, dv, split, request):
    """Two sequences in one step, then continued in portions and single tokens.  Most channels decay by less than 1e-3 a
    token, every fifth one by a third (a kernel that uses one channel's factor for a whole head, or the wrong row's, shows);
    a value written at token 3 with a key that later queries repeat; slots that held rubbish; slot 0 used again."""
    ops.delta_rule_split(split)
    request.addfinalizer(lambda: ops.delta_rule_split(0))
    lens, portions = [330, 97], [[203, 1, 1, 61, 64], [90, 1, 1, 3, 2]]
    state = torch.full((3, H, dk, dv), 3.0, device="cuda")

    def make(T, seed):
        r = np.random.default_rng(seed)
        q, k = r.standard_normal((T, G, dk)), r.standard_normal((T, G, dk))
        unit = k[3] / np.sqrt((k[3] * k[3]).sum(-1, keepdims=True))
        for t in range(T):                                            # no other token writes along token 3's key
            if t != 3:
                k[t] -= (k[t] * unit).sum(-1, keepdims=True) * unit
        q[5:] = 0.15 * q[5:] + k[3][None] * 2.0                       # later queries ask for token 3's key
        v = r.standard_normal((T, H, dv)) * 0.1
        v[3] = r.standard_normal((H, dv)) * 3.0
        beta = plain.sigmoid(r.standard_normal((T, H)))
        beta[3] = 0.97
        a = -7.0 - r.random((T, H, dk))                               # softplus(a) ~ 1e-3
        a[:, :, ::5] = 0.5                                            # these channels fade fast
        f = lambda x: x.astype(np.float32).astype(np.float64)
        return [f(x) for x in (q, k, v, beta, a)]

    A = -np.exp(np.linspace(-0.3, 0.2, H))

    def run(seqs, slots, cuts):
        outs, at = [[] for _ in seqs], [0] * len(seqs)
        for s in range(max(len(c) for c in cuts)):
            live = [i for i in range(len(seqs)) if s < len(cuts[i])]
            counts = [cuts[i][s] for i in live]
            T = sum(counts)
            qkv = np.zeros((T, 2 * G * dk + H * dv + 4), dtype=np.float32)
            proj_b = np.zeros((T, H + 1), dtype=np.float32)
            chan = np.zeros((T, H * dk), dtype=np.float32)
            o = 0
            for i, n in zip(live, counts):
                q, k, v, beta, a = [x[at[i]:at[i] + n] for x in seqs[i]]
                qkv[o:o + n, 4:4 + G * dk] = q.reshape(n, -1)
                qkv[o:o + n, 4 + G * dk:4 + 2 * G * dk] = k.reshape(n, -1)
                qkv[o:o + n, 4 + 2 * G * dk:] = v.reshape(n, -1)
                proj_b[o:o + n, 1:] = np.log(beta / (1.0 - beta))
                chan[o:o + n] = a.reshape(n, -1)
                o += n
            step = _Step()
            step.n_seqs, step.n_rows = len(live), T
            step.cu_seqlens = dev(np.concatenate([[0], np.cumsum(counts)]), torch.int32)
            step.slots = dev([slots[i] for i in live], torch.int32)
            step.start_pos = dev([at[i] for i in live], torch.int32)
            qd, bd, cd = dev(qkv), torch.empty((T, H), device="cuda"), dev(chan)
            ops.delta_prepare(qd, 4, 4 + G * dk, G, dk, 1e-6, dk ** -0.5, dev(proj_b), 1, H, bd, cd, dev(A))
            y = torch.empty((T, H * dv), device="cuda")
            ops.delta_rule(qd, 4, 4 + G * dk, 4 + 2 * G * dk, bd, cd, state, step, y, H, G, dk, dv, per_channel=True)
            torch.cuda.synchronize()
            y = y.cpu().numpy().astype(np.float64)
            o = 0
            for i, n in zip(live, counts):
                outs[i].append(y[o:o + n])
                at[i] += n
                o += n
        return [np.concatenate(x).reshape(-1, H, dv) for x in outs]

    def want_of(seq):
        q, k, v, beta, a = seq
        qn = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dk ** -0.5
        kn = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
        decay = np.exp(A[None, :, None] * plain.softplus(a))
        return np.stack([plain.delta_scan(qn[:, h // (H // G)], kn[:, h // (H // G)], v[:, h], beta[:, h], decay[:, h]) for h in range(H)], axis=1)

    seqs = [make(n, 10 + i) for i, n in enumerate(lens)]
    got = run(seqs, [0, 2], portions)
    for i, seq in enumerate(seqs):
        want = want_of(seq)
        assert np.abs(got[i] - want).max() <= 3e-4 * np.abs(want).max(), f"sequence {i}"
        # the read-out long after token 3 still carries its value in the channels that barely decay
        assert np.abs(want[-1]).max() > 0.003 * np.abs(seq[2][3]).max()
    third = make(70, 33)
    got = run([third], [0], [[64, 6]])
    want = want_of(third)
    assert np.abs(got[0] - want).max() <= 3e-4 * np.abs(want).max(), "a slot that is used again"


# ---- routing, the dense feed-forward, the sigmoid gate --------------------------------------------------------------------------------
@pytest.mark.parametrize("E,top,sum_to", [(8, 3, 2.0), (5, 5, 1.0), (1, 1, 0.5), (40, 4, 2.5), (6, 2, 0.0)])
def test_routing_over_all_experts_with_weights_normed_to_a_sum(E, top, sum_to):
    g = np.random.default_rng(7)
    T = 50
    z = g.standard_normal((T, E + 2)).astype(np.float32)
    corr = (g.standard_normal(E) * 0.3).astype(np.float32)
    if E > 2:
        z[0, :E] = 0.0                      # exact ties: the lowest indices win
        corr[:] = np.where(np.arange(E) == E - 1, 0.5, corr)        # the last expert is chosen often for its correction alone
    ids, wts = ops.moe_route(dev(z), E, top, 32, "softmax_all", dev(corr), 0, sum_to)[:2]
    ids, wts = ids.cpu().numpy().reshape(T, top), wts.cpu().numpy().reshape(T, top).astype(np.float64)
    flipped = 0
    for t in range(T):
        if E > 2 and t == 0:
            continue
        order, w = plain.route(z[t, :E].astype(np.float64), corr.astype(np.float64), top, sum_to if sum_to else 1.0)
        if not sum_to:                      # scores as they are
            e = np.exp(z[t, :E].astype(np.float64) - z[t, :E].max())
            w = np.array([(e / e.sum())[i] for i in order])
        assert list(ids[t]) == order, f"row {t}"
        assert np.abs(wts[t] - w).max() <= 1e-5 * max(w.max(), 1e-3), f"row {t}"
        flipped += order != sorted(range(E), key=lambda i: (-z[t, i], i))[:top]
    if E > 2 and top < E:
        assert flipped > 0                  # the correction changed choices
        assert abs(wts[1].sum() - (sum_to or wts[1].sum())) < 1e-5


@pytest.mark.parametrize("dtype", list(DT))
def test_squared_relu_between_two_products(dtype):
    g = np.random.default_rng(8)
    x = (g.standard_normal((33, 70)) * 2).astype(np.float32)
    out = torch.empty((33, 70), dtype=DT[dtype], device="cuda")
    ops.convert(dev(x), out, "relu_squared")
    want = np.maximum(x.astype(np.float64), 0.0) ** 2
    assert np.abs(out.float().cpu().numpy() - want).max() <= (1e-6 if dtype == "float32" else 5e-3) * want.max()
    assert float(out[x < 0].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("H,dv", [(4, 12), (2, 64), (3, 200)])
def test_normed_read_out_with_a_sigmoid_gate(dtype, H, dv):
    g = np.random.default_rng(9)
    T = 21
    y, z = g.standard_normal((T, H * dv)).astype(np.float32) * 3, g.standard_normal((T, H * dv)).astype(np.float32) * 2
    w = (1 + 0.2 * g.standard_normal(dv)).astype(np.float32)
    out = torch.empty((T, H * dv), dtype=DT[dtype], device="cuda")
    ops.gated_rmsnorm(dev(y), dev(z), dev(np.tile(w, H)), 1e-5, H, True, out, gate="sigmoid")
    want = (plain.unit_rms(y.astype(np.float64).reshape(T, H, dv), 1e-5) * w).reshape(T, -1) * plain.sigmoid(z.astype(np.float64))
    assert np.abs(out.float().cpu().numpy() - want).max() <= (3e-5 if dtype == "float32" else 8e-3) * np.abs(want).max()
