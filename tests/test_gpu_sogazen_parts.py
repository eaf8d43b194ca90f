"""Each Sogazen mechanism alone on the GPU against its plain function, on inputs made so that a fault shows: attention
with a capped score and a sink in all its kernels (prompts on tcgen05 with the keys whole and in ranges, the warp kernel,
single tokens with the keys split), with one far key whose raw score lies far above the cap, rows whose scores are all
so low that the sink takes nearly everything, and first rows where the sink is half the denominator; the attention mixer
whose values are the keys as projected (biases, a norm over all heads at once, part of every head rotated); the mixer
with a decaying matrix state, with a state that barely decays (what was written hundreds of tokens back still decides the
output), a bonus that only the current token gets, steps that continue a sequence, and a slot that is used again; the
norm that joins two mixers; the clamped dense feed-forward with both clamps at work; routing over all outputs with a
correction that changes the choice but not the weight, identity outputs, and experts without a gate.
"""
import math

import numpy as np
import pytest
import torch

from tinyllama_c_b200 import ops
from tinyllama_c_b200.parts.base import PartSpec
from plain import ops_plain
from plain import sogazen_plain as plain
from test_gpu_kernels import TOL as KTOL, _paged_setup, _step_arrays, cmp, gen, rnd
from test_gpu_turevik_parts import DECODED, DT, LENS, compare, dev, draw, rnd_of, run_steps

pytestmark = pytest.mark.gpu


# ---- attention with a capped score and a sink: the kernels ---------------------------------------------------------------
def _mark_keys(k_pages, table, slots, seq, marks):
    """Scales single cached keys of sequence `seq` (position -> factor) so that they stand out, or sink, for every query."""
    for p, f in marks.items():
        k_pages[int(table[int(slots[seq]), p // 64]), :, p % 64, :] *= f


@pytest.mark.parametrize("key_ranges", [0, 3])
@pytest.mark.parametrize("softcap,sink", [(0.0, True), (3.0, True), (25.0, False), (40.0, True)])
@pytest.mark.parametrize("H,KV,hd", [(8, 2, 128), (6, 1, 64), (3, 3, 64)])
def test_capped_scores_and_sink_of_prompts_on_tcgen05(H, KV, hd, softcap, sink, key_ranges):
    """Prompts that cross 128-row tiles, one that continues at position 2,100, single rows.  Position 5 of the first
    sequence has a raw score far above every cap (without the cap it would take the whole row), position 202 makes a
    row's maximum jump in a late key tile.  The third sequence's queries point away from its keys: all its scores are
    low and the sink takes most of the denominator.  First rows: one key and the sink."""
    g = gen(91)
    starts, lens = [0, 2100, 0, 63, 0], [333, 129, 70, 2, 1]
    pos, row_seq, cu, start_pos = _step_arrays(starts, lens)
    totals = [s + n for s, n in zip(starts, lens)]
    slots, table, k_pages, v_pages = _paged_setup(g, 5, totals, KV, hd, torch.bfloat16, n_slots=7)
    T = sum(lens)
    q = rnd(g, T, H * hd, dtype=torch.bfloat16)
    _mark_keys(k_pages, table, slots, 0, {5: 9.0, 202: 14.0})
    _mark_keys(k_pages, table, slots, 1, {73: 6.0, 2059: 7.0})
    # the third sequence: its keys share a component that its queries point away from, so every score is about -8 or lower
    for p in range(70):
        k_pages[int(table[int(slots[2]), p // 64]), :, p % 64, :] += 2.0
    rows3 = slice(int(cu[2]), int(cu[3]))
    q[rows3] = (0.1 * q[rows3].float() - 0.5).to(torch.bfloat16)
    args = [q, k_pages, v_pages, table, pos, row_seq, slots, torch.empty(T, H * hd, dtype=torch.bfloat16), H, KV, hd,
            1.0 / math.sqrt(hd), 0, 0, cu, start_pos, max(totals), 0, key_ranges, softcap, sink]
    cmp("attention", args, [7], tol_of=KTOL[torch.bfloat16] * 2.5)
    torch.cuda.synchronize()
    ops.check_errors()
    if sink and key_ranges == 0 and H == 3:         # the sink shows: the same call without it differs by far more than the allowance
        with_sink = args[7].float()
        ops_plain.attention(*args[:-1], False)
        assert (args[7].float() - with_sink).abs().max() > 0.2 * with_sink.abs().max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,KV,hd,softcap,sink", [(6, 3, 24, 2.0, True), (4, 1, 48, 30.0, True), (9, 1, 64, 5.0, True),
                                                  (8, 2, 128, 10.0, False), (5, 5, 80, 0.0, True)])
def test_capped_scores_and_sink_of_any_rows_and_of_single_tokens(dtype, H, KV, hd, softcap, sink):
    """The warp kernel (any sizes, both types; here a step that mixes a prompt with single rows) and the split-key
    kernels of single-token steps, the far key at position 3 of a sequence of 701 among them."""
    g = gen(92)
    starts, lens = [0, 200, 63, 5], [70, 1, 2, 1]
    pos, row_seq, cu, _ = _step_arrays(starts, lens)
    slots, table, k_pages, v_pages = _paged_setup(g, 4, [s + n for s, n in zip(starts, lens)], KV, hd, DT[dtype])
    T = sum(lens)
    q = rnd(g, T, H * hd, dtype=DT[dtype])
    _mark_keys(k_pages, table, slots, 1, {3: 8.0})
    cmp("attention", [q, k_pages, v_pages, table, pos, row_seq, slots, torch.empty(T, H * hd, dtype=DT[dtype]), H, KV, hd,
                      1.0 / math.sqrt(hd), 0, 0, None, None, 0, 0, 0, softcap, sink], [7], tol_of=KTOL[DT[dtype]] * 2)
    starts, lens = [0, 200, 63, 700, 128], [1, 1, 1, 1, 1]
    pos, row_seq, cu, _ = _step_arrays(starts, lens)
    slots, table, k_pages, v_pages = _paged_setup(g, 5, [s + n for s, n in zip(starts, lens)], KV, hd, DT[dtype], n_slots=6)
    q = rnd(g, 5, H * hd, dtype=DT[dtype])
    _mark_keys(k_pages, table, slots, 3, {3: 8.0, 640: 0.0})
    q[2] *= -3.0
    for max_keys in (701, 1024):
        cmp("attention", [q, k_pages, v_pages, table, pos, row_seq, slots, torch.empty(5, H * hd, dtype=DT[dtype]), H, KV,
                          hd, 1.0 / math.sqrt(hd), 0, max_keys, None, None, 0, 0, 0, softcap, sink], [7], tol_of=KTOL[DT[dtype]] * 2)



@pytest.mark.parametrize("H,KV,hd,rope,softcap,sink", [(8, 2, 128, 64, 30.0, True), (6, 1, 64, 64, 3.0, True), (6, 3, 64, 32, 0.0, True),
                                                       (4, 4, 128, 0, 8.0, False), (2, 2, 256, 128, 5.0, True)])
def test_capped_scores_and_sink_of_single_tokens_in_one_kernel(H, KV, hd, rope, softcap, sink):
    """Rotation, store of the new row and attention in one launch, with the cap and the sink: a far key whose raw score
    lies above the cap, a first row (its own key and the sink), a row whose query points away from all its keys (the
    sink takes most); the keys in one piece a block, in several pieces that another block merges, and pieces of two rounds."""
    g = gen(93)
    starts = [0, 200, 63, 3300, 127, 128]
    B = len(starts)
    pos, row_seq, cu, _ = _step_arrays(starts, [1] * B)
    slots, table, k_pages, v_pages = _paged_setup(g, B, [s + 1 for s in starts], KV, hd, torch.bfloat16, n_slots=7)
    _mark_keys(k_pages, table, slots, 3, {3: 9.0, 2500: 6.0})
    for p in range(200):
        k_pages[int(table[int(slots[1]), p // 64]), :, p % 64, :] += 1.5
    width = (H + 2 * KV) * hd
    qkv = rnd(g, B, width)
    qkv[1, :H * hd] = 0.1 * qkv[1, :H * hd] - 0.4
    inv = (1.0 / torch.pow(torch.tensor(1e4, dtype=torch.float64),
                           torch.arange(rope // 2, dtype=torch.float64) * 2 / max(rope, 1))).float()
    scale = 1.3 / math.sqrt(hd)
    k_ref, v_ref = k_pages.clone(), v_pages.clone()
    q_ref = torch.empty(B, H * hd, dtype=torch.bfloat16)
    ops_plain.rope_kv_store(qkv, 0, H * hd, (H + KV) * hd, q_ref, k_ref, v_ref, inv, pos, row_seq, slots, table, H, KV, hd, True)
    out_ref = torch.empty(B, H * hd, dtype=torch.bfloat16)
    ops_plain.attention(q_ref, k_ref, v_ref, table, pos, row_seq, slots, out_ref, H, KV, hd, scale, 0, 0, None, None, 0, 0, 0,
                        softcap, sink)
    counters = ops.new_arrival_counters("cuda")
    try:
        for max_keys, passes in ((3301, 0), (4096, 2), (3301, 1000)):
            ops.attention_decode_fused_passes(passes)
            k_gpu, v_gpu = k_pages.cuda(), v_pages.cuda()
            out = torch.empty(B, H * hd, dtype=torch.bfloat16, device="cuda")
            ops.attention_decode_fused(qkv.cuda(), 0, H * hd, (H + KV) * hd, k_gpu, v_gpu, inv.cuda(), True, table.cuda(), pos.cuda(),
                                       row_seq.cuda(), slots.cuda(), out, H, KV, hd, scale, 0, max_keys, counters, softcap, sink)
            torch.cuda.synchronize()
            ops.check_errors()
            ref = out_ref.double()
            err = (ref - out.cpu().double()).abs().max()
            assert err <= KTOL[torch.bfloat16] * 2.5 * ref.abs().max(), f"max_keys {max_keys}, passes {passes}: {err}"
    finally:
        ops.attention_decode_fused_passes(0)
    if sink:                                        # the sink shows: without it the first row would be its own value
        own = v_ref[int(table[int(slots[0]), 0]), :, 0, :].double().repeat_interleave(H // KV, 0).reshape(-1)
        assert (out_ref[0].double() - own).abs().max() > 0.05 * own.abs().max()


# ---- the attention mixer whose values are its keys ---------------------------------------------------------------------
@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("H,G,d,rot,cap", [(4, 2, 16, 6, 3.0), (9, 1, 64, 64, 20.0), (3, 3, 24, 0, 40.0), (8, 2, 128, 32, 12.0)])
def test_attention_mixer_with_keys_as_values(dtype, H, G, d, rot, cap):
    """Biases on q and k, one norm over all query heads and one over all key heads, part of every head rotated, the cap,
    the sink; what is cached as a value is the key as projected.  Prompts in one step, then single tokens."""
    g = np.random.default_rng(11)
    D = 40
    m = dict(heads=H, kv_heads=G, dim=d, vdim=d, scale=float(d ** -0.5) * 1.7, softcap=cap, rot=dict(base=1000.0, dims=rot))
    W = {"a.q": draw(g, (H * d, D), 0.3, dtype), "a.k": draw(g, (G * d, D), 0.3, dtype), "a.o": draw(g, (D, H * d), 0.2, dtype),
         "a.q.b": draw(g, (H * d,), 0.5, dtype), "a.k.b": draw(g, (G * d,), 0.5, dtype),
         "a.q.norm": 1.0 + draw(g, (H * d,), 0.3, dtype), "a.k.norm": 1.0 + draw(g, (G * d,), 0.3, dtype)}
    position = PartSpec("position", "rope_neox", dict(head_dim=d, theta=1000.0, rope_dim=rot)) if rot else \
        PartSpec("position", "none", dict(head_dim=d))
    part = PartSpec("mixer", "attention", dict(
        hidden=D, n_heads=H, n_kv_heads=G, head_dim=d, v_dim=d, prefix="a.", position=position,
        names=dict(q="q", k="k", o="o", q_bias="q.b", k_bias="k.b"), values="keys", scale=m["scale"],
        whole_norm=dict(q="q.norm", k="k.norm", eps=1e-5), softcap=cap, sink=True)).build()
    part.bind({k: torch.tensor(v, dtype=DT[dtype] if v.ndim == 2 else torch.float32) for k, v in W.items()}, DT[dtype], "cuda")
    rows = [draw(g, (n + DECODED, D), 1.0, dtype) for n in LENS]

    def forward(x, step, views):
        out = torch.zeros((x.shape[0], D), dtype=torch.float32, device="cuda")
        part.forward(x, step, views[0], out)
        return out
    got = run_steps(forward, part.cache_requests(), rows, dtype, DT[dtype])
    want = [plain.key_value_attention(x, W, "a.", m, 1e-5, np.arange(len(x)), rnd_of(dtype)) for x in rows]
    compare(got, want, dtype, "attention with keys as values", tol=3e-5 if dtype == "float32" else 4e-2)


# ---- the mixer with a decaying matrix state ------------------------------------------------------------------------------
class _Step:
    pass


def _wkv_plain(r, k, v, w, u):
    T, H, d = r.shape
    o, S = np.zeros((T, H, d)), np.zeros((H, d, d))
    for t in range(T):
        for h in range(H):
            kv = np.outer(k[t, h], v[t, h])
            o[t, h] = (S[h] + u[h][:, None] * kv).T @ r[t, h]
            S[h] = w[t, h][:, None] * S[h] + kv
    return o


@pytest.mark.parametrize("H,d", [(2, 8), (3, 32), (2, 64), (1, 72), (2, 40), (1, 130)])
def test_wkv_state_keeps_what_was_written_hundreds_of_tokens_back(H, d):
    """Two sequences in one step, then continued in portions and single tokens.  The decay stays within 1e-3 of one and
    token 3 writes a large value along a key that later receptances repeat, so hundreds of tokens on the read-out is
    still mostly that value: a state that is lost, reset, decayed twice or mixed up between sequences, heads or slots
    shows.  The bonus differs by far from 1, so leaving it out, or giving it to the state, shows at once.  The slots held
    rubbish before, and slot 0 is then used again by a third sequence."""
    lens, portions = [330, 97], [[203, 1, 1, 61, 64], [90, 1, 1, 3, 2]]
    state = torch.full((3, H, d, d), 3.0, device="cuda")
    u = np.random.default_rng(3).standard_normal((H, d)) * 2.0 + 3.0

    def make(T, seed):
        g = np.random.default_rng(seed)
        r, k = g.standard_normal((T, H, d)), g.standard_normal((T, H, d)) * 0.3
        unit = k[3] / np.sqrt((k[3] * k[3]).sum(-1, keepdims=True))
        for t in range(T):                                            # no other token writes along token 3's key
            if t != 3:
                k[t] -= (k[t] * unit).sum(-1, keepdims=True) * unit
        k[3] = unit
        r[5:] = 0.05 * r[5:] + unit[None] * 2.0                       # later tokens ask for token 3's key
        v = g.standard_normal((T, H, d)) * 0.1
        v[3] = g.standard_normal((H, d)) * 3.0
        a = np.log(-np.log(1.0 - 1e-3 * g.random((T, H, d))))        # w = exp(-exp(a)) within 1e-3 of one
        f = lambda x: x.astype(np.float32).astype(np.float64)
        return [f(x) for x in (r, k, v, a)]

    def run(seqs, slots, cuts):
        outs, at = [[] for _ in seqs], [0] * len(seqs)
        HD = H * d
        for s in range(max(len(c) for c in cuts)):
            live = [i for i in range(len(seqs)) if s < len(cuts[i])]
            counts = [cuts[i][s] for i in live]
            T = sum(counts)
            rkv = np.zeros((T, 3 * HD + 5), dtype=np.float32)       # v, r, k from columns 2, 2 + HD + 1, ...: any offsets
            a = np.zeros((T, HD), dtype=np.float32)
            o = 0
            for i, n in zip(live, counts):
                r_, k_, v_, a_ = [x[at[i]:at[i] + n].reshape(n, HD) for x in seqs[i]]
                rkv[o:o + n, 2:2 + HD], rkv[o:o + n, 3 + HD:3 + 2 * HD], rkv[o:o + n, 5 + 2 * HD:5 + 3 * HD] = v_, r_, k_
                a[o:o + n] = a_
                o += n
            step = _Step()
            step.n_seqs, step.n_rows = len(live), T
            step.cu_seqlens = dev(np.concatenate([[0], np.cumsum(counts)]), torch.int32)
            step.slots = dev([slots[i] for i in live], torch.int32)
            step.start_pos = dev([at[i] for i in live], torch.int32)
            y = torch.empty((T, HD), device="cuda")
            ops.wkv_scan(dev(rkv), 3 + HD, 5 + 2 * HD, 2, dev(a), dev(u), state, step, H, d, y)
            torch.cuda.synchronize()
            ops.check_errors()
            y = y.cpu().numpy().astype(np.float64)
            o = 0
            for i, n in zip(live, counts):
                outs[i].append(y[o:o + n])
                at[i] += n
                o += n
        return [np.concatenate(x).reshape(-1, H, d) for x in outs]

    want_of = lambda seq: _wkv_plain(seq[0], seq[1], seq[2], np.exp(-np.exp(seq[3])), u)
    seqs = [make(n, 20 + i) for i, n in enumerate(lens)]
    got = run(seqs, [2, 0], portions)
    for i, seq in enumerate(seqs):
        want = want_of(seq)
        err = np.abs(got[i] - want).max()
        assert err <= 3e-5 * np.abs(want).max(), f"sequence {i}: error {err:.3e} of {np.abs(want).max():.3e}"
        assert np.abs(want[-1] / 2.0 - seq[2][3]).max() < 0.5 * np.abs(seq[2][3]).max()      # far on, still token 3's value
        # the bonus shows: token 3's own read-out is u times what the state alone would give
        assert np.abs(want[3] - _wkv_plain(seq[0][:4], seq[1][:4], seq[2][:4], np.exp(-np.exp(seq[3][:4])), np.ones((H, d)))[3]).max() > 0.1
    third = make(40, 33)
    got3, want3 = run([third], [0], [[1, 1, 30, 8]])[0], want_of(third)
    assert np.abs(got3 - want3).max() <= 3e-5 * np.abs(want3).max(), "a slot used again"


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("H,d,R", [(3, 8, 5), (2, 64, 16), (1, 72, 7), (5, 16, 8)])
def test_wkv_mixer_with_its_mixes_gate_and_norm(dtype, H, d, R):
    """The whole mixer: five mixes with the previous token's input (kept across steps, zeros at position 0), the decay's
    two small products, the scan, each head divided by its root mean square, the weight, the gate, the output."""
    g = np.random.default_rng(13)
    D, HD = (128 if d == 64 else 44), H * d        # 128: rows of 16-byte multiples, which the tiled product of prompts takes
    names = {k: "w." + k for k in ("r", "k", "v", "g", "w1", "w2", "w0", "u", "norm", "o")}
    names.update({"mu_" + s: "w.mu." + s for s in ("r", "k", "v", "g", "w")})
    W = {"w." + s: draw(g, (HD, D), 0.25, dtype) for s in ("r", "k", "v", "g")}
    W.update({"w.mu." + s: plain.bf16_round(g.random(D)) for s in ("r", "k", "v", "g", "w")})
    W.update({"w.w1": draw(g, (R, D), 0.3, dtype), "w.w2": draw(g, (HD, R), 0.5, dtype), "w.w0": draw(g, (HD,), 1.0, dtype) - 2.0,
              "w.u": draw(g, (H, d), 1.0, dtype), "w.norm": 1.0 + draw(g, (HD,), 0.2, dtype), "w.o": draw(g, (D, HD), 0.2, dtype)})
    part = PartSpec("mixer", "wkv", dict(hidden=D, n_heads=H, head_dim=d, eps=1e-5, names=names, decay_rank=R)).build()
    part.bind({k: torch.tensor(v, dtype=DT[dtype] if v.ndim == 2 and "u" != k[-1] else torch.float32) for k, v in W.items()},
              DT[dtype], "cuda")
    rows = [g.standard_normal((n + DECODED, D)).astype(np.float32).astype(np.float64) for n in LENS]

    def forward(x, step, views):
        out = torch.zeros((x.shape[0], D), dtype=torch.float32, device="cuda")
        part.forward(x, step, views[0], out, accumulate=False)
        return out
    got = run_steps(forward, part.cache_requests(), rows, dtype, torch.float32)
    want = [plain.wkv_mixer(x, W, "w.", dict(heads=H, dim=d), 1e-5, rnd_of(dtype)) for x in rows]
    compare(got, want, dtype, "wkv mixer", tol=3e-5 if dtype == "float32" else 4e-2)


# ---- the norm that joins two mixers, the dense feed-forward ----------------------------------------------------------------
@pytest.mark.parametrize("n,D", [(2, 44), (2, 256), (3, 64)])
def test_mixers_joined_by_their_own_norms(n, D):
    """Every summand divided by its OWN root mean square (summands of very different sizes: a shared root mean square
    would let the largest one drown the others), then the layer's norm on the mean."""
    g = np.random.default_rng(14)
    T = 37
    parts = g.standard_normal((T, n, D)) * np.array([0.01, 30.0, 1.0][:n])[None, :, None]
    w, outer, res = 1.0 + g.standard_normal((n, D)) * 0.2, 1.0 + g.standard_normal(D) * 0.2, g.standard_normal((T, D))
    f32 = lambda a: np.asarray(a, dtype=np.float32).astype(np.float64)
    parts, w, outer, res = f32(parts), f32(w), f32(outer), f32(res)
    part = PartSpec("norm", "rmsnorm_mean", dict(width=D, eps=1e-6, weight_names=tuple(f"j{i}" for i in range(n)))).build()
    part.bind({f"j{i}": torch.tensor(w[i], dtype=torch.float32) for i in range(n)}, torch.float32, "cuda")
    out_norm = PartSpec("norm", "rmsnorm", dict(width=D, eps=1e-6, weight_name="o")).build()
    out_norm.bind({"o": torch.tensor(outer, dtype=torch.float32)}, torch.float32, "cuda")
    y = sum(plain.rms_norm(parts[:, i], w[i], 1e-6) for i in range(n)) / n
    r = dev(res)
    part.add_joined(dev(parts), r, out_norm)
    want = res + plain.rms_norm(y, outer, 1e-6)
    assert np.abs(r.cpu().numpy() - want).max() <= 1e-5 * np.abs(want).max()
    r = dev(res)
    part.add_joined(dev(parts), r)
    assert np.abs(r.cpu().numpy() - (res + y)).max() <= 1e-5 * np.abs(res + y).max()


@pytest.mark.parametrize("T", [5, 600])
@pytest.mark.parametrize("n,D", [(2, 256), (2, 50), (3, 64), (1, 1536)])
@pytest.mark.parametrize("copy_dtype", ["bfloat16", "float32"])
def test_adding_norms_leave_the_stream_in_a_second_type(T, n, D, copy_dtype):
    """The kernels that add a normed sublayer result into the 32-bit stream also write the new rows in the type of the
    next sublayer's input: the join of the mixers and the plain output norm, few rows and many, widths with and
    without 16-byte rows."""
    g = np.random.default_rng(15)
    f32 = lambda a: np.asarray(a, dtype=np.float32).astype(np.float64)
    parts, res = f32(g.standard_normal((T, n, D))), f32(g.standard_normal((T, D)))
    w, outer = f32(1.0 + g.standard_normal((n, D)) * 0.2), f32(1.0 + g.standard_normal(D) * 0.2)
    for joined in (True, False):
        r, copy = dev(res), torch.full((T, D), 7.0, dtype=DT[copy_dtype], device="cuda")
        if joined:
            ops.rmsnorm_mean_add(dev(parts), dev(w), 1e-6, 1.0 / n, r, dev(outer), 1e-6, copy=copy)
            want = res + plain.rms_norm(sum(plain.rms_norm(parts[:, i], w[i], 1e-6) for i in range(n)) / n, outer, 1e-6)
        else:
            ops.rmsnorm_add(dev(parts), dev(outer), 1e-6, r, copy=copy)
            want = res + plain.rms_norm(parts.sum(axis=1), outer, 1e-6)
        assert np.abs(r.cpu().numpy() - want).max() <= 1e-5 * np.abs(want).max()
        assert torch.equal(copy, r.to(DT[copy_dtype]))          # the copy is the stream itself, rounded once


@pytest.mark.parametrize("dtype,D,F", [("bfloat16", 256, 512), ("bfloat16", 64, 40), ("bfloat16", 44, 28), ("float32", 64, 40)])
def test_dense_feed_forward_with_both_clamps_at_work(dtype, D, F):
    g = np.random.default_rng(15)
    limit = 0.9
    W = {"f.gate": draw(g, (F, D), 0.2, dtype), "f.up": draw(g, (F, D), 0.2, dtype), "f.down": draw(g, (D, F), 0.1, dtype)}
    part = PartSpec("feed_forward", "swiglu", dict(hidden=D, intermediate=F, prefix="f.", act="swish_clamped", limit=limit,
                                                   alpha=plain.SWISH_ALPHA, names=dict(gate="gate", up="up", down="down"))).build()
    part.bind({k: torch.tensor(v, dtype=DT[dtype]) for k, v in W.items()}, DT[dtype], "cuda")
    for T in (1, 20, 100, 300):
        x = draw(g, (T, D), 1.0, dtype)
        out = torch.zeros((T, D), dtype=torch.float32, device="cuda")
        part.forward(dev(x, DT[dtype]), out, accumulate=False)
        want = plain.dense_ff(x, W, "f.", dict(limit=limit), rnd_of(dtype))
        err = np.abs(out.cpu().numpy() - want).max()
        assert err <= (3e-5 if dtype == "float32" else 2e-2) * np.abs(want).max(), f"T={T}: {err:.3e} of {np.abs(want).max():.3e}"
        gate, up = x @ W["f.gate"].T, x @ W["f.up"].T
        if T >= 100:
            assert (gate > limit).mean() > 0.1 and (up > limit).mean() > 0.1 and (up < -limit).mean() > 0.1


# ---- routing over all outputs with a correction, identity outputs, experts without a gate -----------------------------------
def test_routing_where_the_correction_changes_the_choice_but_not_the_weight():
    g = np.random.default_rng(16)
    for E, ident, top in ((4, 4, 2), (3, 0, 3), (1, 2, 1), (6, 1, 7), (40, 5, 6)):
        T, n = 60, E + ident
        z = g.standard_normal((T, n + 1)).astype(np.float32)            # (one more column than outputs: it takes no part)
        corr = (g.standard_normal(n) * 0.5).astype(np.float32)
        corr[n - 1] = 0.9                                               # the last output is chosen far more often than its score earns
        ids, wts, order, offsets, tile_off, _ = ops.moe_route(dev(z), n, top, 32, "softmax_all", dev(corr), ident)
        torch.cuda.synchronize()
        ids, wts = ids.cpu().numpy().reshape(T, top), wts.cpu().numpy().reshape(T, top)
        W = {"m.router": np.eye(n), "m.correction": corr.astype(np.float64)}
        mlp = dict(router=dict(experts=E, identity=ident, top=top))
        want_ids, want_w = plain.route(z[:, :n].astype(np.float64), W, "m.", mlp)
        changed = 0
        for t in range(T):
            assert list(ids[t]) == list(want_ids[t]), f"E={E}+{ident} top={top} token {t}"
            assert np.abs(wts[t] - want_w[t]).max() <= 1e-6
            changed += set(want_ids[t]) != set(np.argsort(-z[t, :n], kind="stable")[:top])
        assert top == n or changed > 0
        if top < n:
            assert wts.sum(-1).max() < 1.0 - 1e-3                       # the weights are the scores: not renormalised
        order, offsets = order.cpu().numpy(), offsets.cpu().numpy()
        flat = ids.reshape(-1)
        for e in range(E):                                              # the lists of the experts that have weights
            assert all(flat[i] == e for i in order[offsets[e]:offsets[e + 1]])
            assert offsets[e + 1] - offsets[e] == (flat == e).sum()


@pytest.mark.parametrize("dtype,D,F", [("float32", 44, 20), ("bfloat16", 64, 24), ("bfloat16", 44, 12), ("bfloat16", 128, 72)])
@pytest.mark.parametrize("E,ident,top", [(4, 4, 2), (1, 0, 1), (2, 3, 5), (6, 1, 3)])
def test_experts_without_gates_beside_identity_outputs(dtype, D, F, E, ident, top):
    """The part as a layer runs it: the input in the activation type for the products, the 32-bit rows for the outputs
    that return their input."""
    g = np.random.default_rng(17)
    n = E + ident
    W = {"m.router": draw(g, (n, D), 0.3, dtype), "m.correction": draw(g, (n,), 0.3, dtype)}
    for e in range(E):
        W[f"m.e{e}.up"], W[f"m.e{e}.down"] = draw(g, (F, D), 0.3, dtype), draw(g, (D, F), 0.3, dtype)
    part = PartSpec("feed_forward", "moe", dict(
        hidden=D, n_experts=E, top=top, expert_ff=F, router_name="m.router", choice_bias_name="m.correction", n_identity=ident,
        expert_names={k: "m.e{e}." + k for k in ("up", "down")}, weights="softmax_all", weight_on="output", act="relu_squared")).build()
    part.bind({k: torch.tensor(v, dtype=DT[dtype] if v.ndim == 2 else torch.float32) for k, v in W.items()}, DT[dtype], "cuda")
    mlp = dict(router=dict(experts=E, identity=ident, top=top))
    for T in (1, 33, 150):
        x = g.standard_normal((T, D)).astype(np.float32).astype(np.float64)
        out = torch.zeros((T, D), dtype=torch.float32, device="cuda")
        part.forward(dev(x).to(DT[dtype]), out, accumulate=False, stream=dev(x))
        torch.cuda.synchronize()
        ops.check_errors()
        want = plain.expert_ff(x, W, "m.", mlp, rnd_of(dtype))
        err = np.abs(out.cpu().numpy() - want).max()
        assert err <= (3e-5 if dtype == "float32" else 2e-2) * np.abs(want).max(), f"T={T}: {err:.3e} of {np.abs(want).max():.3e}"
