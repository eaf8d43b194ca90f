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
