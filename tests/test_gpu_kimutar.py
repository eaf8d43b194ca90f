"""Kimutar on the GPU against the plain implementation (tests/plain/kimutar_plain.py), in 32-bit and in bfloat16: whole
prompts and the first tokens of a sequence; prompts then tokens one by one across page borders and past every window;
prompts in portions down to two tokens; unequal batches whose shorter requests end earlier, with slots and pages freed and
used again; long decoding; greedy generation through the entry point and its scheduler; configurations drawn at random.

float32 is held to the exact plain result (what differs is the order of sums).  In bfloat16 the engine is held to three
times the distance that the plain model of a bfloat16 run has from exact arithmetic, row by row in root mean square; a
cache, state or batching fault moves logits by about their own size.  Routing is a discrete choice that rounding noise
can tip, so the bfloat16 runs use the same layers with every router output chosen (weights and sums are then continuous);
the choice itself is tested in 32-bit and at the kernel.
"""
import copy

import numpy as np
import pytest

import tinyllama_c_b200 as tlc
from tinyllama_c_b200.engine import StepEntry

import configs
from helpers import make_model_dir, random_tokens, read_config, read_weights, release_all
from plain import kimutar_plain as plain

pytestmark = pytest.mark.gpu


def all_outputs(cfg: dict) -> dict:
    cfg = copy.deepcopy(cfg)
    for layer in cfg["layers"]:
        if layer.get("mlp") and layer["mlp"]["kind"] == "moe":
            r = layer["mlp"]["router"]
            r["top"] = r["experts"]
    return cfg


CONFIGS = {("KA", "float32"): configs.KIMUTAR_A, ("KB", "float32"): configs.KIMUTAR_B,
           ("KA", "bfloat16"): all_outputs(configs.KIMUTAR_A), ("KB", "bfloat16"): all_outputs(configs.KIMUTAR_B)}
CASES = sorted(CONFIGS)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("kimutar")
    return {key: make_model_dir(root, cfg, seed=80 + i, std=0.2, name="-".join(key)) for i, (key, cfg) in enumerate(sorted(CONFIGS.items()))}


@pytest.fixture(scope="module")
def engines(folders):
    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            made[(name, dtype)] = tlc.LLM(folders[(name, dtype)], dtype=dtype, max_tokens=64 * 20, max_seqs=5)
        release_all(made[(name, dtype)])
        return made[(name, dtype)]
    return get


_plain_cache = {}


def plain_logits(folder, toks, rnd=plain._same):
    key = (folder, tuple(toks), rnd is plain._same)
    if key not in _plain_cache:
        _plain_cache[key] = plain.forward(read_config(folder), read_weights(folder), list(toks), rnd=rnd)
    return _plain_cache[key]


def check(got, folder, toks, rows, dtype, what):
    """got [n, V]: the engine's logits at positions `rows` of request `toks`."""
    exact = plain_logits(folder, toks)[rows]
    got = np.asarray(got, dtype=np.float64)
    assert got.shape == exact.shape, what
    if dtype == "float32":
        scale = np.abs(plain_logits(folder, toks)).max()
        err = np.abs(got - exact)
        assert err.max() <= 1e-4 * scale, f"{what}: max error {err.max():.3e} of {scale:.3e} at row {rows[int(err.max(1).argmax())]}"
        assert err.mean() <= 2e-5 * scale, f"{what}: mean error {err.mean():.3e} of {scale:.3e}"
        return
    model = plain_logits(folder, toks, plain.bf16_round)
    noise = np.sqrt(((model - plain_logits(folder, toks)) ** 2).mean(axis=1)).max()
    err = np.sqrt(((got - exact) ** 2).mean(axis=1))
    assert err.max() <= 3.0 * noise, f"{what}: row error {err.max():.3e} at row {rows[int(err.argmax())]}, rounding noise {noise:.3e}"


def run_whole(llm, toks, want=None):
    want = list(range(len(toks))) if want is None else want
    s = llm.cache.acquire()
    out = llm.step([StepEntry(s, toks, want)]).cpu().numpy()
    llm.cache.release(s)
    return out


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_prompts_and_first_tokens(engines, folders, name, dtype):
    llm, folder = engines(name, dtype), folders[(name, dtype)]
    vocab = read_config(folder)["vocab"]
    for i, n in enumerate([1, 2, 3, 65, 150, 200]):
        toks = random_tokens(vocab, n, 700 + i)
        check(run_whole(llm, toks), folder, toks, list(range(n)), dtype, f"{name} whole prompt of {n}")
    llm.cache.check()


@pytest.mark.parametrize("name,dtype", CASES)
def test_prompt_then_tokens_one_by_one_across_page_borders(engines, folders, name, dtype):
    llm, folder = engines(name, dtype), folders[(name, dtype)]
    toks = random_tokens(read_config(folder)["vocab"], 180, 711)
    for cut in (1, 50, 63, 129):
        s = llm.cache.acquire()
        rows = [llm.step([StepEntry(s, toks[:cut], [cut - 1])]).cpu().numpy()[0]]
        for p in range(cut, len(toks)):
            rows.append(llm.step([StepEntry(s, [toks[p]], [0])]).cpu().numpy()[0])
        llm.cache.release(s)
        check(np.stack(rows), folder, toks, list(range(cut - 1, len(toks))), dtype, f"{name} prompt of {cut}, then one by one")
    llm.cache.check()


@pytest.mark.parametrize("name,dtype", CASES)
def test_prompt_in_portions(engines, folders, name, dtype):
    llm, folder = engines(name, dtype), folders[(name, dtype)]
    toks = random_tokens(read_config(folder)["vocab"], 200, 712)
    for sizes in ([2] * 100, [64, 64, 64, 8], [63, 2, 1, 70, 64], [3, 129, 5, 63], [130, 70]):
        assert sum(sizes) == len(toks)
        s, at, rows = llm.cache.acquire(), 0, []
        for n in sizes:
            rows.append(llm.step([StepEntry(s, toks[at:at + n], list(range(n)))]).cpu().numpy())
            at += n
        llm.cache.release(s)
        check(np.concatenate(rows), folder, toks, list(range(len(toks))), dtype, f"{name} in portions {sizes[:5]}")


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_batches_with_slots_and_pages_used_again(engines, folders, name, dtype):
    """Three batches one after another in a cache of five slots: requests of unequal length start together, go on one
    token at a time, the shorter ones end earlier and their slots, pages and recurrent states go to the next batch (a
    state that is not reset at position 0 shows there)."""
    llm, folder = engines(name, dtype), folders[(name, dtype)]
    vocab = read_config(folder)["vocab"]
    for wave in range(3):
        lens = [[1, 70, 140], [66, 3, 129, 20], [150, 64]][wave]
        tail = [6, 3, 9, 1][:len(lens)]
        reqs = [random_tokens(vocab, n + k, 800 + 10 * wave + i) for i, (n, k) in enumerate(zip(lens, tail))]
        slots = [llm.cache.acquire() for _ in reqs]
        got = [[] for _ in reqs]
        out = llm.step([StepEntry(s, q[:n], [n - 1]) for s, q, n in zip(slots, reqs, lens)]).cpu().numpy()
        for i in range(len(reqs)):
            got[i].append(out[i])
        at = list(lens)
        live = list(range(len(reqs)))
        while live:
            live = [i for i in live if at[i] < len(reqs[i])]
            if not live:
                break
            out = llm.step([StepEntry(slots[i], [reqs[i][at[i]]], [0]) for i in live]).cpu().numpy()
            for j, i in enumerate(live):
                got[i].append(out[j])
                at[i] += 1
                if at[i] == len(reqs[i]):
                    llm.cache.release(slots[i])
                    slots[i] = None
        for i, q in enumerate(reqs):
            if slots[i] is not None:
                llm.cache.release(slots[i])
            check(np.stack(got[i]), folder, q, list(range(lens[i] - 1, len(q))), dtype, f"{name} batch {wave} request {i}")
        llm.cache.check()


@pytest.mark.parametrize("name", ["KA", "KB"])
def test_long_decoding(engines, folders, name):
    llm, folder = engines(name, "float32"), folders[(name, "float32")]
    toks = random_tokens(read_config(folder)["vocab"], 230, 713)
    s = llm.cache.acquire()
    rows = [llm.step([StepEntry(s, toks[:4], [3])]).cpu().numpy()[0]]
    for p in range(4, len(toks)):
        rows.append(llm.step([StepEntry(s, [toks[p]], [0])]).cpu().numpy()[0])
    llm.cache.release(s)
    check(np.stack(rows), folder, toks, list(range(3, len(toks))), "float32", f"{name} 226 tokens one by one")
    llm.cache.check()


@pytest.mark.parametrize("name,dtype", [("KA", "float32"), ("KB", "float32"), ("KB", "bfloat16")])
def test_greedy_generation_through_the_entry_point(engines, folders, name, dtype):
    """LLM.generate (scheduler, batches, captured one-token steps) against greedy decoding with the plain implementation.
    A step whose two best logits lie closer than the run's rounding could tell apart ends the comparison there."""
    llm, folder = engines(name, dtype), folders[(name, dtype)]
    cfg, W = read_config(folder), read_weights(folder)
    prompts = [random_tokens(cfg["vocab"], n, 900 + i) for i, n in enumerate([5, 70, 1, 33])]
    n_new = 12
    results = llm.generate(prompts, tlc.GREEDY, max_new_tokens=n_new, stop_ids=(), ignore_eos=True)
    llm.cache.check()
    margin = 1e-3 if dtype == "float32" else 0.25
    for prompt, res in zip(prompts, results):
        got = list(res.tokens)
        assert len(got) == n_new
        seq = list(prompt)
        for k in range(n_new):
            row = plain.forward(cfg, W, seq)[-1]
            best = np.sort(row)[-2:]
            if best[1] - best[0] < margin * np.abs(row).max():
                break
            assert got[k] == int(np.argmax(row)), f"{name} {dtype}: token {k} of a prompt of {len(prompt)}"
            seq.append(got[k])


@pytest.mark.parametrize("seed", list(range(1, 11)))
def test_configurations_drawn_at_random(tmp_path, seed):
    """Layer order, kinds, the repeated range, sizes, rotated dimensions, scalings, windows, taps, experts and constants drawn from a seed: a prompt
    in two portions (the second starts inside a page), then tokens one by one, in 32-bit against the exact plain result and
    in bfloat16 (every router output chosen) within three times the plain bfloat16 model's distance from it."""
    base = configs.kimutar_random(seed)
    g = np.random.default_rng(3000 + seed)
    n, tail = int(g.choice([40, 70, 131])), 10
    toks = g.integers(0, base["vocab"], n + tail).tolist()
    for dtype, cfg in (("float32", base), ("bfloat16", all_outputs(base))):
        folder = make_model_dir(tmp_path, cfg, seed=seed, std=0.2, name=dtype)
        llm = tlc.LLM(folder, dtype=dtype, max_tokens=64 * 6, max_seqs=2)
        s, cut = llm.cache.acquire(), n // 3
        rows = [llm.step([StepEntry(s, toks[:cut], list(range(cut)))]).cpu().numpy(),
                llm.step([StepEntry(s, toks[cut:n], list(range(n - cut)))]).cpu().numpy()]
        for p in range(n, n + tail):
            rows.append(llm.step([StepEntry(s, [toks[p]], [0])]).cpu().numpy())
        llm.cache.release(s)
        llm.cache.check()
        check(np.concatenate(rows), folder, toks, list(range(n + tail)), dtype, f"seed {seed} {dtype}")
        del llm
