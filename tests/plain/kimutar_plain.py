"""Plain, slow Kimutar forward pass: whole sequences, no cache, one function per mechanism.

The oracle of the Kimutar tests.  It shares no code with the product package: it takes the configuration as a plain
``dict`` (the keys of config.json) and the weights as a ``dict`` of numpy arrays keyed by tensor name, and computes
everything in float64 except the rotary angle, which is the float32 product of position and frequency.  Attention walks
query by query over keys that are picked by the mask's own definition, the delta rule walks token by token with the
state as a matrix, and every expert is applied to one token at a time.

Notation: D model width, T tokens of one sequence.  A layer is  x <- x + (mixer(n1(x)) + ff(n2(x)))  with
n(x) = (x - mean(x)) / sqrt(var(x) + eps) * w.  `rnd` models a bfloat16 engine: it is applied where such an engine must
round (inputs of matrix products, cached rows); the identity gives exact arithmetic.
"""
from __future__ import annotations

import math

import numpy as np

UNIT_EPS = 1e-6          # under the root when the delta rule's queries and keys are made unit vectors
WEIGHT_SUM_EPS = 1e-20   # added to the sum of the chosen experts' scores


def _same(x):
    return x


def bf16_round(x):
    """Nearest bfloat16 (ties to even) of every element, returned as float64."""
    x32 = np.ascontiguousarray(x, dtype=np.float32)
    bits = x32.view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32).astype(np.float64).reshape(np.shape(x))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def unit_rms(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def layer_norm(x, w, eps):
    d = x - x.mean(-1, keepdims=True)
    return d / np.sqrt((d * d).mean(-1, keepdims=True) + eps) * w


# ---- rotations ----------------------------------------------------------------------------------------------------
def plain_frequencies(base, dims):
    return np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)


def ramp_frequencies(base, dims, sc):
    """Frequencies blended between f and f / factor along a linear ramp over the pair index, and the factor by which
    cosines and sines grow: sc = {factor, original, fast, slow}."""
    f = plain_frequencies(base, dims)

    def index_of(turns):      # the (real-valued) pair index whose wave makes `turns` turns over `original` positions
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(sc["fast"])), 0)
    hi = min(math.ceil(index_of(sc["slow"])), dims - 1)
    out = np.empty_like(f)
    for i in range(dims // 2):
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out[i] = f[i] / sc["factor"] * r + f[i] * (1.0 - r)
    return out, 0.1 * math.log(sc["factor"]) + 1.0


def band_frequencies(base, dims, sc):
    """Frequencies kept where the wave is short, divided by factor where it is long, blended between:
    sc = {factor, low, high, original}."""
    f = plain_frequencies(base, dims)
    out = np.empty_like(f)
    for i, fi in enumerate(f):
        wave = 2.0 * math.pi / fi
        if wave < sc["original"] / sc["high"]:
            out[i] = fi
        elif wave > sc["original"] / sc["low"]:
            out[i] = fi / sc["factor"]
        else:
            s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
            out[i] = (1.0 - s) * fi / sc["factor"] + s * fi
    return out


def _angles(pos, freq):
    return (np.asarray(pos, dtype=np.float32)[:, None] * freq.astype(np.float32)[None, :]).astype(np.float64)   # a 32-bit product


def rotate_halves(x, pos, freq, grow=1.0):
    """x [T, heads, d]: dimension i of the first 2 * len(freq) is paired with i + len(freq)."""
    x = x.copy()
    n = len(freq)
    if n == 0:
        return x
    ang = _angles(pos, freq)
    cs, sn = np.cos(ang)[:, None, :] * grow, np.sin(ang)[:, None, :] * grow
    u, v = x[..., :n].copy(), x[..., n:2 * n].copy()
    x[..., :n] = u * cs - v * sn
    x[..., n:2 * n] = v * cs + u * sn
    return x


def rotate_neighbours(x, pos, freq):
    """x [T, heads, d]: pairs (2i, 2i+1) of the first 2 * len(freq) dimensions."""
    x = x.copy()
    n = len(freq)
    if n == 0:
        return x
    ang = _angles(pos, freq)
    cs, sn = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    u, v = x[..., 0:2 * n:2].copy(), x[..., 1:2 * n:2].copy()
    x[..., 0:2 * n:2] = u * cs - v * sn
    x[..., 1:2 * n:2] = v * cs + u * sn
    return x


def _frequencies(rot, scaled):
    """(frequencies, amplitude of cosines and sines) of a mixer's 'rot': none rotated, plain, or stretched by `scaled`."""
    if not rot["dims"]:
        return np.zeros(0), 1.0
    if rot.get("scaling") is None:
        return plain_frequencies(rot["base"], rot["dims"]), 1.0
    return scaled(rot["base"], rot["dims"], rot["scaling"])


# ---- attention ------------------------------------------------------------------------------------------------------
def visible(i, j, size=None, keep_first=0):
    """Whether query position i sees key position j: causal, and with a window only the last `size` positions and the
    first `keep_first` of the sequence."""
    if j > i:
        return False
    return size is None or i - j < size or j < keep_first


def attend(q, k, v, scale, size=None, keep_first=0, sink=None):
    """One head: q [T, d], k [T, d], v [T, dv] -> [T, dv].  sink: a number whose exponential joins the denominator."""
    T = q.shape[0]
    out = np.zeros((T, v.shape[1]))
    for i in range(T):
        js = [j for j in range(i + 1) if visible(i, j, size, keep_first)]
        s = (k[js] @ q[i]) * scale
        top = s.max() if sink is None else max(s.max(), sink)
        e = np.exp(s - top)
        den = e.sum() + (0.0 if sink is None else math.exp(sink - top))
        out[i] = (e / den) @ v[js]
    return out


def difference_attention(h, W, p, m, eps, rnd=_same):
    """Two score maps per head over the same values; the second is subtracted, times lambda."""
    T = h.shape[0]
    H, G, d, dv, diff = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["diff"]
    pos = np.arange(T)
    freq, grow = _frequencies(m["rot"], ramp_frequencies)
    q = (h @ W[p + "q"].T).reshape(T, H * 2, d)
    k = (h @ W[p + "k"].T).reshape(T, G * 2, d)
    v = rnd(h @ W[p + "v"].T).reshape(T, G, dv)
    q = rnd(rotate_halves(unit_rms(q, eps) * W[p + "q.norm"], pos, freq, grow))
    k = rnd(rotate_halves(unit_rms(k, eps) * W[p + "k.norm"], pos, freq, grow))
    lam = math.exp(float(W[p + "lq1"] @ W[p + "lk1"])) - math.exp(float(W[p + "lq2"] @ W[p + "lk2"])) + diff
    out = np.zeros((T, H, dv))
    for hh in range(H):
        g = hh // (H // G)
        a1 = attend(q[:, 2 * hh], k[:, 2 * g], v[:, g], m["scale"])
        a2 = attend(q[:, 2 * hh + 1], k[:, 2 * g + 1], v[:, g], m["scale"])
        out[:, hh] = unit_rms(a1 - lam * a2, eps) * (1.0 - diff)
    return rnd(out.reshape(T, H * dv)) @ W[p + "o"].T


def window_attention(h, W, p, m, eps, rnd=_same):
    """Biased projections, normed heads, neighbour rotation, a window that keeps the first tokens, a sink per head."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(T)
    freq, _ = _frequencies(m["rot"], lambda base, dims, sc: (band_frequencies(base, dims, sc), 1.0))
    mask = m.get("mask") or {}
    q = (h @ W[p + "q"].T + W[p + "q.b"]).reshape(T, H, d)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).reshape(T, G, d)
    v = rnd(h @ W[p + "v"].T + W[p + "v.b"]).reshape(T, G, dv)
    q = rnd(rotate_neighbours(unit_rms(q, eps) * W[p + "q.norm"], pos, freq))
    k = rnd(rotate_neighbours(unit_rms(k, eps) * W[p + "k.norm"], pos, freq))
    out = np.zeros((T, H, dv))
    for hh in range(H):
        g = hh // (H // G)
        out[:, hh] = attend(q[:, hh], k[:, g], v[:, g], m["scale"], mask.get("size"), mask.get("keep_first", 0), float(W[p + "sink"][hh]))
    return rnd(out.reshape(T, H * dv)) @ W[p + "o"].T + W[p + "o.b"]


# ---- the delta rule with a decay per key channel ----------------------------------------------------------------
def short_conv(x, w):
    """x [T, C], w [C, taps]: the last tap weighs the current row, zeros stand before the first."""
    T, C = x.shape
    taps = w.shape[1]
    out = np.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            src = t - (taps - 1) + j
            if src >= 0:
                out[t] += x[src] * w[:, j]
    return out


def delta_scan(q, k, v, beta, decay):
    """One head.  q, k [T, dk] (k a unit vector), v [T, dv], beta [T], decay [T, dk] -> read-outs [T, dv].
    S [dk, dv]:  S <- diag(decay) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q."""
    T, dk = k.shape
    S = np.zeros((dk, v.shape[1]))
    o = np.zeros((T, v.shape[1]))
    for t in range(T):
        S = decay[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + np.outer(k[t], u)
        o[t] = S.T @ q[t]
    return o


def channel_delta(h, W, p, m, eps, rnd=_same):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ W[p + "q"].T, W[p + "q.conv"])).reshape(T, G, dk)
    k = silu(short_conv(h @ W[p + "k"].T, W[p + "k.conv"])).reshape(T, G, dk)
    v = silu(short_conv(h @ W[p + "v"].T, W[p + "v.conv"])).reshape(T, H, dv)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + UNIT_EPS) * dk ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + UNIT_EPS)
    beta = sigmoid(h @ W[p + "b"].T)
    a = rnd(h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]
    decay = np.exp(-np.exp(W[p + "A_log"])[None, :, None] * softplus(a).reshape(T, H, dk))
    gate = sigmoid(rnd(h @ W[p + "g1"].T) @ W[p + "g2"].T)
    o = np.zeros((T, H, dv))
    for hh in range(H):
        g = hh // (H // G)
        o[:, hh] = delta_scan(q[:, g], k[:, g], v[:, hh], beta[:, hh], decay[:, hh])
    o = unit_rms(o, eps) * W[p + "norm"][None, None, :]
    return rnd(o.reshape(T, H * dv) * gate) @ W[p + "o"].T


# ---- feed-forward ----------------------------------------------------------------------------------------------------
def dense(h, W, p, rnd=_same):
    return rnd(np.maximum(h @ W[p + "up"].T, 0.0) ** 2) @ W[p + "down"].T


def gated_expert(x, W, p, rnd=_same):
    return W[p + "down"] @ rnd(silu(W[p + "gate"] @ x) * (W[p + "up"] @ x))


def route(z, correction, top, scale):
    """z [E] logits -> (chosen experts, their weights): scores are the softmax over all experts; the choice goes by score
    plus correction (lowest index first on ties), the weights by the scores alone, normed to sum to `scale`."""
    e = np.exp(z - z.max())
    s = e / e.sum()
    order = sorted(range(len(z)), key=lambda i: (-(s[i] + correction[i]), i))[:top]
    w = np.array([s[i] for i in order])
    return order, w / (w.sum() + WEIGHT_SUM_EPS) * scale


def moe(h, W, p, mlp, rnd=_same):
    r = mlp["router"]
    z = h @ W[p + "router"].T
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(*route(z[t], W[p + "correction"], r["top"], r["scale"])):
            out[t] += w * gated_expert(h[t], W, f"{p}e{e}.", rnd)
        if mlp.get("shared") is not None:
            out[t] += sigmoid(float(W[p + "shared.sg"][0] @ h[t])) * gated_expert(h[t], W, p + "shared.", rnd)
    return out


# ---- the model ------------------------------------------------------------------------------------------------------------
def run_order(cfg):
    """[(layer, pass or None)]: the looped range repeats, every pass after a learned vector has been added."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg, W, tokens, rnd=_same, layers_out=None):
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)].astype(np.float64)
    for i, first_of_pass in run_order(cfg):
        layer, L = cfg["layers"][i], f"l{i}."
        if first_of_pass is not None:
            x = x + W["loop.step"][first_of_pass]
        h = rnd(layer_norm(x, W[L + "norm1"], eps))
        m, kind = layer["mixer"], layer["type"]
        if kind == "attention":
            y = difference_attention(h, W, L + "mix.", m, eps, rnd)
        elif kind == "attention_2":
            y = window_attention(h, W, L + "mix.", m, eps, rnd)
        elif kind == "channel_delta":
            y = channel_delta(h, W, L + "mix.", m, eps, rnd)
        else:
            raise ValueError(kind)
        mlp = layer.get("mlp")
        if mlp is not None:
            h2 = rnd(layer_norm(x, W[L + "norm2"], eps))
            y = y + (dense(h2, W, L + "mlp.", rnd) if mlp["kind"] == "dense" else moe(h2, W, L + "mlp.", mlp, rnd))
        x = x + y
        if layers_out is not None:
            layers_out.append(x.copy())
    return rnd(layer_norm(x, W["final.norm"], eps)) @ W["head"].T
