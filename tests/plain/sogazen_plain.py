"""Plain, slow Sogazen forward pass: whole sequences, no cache, one function per mechanism.

The oracle of the Sogazen tests.  It shares no code with the product package: it takes the configuration as a plain
``dict`` (the keys of config.json) and the weights as a ``dict`` of numpy arrays keyed by tensor name, and computes
everything in float64 except the rotary angle, which is the float32 product of position and frequency.  Both
recurrences walk token by token, attention builds every row of scores, every expert is applied to one token at a time.

Notation: D model width, T tokens of one sequence, n(y; w) = y / sqrt(mean(y^2) + eps) * w.  A layer is
x <- x + n(mixer(x); norm1), then x <- x + n(ff(x); norm2): the sublayers read the stream itself and the norm sits on
what they return.  `rnd` models a bfloat16 engine: it is applied where such an engine must round (inputs of matrix
products, cached keys); the identity gives exact arithmetic.
"""
from __future__ import annotations

import numpy as np

SWISH_ALPHA = 1.702        # dense feed-forward: g * sigmoid(SWISH_ALPHA * g) * (u + 1)


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


def rms_norm(y, w, eps):
    return y / np.sqrt((y * y).mean(-1, keepdims=True) + eps) * w


# ---- attention whose values are its keys, with a capped score and a sink ---------------------------------------------
def rotate_halves(x, pos, base, dims):
    """x [T, heads, d]: dimension i of the first `dims` pairs with i + dims/2 and the pair turns by
    pos * base^(-2i/dims); the other dimensions stay."""
    half = dims // 2
    inv = (1.0 / np.power(np.float64(base), 2.0 * np.arange(half, dtype=np.float64) / dims)).astype(np.float32)
    ang = (np.asarray(pos, dtype=np.float32)[:, None] * inv[None, :]).astype(np.float64)       # 32-bit product
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def sink_softmax(s):
    """p_j = exp(s_j) / (1 + sum_i exp(s_i)): one more term of score 0 in the denominator, which carries no value."""
    m = max(0.0, float(s.max()))
    e = np.exp(s - m)
    return e / (np.exp(-m) + e.sum())


def capped(s, cap):
    return cap * np.tanh(s / cap)


def key_value_attention(h, W, p, m, eps, pos, rnd=_same):
    """h [T, D].  q = W_q h + b_q, k = W_k h + b_k; the VALUES are k as projected; q and k are then normed over their
    whole width (all heads at once), turned, and scored with a cap; causal; softmax with a sink."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    hr = rnd(h)
    q = hr @ W[p + "q"].T + W[p + "q.b"]
    k = hr @ W[p + "k"].T + W[p + "k.b"]
    v = rnd(k).reshape(T, G, m["vdim"])
    q = rms_norm(q, W[p + "q.norm"], eps).reshape(T, H, d)
    k = rms_norm(k, W[p + "k.norm"], eps).reshape(T, G, d)
    q = rnd(rotate_halves(q, pos, m["rot"]["base"], m["rot"]["dims"]))
    k = rnd(rotate_halves(k, pos, m["rot"]["base"], m["rot"]["dims"]))
    out = np.zeros((T, H, m["vdim"]))
    for i in range(T):
        for hh in range(H):
            g = hh // (H // G)
            s = capped((k[:i + 1, g] @ q[i, hh]) * m["scale"], m["softcap"])
            out[i, hh] = sink_softmax(s) @ v[:i + 1, g]
    return rnd(out.reshape(T, -1)) @ W[p + "o"].T


# ---- the state-space mixer -------------------------------------------------------------------------------------------
def causal_conv(x, w, b):
    """x [T, C], w [C, taps] with the last column on the current token, zeros before the start."""
    T, taps = x.shape[0], w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, x.shape[1])), x], axis=0)
    out = np.tile(b, (T, 1)).astype(np.float64)
    for j in range(taps):
        out += padded[j:j + T] * w[:, j]
    return out


def state_space(h, W, p, m, eps, rnd=_same):
    T = h.shape[0]
    Hs, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = Hs * P
    proj = rnd(h) @ W[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W[p + "conv"], W[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, Hs, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + W[p + "dt_bias"])
    rate = np.exp(W[p + "A_log"])
    y = np.zeros((T, Hs, P))
    S = np.zeros((Hs, N, P))
    for t in range(T):
        for hh in range(Hs):
            g = hh // (Hs // G)
            S[hh] = np.exp(-rate[hh] * dt[t, hh]) * S[hh] + dt[t, hh] * np.outer(B[t, g], x[t, hh])
            y[t, hh] = S[hh].T @ C[t, g] + W[p + "D"][hh] * x[t, hh]
    y = y.reshape(T, inner) * silu(z)                      # the gate first, then the norm in equal parts
    parts = m["norm_groups"]
    y = rms_norm(y.reshape(T, parts, inner // parts), 1.0, eps).reshape(T, inner) * W[p + "norm"]
    return rnd(y) @ W[p + "o"].T


def parallel_mixer(h, W, p, m, eps, pos, rnd=_same):
    a = key_value_attention(h, W, p + "left.", m["left"], eps, pos, rnd)
    b = state_space(h, W, p + "right.", m["right"], eps, rnd)
    return 0.5 * (rms_norm(a, W[p + "left.out"], eps) + rms_norm(b, W[p + "right.out"], eps))


# ---- the mixer with a decaying matrix state and a bonus for the current token ------------------------------------
def wkv_mixer(h, W, p, m, eps, rnd=_same):
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    prev = np.concatenate([np.zeros((1, h.shape[1])), h[:-1]], axis=0)
    mix = lambda s: rnd(h + (prev - h) * W[p + "mu." + s])
    r = (mix("r") @ W[p + "r"].T).reshape(T, H, d)
    k = (mix("k") @ W[p + "k"].T).reshape(T, H, d)
    v = (mix("v") @ W[p + "v"].T).reshape(T, H, d)
    gate = silu(mix("g") @ W[p + "g"].T)
    lora = rnd(np.tanh(mix("w") @ W[p + "w1"].T)) @ W[p + "w2"].T + W[p + "w0"]
    w = np.exp(-np.exp(lora)).reshape(T, H, d)
    u = W[p + "u"]
    o = np.zeros((T, H, d))
    S = np.zeros((H, d, d))                                 # rows: key channels, columns: value channels
    for t in range(T):
        for hh in range(H):
            kv = np.outer(k[t, hh], v[t, hh])
            o[t, hh] = (S[hh] + u[hh][:, None] * kv).T @ r[t, hh]
            S[hh] = w[t, hh][:, None] * S[hh] + kv
    o = rms_norm(o, 1.0, eps).reshape(T, H * d) * W[p + "norm"] * gate
    return rnd(o) @ W[p + "o"].T


# ---- feed-forwards -----------------------------------------------------------------------------------------------------
def dense_ff(h, W, p, mlp, rnd=_same):
    lim = mlp["limit"]
    hr = rnd(h)
    g = np.minimum(hr @ W[p + "gate"].T, lim)
    u = np.clip(hr @ W[p + "up"].T, -lim, lim)
    return rnd(g * sigmoid(SWISH_ALPHA * g) * (u + 1.0)) @ W[p + "down"].T


def route(h, W, p, mlp):
    """(chosen [T, top], weights [T, top]): softmax over ALL router outputs; the choice adds a correction to the scores,
    the weights are the scores themselves."""
    z = h @ W[p + "router"].T
    e = np.exp(z - z.max(-1, keepdims=True))
    s = e / e.sum(-1, keepdims=True)
    order = np.argsort(-(s + W[p + "correction"]), axis=-1, kind="stable")[:, :mlp["router"]["top"]]
    return order, np.take_along_axis(s, order, axis=-1)


def expert_ff(h, W, p, mlp, rnd=_same):
    """The last `identity` router outputs stand for experts that return their input."""
    E = mlp["router"]["experts"]
    hr = rnd(h)
    chosen, weight = route(hr, W, p, mlp)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(chosen[t], weight[t]):
            if e >= E:
                out[t] += s * h[t]
            else:
                a = np.maximum(hr[t] @ W[f"{p}e{e}.up"].T, 0.0) ** 2
                out[t] += s * (rnd(a) @ W[f"{p}e{e}.down"].T)
    return out


# ---- the model -----------------------------------------------------------------------------------------------------------
def forward(cfg, W, tokens, rnd=_same, layers_out=None):
    """Logits [T, vocab] of one sequence; layers_out, a list, receives the stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)].astype(np.float64)
    pos = np.arange(len(tokens))
    for i, layer in enumerate(cfg["layers"]):
        L = f"l{i}."
        if layer["type"] == "parallel":
            y = parallel_mixer(x, W, L + "mix.", layer["mixer"], eps, pos, rnd)
        elif layer["type"] == "wkv":
            y = wkv_mixer(x, W, L + "mix.", layer["mixer"], eps, rnd)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(y, W[L + "norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            y = dense_ff(x, W, L + "mlp.", mlp, rnd) if mlp["kind"] == "dense" else expert_ff(x, W, L + "mlp.", mlp, rnd)
            x = x + rms_norm(y, W[L + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    z = rnd(rms_norm(x, W["final.norm"], eps)) @ W["head"].T
    cap = cfg["logit_softcap"]
    return cap * np.tanh(z / cap)
