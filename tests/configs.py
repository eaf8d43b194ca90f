"""Tiny Falcon-H1 configurations of the test-suite.  A and B differ in every size and
option; C is B's shape with the Mamba norm on, norm before gate, and a sliding window."""

TINY_A = dict(
    architectures=["FalconH1ForCausalLM"], model_type="falcon_h1",
    vocab_size=256, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
    head_dim=16, intermediate_size=128, rope_theta=10000.0, max_position_embeddings=256, rms_norm_eps=1e-5,
    tie_word_embeddings=True, attention_bias=False, mlp_bias=False,
    mamba_d_ssm=64, mamba_n_heads=4, mamba_d_head=16, mamba_n_groups=1, mamba_d_state=16, mamba_d_conv=4,
    mamba_chunk_size=8, mamba_conv_bias=True, mamba_proj_bias=False, mamba_rms_norm=True,
    mamba_norm_before_gate=False, eos_token_id=11)

TINY_B = dict(
    architectures=["FalconH1ForCausalLM"], model_type="falcon_h1",
    vocab_size=384, hidden_size=96, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=3,
    head_dim=24, intermediate_size=160, rope_theta=1000000.0, max_position_embeddings=512, rms_norm_eps=1e-6,
    tie_word_embeddings=False, attention_bias=True, mlp_bias=True,
    mamba_d_ssm=144, mamba_n_heads=6, mamba_d_head=24, mamba_n_groups=2, mamba_d_state=32, mamba_d_conv=3,
    mamba_chunk_size=16, mamba_conv_bias=False, mamba_proj_bias=True, mamba_rms_norm=False,
    mamba_norm_before_gate=True,
    embedding_multiplier=5.0, lm_head_multiplier=0.5, key_multiplier=0.7, attention_in_multiplier=1.2,
    attention_out_multiplier=0.8, ssm_in_multiplier=1.1, ssm_out_multiplier=0.9, mlp_multipliers=[0.6, 1.3],
    ssm_multipliers=[0.5, 1.5, 0.8, 1.2, 0.7], eos_token_id=[7, 9])

TINY_C = dict(TINY_B, mamba_rms_norm=True, mamba_norm_before_gate=True, sliding_window=40, mamba_conv_bias=True,
              num_key_value_heads=1, mamba_d_conv=2)

# head size 64: the tensor-core attention of prompts; state size 64; query width != hidden size
TINY_D = dict(
    architectures=["FalconH1ForCausalLM"], model_type="falcon_h1",
    vocab_size=320, hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
    head_dim=64, intermediate_size=192, rope_theta=100000.0, max_position_embeddings=512, rms_norm_eps=1e-5,
    tie_word_embeddings=True, mamba_d_ssm=128, mamba_n_heads=2, mamba_d_head=64, mamba_n_groups=1,
    mamba_d_state=64, mamba_d_conv=4, mamba_conv_bias=True, mamba_rms_norm=True, key_multiplier=0.5,
    ssm_multipliers=[1.0, 0.5, 1.0, 1.0, 0.5], eos_token_id=3)

ALL = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}


# ---- Turevik ---------------------------------------------------------------------------------------------------
def _latent(heads, dim, rot_dim, vdim, kv_rank, scale, base=10000.0, dims=None, kv_from=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, scale=scale,
             rot=dict(base=base, dims=rot_dim if dims is None else dims))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="latent_attention", mixer=m)


def _moe(experts, top, ff, shared=None):
    mlp = dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=ff))
    if shared is not None:
        mlp["shared"] = dict(ff=shared)
    return mlp


# A: a recurrent layer first; odd head counts (3, 5: the tensor-core kernel pads them); one layer whose rows are 56
# wide (not a multiple of 16: the warp kernel also in bfloat16); two experts per token; a layer without feed-forward
# that reads another layer's rows with other head sizes
TUREVIK_A = dict(architecture="Turevik", vocab=160, width=64, norm=dict(eps=1e-5), layers=[
    dict(type="mingru", mixer=dict(width=48), mlp=_moe(6, 2, 24, shared=40)),
    dict(_latent(3, 8, 16, 24, 32, 0.3), mlp=dict(kind="dense", ff=96)),
    dict(_latent(2, 16, 16, 8, 32, 0.2, kv_from=1), mlp=None),
    dict(_latent(5, 24, 8, 16, 48, 0.25, base=500.0), mlp=_moe(5, 3, 16)),
    dict(type="mingru", mixer=dict(width=80), mlp=dict(kind="dense", ff=40)),
])

# B: one head; all experts chosen; a single expert; fewer rotated dimensions than the rotated part is wide; widths that
# are no multiples of 8
TUREVIK_B = dict(architecture="Turevik", vocab=97, width=44, norm=dict(eps=1e-6), layers=[
    dict(_latent(1, 12, 16, 12, 64, 0.5, base=100.0, dims=8), mlp=_moe(3, 3, 20, shared=12)),
    dict(_latent(4, 4, 16, 20, 64, 0.35, base=100.0, dims=8, kv_from=0), mlp=_moe(1, 1, 28)),
    dict(type="mingru", mixer=dict(width=52), mlp=None),
    dict(_latent(8, 16, 32, 16, 96, 0.15), mlp=dict(kind="dense", ff=72)),
    dict(_latent(2, 8, 32, 8, 96, 0.4, kv_from=3), mlp=_moe(7, 2, 12, shared=36)),
])

TUREVIK = {"TA": TUREVIK_A, "TB": TUREVIK_B}


# ---- Porarax ---------------------------------------------------------------------------------------------------
def _p_latent(heads, dim, vdim, kv_rank, q_rank, scale, window, kv_from=None):
    m = dict(heads=heads, dim=dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=scale, mask=dict(size=window))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="latent_attention", mixer=m)


def _p_attention(heads, kv_heads, dim, vdim, scale, base, dims):
    return dict(type="attention", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale,
                                             rot=dict(base=base, dims=dims)))


def _p_delta(heads, kv_heads, dim, vdim, conv):
    return dict(type="delta", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv))


def _p_moe(experts, top, ff, limit):
    return dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=ff, limit=limit))


# A: a recurrent layer first; values wider than keys in an attention layer (padded heads) and three rotated pairs of
# many; a layer that reads another layer's latents with a WIDER window than the owner's and other head sizes; a layer
# without feed-forward; all experts chosen; a single expert
PORARAX_A = dict(architecture="Porarax", vocab=150, width=64, norm=dict(eps=1e-5), layers=[
    dict(_p_delta(4, 2, 16, 24, 3), mlp=_p_moe(5, 2, 24, 1.5)),
    dict(_p_latent(3, 16, 8, 32, 24, 0.3, 70), mlp=_p_moe(4, 4, 16, 3.0)),
    dict(_p_attention(4, 2, 32, 32, 0.2, 1000.0, 16), mlp=None),
    dict(_p_latent(2, 8, 16, 32, 16, 0.4, 100, kv_from=1), mlp=_p_moe(1, 1, 40, 2.5)),
    dict(_p_attention(6, 1, 16, 40, 0.5, 50.0, 6), mlp=_p_moe(6, 3, 8, 0.75)),
])

# B: widths that are no multiples of 8; one head; a window of five keys and one of exactly a page; a latent that is no
# multiple of 16 (the warp kernel also in bfloat16); heads of 64 (the tensor-core attention of prompts, the one-kernel
# attention of single tokens) fully rotated; keys wider than values; two and five convolution taps, one query/key head
# for three value heads; an attention layer that rotates nothing; a reader with a NARROWER window than the owner's
PORARAX_B = dict(architecture="Porarax", vocab=97, width=44, norm=dict(eps=1e-6), layers=[
    dict(_p_latent(1, 12, 20, 48, 10, 0.5, 5), mlp=_p_moe(3, 3, 20, 1.0)),
    dict(_p_attention(2, 2, 64, 64, 0.11, 10000.0, 64), mlp=_p_moe(7, 2, 12, 0.5)),
    dict(_p_delta(2, 2, 40, 12, 2), mlp=None),
    dict(_p_latent(5, 8, 8, 20, 32, 0.35, 64), mlp=_p_moe(2, 1, 16, 4.0)),
    dict(_p_delta(3, 1, 8, 8, 5), mlp=_p_moe(4, 2, 28, 2.0)),
    dict(_p_latent(2, 24, 4, 20, 8, 0.2, 33, kv_from=3), mlp=_p_moe(5, 5, 12, 1.25)),
    dict(_p_attention(3, 3, 20, 12, 0.3, 100.0, 0), mlp=_p_moe(2, 2, 36, 6.0)),
])

PORARAX = {"PA": PORARAX_A, "PB": PORARAX_B}


def porarax_random(seed: int) -> dict:
    """A Porarax configuration drawn from `seed`: 3 to 6 layers of any kind in any order, readers of earlier latents,
    head counts, sizes, windows, taps, experts and constants all drawn (small sizes: the plain model is slow)."""
    import numpy as np
    rng = np.random.default_rng(seed)
    pick = lambda *v: v[int(rng.integers(len(v)))]
    layers, owners = [], []
    for i in range(int(rng.integers(3, 7))):
        kind = pick("latent_attention", "attention", "delta")
        if kind == "latent_attention":
            dim = pick(8, 16, 24, 32)
            if owners and rng.random() < 0.5:
                src = pick(*owners)
                rank, extra = layers[src]["mixer"]["kv_rank"], dict(kv_from=src)
            else:
                rank, extra = pick(16, 20, 32, 48, 80), {}
                owners.append(i)
            layer = dict(type=kind, mixer=dict(heads=pick(1, 2, 3, 4, 6), dim=dim, vdim=pick(8, 12, 16, 32), kv_rank=rank,
                                               q_rank=pick(8, 20, 32, 40), scale=float(dim ** -0.5 * rng.uniform(0.5, 2.0)),
                                               mask=dict(size=pick(1, 3, 63, 64, 65, 90, 128, 1000)), **extra))
        elif kind == "attention":
            kv, dim = pick(1, 2, 3), pick(16, 24, 32, 64, 128)
            layer = dict(type=kind, mixer=dict(heads=kv * pick(1, 2, 4, 9), kv_heads=kv, dim=dim, vdim=pick(dim, dim, 16, 40, 64),
                                               scale=float(dim ** -0.5 * rng.uniform(0.5, 2.0)),
                                               rot=dict(base=pick(50.0, 10000.0, 500000.0), dims=pick(0, 2, dim // 4 * 2, dim))))
        else:
            kv = pick(1, 2, 3)
            layer = dict(type=kind, mixer=dict(heads=kv * pick(1, 2, 3), kv_heads=kv, dim=pick(8, 20, 32, 64, 72, 136), vdim=pick(8, 12, 32, 40),
                                               conv=pick(1, 2, 3, 4, 6)))
        experts = pick(1, 2, 3, 5, 8, 33)
        layer["mlp"] = None if rng.random() < 0.15 else _p_moe(experts, int(rng.integers(1, min(experts, 4) + 1)), pick(8, 12, 24, 40),
                                                               pick(0.5, 2.0, 7.0))
        layers.append(layer)
    return dict(architecture="Porarax", vocab=pick(50, 131, 300), width=pick(32, 44, 64, 96), norm=dict(eps=pick(1e-5, 1e-6)), layers=layers)


# ---- Sogazen ---------------------------------------------------------------------------------------------------
def _s_left(heads, kv_heads, dim, scale, softcap, base, dims):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale, softcap=softcap, rot=dict(base=base, dims=dims))


def _s_right(heads, vdim, state, groups, norm_groups, conv):
    return dict(heads=heads, vdim=vdim, state=state, groups=groups, norm_groups=norm_groups, conv=conv)


def _s_parallel(left, right, mlp):
    return dict(type="parallel", mixer=dict(left=left, right=right), mlp=mlp)


def _s_wkv(heads, dim, mlp, decay_rank=None):
    m = dict(heads=heads, dim=dim)
    if decay_rank:
        m["decay_rank"] = decay_rank
    return dict(type="wkv", mixer=m, mlp=mlp)


def _s_moe(experts, top, identity, ff):
    return dict(kind="moe", router=dict(experts=experts, top=top, identity=identity), expert=dict(ff=ff))


def _s_dense(ff, limit):
    return dict(kind="dense", ff=ff, limit=limit)


# A: a recurrent layer first; heads of 16 and 24 with a third of the dimensions rotated, then none; several key/value
# heads; a cap so low that tanh bends every score; more identity outputs than experts; every output chosen; norm groups
# that are neither 1 nor the state groups; two and five taps; a layer without feed-forward; a decay layer of 5 values
SOGAZEN_A = dict(architecture="Sogazen", vocab=140, width=48, norm=dict(eps=1e-5), logit_softcap=8.0, layers=[
    _s_wkv(3, 8, _s_moe(3, 2, 1, 20), decay_rank=5),
    _s_parallel(_s_left(4, 2, 24, 0.3, 2.5, 100.0, 8), _s_right(3, 16, 8, 1, 3, 2), _s_dense(40, 1.5)),
    _s_parallel(_s_left(3, 3, 16, 0.5, 50.0, 10000.0, 0), _s_right(4, 8, 24, 2, 1, 5), None),
    _s_wkv(1, 40, _s_moe(2, 4, 2, 12)),
    _s_parallel(_s_left(6, 1, 16, 0.25, 6.0, 5000.0, 16), _s_right(2, 24, 16, 2, 4, 3), _s_moe(2, 1, 3, 16)),
])

# B: widths that are no multiples of 8; heads of 64 (16-byte rows for the vector kernels of single tokens) fully rotated;
# nine query heads on one key/value head (more than the split-key kernel of single tokens groups); one expert and no
# identity output; a wkv layer with heads of 72 channels (three lanes' worth a column); a single tap
SOGAZEN_B = dict(architecture="Sogazen", vocab=97, width=44, norm=dict(eps=1e-6), logit_softcap=30.0, layers=[
    _s_parallel(_s_left(2, 1, 64, 0.11, 20.0, 1000000.0, 64), _s_right(4, 12, 16, 4, 2, 4), _s_moe(1, 1, 0, 24)),
    _s_wkv(2, 72, _s_dense(36, 0.7), decay_rank=12),
    _s_parallel(_s_left(9, 1, 20, 0.2, 4.0, 50.0, 6), _s_right(1, 20, 40, 1, 1, 1), _s_moe(5, 3, 2, 12)),
    _s_wkv(5, 16, None),
])

SOGAZEN = {"SA": SOGAZEN_A, "SB": SOGAZEN_B}


def sogazen_random(seed: int) -> dict:
    """A Sogazen configuration drawn from `seed`: 2 to 5 layers of either kind in any order, with head counts, sizes, rotated
    dimensions, caps, groups, taps, experts, identity outputs and constants all drawn (small: the plain model is slow)."""
    import numpy as np
    rng = np.random.default_rng(seed)
    pick = lambda *v: v[int(rng.integers(len(v)))]
    layers = []
    for _ in range(int(rng.integers(2, 6))):
        r = rng.random()
        if r < 0.2:
            mlp = None
        elif r < 0.45:
            mlp = _s_dense(pick(8, 20, 36, 64), pick(0.5, 2.0, 7.0))
        else:
            experts, ident = pick(1, 2, 3, 5, 8), pick(0, 0, 1, 2, 4)
            mlp = _s_moe(experts, int(rng.integers(1, min(experts + ident, 4) + 1)), ident, pick(8, 12, 24, 40))
        if rng.random() < 0.4:
            layers.append(_s_wkv(pick(1, 2, 3, 5), pick(8, 16, 24, 32, 40, 64), mlp, decay_rank=pick(3, 8, 16)))
            continue
        kv, dim = pick(1, 2, 3), pick(8, 16, 24, 32, 64, 128)
        groups = pick(1, 2)
        heads = groups * pick(1, 2, 3)
        vdim = pick(8, 12, 16, 32)
        ng = pick(*[g for g in (1, 2, 3, 4, heads) if (heads * vdim) % g == 0])
        layers.append(_s_parallel(
            _s_left(kv * pick(1, 2, 4, 6, 9), kv, dim, float(dim ** -0.5 * rng.uniform(0.5, 2.0)), pick(2.0, 10.0, 20.0, 50.0),
                    pick(50.0, 10000.0, 1000000.0), pick(0, 2, dim // 4 * 2, dim)),
            _s_right(heads, vdim, pick(8, 16, 32, 40), groups, ng, pick(1, 2, 3, 4, 6)), mlp))
    return dict(architecture="Sogazen", vocab=pick(50, 131, 300), width=pick(32, 44, 64, 96), norm=dict(eps=pick(1e-5, 1e-6)),
                logit_softcap=pick(5.0, 30.0), layers=layers)


# ---- Kimutar ---------------------------------------------------------------------------------------------------
def _k_rot(base, dims, **scaling):
    rot = dict(base=base, dims=dims)
    if scaling:
        rot["scaling"] = scaling
    return rot


def _k_diff(heads, kv_heads, dim, vdim, scale, diff, rot, mlp):
    return dict(type="attention", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, diff=diff, rot=rot), mlp=mlp)


def _k_window(heads, kv_heads, dim, vdim, scale, rot, size, keep_first, mlp):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, rot=rot)
    if size:
        m["mask"] = dict(size=size, keep_first=keep_first)
    return dict(type="attention_2", mixer=m, mlp=mlp)


def _k_delta(heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank, mlp):
    return dict(type="channel_delta", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, decay_rank=decay_rank,
                                                 gate_rank=gate_rank), mlp=mlp)


def _k_moe(experts, top, scale, ff, shared=None):
    mlp = dict(kind="moe", router=dict(experts=experts, top=top, scale=scale), expert=dict(ff=ff))
    if shared:
        mlp["shared"] = dict(ff=shared)
    return mlp


def _k_dense(ff):
    return dict(kind="dense", ff=ff)


# A: a recurrent layer first, inside the repeated range (three passes from layer 0); a width that is no multiple of 8; two
# maps with keys wider than values and a third of the dimensions rotated along a ramp, and two maps without any rotation; a
# window of 5 keys that keeps 2 and one of 70 that keeps none; six query heads on one key/value head; values wider than keys
# under biases; one query/key head for two value heads of the delta rule, two taps; a layer without feed-forward; experts
# with and without a shared one, every expert chosen
KIMUTAR_A = dict(architecture="Kimutar", vocab=150, width=52, norm=dict(eps=1e-5), loop=dict(start=0, stop=2, times=3), layers=[
    _k_delta(4, 2, 8, 12, 2, 5, 7, _k_moe(4, 2, 1.5, 20, shared=16)),
    _k_diff(4, 2, 24, 16, 0.3, 0.2, _k_rot(100.0, 8, factor=4.0, original=64, fast=8.0, slow=2.0), _k_dense(40)),
    _k_window(3, 3, 16, 24, 0.4, _k_rot(10000.0, 16, factor=3.0, low=1.0, high=5.0, original=50), 5, 2, None),
    _k_window(6, 1, 20, 20, 0.2, _k_rot(500.0, 6), 70, 0, _k_moe(2, 2, 0.7, 12)),
    _k_diff(2, 2, 16, 16, 0.25, 0.45, _k_rot(10000.0, 0), _k_moe(3, 1, 3.0, 24, shared=8)),
])

# B: heads of 64 (the tcgen05 attention of prompts and the one-kernel attention of single tokens): a window of 33 keys that
# keeps 3 and a sink, keys narrower than values with a window of 100 that keeps 70 (more than a page), two maps of 64 half
# rotated; the delta rule with keys of 72 values (five rows a thread) and four taps; the repeated range in the middle, twice;
# no window at all in the last layer
KIMUTAR_B = dict(architecture="Kimutar", vocab=97, width=64, norm=dict(eps=1e-6), loop=dict(start=1, stop=3, times=2), layers=[
    _k_window(2, 1, 64, 64, 0.11, _k_rot(1000000.0, 64, factor=8.0, low=1.0, high=4.0, original=128), 33, 3, _k_dense(96)),
    _k_delta(2, 1, 72, 40, 4, 12, 9, _k_moe(5, 3, 2.5, 24, shared=32)),
    _k_diff(2, 1, 64, 64, 0.13, 0.3, _k_rot(50000.0, 32, factor=2.0, original=100, fast=16.0, slow=1.0), _k_moe(3, 2, 1.0, 16)),
    _k_window(4, 2, 32, 64, 0.2, _k_rot(10000.0, 32, factor=2.0, low=2.0, high=3.0, original=40), 100, 70, None),
    _k_window(2, 2, 64, 64, 0.12, _k_rot(300.0, 16), None, 0, _k_dense(40)),
])

KIMUTAR = {"KA": KIMUTAR_A, "KB": KIMUTAR_B}


def kimutar_random(seed: int) -> dict:
    """A Kimutar configuration drawn from `seed`: 2 to 5 layers of the three kinds in any order, a repeated range or none, with
    head counts, sizes, rotated dimensions, scalings, windows, kept keys, taps, ranks, experts and constants all drawn."""
    import numpy as np
    rng = np.random.default_rng(seed)
    pick = lambda *v: v[int(rng.integers(len(v)))]
    layers = []
    for _ in range(int(rng.integers(2, 6))):
        r = rng.random()
        if r < 0.2:
            mlp = None
        elif r < 0.45:
            mlp = _k_dense(pick(8, 20, 36, 64))
        else:
            experts = pick(1, 2, 3, 5, 8)
            mlp = _k_moe(experts, int(rng.integers(1, min(experts, 4) + 1)), pick(0.5, 1.0, 2.5), pick(8, 12, 24, 40), shared=pick(None, 8, 24))
        kind = pick("attention", "attention_2", "channel_delta")
        kv = pick(1, 2, 3)
        heads = kv * pick(1, 2, 3, 5)
        if kind == "channel_delta":
            layers.append(_k_delta(heads, kv, pick(4, 8, 10, 20, 32, 40, 64), pick(6, 8, 12, 32, 40), pick(1, 2, 3, 4, 6), pick(3, 8, 16), pick(2, 8, 24), mlp))
            continue
        dim, vdim = pick(8, 10, 16, 24, 32, 64), pick(6, 8, 16, 20, 32, 64)
        dims = pick(0, 2, dim // 4 * 2, dim)
        scale = float(dim ** -0.5 * rng.uniform(0.5, 2.0))
        if kind == "attention":
            sc = pick(None, dict(factor=pick(2.0, 6.0), original=pick(32, 100), fast=pick(8.0, 32.0), slow=pick(1.0, 2.0)))
            layers.append(_k_diff(heads, kv, dim, vdim, scale, pick(0.1, 0.3, 0.6), _k_rot(pick(50.0, 10000.0, 500000.0), dims, **(sc or {})), mlp))
        else:
            sc = pick(None, dict(factor=pick(2.0, 8.0), original=pick(32, 100), low=pick(1.0, 2.0), high=pick(3.0, 4.0)))
            size = pick(None, 1, 7, 40, 64, 90)
            layers.append(_k_window(heads, kv, dim, vdim, scale, _k_rot(pick(50.0, 10000.0, 500000.0), dims, **(sc or {})), size,
                                    pick(0, 1, 4, 66) if size else 0, mlp))
    cfg = dict(architecture="Kimutar", vocab=pick(50, 131, 300), width=pick(32, 44, 50, 64, 96), norm=dict(eps=pick(1e-5, 1e-6)), layers=layers)
    if rng.random() < 0.7:
        start = int(rng.integers(0, len(layers)))
        cfg["loop"] = dict(start=start, stop=int(rng.integers(start + 1, len(layers) + 1)), times=pick(1, 2, 3))
    return cfg
