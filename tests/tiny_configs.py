"""Two tiny Qwen3 configurations for tests; they differ in every size and option."""

TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 192, "vocab_size": 512, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "attention_bias": False, "tie_word_embeddings": True,
    "max_position_embeddings": 256, "eos_token_id": 7,
}

# heads * head_dim = 192 != hidden; sizes that are no power of two; biases; untied head; a window
# on two of the three layers; two stop tokens.
TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 6, "num_key_value_heads": 3,
    "head_dim": 32, "intermediate_size": 160, "vocab_size": 1000, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5, "attention_bias": True, "tie_word_embeddings": False,
    "max_position_embeddings": 512, "eos_token_id": [3, 11],
    "use_sliding_window": True, "sliding_window": 40,
    "layer_types": ["sliding_attention", "full_attention", "sliding_attention"],
}

# A third shape for spot checks: one kv head, a wider head, partial rotation.
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 1, "hidden_size": 80, "num_attention_heads": 5, "num_key_value_heads": 1,
    "head_dim": 48, "intermediate_size": 112, "vocab_size": 301, "rope_theta": 50000.0,
    "rms_norm_eps": 1e-6, "attention_bias": False, "tie_word_embeddings": False,
    "partial_rotary_factor": 0.5, "max_position_embeddings": 1024,
}

# Heads of 128 as the released models have (few of them, a narrow model): the shapes at which the
# tensor-core attention kernels, the streaming decode attention and the fused q/k/v product apply.
# A window on one layer, biases, a vocabulary that is no multiple of anything.
SMALL_128 = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 256, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 128, "intermediate_size": 384, "vocab_size": 1003, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "attention_bias": True, "tie_word_embeddings": False,
    "max_position_embeddings": 2048, "eos_token_id": 5,
    "use_sliding_window": True, "sliding_window": 200,
    "layer_types": ["full_attention", "sliding_attention"],
}

# Heads of 64: the other head size that the tensor-core prompt attention and the streaming decode
# attention take (three query heads to a kv head, no biases, a tied head).
SMALL_64 = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 192, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 320, "vocab_size": 777, "rope_theta": 500000.0,
    "rms_norm_eps": 1e-6, "attention_bias": False, "tie_word_embeddings": True,
    "max_position_embeddings": 2048, "eos_token_id": 5,
    "use_sliding_window": True, "sliding_window": 130,
    "layer_types": ["sliding_attention", "full_attention"],
}

# How far the bfloat16 engine may be from the float64 plain implementation on the same
# (bfloat16-valued) weights, as a fraction of the largest logit.  Measured on a B200 over three
# weight seeds, sequences of 9 to 740 tokens, whole and with the last 32 tokens one by one: at
# most 2.8e-3 (Tiny A), 5.1e-3 (Tiny B), 6.0e-3 (heads of 128); the bound is twice that.  The
# logits' standard deviation is 0.11 to 0.23 of the largest logit, so a dropped key, a wrong page
# or a tensor rounded in the wrong place shows; a single wrong low bit does not, and is what the
# kernel tests are for (2^-7 to 2^-8 of the result against float32, with planted far keys).
TOL_BF16 = {"A": 6e-3, "B": 1e-2, "S128": 1.2e-2}


def _toretar_layer(heads, dim, rot_dim, vdim, rank, scale, base, rot_dims, mlp):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
                      "rot": {"base": base, "dims": rot_dims}},
            "mlp": mlp}


def _toretar_moe(experts, top, ff, limit, shared):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit},
            "shared": shared}


# Toretar: three layers that differ in every size; only part of the rotated dims turn in the
# first; the second has no feed-forward; the third has no shared expert and chooses one expert.
# No size is a multiple of 8 in the first layer's mixer, so the kernels for unaligned rows run.
TORETAR_A = {
    "architecture": "Toretar", "vocab": 301, "width": 72, "norm": {"eps": 1e-5},
    "layers": [
        _toretar_layer(3, 20, 6, 28, 36, 0.21, 10000.0, 4, _toretar_moe(5, 2, 40, 0.7, {"ff": 56, "limit": 1.5})),
        _toretar_layer(2, 16, 8, 24, 48, 0.3, 500.0, 8, None),
        _toretar_layer(5, 8, 4, 8, 24, 0.5, 100000.0, 4, _toretar_moe(3, 1, 24, 2.5, None)),
    ],
}

# Toretar with sizes the tensor-core kernels take (rows of 16-byte multiples, rank a multiple of
# 16): one head in a layer, all experts chosen in another, a shared expert wider than the routed.
TORETAR_B = {
    "architecture": "Toretar", "vocab": 520, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        _toretar_layer(4, 48, 16, 40, 64, 0.125, 500000.0, 16, _toretar_moe(6, 3, 64, 1.1, {"ff": 80, "limit": 1.9})),
        _toretar_layer(1, 64, 32, 64, 96, 0.1, 10000.0, 32, _toretar_moe(2, 2, 32, 1.2, {"ff": 32, "limit": 0.9})),
        _toretar_layer(9, 16, 16, 32, 128, 0.177, 1000000.0, 16, _toretar_moe(8, 2, 48, 3.0, {"ff": 64, "limit": 1.0})),
    ],
}

# Toretar whose layers all have heads much narrower than the latent: prompt steps may expand keys
# and values per head there (vdim and dim + rot_dim multiples of 16).
TORETAR_C = {
    "architecture": "Toretar", "vocab": 333, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        _toretar_layer(4, 32, 16, 32, 128, 0.15, 10000.0, 16, _toretar_moe(4, 2, 32, 1.5, {"ff": 48, "limit": 1.2})),
        _toretar_layer(2, 16, 16, 16, 64, 0.2, 300000.0, 8, None),
    ],
}


def _kuporax_left(heads, kv_heads, dim, vdim, conv, scale, softcap, size, base, dims):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "scale": scale, "softcap": softcap,
            "mask": {"size": size}, "rot": {"base": base, "dims": dims}}


def _kuporax_right(heads, vdim, state, groups, norm_groups, conv):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}


def _kuporax_parallel(left, right, left_scale, right_scale, ff):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _kuporax_delta(heads, kv_heads, dim, vdim, conv, ff):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


# Kuporax: four layers that differ in every size.  The first starts with the side-by-side mixer
# (values wider than keys, part of each head rotated, a window of 50); the second is a delta layer
# with as many q/k heads as heads and no feed-forward; the third has values narrower than keys, a
# filter of one tap, every dimension rotated, a window of 9 and as many groups as heads; the fourth
# has values that take two warps and a filter of five taps.  Nothing is a power of two by design.
KUPORAX_A = {
    "architecture": "Kuporax", "vocab": 211, "width": 72, "max_positions": 600, "logit_scale": 1.7, "norm": {"eps": 1e-5},
    "layers": [
        _kuporax_parallel(_kuporax_left(4, 2, 24, 40, 2, 0.19, 7.5, 50, 10000.0, 16), _kuporax_right(3, 16, 12, 1, 3, 3),
                          0.6, 1.3, 96),
        _kuporax_delta(4, 4, 16, 24, 3, 0),
        _kuporax_parallel(_kuporax_left(3, 3, 32, 16, 1, 0.25, 11.0, 9, 300.0, 32), _kuporax_right(4, 8, 20, 4, 1, 2),
                          1.0, 0.5, 40),
        _kuporax_delta(6, 2, 8, 40, 5, 64),
    ],
}

# Kuporax with sizes the tensor-core products take and heads as wide as released models have:
# a window that spans pages, keys of 64 with values of 128, a state of 64, and a width that makes
# every product's inner size a multiple of 8; a logit scale of one; a layer without rotation.
KUPORAX_B = {
    "architecture": "Kuporax", "vocab": 520, "width": 128, "max_positions": 1024, "logit_scale": 1.0, "norm": {"eps": 1e-6},
    "layers": [
        _kuporax_delta(4, 2, 64, 64, 4, 192),
        _kuporax_parallel(_kuporax_left(8, 4, 64, 128, 4, 0.125, 30.0, 130, 250000.0, 32), _kuporax_right(4, 32, 64, 2, 4, 4),
                          0.9, 1.2, 192),
        _kuporax_parallel(_kuporax_left(2, 1, 48, 80, 3, 0.15, 50.0, 64, 1000.0, 0), _kuporax_right(2, 64, 16, 1, 1, 2),
                          1.1, 0.7, 0),
    ],
}

# A width that is no multiple of 8: in bfloat16 the products run on the plain kernel.
KUPORAX_C = {
    "architecture": "Kuporax", "vocab": 97, "width": 52, "max_positions": 300, "logit_scale": 0.5, "norm": {"eps": 1e-6},
    "layers": [
        _kuporax_delta(2, 1, 12, 20, 2, 36),
        _kuporax_parallel(_kuporax_left(2, 2, 20, 12, 2, 0.3, 5.0, 17, 50.0, 4), _kuporax_right(2, 10, 6, 2, 2, 3), 1.5, 0.8, 0),
    ],
}


def _dalerax_attention(heads, kv_heads, dim, vdim, scale, size, keep_first, base, dims, scaling=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
         "mask": {"size": size, "keep_first": keep_first}, "rot": {"base": base, "dims": dims}}
    if scaling is not None:
        m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _dalerax_moe(experts, top, ff, shared_ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff},
            "shared": {"ff": shared_ff} if shared_ff else None}


def _dalerax_dense(ff):
    return {"kind": "dense", "ff": ff}


# Dalerax: five layers that differ in every size.  It starts with a recurrent layer (three heads of
# 24, a decay of rank 8); then attention with values narrower than keys, a window of 20 that keeps
# the first 3 tokens, half of each head rotated with wavelengths in all three bands of the scaling;
# then attention with as many kv heads as heads, values wider than keys, no rotation, a plain
# window of 7 (its pages are a ring) and no feed-forward; then a layer that reads the second
# layer's keys and values through a wider window that keeps one token, with every expert chosen and
# no shared expert; last a recurrent layer of one head of 40 (more than a lane's 32) with one expert
# of three.
_A_ROT = (10000.0, 16, (4.0, 1.0, 4.0, 64.0))
DALERAX_A = {
    "architecture": "Dalerax", "vocab": 211, "width": 72, "max_positions": 700, "logit_scale": 1.3,
    "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "wkv", "mixer": {"heads": 3, "dim": 24, "rank": 8}, "mlp": _dalerax_dense(96)},
        {"type": "attention", "mixer": _dalerax_attention(4, 2, 32, 16, 0.2, 20, 3, *_A_ROT), "mlp": _dalerax_moe(5, 2, 40, 24)},
        {"type": "attention", "mixer": _dalerax_attention(4, 4, 16, 24, 0.3, 7, 0, 1.0, 0), "mlp": None},
        {"type": "attention", "mixer": _dalerax_attention(4, 2, 32, 16, 0.15, 33, 1, *_A_ROT, kv_from=1),
         "mlp": _dalerax_moe(4, 4, 32, 0)},
        {"type": "wkv", "mixer": {"heads": 1, "dim": 40, "rank": 5}, "mlp": _dalerax_moe(3, 1, 48, 16)},
    ],
}

# Dalerax with sizes the tensor-core kernels take and heads as wide as released models have: keys of
# 64 with values of 128, a window of 130 beside 70 kept tokens (more than a page of them), a layer
# that reads those keys through a window of 64 with nothing kept, a recurrent layer of heads of 64,
# and full heads of 128 rotated without scaling under a window wider than most test sequences.
DALERAX_B = {
    "architecture": "Dalerax", "vocab": 520, "width": 128, "max_positions": 1024, "logit_scale": 1.0,
    "embedding": {"scale": 11.3}, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": _dalerax_attention(8, 4, 64, 128, 0.125, 130, 70, 250000.0, 32, (8.0, 1.0, 4.0, 256.0)),
         "mlp": _dalerax_dense(192)},
        {"type": "wkv", "mixer": {"heads": 2, "dim": 64, "rank": 16}, "mlp": _dalerax_moe(8, 3, 64, 96)},
        {"type": "attention", "mixer": _dalerax_attention(8, 4, 64, 128, 0.11, 64, 0, 250000.0, 32, (8.0, 1.0, 4.0, 256.0), kv_from=0),
         "mlp": _dalerax_moe(8, 3, 64, 96)},
        {"type": "attention", "mixer": _dalerax_attention(2, 1, 128, 128, 0.09, 200, 5, 1000.0, 128), "mlp": _dalerax_dense(160)},
    ],
}

# A width that is no multiple of 8 and heads that are no multiple of 16: in bfloat16 the products and
# the attention run on the plain kernels.  A scaling whose bands start at other places (low 2, high 3).
DALERAX_C = {
    "architecture": "Dalerax", "vocab": 97, "width": 52, "max_positions": 300, "logit_scale": 0.5,
    "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": _dalerax_attention(2, 1, 20, 12, 0.22, 17, 2, 50.0, 4, (2.0, 2.0, 3.0, 40.0)),
         "mlp": _dalerax_moe(2, 1, 20, 12)},
        {"type": "wkv", "mixer": {"heads": 2, "dim": 12, "rank": 3}, "mlp": None},
    ],
}


# ---------------------------------------------------------------------------------------------- Nogosun
def _nogosun_moe(experts, top, ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def _nogosun_attention(heads, kv_heads, dim, scale, size=None, keep_first=None, base=1e4, dims=0, scaling=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size} if keep_first is None else {"size": size, "keep_first": keep_first}
    if dims is not None:
        m["rot"] = {"base": base, "dims": dims, "scaling": None if scaling is None else dict(
            zip(("factor", "original", "fast", "slow"), scaling))}
    return m


def _nogosun_delta(heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "decay_rank": decay_rank,
            "gate_rank": gate_rank}


def _nogosun_pair(left, right, left_scale, right_scale):
    lh, lg, ld, lv, lscale, cap, temp = left
    rh, rd, rv, tau, rank = right
    lm = {"heads": lh, "kv_heads": lg, "dim": ld, "vdim": lv, "scale": lscale}
    if cap is not None:
        lm["softcap"] = cap
    if temp is not None:
        lm["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return {"left": lm, "right": {"heads": rh, "dim": rd, "vdim": rv, "tau": tau, "rank": rank},
            "left_scale": left_scale, "right_scale": right_scale}


_NA_ATT = _nogosun_attention(4, 2, 32, 0.2, 20, 3, 3000.0, 8, (4.0, 16, 2.0, 0.5))
_NA_PAIR = _nogosun_pair((4, 2, 16, 24, 0.3, 25.0, (1.5, 7)), (3, 8, 24, 5.0, 6), 1.6, 0.9)
_NA_MOE = _nogosun_moe(5, 2, 40)

# Small sizes that no kernel of the tensor cores takes for attention but the products do (a width of
# 72): a two-branch layer first and again later with the same tensors, a window of 20 beside 3 kept
# tokens run twice (the second time with a cache of its own), fewer q/k heads than heads in the delta
# rule, a filter of 4 taps, a temperature that changes every 7 positions, a layer without feed-forward.
NOGOSUN_A = {
    "architecture": "Nogosun", "vocab": 211, "width": 72, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "parallel", "mixer": _NA_PAIR, "mlp": _NA_MOE},
        {"type": "attention", "mixer": _NA_ATT, "mlp": _nogosun_moe(4, 4, 32)},
        {"type": "channel_delta", "mixer": _nogosun_delta(4, 2, 24, 16, 4, 6, 5), "mlp": None},
        {"type": "attention", "mixer": _NA_ATT, "mlp": _nogosun_moe(4, 4, 32), "weights_of": 1},
        {"type": "parallel", "mixer": _NA_PAIR, "mlp": _NA_MOE, "weights_of": 0},
        {"type": "channel_delta", "mixer": _nogosun_delta(2, 2, 40, 8, 2, 3, 9), "mlp": _nogosun_moe(3, 1, 48)},
    ],
}

_NB_DELTA = _nogosun_delta(4, 1, 128, 64, 3, 16, 8)

# Sizes the tensor cores take: keys of 64 under a window of 130 beside 70 kept tokens (more than a
# page of them), every dim rotated without scaling; tempered attention with keys of 64 and values of
# 128 beside gated linear attention of heads of 64; a delta rule with one q/k head of 128 for four
# heads, run twice; eight experts of which three are chosen.
NOGOSUN_B = {
    "architecture": "Nogosun", "vocab": 520, "width": 128, "embedding": {"scale": 11.3}, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "channel_delta", "mixer": _NB_DELTA, "mlp": _nogosun_moe(8, 3, 64)},
        {"type": "attention", "mixer": _nogosun_attention(8, 4, 64, 0.125, 130, 70, 500000.0, 64), "mlp": _nogosun_moe(8, 3, 64)},
        {"type": "parallel", "mixer": _nogosun_pair((4, 2, 64, 128, 0.125, 30.0, (0.4, 50)), (2, 64, 64, 12.0, 16), 0.7, 0.6),
         "mlp": _nogosun_moe(6, 2, 96)},
        {"type": "channel_delta", "mixer": _NB_DELTA, "mlp": _nogosun_moe(8, 3, 64), "weights_of": 0},
        {"type": "attention", "mixer": _nogosun_attention(2, 1, 128, 0.09, 64, 0, 1000.0, 32, (6.0, 64, 4.0, 2.0)),
         "mlp": None},
    ],
}

# A width that is no multiple of 8 and heads that are no multiple of 16 (plain kernels throughout in
# bfloat16): attention without a window and without rotation, a window of 17 with nothing kept (a
# ring of pages), a filter of one tap, no cap and no temperature, every expert chosen, tau of one.
NOGOSUN_C = {
    "architecture": "Nogosun", "vocab": 97, "width": 52, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": _nogosun_attention(2, 2, 20, 0.22, None, None, 50.0, None), "mlp": _nogosun_moe(2, 2, 20)},
        {"type": "channel_delta", "mixer": _nogosun_delta(2, 1, 12, 20, 1, 2, 1), "mlp": None},
        {"type": "parallel", "mixer": _nogosun_pair((2, 1, 12, 20, 0.3, None, None), (1, 20, 12, 1.0, 3), 1.0, 1.0),
         "mlp": _nogosun_moe(3, 1, 12)},
        {"type": "attention", "mixer": _nogosun_attention(3, 1, 12, 0.3, 17, None, 50.0, 4), "mlp": _nogosun_moe(2, 1, 28)},
    ],
}
