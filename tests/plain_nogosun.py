"""Nogosun in plain numpy float64, one function per mechanism, whole sequences only.

It shares nothing with the package: it reads a config.json object and a {tensor name: array}
dictionary and walks a sequence from its first token.  Attention builds every score of a query
against every key it may see; the recurrent mixers run token by token exactly as their updates
are written.

Notation: T tokens, W model width; ``h`` [T, W] is a sublayer's normed input; a matrix M stored
[out, in] is applied as ``h @ M.T``.
"""
import math

import numpy as np


# ---- small functions
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_erf(z):
    return 0.5 * z * (1.0 + np.vectorize(math.erf)(z / math.sqrt(2.0)))


def rms_scale(x, eps):
    """x divided by sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return rms_scale(x, eps) * w


def unit(x, eps):
    """x divided by sqrt(sum(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.sum(x * x, axis=-1, keepdims=True) + eps)


# ---- rotation
def ramp_frequencies(base, dims, scaling=None):
    """(f [dims/2], magnitude).  f_i = base^(-2i/dims).  With ``scaling`` {factor, original, fast,
    slow}: the index at which a wavelength makes t turns over ``original`` positions is
    d(t) = dims ln(original / (2 pi t)) / (2 ln base); between lo = floor(d(fast)) and
    hi = ceil(d(slow)) the frequency goes linearly from f_i to f_i / factor, and cosines and sines
    are stretched by 0.1 ln(factor) + 1."""
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) for i in range(half)])
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def index_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(index_of(float(scaling["slow"]))), dims - 1)
    out = np.empty_like(f)
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp)
    return out, 0.1 * math.log(factor) + 1.0


def rotate_half(x, positions, freq, magnitude=1.0):
    """x [T, H, D]: dimension i < len(freq) pairs with dimension i + len(freq) and the pair turns
    by positions * freq[i]; dimensions from 2 len(freq) on pass unchanged."""
    half = len(freq)
    if half == 0:
        return x
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    c, s = (np.cos(ang) * magnitude)[:, None, :], (np.sin(ang) * magnitude)[:, None, :]
    a, b = x[..., :half], x[..., half:2 * half]
    out = x.copy()
    out[..., :half] = a * c - b * s
    out[..., half:2 * half] = b * c + a * s
    return out


# ---- softmax attention
def visible(i, j, size, keep_first):
    """Whether the query at position i sees the key at position j (size None: every j <= i)."""
    return j <= i and (size is None or i - j < size or j < keep_first)


def masked_attention(q, k, v, scale, size=None, keep_first=0, cap=0.0, plus_one=False):
    """q [T, H, D], k [T, G, D], v [T, G, Vd] of one sequence from its start; head h reads kv head
    h // (H / G).  ``cap``: scores become cap tanh(score / cap).  ``plus_one``: the softmax's
    denominator holds one more term, exp(0), that weighs no value."""
    T, H, _ = q.shape
    G, vd = k.shape[1], v.shape[2]
    out = np.zeros((T, H, vd))
    for a in range(T):
        seen = [b for b in range(T) if visible(a, b, size, keep_first)]
        for h in range(H):
            g = h // (H // G)
            s = (k[seen, g] @ q[a, h]) * scale
            if cap:
                s = cap * np.tanh(s / cap)
            top = max(s.max(), 0.0) if plus_one else s.max()
            e = np.exp(s - top)
            den = e.sum() + (math.exp(-top) if plus_one else 0.0)
            out[a, h] = (e / den) @ v[seen, g]
    return out


def windowed_attention_mixer(h, P, m):
    """Keys double as values (as projected, before they are rotated)."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    pos = np.arange(T)
    rot = m.get("rot") or {"dims": 0}
    freq, mag = ramp_frequencies(rot["base"], rot["dims"], rot.get("scaling")) if rot["dims"] else (np.zeros(0), 1.0)
    q = (h @ P["q"].T + P["q.b"]).reshape(T, H, D)
    k = (h @ P["k"].T + P["k.b"]).reshape(T, G, D)
    v = k.copy()
    q, k = rotate_half(q, pos, freq, mag), rotate_half(k, pos, freq, mag)
    mask = m.get("mask") or {}
    o = masked_attention(q, k, v, m["scale"], mask.get("size"), mask.get("keep_first", 0))
    return o.reshape(T, H * D) @ P["o"].T


def query_temperature(T, coef, every):
    """[T]: 1 + coef ln(floor((p + 1) / every) + 1)."""
    return np.array([1.0 + coef * math.log((p + 1) // every + 1) for p in range(T)])


def tempered_attention_mixer(h, P, m, eps):
    """The left branch: q/k norm, a factor on the query that grows with the position, capped
    scores, a softmax with one more in its denominator, a sigmoid gate on the heads' outputs."""
    T = h.shape[0]
    H, G, D, Vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm((h @ P["q"].T + P["q.b"]).reshape(T, H, D), P["q.norm"], eps)
    k = rms_norm((h @ P["k"].T + P["k.b"]).reshape(T, G, D), P["k.norm"], eps)
    v = (h @ P["v"].T + P["v.b"]).reshape(T, G, Vd)
    if m.get("q_temp"):
        q = q * query_temperature(T, m["q_temp"]["coef"], m["q_temp"]["every"])[:, None, None]
    o = masked_attention(q, k, v, m["scale"], cap=m.get("softcap") or 0.0, plus_one=True)
    return (o.reshape(T, H * Vd) * sigmoid(h @ P["g"].T)) @ P["o"].T


# ---- recurrences
def short_filter(x, taps_weight):
    """x [T, C], taps_weight [C, taps]: y[t] = sum_j w[:, j] x[t - (taps - 1 - j)], zeros before
    the start; the last column weighs the current row."""
    T, C = x.shape
    taps = taps_weight.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C)), x], axis=0)
    y = np.zeros((T, C))
    for j in range(taps):
        y += padded[j:j + T] * taps_weight[:, j]
    return y


def channel_delta_scan(q, k, v, beta, g, state=None):
    """q, k, g [T, H, D], v [T, H, Vd], beta [T, H].  Per head and token:
    S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, H, D = q.shape
    Vd = v.shape[2]
    S = np.zeros((H, D, Vd)) if state is None else state.copy()
    o = np.zeros((T, H, Vd))
    for t in range(T):
        for h in range(H):
            S[h] = g[t, h][:, None] * S[h]
            u = beta[t, h] * (v[t, h] - S[h].T @ k[t, h])
            S[h] = S[h] + np.outer(k[t, h], u)
            o[t, h] = S[h].T @ q[t, h]
    return o, S


def channel_delta_mixer(h, P, m, eps):
    T = h.shape[0]
    H, G, D, Vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rep = H // G
    q = silu(short_filter(h @ P["q"].T, P["q.conv"])).reshape(T, G, D)
    k = silu(short_filter(h @ P["k"].T, P["k.conv"])).reshape(T, G, D)
    v = silu(short_filter(h @ P["v"].T, P["v.conv"])).reshape(T, H, Vd)
    q = np.repeat(unit(q, 1e-6) * D ** -0.5, rep, axis=1)
    k = np.repeat(unit(k, 1e-6), rep, axis=1)
    beta = sigmoid(h @ P["b"].T)
    step = softplus((h @ P["a1"].T) @ P["a2"].T + P["dt_bias"]).reshape(T, H, D)
    g = np.exp(-np.exp(P["A_log"])[None, :, None] * step)
    o, _ = channel_delta_scan(q, k, v, beta, g)
    gate = sigmoid((h @ P["g1"].T) @ P["g2"].T).reshape(T, H, Vd)
    o = rms_scale(o, eps) * P["norm"] * gate
    return o.reshape(T, H * Vd) @ P["o"].T


def decayed_outer_scan(q, k, v, alpha, state=None):
    """q, k, alpha [T, H, D], v [T, H, Vd].  Per head and token: S <- diag(alpha) S + k v^T,
    then o = S^T q (the read-out sees the token's own write)."""
    T, H, D = q.shape
    Vd = v.shape[2]
    S = np.zeros((H, D, Vd)) if state is None else state.copy()
    o = np.zeros((T, H, Vd))
    for t in range(T):
        for h in range(H):
            S[h] = alpha[t, h][:, None] * S[h] + np.outer(k[t, h], v[t, h])
            o[t, h] = S[h].T @ q[t, h]
    return o, S


def gated_linear_mixer(h, P, m, eps):
    """The right branch."""
    T = h.shape[0]
    H, D, Vd = m["heads"], m["dim"], m["vdim"]
    q = (h @ P["q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ P["k"].T).reshape(T, H, D)
    v = (h @ P["v"].T).reshape(T, H, Vd)
    z = (h @ P["a1"].T) @ P["a2"].T + P["a2.b"]
    alpha = (sigmoid(z) ** (1.0 / m["tau"])).reshape(T, H, D)
    o, _ = decayed_outer_scan(q, k, v, alpha)
    o = rms_norm(o, P["norm"], eps).reshape(T, H * Vd) * silu(h @ P["g"].T)
    return o @ P["o"].T


def two_branch_mixer(h, P, m, eps):
    left = tempered_attention_mixer(h, sub(P, "left."), m["left"], eps)
    right = gated_linear_mixer(h, sub(P, "right."), m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


# ---- feed-forward
def route_all(z, top):
    """z [experts]: softmax over all of them; (the ``top`` largest, the lower index first among
    equals; their probabilities as they are)."""
    p = np.exp(z - z.max())
    p = p / p.sum()
    order = sorted(range(len(z)), key=lambda e: (-p[e], e))[:top]
    return order, p[order]


def routed_ffn(h, P, mlp):
    out = np.zeros((h.shape[0], P["e0.down"].shape[0]))
    z = h @ P["router"].T
    for t in range(h.shape[0]):
        chosen, weights = route_all(z[t], mlp["router"]["top"])
        for e, wt in zip(chosen, weights):
            out[t] += wt * (gelu_erf(h[t] @ P[f"e{e}.up"].T) @ P[f"e{e}.down"].T)
    return out


# ---- the model
def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


MIXERS = {
    "attention": lambda h, P, m, eps: windowed_attention_mixer(h, P, m),
    "channel_delta": channel_delta_mixer,
    "parallel": two_branch_mixer,
}


def forward(config, tensors, tokens, return_layers=False):
    """Logits [T, vocab] of a whole sequence; with ``return_layers`` also the residual stream after
    every layer."""
    tokens = np.asarray(tokens)
    eps = config["norm"]["eps"]
    x = tensors["embed"][tokens] * config["embedding"]["scale"]
    layers = []
    for i, layer in enumerate(config["layers"]):
        src = i
        while "weights_of" in config["layers"][src]:          # the layer whose tensors this one runs
            src = config["layers"][src]["weights_of"]
        y = MIXERS[layer["type"]](rms_norm(x, tensors[f"l{src}.norm1"], eps), sub(tensors, f"l{src}.mix."), layer["mixer"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            y = y + routed_ffn(rms_norm(x, tensors[f"l{src}.norm2"], eps), sub(tensors, f"l{src}.mlp."), mlp)
        x = x + y
        layers.append(x.copy())
    logits = rms_norm(x, tensors["final.norm"], eps) @ tensors["head"].T
    return (logits, layers) if return_layers else logits


def load_folder(folder):
    """(config.json object, {tensor name: float64 array}) of a model folder; the safetensors file
    is read here, by hand: 8 bytes of header length, the JSON header, then the data."""
    import json
    import os
    import struct
    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    tensors = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw = data[lo:hi]
        if info["dtype"] == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif info["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4")
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
        tensors[name] = a.astype(np.float64).reshape(info["shape"])
    return config, tensors


def generate(config, tensors, prompt, n, stop=()):
    """Greedy continuation: (tokens, reason); the first largest logit wins; a stop token ends the
    run and is the last token returned."""
    toks, out = list(prompt), []
    for _ in range(n):
        nxt = int(np.argmax(forward(config, tensors, toks)[-1]))
        out.append(nxt)
        if nxt in stop:
            return out, "stop"
        toks.append(nxt)
    return out, "length"
