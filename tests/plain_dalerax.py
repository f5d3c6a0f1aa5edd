"""Dalerax in plain numpy float64, one function per mechanism, whole sequences only.

It shares nothing with the package: it reads a config.json object and a {tensor name: array}
dictionary and walks a sequence from its first token.  Attention builds the full score matrix
and the full mask; the recurrent mixer runs token by token exactly as its update is written.

Notation: T tokens, W model width; ``h`` [T, W] is a layer's normed input; a matrix M stored
[out, in] is applied as ``h @ M.T``.
"""
import math

import numpy as np


# ---- small functions
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def rms_scale(x, eps):
    """x divided by sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose stored weight is a deviation from one."""
    return rms_scale(x, eps) * (1.0 + w)


# ---- rotation
def rotary_frequencies(base, dims, scaling=None):
    """f_i = base^(-2i/dims), i < dims/2; with ``scaling`` the long wavelengths are stretched:
    unchanged below original/high, divided by factor above original/low, blended in between."""
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])
    if not scaling:
        return f
    factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = np.empty_like(f)
    for i, fi in enumerate(f):
        wavelength = 2.0 * math.pi / fi
        if wavelength < original / high:
            out[i] = fi
        elif wavelength > original / low:
            out[i] = fi / factor
        else:
            s = (original / wavelength - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out


def rotate_half(x, positions, freq):
    """x [T, H, D]: dimension i < len(freq) pairs with dimension i + len(freq) and the pair turns
    by positions * freq[i]; dimensions from 2 len(freq) on pass unchanged."""
    half = len(freq)
    if half == 0:
        return x
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:2 * half]
    out = x.copy()
    out[..., :half] = a * c - b * s
    out[..., half:2 * half] = b * c + a * s
    return out


# ---- attention
def visible(i, j, size, keep_first):
    """Whether the query at position i sees the key at position j."""
    return j <= i and (i - j < size or j < keep_first)


def sink_attention(q, k, v, q_pos, k_pos, scale, size, keep_first, sink):
    """q [Tq, H, D], k [Tk, G, D], v [Tk, G, Vd]; head h reads kv head h // (H / G).  The softmax's
    denominator holds one more term, exp(sink[h]), that weighs no value."""
    tq, H, _ = q.shape
    G, vd = k.shape[1], v.shape[2]
    out = np.zeros((tq, H, vd))
    for a in range(tq):
        seen = [b for b in range(len(k_pos)) if visible(q_pos[a], k_pos[b], size, keep_first)]
        for h in range(H):
            g = h // (H // G)
            s = np.array([np.dot(q[a, h], k[b, g]) * scale for b in seen])
            top = max(s.max(), sink[h])
            e = np.exp(s - top)
            den = e.sum() + math.exp(sink[h] - top)
            out[a, h] = (e / den) @ v[seen, g]
    return out


def attention_mixer(h, P, m, borrowed=None):
    """Returns (output [T, W], (rotated keys, values)).  ``borrowed``: another layer's (keys,
    values) to read in place of this layer's own."""
    T = h.shape[0]
    H, G, D, Vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(T)
    freq = rotary_frequencies(m["rot"]["base"], m["rot"]["dims"], m["rot"].get("scaling")) if m["rot"]["dims"] else np.zeros(0)
    q = rotate_half((h @ P["q"].T).reshape(T, H, D), pos, freq)
    if borrowed is None:
        k = rotate_half((h @ P["k"].T).reshape(T, G, D), pos, freq)
        v = (h @ P["v"].T).reshape(T, G, Vd)
    else:
        k, v = borrowed
    o = sink_attention(q, k, v, pos, pos, m["scale"], m["mask"]["size"], m["mask"]["keep_first"], P["sink"])
    return o.reshape(T, H * Vd) @ P["o"].T, (k, v)


# ---- linear attention with decays
def shifted(h, before=None):
    """Row t is h[t - 1]; row 0 is ``before`` (zeros for a sequence's start)."""
    first = np.zeros((1, h.shape[1])) if before is None else np.asarray(before).reshape(1, -1)
    return np.concatenate([first, h[:-1]], axis=0)


def wkv_scan(r, k, v, w, u, state=None):
    """r, k, w [T, H, D], v [T, H, Vd], u [H, D].  Per head, for each token in turn:
    y = (S + diag(u) k v^T)^T r, then S <- diag(w) S + k v^T.  Returns (y [T, H, Vd], S)."""
    T, H, D = r.shape
    S = np.zeros((H, D, v.shape[2])) if state is None else state.copy()
    y = np.zeros((T, H, v.shape[2]))
    for t in range(T):
        for h in range(H):
            kv = np.outer(k[t, h], v[t, h])
            y[t, h] = (S[h] + u[h][:, None] * kv).T @ r[t, h]
            S[h] = w[t, h][:, None] * S[h] + kv
    return y, S


def wkv_mixer(h, P, m, eps):
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    prev = shifted(h)
    blend = {s: h + (prev - h) * P["mu." + s] for s in ("r", "k", "v", "g", "w")}
    r = (blend["r"] @ P["r"].T).reshape(T, H, D)
    k = (blend["k"] @ P["k"].T).reshape(T, H, D)
    v = (blend["v"] @ P["v"].T).reshape(T, H, D)
    gate = silu(blend["g"] @ P["g"].T)
    w = np.exp(-np.exp(np.tanh(blend["w"] @ P["w1"].T) @ P["w2"].T + P["w0"])).reshape(T, H, D)
    y, _ = wkv_scan(r, k, v, w, P["u"])
    y = rms_scale(y, eps).reshape(T, H * D) * P["norm"] * gate
    return y @ P["o"].T


# ---- feed-forward
def gated_ffn(h, P):
    return (silu(h @ P["gate"].T) * (h @ P["up"].T)) @ P["down"].T


def route(z, top):
    """z [experts]: (indices of the ``top`` largest, the lower index first among equals; softmax over them)."""
    order = sorted(range(len(z)), key=lambda e: (-z[e], e))[:top]
    e = np.exp(z[order] - z[order].max())
    return order, e / e.sum()


def routed_ffn(h, P, mlp):
    out = np.zeros((h.shape[0], P["e0.down"].shape[0]))
    z = h @ P["router"].T + P["router.b"]
    for t in range(h.shape[0]):
        chosen, weights = route(z[t], mlp["router"]["top"])
        for e, wt in zip(chosen, weights):
            out[t] += wt * gated_ffn(h[t:t + 1], sub(P, f"e{e}."))[0]
    if mlp.get("shared") is not None:
        out += gated_ffn(h, sub(P, "shared."))
    return out


# ---- the model
def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, tokens, return_layers=False):
    """Logits [T, vocab] of a whole sequence; with ``return_layers`` also the residual stream after
    every layer."""
    tokens = np.asarray(tokens)
    eps = config["norm"]["eps"]
    x = tensors["embed"][tokens] * config["embedding"]["scale"] + tensors["pos"][:len(tokens)]
    layers, kept = [], {}
    for i, layer in enumerate(config["layers"]):
        h = offset_norm(x, tensors[f"l{i}.norm1"], eps)
        m, P = layer["mixer"], sub(tensors, f"l{i}.mix.")
        if layer["type"] == "attention":
            y, kv = attention_mixer(h, P, m, kept[m["kv_from"]] if "kv_from" in m else None)
            kept[i] = kv
        else:
            y = wkv_mixer(h, P, m, eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            F = sub(tensors, f"l{i}.mlp.")
            y = y + (gated_ffn(h, F) if mlp["kind"] == "dense" else routed_ffn(h, F, mlp))
        x = x + y
        layers.append(x.copy())
    logits = offset_norm(x, tensors["final.norm"], eps) @ tensors["head"].T * config["logit_scale"]
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
