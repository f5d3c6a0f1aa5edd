"""Nogosun: configuration, plan, tensor names.

A decoder of parallel blocks with two RMS norms a layer: x += mixer(norm1(x)) + ffn(norm2(x)), both
norms of the same x, weights as stored.  The configuration lists the layers one by one; a layer with
``weights_of: j`` runs layer j's tensors (j before or after it) with a cache and state of its own.  Three mixers:

* ``attention``: grouped-query softmax attention whose values are its keys as projected (no value
  matrix), biases on q and k, the first ``rot.dims`` dims of every head rotated in the half layout
  with frequencies blended along the index and stretched cosines and sines (``rot.scaling``), a
  sliding window beside which the sequence's first ``mask.keep_first`` positions stay visible.
* ``channel_delta``: a delta rule with a decay per head and key channel made by a two-matrix
  projection, short causal filters with SiLU on q, k and v, unit q and k, a norm and a sigmoid gate
  (two matrices again) on the read-out.
* ``parallel``: two mixers on the same input, each times a factor: ``left``, causal softmax
  attention with biases, q/k norm, a factor on the query that grows with the position, capped
  scores, one added to the softmax's denominator and a sigmoid gate on the heads' outputs; ``right``,
  gated linear attention with a decay per key channel, read after the token's own write.

The feed-forward routes every token to ``top`` of ``experts`` small layers down gelu(up h) (exact
GELU), weighted by their shares of the softmax over all experts; or there is none (``mlp: null``).

config.json::

    {"architecture": "Nogosun", "vocab": V, "width": W, "embedding": {"scale": s}, "norm": {"eps": e},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size", "keep_first"},
                           "rot": {"base", "dims", "scaling": null | {"factor", "original", "fast", "slow"}}},
                 "mlp": null | {"kind": "moe", "router": {"experts", "top"}, "expert": {"ff"}}},
                {"type": "channel_delta", "mixer": {"heads", "kv_heads", "dim", "vdim", "conv"}, "mlp": ...},
                {"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap", "q_temp": {"coef", "every"}},
                           "right": {"heads", "dim", "vdim", "tau"}, "left_scale", "right_scale"}, "mlp": ...},
                {"type": ..., "weights_of": j, ...}, ...]}

Tensors: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``final.norm``, ``head``;
``l<i>.mix.{q,q.b,k,k.b,o}`` (attention);
``l<i>.mix.{q,q.conv,k,k.conv,v,v.conv,b,A_log,a1,a2,dt_bias,g1,g2,norm,o}`` (channel_delta);
``l<i>.mix.left.{q,q.b,k,k.b,v,v.b,q.norm,k.norm,g,o}`` and
``l<i>.mix.right.{q,k,v,g,o,norm,a1,a2,a2.b}`` (parallel);
``l<i>.mlp.{router,e<j>.up,e<j>.down}``.  The inner sizes of the two-matrix projections (rows of
``a1``, ``g1``) are read from the checkpoint's shapes; a configuration without a checkpoint (random
weights) may name them as ``mixer.decay_rank``, ``mixer.gate_rank`` and ``mixer.right.rank``.

This module is all that knows the architecture: it turns the configuration into a ``ModelPlan`` of
generic parts (``parallel`` block with a norm of its own for the feed-forward, ``capped_attention``,
``channel_delta``, ``gated_linear``, ``side_by_side``, ``moe`` without gates, ``rmsnorm``, ``rotary``).
"""
from __future__ import annotations

import dataclasses
from typing import Tuple

from ..config.base import ConfigError, ModelConfig
from ..config.registry import register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry

MIXERS = ("attention", "channel_delta", "parallel")
#: inner size of a two-matrix projection when neither a checkpoint nor the configuration gives one
DEFAULT_RANK = 16


def _num(problems, where, obj, name, kind=int, allow_zero=False, optional=False):
    v = obj.get(name) if isinstance(obj, dict) else None
    if v is None and optional:
        return None
    if kind is int and isinstance(v, float) and v.is_integer():
        v = int(v)                                   # a count written as 256.0
    ok = isinstance(v, int) and not isinstance(v, bool) if kind is int else (
        isinstance(v, (int, float)) and not isinstance(v, bool))
    if not ok:
        problems.append(f"{where}.{name}: expected {'an integer' if kind is int else 'a number'}, got {v!r}")
        return None
    if v < 0 or (v == 0 and not allow_zero):
        problems.append(f"{where}.{name}: must be positive, got {v!r}")
        return None
    return kind(v)


def _check_heads(p, w, m, kv=True):
    heads = _num(p, w, m, "heads")
    _num(p, w, m, "dim")
    _num(p, w, m, "vdim")
    if kv:
        g = _num(p, w, m, "kv_heads")
        if heads and g and heads % g:
            p.append(f"{w}: {heads} heads are not a multiple of {g} kv_heads")


def _check_attention(p, w, m):
    _check_heads(p, w, m)
    _num(p, w, m, "scale", float)
    if m.get("dim") != m.get("vdim"):
        p.append(f"{w}: the values are the keys, so vdim ({m.get('vdim')!r}) must equal dim ({m.get('dim')!r})")
    mask = m.get("mask")
    if mask is not None:
        _num(p, w + ".mask", mask, "size")
        _num(p, w + ".mask", mask, "keep_first", allow_zero=True, optional=True)
    rot = m.get("rot")
    if rot is not None:
        dims = _num(p, w + ".rot", rot, "dims", allow_zero=True)
        if dims:
            _num(p, w + ".rot", rot, "base", float)
            if isinstance(m.get("dim"), int) and (dims % 2 or dims > m["dim"]):
                p.append(f"{w}.rot.dims: {dims} is odd or more than dim ({m['dim']})")
        scaling = rot.get("scaling") if isinstance(rot, dict) else None
        if scaling is not None:
            for name in ("factor", "original", "fast", "slow"):
                _num(p, w + ".rot.scaling", scaling, name, float)


def _check_parallel(p, w, m):
    left, right = m.get("left"), m.get("right")
    if not isinstance(left, dict) or not isinstance(right, dict):
        p.append(f"{w}: expected the objects left and right")
        return
    _check_heads(p, w + ".left", left)
    _num(p, w + ".left", left, "scale", float)
    _num(p, w + ".left", left, "softcap", float, allow_zero=True, optional=True)
    if left.get("q_temp") is not None:
        _num(p, w + ".left.q_temp", left["q_temp"], "coef", float, allow_zero=True)
        _num(p, w + ".left.q_temp", left["q_temp"], "every")
    _check_heads(p, w + ".right", right, kv=False)
    _num(p, w + ".right", right, "tau", float)
    _num(p, w + ".right", right, "rank", optional=True)
    _num(p, w, m, "left_scale", float, allow_zero=True)
    _num(p, w, m, "right_scale", float, allow_zero=True)


def _check_mlp(p, w, mlp):
    if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
        got = mlp.get("kind") if isinstance(mlp, dict) else mlp
        p.append(f"{w}.kind: unknown feed-forward {got!r} (known: moe)")
        return
    experts = _num(p, w + ".router", mlp.get("router"), "experts")
    top = _num(p, w + ".router", mlp.get("router"), "top")
    if experts and top and top > experts:
        p.append(f"{w}.router.top: {top} of {experts} experts")
    _num(p, w + ".expert", mlp.get("expert"), "ff")


@dataclasses.dataclass(frozen=True)
class NogosunConfig(ModelConfig):
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    #: one entry per layer, as config.json lists them (checked; plain dicts)
    layers: Tuple[dict, ...]

    @classmethod
    def from_dict(cls, raw):
        if not isinstance(raw, dict):
            raise ConfigError("config.json: the top level must be an object")
        p = []
        vocab = _num(p, "config", raw, "vocab")
        width = _num(p, "config", raw, "width")
        emb = _num(p, "embedding", raw.get("embedding"), "scale", float)
        eps = _num(p, "norm", raw.get("norm"), "eps", float)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            p.append("layers: expected a list of at least one layer")
            layers = []
        for i, layer in enumerate(layers):
            w = f"layers[{i}]"
            if not isinstance(layer, dict):
                p.append(f"{w}: expected an object")
                continue
            kind, m = layer.get("type"), layer.get("mixer")
            if kind not in MIXERS:
                p.append(f"{w}.type: unknown mixer {kind!r} (known: {', '.join(MIXERS)})")
                continue
            if not isinstance(m, dict):
                p.append(f"{w}.mixer: expected an object")
                continue
            if kind == "attention":
                _check_attention(p, w + ".mixer", m)
            elif kind == "channel_delta":
                _check_heads(p, w + ".mixer", m)
                _num(p, w + ".mixer", m, "conv")
                _num(p, w + ".mixer", m, "decay_rank", optional=True)
                _num(p, w + ".mixer", m, "gate_rank", optional=True)
            else:
                _check_parallel(p, w + ".mixer", m)
            if layer.get("mlp") is not None:
                _check_mlp(p, w + ".mlp", layer["mlp"])
            if "weights_of" in layer:
                j = layer["weights_of"]
                if (not isinstance(j, int) or isinstance(j, bool) or not 0 <= j < len(layers) or j == i
                        or not isinstance(layers[j], dict)):
                    p.append(f"{w}.weights_of: {j!r} is not another layer")
                elif layers[j].get("type") != kind:
                    p.append(f"{w}.weights_of: layer {j} is a {layers[j].get('type')!r} layer, this one {kind!r}")
                else:
                    seen, at = {i}, j            # the chain of owners must end at a layer with tensors of its own
                    while isinstance(layers[at], dict) and "weights_of" in layers[at] and at not in seen:
                        seen.add(at)
                        nxt = layers[at]["weights_of"]
                        if not isinstance(nxt, int) or isinstance(nxt, bool) or not 0 <= nxt < len(layers):
                            break
                        at = nxt
                    if isinstance(layers[at], dict) and "weights_of" in layers[at]:
                        p.append(f"{w}.weights_of: the layers that share tensors name one another in a circle")
        if p:
            raise ConfigError("config.json: " + "; ".join(p))
        return cls(vocab=vocab, width=width, embedding_scale=emb, norm_eps=eps, layers=tuple(layers))

    def to_dict(self):
        return {"architecture": "Nogosun", "vocab": self.vocab, "width": self.width,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
                "layers": [dict(layer) for layer in self.layers]}


def owner(cfg, i: int) -> int:
    """The layer whose tensors layer ``i`` runs: itself, or the end of its chain of ``weights_of``."""
    while "weights_of" in cfg.layers[i]:
        i = int(cfg.layers[i]["weights_of"])
    return i


def _rank(m: dict, key: str, tensor: str, shapes) -> int:
    """Inner size of a two-matrix projection: the configuration's ``key`` if it has one, else the
    rows of the checkpoint's first matrix, else DEFAULT_RANK."""
    if m.get(key) is not None:
        return int(m[key])
    shape = shapes.get(tensor) if isinstance(shapes, dict) else None
    return int(shape[0]) if shape else DEFAULT_RANK


def _attention_spec(cfg, m, prefix) -> PartSpec:
    rot = m.get("rot") or {}
    dims = int(rot.get("dims") or 0)
    position = None
    if dims:
        position = PartSpec("rotary", {"head_dim": int(m["dim"]), "rotary_dim": dims, "theta": float(rot["base"]),
                                       "layout": "half", "scaling": rot.get("scaling")})
    mask = m.get("mask") or {}
    names = {"q": prefix + "q", "k": prefix + "k", "o": prefix + "o", "q_bias": prefix + "q.b", "k_bias": prefix + "k.b"}
    return PartSpec("capped_attention", {
        "hidden_size": cfg.width, "heads": int(m["heads"]), "kv_heads": int(m["kv_heads"]), "dim": int(m["dim"]),
        "vdim": int(m["vdim"]), "bias": True, "values_are_keys": True, "scale": float(m["scale"]),
        "window": int(mask["size"]) if mask.get("size") else None, "keep_first": int(mask.get("keep_first") or 0),
        "position": position}, names)


def _channel_delta_spec(cfg, m, prefix, shapes) -> PartSpec:
    names = {k: prefix + k for k in ("q", "k", "v", "b", "a1", "a2", "g1", "g2", "o", "A_log", "dt_bias", "norm")}
    names.update({f"{s}_conv": f"{prefix}{s}.conv" for s in ("q", "k", "v")})
    return PartSpec("channel_delta", {
        "hidden_size": cfg.width, "heads": int(m["heads"]), "kv_heads": int(m["kv_heads"]), "dim": int(m["dim"]),
        "vdim": int(m["vdim"]), "conv": int(m["conv"]), "decay_rank": _rank(m, "decay_rank", prefix + "a1", shapes),
        "gate_rank": _rank(m, "gate_rank", prefix + "g1", shapes), "norm_eps": cfg.norm_eps}, names)


def _parallel_spec(cfg, m, prefix, shapes) -> PartSpec:
    left, right = m["left"], m["right"]
    lp, rp = prefix + "left.", prefix + "right."
    lnames = {k: lp + k for k in ("q", "k", "v", "g", "o")}
    lnames.update({"q_bias": lp + "q.b", "k_bias": lp + "k.b", "v_bias": lp + "v.b", "q_norm": lp + "q.norm",
                   "k_norm": lp + "k.norm"})
    lspec = PartSpec("capped_attention", {
        "hidden_size": cfg.width, "heads": int(left["heads"]), "kv_heads": int(left["kv_heads"]), "dim": int(left["dim"]),
        "vdim": int(left["vdim"]), "bias": True, "scale": float(left["scale"]), "softcap": float(left.get("softcap") or 0.0),
        "window": None, "gate": True, "qk_norm": cfg.norm_eps, "fixed_sink": 0.0,
        "q_temper": dict(left["q_temp"]) if left.get("q_temp") else None, "position": None}, lnames)
    rnames = {k: rp + k for k in ("q", "k", "v", "g", "o", "norm", "a1", "a2")}
    rnames["a2_bias"] = rp + "a2.b"
    rspec = PartSpec("gated_linear", {
        "hidden_size": cfg.width, "heads": int(right["heads"]), "dim": int(right["dim"]), "vdim": int(right["vdim"]),
        "rank": _rank(right, "rank", rp + "a1", shapes), "tau": float(right["tau"]), "norm_eps": cfg.norm_eps}, rnames)
    return PartSpec("side_by_side", {"branches": [{"name": "left", "spec": lspec, "scale": float(m["left_scale"])},
                                                  {"name": "right", "spec": rspec, "scale": float(m["right_scale"])}]})


def _ffn_spec(cfg, mlp, prefix) -> PartSpec:
    experts = int(mlp["router"]["experts"])
    names = {"router": prefix + "router"}
    for e in range(experts):
        names[f"e{e}.up"] = f"{prefix}e{e}.up"
        names[f"e{e}.down"] = f"{prefix}e{e}.down"
    return PartSpec("moe", {"hidden_size": cfg.width, "experts": experts, "top": int(mlp["router"]["top"]),
                            "ff": int(mlp["expert"]["ff"]), "limit": None, "router_bias": False, "gated": False,
                            "routing": "softmax_all", "shared": None}, names)


def build_plan(cfg: NogosunConfig, names=None) -> ModelPlan:
    """``names``: the checkpoint's {tensor name: shape} (None: no checkpoint yet)."""
    def norm(name):
        return PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps}, {"weight": name})

    layers, place, ignored = [], {}, []
    for i, layer in enumerate(cfg.layers):
        if "weights_of" in layer:
            continue
        m, prefix = layer["mixer"], f"l{i}.mix."
        if layer["type"] == "attention":
            mixer = _attention_spec(cfg, m, prefix)
        elif layer["type"] == "channel_delta":
            mixer = _channel_delta_spec(cfg, m, prefix, names)
        else:
            mixer = _parallel_spec(cfg, m, prefix, names)
        parts = {"norm": norm(f"l{i}.norm1"), "mixer": mixer}
        if layer.get("mlp") is not None:
            parts["ffn_norm"] = norm(f"l{i}.norm2")
            parts["ffn"] = _ffn_spec(cfg, layer["mlp"], f"l{i}.mlp.")
        else:
            ignored.append(f"l{i}.norm2")          # a layer without feed-forward has no use for its second norm
        place[i] = len(layers)
        layers.append(LayerSpec(parts, "parallel"))
    # every run of a layer, with tensors of its own or another layer's (named before or after it), keeps its own cache
    schedule = [ScheduleEntry(place[owner(cfg, i)]) for i in range(len(cfg.layers))]
    plan = ModelPlan(
        hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "scale": cfg.embedding_scale},
                           {"weight": "embed"}),
        layers=layers, schedule=schedule, final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width}, {"weight": "head"}),
        max_positions=0, stop_ids=[], ignored_tensors=ignored)
    plan.validate()
    return plan


def checkpoint_layout(cfg: NogosunConfig) -> dict:
    """{tensor name: (shape, kind)} of a complete checkpoint (kind as weights.random_init reads it)."""
    w = cfg.width
    out = {"embed": ((cfg.vocab, w), "matrix")}
    for i, layer in enumerate(cfg.layers):
        if "weights_of" in layer:
            continue
        out[f"l{i}.norm1"] = ((w,), "norm")
        m, p = layer["mixer"], f"l{i}.mix."
        if layer["type"] == "attention":
            nh, g, d = (int(m[x]) for x in ("heads", "kv_heads", "dim"))
            out.update({p + "q": ((nh * d, w), "matrix"), p + "q.b": ((nh * d,), "bias"), p + "k": ((g * d, w), "matrix"),
                        p + "k.b": ((g * d,), "bias"), p + "o": ((w, nh * d), "matrix")})
        elif layer["type"] == "channel_delta":
            nh, g, d, vd, taps = (int(m[x]) for x in ("heads", "kv_heads", "dim", "vdim", "conv"))
            ra, rg = _rank(m, "decay_rank", p + "a1", None), _rank(m, "gate_rank", p + "g1", None)
            for s, rows in (("q", g * d), ("k", g * d), ("v", nh * vd)):
                out[p + s] = ((rows, w), "matrix")
                out[f"{p}{s}.conv"] = ((rows, taps), "filter")
            out.update({p + "b": ((nh, w), "matrix"), p + "A_log": ((nh,), "log_rate"), p + "norm": ((vd,), "norm"),
                        p + "a1": ((ra, w), "matrix"), p + "a2": ((nh * d, ra), "lowrank"), p + "dt_bias": ((nh * d,), "small"),
                        p + "g1": ((rg, w), "matrix"), p + "g2": ((nh * vd, rg), "lowrank"), p + "o": ((w, nh * vd), "matrix")})
        else:
            left, right = m["left"], m["right"]
            nh, g, d, vd = (int(left[x]) for x in ("heads", "kv_heads", "dim", "vdim"))
            lp, rp = p + "left.", p + "right."
            for s, rows in (("q", nh * d), ("k", g * d), ("v", g * vd)):
                out[lp + s] = ((rows, w), "matrix")
                out[f"{lp}{s}.b"] = ((rows,), "bias")
            out.update({lp + "q.norm": ((d,), "norm"), lp + "k.norm": ((d,), "norm"), lp + "g": ((nh * vd, w), "matrix"),
                        lp + "o": ((w, nh * vd), "matrix")})
            rh, rd, rv = (int(right[x]) for x in ("heads", "dim", "vdim"))
            rank = _rank(right, "rank", rp + "a1", None)
            out.update({rp + "q": ((rh * rd, w), "matrix"), rp + "k": ((rh * rd, w), "matrix"), rp + "v": ((rh * rv, w), "matrix"),
                        rp + "g": ((rh * rv, w), "matrix"), rp + "o": ((w, rh * rv), "matrix"), rp + "norm": ((rv,), "norm"),
                        rp + "a1": ((rank, w), "matrix"), rp + "a2": ((rh * rd, rank), "lowrank"),
                        rp + "a2.b": ((rh * rd,), "bonus")})
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        out[f"l{i}.norm2"] = ((w,), "norm")
        p = f"l{i}.mlp."
        ff, experts = int(mlp["expert"]["ff"]), int(mlp["router"]["experts"])
        for e in range(experts):
            out[f"{p}e{e}.up"] = ((ff, w), "matrix")
            out[f"{p}e{e}.down"] = ((w, ff), "matrix")
        out[p + "router"] = ((experts, w), "matrix")
    out["final.norm"] = ((w,), "norm")
    out["head"] = ((cfg.vocab, w), "matrix")
    return out


register_architecture(["Nogosun", "nogosun"], NogosunConfig, build_plan, checkpoint_layout)
