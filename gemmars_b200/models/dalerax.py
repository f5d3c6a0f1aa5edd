"""Dalerax: configuration, plan, tensor names.

A decoder of parallel blocks: one RMS norm a layer (its weight stored around zero), whose output
feeds a mixer and a feed-forward that both add into the residual stream.  The configuration lists
the layers one by one.  A layer's mixer is ``attention`` (grouped-query softmax attention over a
sliding window beside which the sequence's first tokens stay visible, a learned sink per head in
the softmax's denominator, part of each head rotated with stretched long wavelengths, and
optionally the keys and values of an earlier layer in place of its own) or ``wkv`` (linear
attention with a decay per key channel and mixes with the token before).  Its feed-forward is
dense (SiLU-gated), routed (top experts by router logits, softmax over the chosen, a shared expert
beside them), or absent.  A learned vector per position is added to the scaled token embedding;
the logits are multiplied by a constant.

config.json::

    {"architecture": "Dalerax", "vocab": V, "width": W, "max_positions": P, "logit_scale": s,
     "embedding": {"scale": e}, "norm": {"eps": e},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size", "keep_first"},
                           "rot": {"base", "dims", "scaling": null | {"factor", "low", "high", "original"}},
                           "kv_from": j (optional: the layer whose keys and values this one reads)},
                 "mlp": null | {"kind": "dense", "ff"}
                             | {"kind": "moe", "router": {"experts", "top"}, "expert": {"ff"}, "shared": null | {"ff"}}},
                {"type": "wkv", "mixer": {"heads", "dim"}, "mlp": ...}, ...]}

Tensors: ``embed``, ``pos``, ``l<i>.norm1``, ``l<i>.mix.{q,k,v,sink,o}`` (no k, v with ``kv_from``),
``l<i>.mix.{mu.{r,k,v,g,w},r,k,v,g,w1,w2,w0,u,norm,o}``, ``l<i>.mlp.{gate,up,down}`` or
``l<i>.mlp.{router,router.b,e<j>.{gate,up,down},shared.{gate,up,down}}``, ``final.norm``, ``head``.
The inner size of a wkv layer's decay (rows of ``w1``) is read from the checkpoint's shapes; a
configuration without a checkpoint (random weights) names it as ``mixer.rank``.

This module is all that knows the architecture: it turns the configuration into a ``ModelPlan``
of generic parts (``parallel`` block, ``capped_attention`` with a sink and kept first positions,
``wkv``, ``gated_mlp``, ``moe`` without clamps, ``rmsnorm`` with offset 1, ``rotary`` with scaling).
"""
from __future__ import annotations

import dataclasses
from typing import Tuple

from ..config.base import ConfigError, ModelConfig
from ..config.registry import register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry

MIXERS = ("attention", "wkv")
FFN_KINDS = ("dense", "moe")
#: inner size of a wkv layer's decay when neither a checkpoint nor the configuration gives one
DEFAULT_RANK = 32


def _num(problems, where, obj, name, kind=int, allow_zero=False):
    v = obj.get(name) if isinstance(obj, dict) else None
    ok = isinstance(v, int) and not isinstance(v, bool) if kind is int else (
        isinstance(v, (int, float)) and not isinstance(v, bool))
    if not ok:
        problems.append(f"{where}.{name}: expected {'an integer' if kind is int else 'a number'}, got {v!r}")
        return None
    if v < 0 or (v == 0 and not allow_zero):
        problems.append(f"{where}.{name}: must be positive, got {v!r}")
        return None
    return kind(v)


def _check_attention(p, w, m, i, layers):
    heads = _num(p, w, m, "heads")
    kv = _num(p, w, m, "kv_heads")
    dim = _num(p, w, m, "dim")
    _num(p, w, m, "vdim")
    _num(p, w, m, "scale", float)
    if heads and kv and heads % kv:
        p.append(f"{w}: {heads} heads are not a multiple of {kv} kv_heads")
    mask = m.get("mask")
    _num(p, w + ".mask", mask, "size")
    if isinstance(mask, dict) and "keep_first" in mask:      # absent: no first token is kept
        _num(p, w + ".mask", mask, "keep_first", allow_zero=True)
    rot = m.get("rot")
    _num(p, w + ".rot", rot, "base", float)
    dims = _num(p, w + ".rot", rot, "dims", allow_zero=True)
    if dims is not None and dim and (dims % 2 or dims > dim):
        p.append(f"{w}.rot.dims: {dims} is odd or more than dim ({dim})")
    scaling = rot.get("scaling") if isinstance(rot, dict) else None
    if scaling is not None:
        for name in ("factor", "low", "high", "original"):
            _num(p, w + ".rot.scaling", scaling, name, float)
    if "kv_from" in m:
        j = m["kv_from"]
        if not isinstance(j, int) or isinstance(j, bool) or not 0 <= j < i:
            p.append(f"{w}.kv_from: {j!r} is not a layer before this one")
            return
        other = layers[j] if isinstance(layers[j], dict) else {}
        om = other.get("mixer") if isinstance(other.get("mixer"), dict) else {}
        if other.get("type") != "attention" or "kv_from" in om:
            p.append(f"{w}.kv_from: layer {j} is not an attention layer with keys and values of its own")
            return
        for name in ("kv_heads", "dim", "vdim"):
            if om.get(name) != m.get(name):
                p.append(f"{w}.kv_from: {name} is {m.get(name)!r} here and {om.get(name)!r} in layer {j}")
        if om.get("rot") != m.get("rot"):
            p.append(f"{w}.kv_from: the rotation differs from layer {j}'s")


def _check_mlp(p, w, mlp):
    if not isinstance(mlp, dict) or mlp.get("kind") not in FFN_KINDS:
        got = mlp.get("kind") if isinstance(mlp, dict) else mlp
        p.append(f"{w}.kind: unknown feed-forward {got!r} (known: {', '.join(FFN_KINDS)})")
        return
    if mlp["kind"] == "dense":
        _num(p, w, mlp, "ff")
        return
    experts = _num(p, w + ".router", mlp.get("router"), "experts")
    top = _num(p, w + ".router", mlp.get("router"), "top")
    if experts and top and top > experts:
        p.append(f"{w}.router.top: {top} of {experts} experts")
    _num(p, w + ".expert", mlp.get("expert"), "ff")
    if mlp.get("shared") is not None:
        _num(p, w + ".shared", mlp.get("shared"), "ff")


@dataclasses.dataclass(frozen=True)
class DaleraxConfig(ModelConfig):
    vocab: int
    width: int
    max_positions: int
    logit_scale: float
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
        max_positions = _num(p, "config", raw, "max_positions")
        logit_scale = _num(p, "config", raw, "logit_scale", float)
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
                _check_attention(p, w + ".mixer", m, i, layers)
            else:
                _num(p, w + ".mixer", m, "heads")
                _num(p, w + ".mixer", m, "dim")
                if "rank" in m:
                    _num(p, w + ".mixer", m, "rank")
            if layer.get("mlp") is not None:
                _check_mlp(p, w + ".mlp", layer["mlp"])
        if p:
            raise ConfigError("config.json: " + "; ".join(p))
        return cls(vocab=vocab, width=width, max_positions=max_positions, logit_scale=logit_scale, embedding_scale=emb,
                   norm_eps=eps, layers=tuple(layers))

    def to_dict(self):
        return {"architecture": "Dalerax", "vocab": self.vocab, "width": self.width, "max_positions": self.max_positions,
                "logit_scale": self.logit_scale, "embedding": {"scale": self.embedding_scale},
                "norm": {"eps": self.norm_eps}, "layers": [dict(layer) for layer in self.layers]}


def _shared_caches(cfg) -> set:
    """Layers whose keys and values another layer reads, and those readers."""
    out = set()
    for i, layer in enumerate(cfg.layers):
        if layer["type"] == "attention" and "kv_from" in layer["mixer"]:
            out.update((i, int(layer["mixer"]["kv_from"])))
    return out


def _attention_spec(cfg, m, prefix, shared: bool) -> PartSpec:
    dims = int(m["rot"]["dims"])
    position = None
    if dims:
        position = PartSpec("rotary", {"head_dim": int(m["dim"]), "rotary_dim": dims, "theta": float(m["rot"]["base"]),
                                       "layout": "half", "scaling": m["rot"].get("scaling")})
    has_kv = "kv_from" not in m
    names = {k: prefix + k for k in (("q", "k", "v", "o", "sink") if has_kv else ("q", "o", "sink"))}
    return PartSpec("capped_attention", {
        "hidden_size": cfg.width, "heads": int(m["heads"]), "kv_heads": int(m["kv_heads"]), "dim": int(m["dim"]),
        "vdim": int(m["vdim"]), "window": int(m["mask"]["size"]), "keep_first": int(m["mask"].get("keep_first", 0)),
        "sink": True, "scale": float(m["scale"]), "position": position, "has_kv": has_kv,
        # a cache that several layers read keeps every page: each reader masks for itself
        "ring": not shared}, names)


def wkv_rank(m: dict, prefix: str, shapes) -> int:
    """Inner size of the decay's two matrices: the configuration's ``rank`` if it has one, else the
    rows of the checkpoint's ``w1``, else DEFAULT_RANK."""
    if "rank" in m:
        return int(m["rank"])
    shape = shapes.get(prefix + "w1") if isinstance(shapes, dict) else None
    return int(shape[0]) if shape else DEFAULT_RANK


def _wkv_spec(cfg, m, prefix, shapes) -> PartSpec:
    names = {k: prefix + k for k in ("r", "k", "v", "g", "w1", "w2", "w0", "u", "norm", "o")}
    names.update({f"mu_{s}": f"{prefix}mu.{s}" for s in ("r", "k", "v", "g", "w")})
    return PartSpec("wkv", {"hidden_size": cfg.width, "heads": int(m["heads"]), "dim": int(m["dim"]),
                            "rank": wkv_rank(m, prefix, shapes), "norm_eps": cfg.norm_eps}, names)


def _ffn_spec(cfg, mlp, prefix) -> PartSpec:
    if mlp["kind"] == "dense":
        return PartSpec("gated_mlp", {"hidden_size": cfg.width, "intermediate_size": int(mlp["ff"]), "activation": "silu"},
                        {k: prefix + k for k in ("gate", "up", "down")})
    experts = int(mlp["router"]["experts"])
    shared = mlp.get("shared")
    names = {"router": prefix + "router", "router_bias": prefix + "router.b"}
    for e in range(experts):
        for part in ("gate", "up", "down"):
            names[f"e{e}.{part}"] = f"{prefix}e{e}.{part}"
    if shared is not None:
        for part in ("gate", "up", "down"):
            names[f"shared.{part}"] = f"{prefix}shared.{part}"
    # the experts are the plain gated form: no clamps, silu(g) * u
    return PartSpec("moe", {"hidden_size": cfg.width, "experts": experts, "top": int(mlp["router"]["top"]),
                            "ff": int(mlp["expert"]["ff"]), "limit": None, "alpha": 1.0, "shift": 0.0, "router_bias": True,
                            "shared": None if shared is None else {"ff": int(shared["ff"]), "limit": None, "gate": False}},
                    names)


def build_plan(cfg: DaleraxConfig, names=None) -> ModelPlan:
    """``names``: the checkpoint's {tensor name: shape} (None: no checkpoint yet)."""
    def norm(name):
        return PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "offset": 1.0}, {"weight": name})

    shared = _shared_caches(cfg)
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        m, prefix = layer["mixer"], f"l{i}.mix."
        mixer = (_attention_spec(cfg, m, prefix, i in shared) if layer["type"] == "attention"
                 else _wkv_spec(cfg, m, prefix, names))
        parts = {"norm": norm(f"l{i}.norm1"), "mixer": mixer}
        if layer.get("mlp") is not None:
            parts["ffn"] = _ffn_spec(cfg, layer["mlp"], f"l{i}.mlp.")
        layers.append(LayerSpec(parts, "parallel"))
        schedule.append(ScheduleEntry(i, cache_of=int(m["kv_from"]) if "kv_from" in m else None))
    plan = ModelPlan(
        hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "scale": cfg.embedding_scale,
                                         "positions": cfg.max_positions}, {"weight": "embed", "positions": "pos"}),
        layers=layers, schedule=schedule, final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "logit_scale": cfg.logit_scale},
                      {"weight": "head"}),
        max_positions=cfg.max_positions, stop_ids=[])
    plan.validate()
    return plan


def checkpoint_layout(cfg: DaleraxConfig) -> dict:
    """{tensor name: (shape, kind)} of a complete checkpoint (kind as weights.random_init reads it)."""
    w = cfg.width
    out = {"embed": ((cfg.vocab, w), "matrix"), "pos": ((cfg.max_positions, w), "matrix")}
    for i, layer in enumerate(cfg.layers):
        out[f"l{i}.norm1"] = ((w,), "small")
        m, p = layer["mixer"], f"l{i}.mix."
        if layer["type"] == "attention":
            nh, g, d, vd = (int(m[x]) for x in ("heads", "kv_heads", "dim", "vdim"))
            out[p + "q"] = ((nh * d, w), "matrix")
            if "kv_from" not in m:
                out[p + "k"] = ((g * d, w), "matrix")
                out[p + "v"] = ((g * vd, w), "matrix")
            out[p + "sink"] = ((nh,), "bonus")
            out[p + "o"] = ((w, nh * vd), "matrix")
        else:
            nh, d = int(m["heads"]), int(m["dim"])
            rank = wkv_rank(m, p, None)
            for s in ("r", "k", "v", "g", "w"):
                out[f"{p}mu.{s}"] = ((w,), "blend")
            for s in ("r", "k", "v", "g"):
                out[p + s] = ((nh * d, w), "matrix")
            out[p + "w1"] = ((rank, w), "matrix")
            out[p + "w2"] = ((nh * d, rank), "lowrank")
            out[p + "w0"] = ((nh * d,), "decay_base")
            out[p + "u"] = ((nh, d), "bonus")
            out[p + "norm"] = ((nh * d,), "norm")
            out[p + "o"] = ((w, nh * d), "matrix")
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        p = f"l{i}.mlp."
        if mlp["kind"] == "dense":
            ff = int(mlp["ff"])
            out.update({p + "gate": ((ff, w), "matrix"), p + "up": ((ff, w), "matrix"), p + "down": ((w, ff), "matrix")})
            continue
        ff, experts = int(mlp["expert"]["ff"]), int(mlp["router"]["experts"])
        for e in range(experts):
            out[f"{p}e{e}.gate"] = ((ff, w), "matrix")
            out[f"{p}e{e}.up"] = ((ff, w), "matrix")
            out[f"{p}e{e}.down"] = ((w, ff), "matrix")
        out[p + "router"] = ((experts, w), "matrix")
        out[p + "router.b"] = ((experts,), "bias")
        if mlp.get("shared") is not None:
            fs = int(mlp["shared"]["ff"])
            out.update({p + "shared.gate": ((fs, w), "matrix"), p + "shared.up": ((fs, w), "matrix"),
                        p + "shared.down": ((w, fs), "matrix")})
    out["final.norm"] = ((w,), "small")
    out["head"] = ((cfg.vocab, w), "matrix")
    return out


register_architecture(["Dalerax", "dalerax"], DaleraxConfig, build_plan, checkpoint_layout)
