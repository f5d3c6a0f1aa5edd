"""Softmax attention beside ``Attention`` for designs whose scores are capped, whose values are
wider or narrower than their keys, or whose q, k and v pass a short filter over time.

For one token, with h the mixer's input:
  q, k, v = W_q h, W_k h, W_v h (+ biases), heads x dim, kv_heads x dim, kv_heads x vdim;
  each channel passes a causal filter over time (``conv`` taps, no bias, no activation; 0: none);
  the position encoding turns q and k (a ``rotary`` part with the "half" layout, or None);
  score = (q . k) * scale, then cap * tanh(score / cap) when ``softcap``; a query sees itself and
  the ``window`` - 1 positions before it (None: all), and with ``keep_first`` the sequence's first
  ``keep_first`` positions as well, at their true places, however far the window has moved on;
  softmax, whose denominator with ``sink`` also holds exp(s_head), a learned number per head that
  has no key and no value; the heads side by side are multiplied by sigmoid(W_g h) when ``gate``,
  then W_o, added into the residual.

Keys (filtered and rotated) and values (filtered) live in the paged cache that every attention
of the package uses (a window's pages are a ring); the filter's last ``conv`` - 1 inputs are a
state per sequence.  Scores, softmax, angles and the gate are float32.  bfloat16 steps run on
the tensor cores where the head sizes allow (kernels.attention_capped).  A part with ``has_kv``
False has no k and v matrices: it runs its own queries, mask and sink over the keys and values of
the schedule entry whose cache it is given.  A window's pages are a ring only with ``ring`` (the
default) and no kept first positions; otherwise every page stays and the window is the kernels'
mask alone, which is what a layer needs whose cache another layer with another mask reads.
Four more parameters, all off by default.  ``values_are_keys``: there is no W_v; a value head is
its key head as projected (with its bias), before norm and rotation, so vdim == dim.  ``qk_norm``
(an eps): every q and k head is divided by its root mean square and multiplied by a weight over
its dims (``q_norm``, ``k_norm``, shared by the heads) before the rotation.  ``q_temper`` {"coef",
"every"}: the query at position p is multiplied by 1 + coef ln(floor((p + 1) / every) + 1).
``fixed_sink`` (a number s): exp(s) joins the softmax's denominator for every head, without a
tensor (0.0: one is added to the denominator).
Parameters: hidden_size, heads, kv_heads, dim, vdim, bias, conv, window, keep_first, sink, scale,
softcap, gate, position, has_kv, ring, out_scale, values_are_keys, qk_norm, q_temper, fixed_sink.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.pool import KVNeed, StateNeed
from .base import Part, TensorWant, build_part, register_part
from .linear import Linear
from .rotary import Rotary


class CappedAttention(Part):
    category = "mixer"

    def __init__(self, spec, compute):
        super().__init__(spec, compute)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.heads, self.kv_heads = int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.bias, self.gate = bool(p.get("bias", False)), bool(p.get("gate", False))
        self.taps = int(p.get("conv") or 0)
        self.window = p.get("window")
        self.keep_first = int(p.get("keep_first") or 0)
        self.sink = bool(p.get("sink", False))
        self.has_kv = bool(p.get("has_kv", True))
        self.ring = bool(p.get("ring", True)) and self.keep_first == 0
        self.scale = float(p["scale"]) if p.get("scale") is not None else float(self.dim) ** -0.5
        self.softcap = float(p.get("softcap") or 0.0)
        self.out_scale = float(p.get("out_scale", 1.0))
        self.values_are_keys = bool(p.get("values_are_keys", False))
        self.qk_norm_eps = float(p["qk_norm"]) if p.get("qk_norm") is not None else None
        temper = p.get("q_temper")
        self.q_temper = (float(temper["coef"]), int(temper["every"])) if temper else None
        self.fixed_sink = float(p["fixed_sink"]) if p.get("fixed_sink") is not None else None
        if self.values_are_keys and (self.vdim != self.dim or not self.has_kv or self.taps > 1):
            raise ValueError("capped_attention: values that are the keys need vdim == dim, keys of the part's own and no "
                             "filter with a memory")
        if self.q_temper is not None and self.q_temper[1] < 1:
            raise ValueError(f"capped_attention: q_temper.every must be at least 1, got {self.q_temper[1]}")
        if self.sink and self.fixed_sink is not None:
            raise ValueError("capped_attention: a learned sink and a fixed one exclude each other")
        if self.heads % self.kv_heads:
            raise ValueError(f"capped_attention: {self.heads} heads are not a multiple of {self.kv_heads} kv heads")
        if self.dim > 512:
            raise ValueError(f"capped_attention: keys of {self.dim} are wider than the kernels take (512)")
        if self.vdim > 512:
            raise ValueError(f"capped_attention: values of {self.vdim} are wider than the kernel takes (512)")
        if not 0 <= self.taps <= 8:
            raise ValueError(f"capped_attention: a filter of {self.taps} taps is not supported (0 to 8)")
        if self.taps > 1 and not self.has_kv:
            raise ValueError("capped_attention: a part without keys and values of its own cannot keep a filter's memory")
        if self.keep_first < 0:
            raise ValueError(f"capped_attention: keep_first must not be negative, got {self.keep_first}")
        pos = p.get("position")
        self.position = build_part("position", pos, compute) if pos is not None else None
        if self.position is not None and not (isinstance(self.position, Rotary) and self.position.layout == "half"):
            raise ValueError("capped_attention: the position encoding must be a rotary part with the half layout")
        self.own_kv = self.kv_heads if self.has_kv else 0
        own_v = 0 if self.values_are_keys else self.own_kv
        self.channels = (self.heads + self.own_kv) * self.dim + own_v * self.vdim     # q | k | v
        self.proj = self.o = self.filter = self.sinks = self.q_norm = self.k_norm = None

    def wants(self):
        h, nh, nkv, d, vd = self.hidden_size, self.heads, self.kv_heads, self.dim, self.vdim
        w = {"q": TensorWant((nh * d, h)), "o": TensorWant((h, nh * vd))}
        kv = [("k", nkv * d)] if self.has_kv else []
        if self.has_kv and not self.values_are_keys:
            kv.append(("v", nkv * vd))
        w.update({n: TensorWant((rows, h)) for n, rows in kv})
        if self.bias:
            w["q_bias"] = TensorWant((nh * d,), "vector")
            w.update({n + "_bias": TensorWant((rows,), "vector") for n, rows in kv})
        if self.taps:
            w["q_conv"] = TensorWant((nh * d, self.taps), "vector")
            w.update({n + "_conv": TensorWant((rows, self.taps), "vector") for n, rows in kv})
        if self.qk_norm_eps is not None:
            w["q_norm"] = TensorWant((d,), "vector")
            if self.has_kv:
                w["k_norm"] = TensorWant((d,), "vector")
        if self.gate:
            w["g"] = TensorWant((nh * vd, h))
        if self.sink:
            w["sink"] = TensorWant((nh,), "vector")
        return w

    def load(self, t):
        qkv = (["q", "k"] if self.values_are_keys else ["q", "k", "v"]) if self.has_kv else ["q"]
        names = qkv + (["g"] if self.gate else [])
        bias = None
        if self.bias:
            parts = [t[n + "_bias"] for n in qkv]
            if self.gate:
                parts.append(torch.zeros(self.heads * self.vdim, dtype=torch.float32, device=t["q_bias"].device))
            bias = torch.cat(parts)
        self.proj = Linear(torch.cat([t[n] for n in names], dim=0), bias)     # one product: [q | k | v | gate]
        self.o = Linear(t["o"])
        if self.taps:
            self.filter = torch.cat([t[n + "_conv"] for n in qkv], dim=0).contiguous()
        if self.sink:
            self.sinks = t["sink"].to(torch.float32).contiguous()
        elif self.fixed_sink is not None:
            self.sinks = torch.full((self.heads,), self.fixed_sink, dtype=torch.float32, device=t["q"].device)
        if self.qk_norm_eps is not None:
            self.q_norm = t["q_norm"].to(torch.float32).contiguous()
            self.k_norm = t["k_norm"].to(torch.float32).contiguous() if self.has_kv else None

    def kernel_units(self):
        return (kernels.gemm_units(self.compute) + kernels.attention_capped_units(self.compute, self.dim, self.vdim)
                + ([("recurrent", ())] if self.taps > 1 else []))

    def cache_needs(self):
        if not self.has_kv:
            return []
        needs = [KVNeed(self.kv_heads, self.dim, self.window if self.ring else None, self.vdim)]
        if self.taps > 1:
            needs.append(StateNeed((self.taps - 1, self.channels)))
        return needs

    def weight_bytes(self):
        return self.proj.bytes() + self.o.bytes() + (4 * self.filter.numel() if self.filter is not None else 0)

    def forward(self, ctx, h, residual, caches, writes_cache=True):
        if writes_cache != self.has_kv:
            raise ValueError("capped_attention: a part with keys and values of its own writes its own cache, and one "
                             "without reads another entry's (has_kv and the schedule's cache_of must agree)")
        group, kc, vc = caches[0]
        if tuple(kc.shape[1:]) != (self.kv_heads, group.page_size, self.dim) or vc.shape[2] != self.vdim:
            raise ValueError(f"capped_attention: the cache holds keys {tuple(kc.shape[1:])} and values of {vc.shape[2]}, "
                             f"this part reads {self.kv_heads} heads of {self.dim} and {self.vdim}")
        if group.need.window is not None and (self.keep_first or self.window is None or self.window > group.need.window):
            raise ValueError("capped_attention: the cache keeps a ring of the last positions only, which does not hold "
                             "what this part's mask sees")
        filter_state = caches[1] if self.taps > 1 else None
        nh, d, vd, c = self.heads, self.dim, self.vdim, self.channels
        p = self.proj(h)
        t = p.shape[0]
        rot = self.position.rotary_dim if self.position is not None else 0
        q = torch.empty((t, nh * d), dtype=p.dtype, device=p.device)
        kernels.filter_rope_cache(p[:, :c], self.filter, filter_state, self.position.inv_freq(p.device) if rot else None, rot,
                                  ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, ctx.cu_seqlens, group.page_table, group.page_size,
                                  q, kc if self.has_kv else None, vc if self.has_kv else None, nh, self.own_kv, d, vd,
                                  q_norm=self.q_norm, k_norm=self.k_norm, norm_eps=self.qk_norm_eps or 0.0,
                                  rot_magnitude=self.position.magnitude if rot else 1.0, q_temper=self.q_temper,
                                  values_are_keys=self.values_are_keys)
        if self.taps > 1:
            kernels.short_filter_state(p[:, :c], filter_state, ctx.cu_seqlens, ctx.seq_slot, self.taps)
        att = torch.empty((t, nh * vd), dtype=p.dtype, device=p.device)
        kernels.attention_capped(ctx, q, att, nh, kc, vc, group.page_table, group.page_size, self.window, self.scale,
                                 self.softcap, p[:, c:] if self.gate else None, self.out_scale, self.keep_first, self.sinks)
        self.o.add_into(att, residual)


register_part("mixer", "capped_attention", CappedAttention)
