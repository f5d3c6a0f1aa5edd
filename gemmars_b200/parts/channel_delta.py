"""Delta rule with a decay per key channel: a recurrent mixer beside ``gated_delta`` whose state per
head is a matrix S [dim, vdim] and whose decay is a vector over the rows of S.

For one token, with h the mixer's input:
  q, k = W_q h, W_k h (kv_heads x dim), v = W_v h (heads x vdim); each passes a short causal filter
  over time (``conv`` taps per channel, no bias) and SiLU; q and k become unit vectors per head
  (x / sqrt(|x|^2 + 1e-6)), q also times dim^-1/2; head i reads q/k head i // (heads / kv_heads);
  beta = sigmoid(W_b h), one per head;
  g = exp(-exp(A_log[head]) * softplus(W_a2 (W_a1 h) + dt_bias)), one per head and key channel;
  S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q  (the read-out sees this token's write);
  o / rms(o) * norm * sigmoid(W_g2 (W_g1 h)) per head (``norm`` [vdim], shared by the heads),
  then W_o, added into the residual.

The projections that read h are one product written in float32: [q | k | v | b | a1 | g1].  What
follows (filters, unit norms, beta, the second halves of the two low-rank projections, softplus and
exponentials, the state, the read-out, the norm) is float32 work.  Per sequence the part keeps S
and the filter's last ``conv - 1`` inputs.  The inner sizes of the two low-rank projections are
parameters (``decay_rank``, ``gate_rank``).  Parameters: hidden_size, heads, kv_heads, dim, vdim,
conv, decay_rank, gate_rank, norm_eps, out_scale.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.pool import StateNeed
from .base import Part, TensorWant, register_part
from .linear import Linear


class ChannelDeltaRule(Part):
    category = "mixer"

    def __init__(self, spec, compute):
        super().__init__(spec, compute)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.heads, self.kv_heads = int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim, self.taps = int(p["dim"]), int(p["vdim"]), int(p["conv"])
        self.decay_rank, self.gate_rank = int(p["decay_rank"]), int(p["gate_rank"])
        self.eps = float(p["norm_eps"])
        self.out_scale = float(p.get("out_scale", 1.0))
        if self.heads % self.kv_heads:
            raise ValueError(f"channel_delta: {self.heads} heads are not a multiple of {self.kv_heads} q/k heads")
        if not 1 <= self.taps <= 8:
            raise ValueError(f"channel_delta: a filter of {self.taps} taps is not supported (1 to 8)")
        if not 1 <= self.dim <= 256:
            raise ValueError(f"channel_delta: q/k heads of {self.dim} are not supported by the kernel (1 to 256)")
        if self.decay_rank < 1 or self.gate_rank < 1:
            raise ValueError("channel_delta: the low-rank projections need an inner size of at least 1")
        self.qk, self.hv, self.hd = self.kv_heads * self.dim, self.heads * self.vdim, self.heads * self.dim
        self.channels = 2 * self.qk + self.hv            # what the filter runs over: q | k | v
        self.proj = self.o = self.filter = self.a2 = self.g2 = self.a_log = self.dt_bias = self.norm = None

    def wants(self):
        h, qk, hv, nh, k = self.hidden_size, self.qk, self.hv, self.heads, self.taps
        return {"q": TensorWant((qk, h)), "k": TensorWant((qk, h)), "v": TensorWant((hv, h)), "b": TensorWant((nh, h)),
                "a1": TensorWant((self.decay_rank, h)), "a2": TensorWant((self.hd, self.decay_rank)),
                "g1": TensorWant((self.gate_rank, h)), "g2": TensorWant((hv, self.gate_rank)), "o": TensorWant((h, hv)),
                "q_conv": TensorWant((qk, k), "vector"), "k_conv": TensorWant((qk, k), "vector"),
                "v_conv": TensorWant((hv, k), "vector"), "A_log": TensorWant((nh,), "vector"),
                "dt_bias": TensorWant((self.hd,), "vector"), "norm": TensorWant((self.vdim,), "vector")}

    def load(self, t):
        # one product: [q | k | v | b | a1 | g1]
        self.proj = Linear(torch.cat([t[n] for n in ("q", "k", "v", "b", "a1", "g1")], dim=0))
        self.o = Linear(t["o"])
        self.a2, self.g2 = t["a2"].contiguous(), t["g2"].contiguous()
        self.filter = torch.cat([t["q_conv"], t["k_conv"], t["v_conv"]], dim=0).contiguous()
        self.a_log, self.dt_bias, self.norm = t["A_log"].contiguous(), t["dt_bias"].contiguous(), t["norm"].contiguous()

    def kernel_units(self):
        return kernels.gemm_units(self.compute) + [("recurrent", ())]

    def cache_needs(self):
        return [StateNeed((self.taps - 1, self.channels)), StateNeed((self.heads, kernels.recurrent_state_floats(self.dim, self.vdim)))]

    def weight_bytes(self):
        small = sum(4 * t.numel() for t in (self.filter, self.a_log, self.dt_bias, self.norm) if t is not None)
        low = sum(t.numel() * t.element_size() for t in (self.a2, self.g2) if t is not None)
        return self.proj.bytes() + self.o.bytes() + small + low

    def forward(self, ctx, h, residual, caches, writes_cache=True):
        if not writes_cache:
            raise ValueError("channel_delta: a recurrent mixer cannot run on another layer's state")
        filter_state, state = caches
        qk, hv, nh, c = self.qk, self.hv, self.heads, self.channels
        p = self.proj(h, out_dtype=torch.float32)
        t = p.shape[0]
        a_at = c + nh
        g_at = a_at + self.decay_rank
        f = torch.empty((t, c), dtype=torch.float32, device=p.device)
        kernels.short_filter(p[:, :c], self.filter, None, filter_state, ctx.cu_seqlens, ctx.tok_seq, ctx.seq_slot, f, act=True)
        decay = kernels.lowrank_map(p[:, a_at:g_at], self.a2, self.dt_bias, "rate", rate=self.a_log, rate_group=self.dim)
        gate = kernels.lowrank_map(p[:, g_at:g_at + self.gate_rank], self.g2, None, "plain")
        y = torch.empty((t, hv), dtype=torch.float32, device=p.device)
        kernels.channel_delta_rule(f[:, :qk], f[:, qk:2 * qk], f[:, 2 * qk:], p[:, c:c + nh], decay, state, ctx.cu_seqlens,
                                   ctx.seq_slot, y, nh, self.kv_heads, self.dim, self.vdim, float(self.dim) ** -0.5)
        out = torch.empty((t, hv), dtype=self.act_dtype, device=p.device)
        kernels.gated_group_norm(y, gate, self.norm, out, self.vdim, self.eps, False, self.out_scale, gate_act="sigmoid")
        self.o.add_into(out, residual)


register_part("mixer", "channel_delta", ChannelDeltaRule)
