"""Gated linear attention: a recurrent mixer beside ``wkv`` whose state per head is a matrix
S [dim, vdim] that decays per key channel and is read after the token's own write.

For one token, with h the mixer's input:
  q = W_q h * dim^-1/2, k = W_k h (heads x dim), v = W_v h (heads x vdim);
  alpha = sigmoid(W_a2 (W_a1 h) + a2_bias)^(1 / tau), one number per head and key channel;
  per head  S <- diag(alpha) S + k v^T;  o = S^T q;
  each head's o divided by its root mean square (eps) times ``norm`` [vdim] (shared by the heads),
  the heads side by side times silu(W_g h), then W_o, added into the residual.

The projections that enter the recurrence are one product written in float32, [q | k | v | a1];
the decay's second half, the sigmoid, its root, the state, the read-out and the norm are float32
work (the read-out is linear in q, so dim^-1/2 multiplies the read-out instead of q).  The gate's logits are a product in the activation type.  Per sequence the part keeps S.
Parameters: hidden_size, heads, dim, vdim, rank (inner size of the decay's two matrices), tau,
norm_eps, out_scale.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.pool import StateNeed
from .base import Part, TensorWant, register_part
from .linear import Linear


class GatedLinearAttention(Part):
    category = "mixer"

    def __init__(self, spec, compute):
        super().__init__(spec, compute)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.heads, self.dim, self.vdim, self.rank = int(p["heads"]), int(p["dim"]), int(p["vdim"]), int(p["rank"])
        self.tau = float(p["tau"])
        self.eps = float(p["norm_eps"])
        self.out_scale = float(p.get("out_scale", 1.0))
        if self.heads < 1 or self.rank < 1 or self.vdim < 1:
            raise ValueError("gated_linear: needs at least one head, a value size and a decay rank of at least 1")
        if not 1 <= self.dim <= 256:
            raise ValueError(f"gated_linear: heads of {self.dim} are not supported by the kernel (1 to 256)")
        if not self.tau > 0:
            raise ValueError(f"gated_linear: tau must be positive, got {self.tau}")
        self.hd, self.hv = self.heads * self.dim, self.heads * self.vdim
        self.proj = self.g = self.o = self.a2 = self.a2_bias = self.norm = None

    def wants(self):
        h = self.hidden_size
        return {"q": TensorWant((self.hd, h)), "k": TensorWant((self.hd, h)), "v": TensorWant((self.hv, h)),
                "g": TensorWant((self.hv, h)), "o": TensorWant((h, self.hv)), "a1": TensorWant((self.rank, h)),
                "a2": TensorWant((self.hd, self.rank)), "a2_bias": TensorWant((self.hd,), "vector"),
                "norm": TensorWant((self.vdim,), "vector")}

    def load(self, t):
        self.proj = Linear(torch.cat([t[n] for n in ("q", "k", "v", "a1")], dim=0))    # one product: [q | k | v | a1]
        self.g, self.o = Linear(t["g"]), Linear(t["o"])
        self.a2, self.a2_bias, self.norm = t["a2"].contiguous(), t["a2_bias"].contiguous(), t["norm"].contiguous()

    def kernel_units(self):
        return kernels.gemm_units(self.compute) + [("recurrent", ())]

    def cache_needs(self):
        return [StateNeed((self.heads, kernels.recurrent_state_floats(self.dim, self.vdim)))]

    def weight_bytes(self):
        small = sum(4 * t.numel() for t in (self.a2_bias, self.norm) if t is not None)
        low = self.a2.numel() * self.a2.element_size() if self.a2 is not None else 0
        return self.proj.bytes() + self.g.bytes() + self.o.bytes() + small + low

    def forward(self, ctx, h, residual, caches, writes_cache=True):
        if not writes_cache:
            raise ValueError("gated_linear: a recurrent mixer cannot run on another layer's state")
        (state,) = caches
        hd, hv = self.hd, self.hv
        p = self.proj(h, out_dtype=torch.float32)
        t = p.shape[0]
        alpha = kernels.lowrank_map(p[:, 2 * hd + hv:], self.a2, self.a2_bias, "sigmoid_root", tau=self.tau)
        y = torch.empty((t, hv), dtype=torch.float32, device=p.device)
        kernels.wkv_scan(p[:, :hd], p[:, hd:2 * hd], alpha, p[:, 2 * hd:2 * hd + hv], None, state, ctx.cu_seqlens,
                         ctx.seq_slot, y, self.heads, self.dim, self.vdim, out_scale=float(self.dim) ** -0.5)
        gate = self.g(h, out_dtype=torch.float32)
        out = torch.empty((t, hv), dtype=self.act_dtype, device=p.device)
        kernels.gated_group_norm(y, gate, self.norm, out, self.vdim, self.eps, False, self.out_scale)
        self.o.add_into(out, residual)


register_part("mixer", "gated_linear", GatedLinearAttention)
