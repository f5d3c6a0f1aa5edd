"""Linear attention with a learned decay per key channel and mixes with the token before (the
time mixing of the RWKV family): a recurrent mixer whose state per head is a matrix S [dim, dim].

For one token, with h the mixer's input and h' the input of the token before it in the sequence
(zeros before the first):
  each of r, k, v, g, w reads its own blend  x_s = h + (h' - h) * mu_s;
  r, k, v = W_r x_r, W_k x_k, W_v x_v  (heads x dim each);  gate = silu(W_g x_g);
  decay  w = exp(-exp(w0 + W_w2 tanh(W_w1 x_w))), one number per head and key channel;
  per head  o = (S + diag(u) k v^T)^T r  (the bonus u only for the token itself),
            then S <- diag(w) S + k v^T;
  each head's o divided by its root mean square (eps), the heads side by side times ``norm``,
  times the gate, then W_o, added into the residual.

The projections' results are written in float32, and everything after them that enters the
recurrence is float32 work: tanh, the low-rank sum, both exponentials, the state, the read-out,
the unit norm.  Per sequence the part keeps S and the last input h'.  Parameters: hidden_size,
heads, dim, rank (inner size of the decay's two matrices), norm_eps, out_scale.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.pool import StateNeed
from .base import Part, TensorWant, register_part
from .linear import Linear

MIXES = ("r", "k", "v", "g", "w")


class DecayedLinearAttention(Part):
    category = "mixer"

    def __init__(self, spec, compute):
        super().__init__(spec, compute)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.heads, self.dim, self.rank = int(p["heads"]), int(p["dim"]), int(p["rank"])
        self.eps = float(p["norm_eps"])
        self.out_scale = float(p.get("out_scale", 1.0))
        if self.heads < 1 or self.rank < 1:
            raise ValueError(f"wkv: needs at least one head and a decay rank of at least 1, got {self.heads} and {self.rank}")
        if not 1 <= self.dim <= 256:
            raise ValueError(f"wkv: heads of {self.dim} are not supported by the kernel (1 to 256)")
        self.inner = self.heads * self.dim
        self.mu = self.r = self.k = self.v = self.g = self.w1 = self.w2 = self.w0 = self.u = self.norm = self.o = None

    def wants(self):
        h, n = self.hidden_size, self.inner
        w = {f"mu_{s}": TensorWant((h,), "vector") for s in MIXES}
        w.update({s: TensorWant((n, h)) for s in ("r", "k", "v", "g")})
        w.update({"w1": TensorWant((self.rank, h)), "w2": TensorWant((n, self.rank)), "w0": TensorWant((n,), "vector"),
                  "u": TensorWant((self.heads, self.dim), "vector"), "norm": TensorWant((n,), "vector"),
                  "o": TensorWant((h, n))})
        return w

    def load(self, t):
        self.mu = torch.stack([t[f"mu_{s}"] for s in MIXES]).to(torch.float32).contiguous()
        self.r, self.k, self.v, self.g = (Linear(t[s]) for s in ("r", "k", "v", "g"))
        self.w1, self.w2 = Linear(t["w1"]), t["w2"].contiguous()
        self.w0, self.u, self.norm = t["w0"].contiguous(), t["u"].contiguous(), t["norm"].contiguous()
        self.o = Linear(t["o"])

    def kernel_units(self):
        return kernels.gemm_units(self.compute) + [("recurrent", ())]

    def cache_needs(self):
        return [StateNeed((self.hidden_size,)),
                StateNeed((self.heads, kernels.recurrent_state_floats(self.dim, self.dim)))]

    def weight_bytes(self):
        small = sum(4 * t.numel() for t in (self.mu, self.w0, self.u, self.norm) if t is not None)
        mats = sum(m.bytes() for m in (self.r, self.k, self.v, self.g, self.w1, self.o))
        return mats + self.w2.numel() * self.w2.element_size() + small

    def forward(self, ctx, h, residual, caches, writes_cache=True):
        if not writes_cache:
            raise ValueError("wkv: a recurrent mixer cannot run on another layer's state")
        before, state = caches
        mixes = kernels.shift_mix(h, self.mu, before, ctx.cu_seqlens, ctx.tok_seq, ctx.seq_slot)
        r, k, v, gate = (m(mixes[i], out_dtype=torch.float32) for i, m in enumerate((self.r, self.k, self.v, self.g)))
        decay = kernels.lowrank_decay(self.w1(mixes[4], out_dtype=torch.float32), self.w2, self.w0)
        y = torch.empty((h.shape[0], self.inner), dtype=torch.float32, device=h.device)
        kernels.wkv_scan(r, k, decay, v, self.u, state, ctx.cu_seqlens, ctx.seq_slot, y, self.heads, self.dim, self.dim)
        out = torch.empty((h.shape[0], self.inner), dtype=self.act_dtype, device=h.device)
        kernels.gated_group_norm(y, gate, self.norm, out, self.dim, self.eps, False, self.out_scale)
        self.o.add_into(out, residual)


register_part("mixer", "wkv", DecayedLinearAttention)
