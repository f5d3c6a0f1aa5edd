"""RMSNorm: out = x * (mean(x^2) + eps)^-1/2 * w, statistics in float32
(src/kernels.rs:1385-1392; the weight is used as stored, not as 1 + w: src/qwen.rs:343-346 with
src/config.rs:465-469).  Input: rows of the float32 residual stream; output: activations.

``offset`` (default 0): the stored weight is a deviation from it, w = offset + stored (a
checkpoint that keeps its norm weights around zero has offset 1); the sum is taken once, in
float32, when the weight is loaded.  ``add_normed`` is the norm on the other side of a sublayer:
it norms the sublayer's float32 output and adds it into the residual stream.  ``forward_with`` is two
norms of the same rows in one pass (a block whose mixer and feed-forward each read a norm of their
own of the same x)."""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, TensorWant, register_part


class RMSNorm(Part):
    category = "norm"
    #: the products around this norm may take it into themselves (kernels.UnscaledRows): its
    #: output is x * rstd(x) * weight with the weight as stored
    linkable = True

    def __init__(self, spec, compute):
        super().__init__(spec, compute)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.offset = float(spec.params.get("offset", 0.0))
        self.weight = None

    def wants(self):
        return {"weight": TensorWant((self.size,), "vector")}

    def load(self, tensors):
        w = tensors["weight"].to(torch.float32)
        self.weight = (w + self.offset if self.offset else w).contiguous()

    def kernel_units(self):
        # the unit of ``add_normed`` is built ahead only for a norm whose plan says it sits after a sublayer
        return [("rows", ())] if self.spec.params.get("after_sublayer") else [("elementwise", ())]

    def weight_bytes(self):
        return 0 if self.weight is None else 4 * self.weight.numel()

    def forward(self, ctx, x, rows_index=None):
        rows = x.shape[0] if rows_index is None else rows_index.numel()
        out = torch.empty((rows, self.size), dtype=self.act_dtype, device=x.device)
        kernels.rmsnorm(x, self.weight, out, self.eps, rows_index)
        return out

    def forward_with(self, ctx, x, other: "RMSNorm"):
        """(this norm of x, ``other``'s norm of x) in one pass: two norms of the same rows with the same
        size and eps share their statistics and differ in their weights alone."""
        if not isinstance(other, RMSNorm) or other.size != self.size or other.eps != self.eps or other.act_dtype != self.act_dtype:
            return self.forward(ctx, x), other.forward(ctx, x)
        out = torch.empty((x.shape[0], self.size), dtype=self.act_dtype, device=x.device)
        out2 = torch.empty_like(out)
        kernels.rmsnorm(x, self.weight, out, self.eps, second=(other.weight, out2))
        return out, out2

    def add_normed(self, ctx, y, x, then=None):
        """x += norm(y): ``y`` a sublayer's float32 output, ``x`` the residual stream.  ``then``: an
        RMSNorm part that reads the stream next; its output is made in the same pass and returned."""
        if then is None:
            kernels.rmsnorm_add(y, self.weight, x, self.eps)
            return None
        out = torch.empty(x.shape, dtype=then.act_dtype, device=x.device)
        kernels.rmsnorm_add(y, self.weight, x, self.eps, (then.weight, then.eps, out))
        return out


register_part("norm", "rmsnorm", RMSNorm)
