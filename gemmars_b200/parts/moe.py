"""Routed feed-forward (mixture of experts) with an optional shared expert.

    z        = router h + bias                      float32 (a product of the framework's, written in float32)
    chosen   = the ``top`` largest z;  weights = softmax over the chosen z alone
    expert   : g = min(gate h, limit), u = clamp(up h, -limit, limit)
               y = g * sigmoid(alpha g) * (u + shift);  out = down y        (no biases)
    residual += sum over chosen of weight * expert(h)  +  sigmoid(shared_gate . h) * shared(h)

The experts' matrices are stacked at load ([experts, 2 ff, hidden]: gate rows then up rows, and
[experts, hidden, ff]) so that a kernel finds an expert by its index alone.  Parameters:
hidden_size, experts, top, ff, limit, alpha (1.702), shift (1.0), router_bias, and ``shared``
(None, or {"ff", "limit", "gate"}: its width, its clamp, and whether its output is multiplied by
a sigmoid of one number per token).  A ``limit`` of None clamps nothing; with alpha 1 and shift 0
the expert is then the plain gated form silu(gate h) * (up h).

Two more parameters.  ``gated`` False: an expert has no gate matrix, out = down gelu(up h) with the
exact (erf) GELU (its tensors are ``e<j>.up`` and ``e<j>.down``; no clamps, no shared expert).
``routing`` "softmax_all": the weights are the chosen experts' shares of the softmax over all
experts, as they are (they do not add up to one); the default "softmax_top" is the softmax over the
chosen alone.
"""
from __future__ import annotations

import torch

from .. import kernels
from .base import Part, TensorWant, register_part
from .linear import Linear


class RoutedExperts(Part):
    category = "ffn"

    def __init__(self, spec, compute):
        super().__init__(spec, compute)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.experts = int(p["experts"])
        self.top = int(p["top"])
        self.ff = int(p["ff"])
        self.limit = float(p["limit"]) if p.get("limit") is not None else float("inf")
        self.alpha = float(p.get("alpha", 1.702))
        self.shift = float(p.get("shift", 1.0))
        self.router_bias = bool(p.get("router_bias", True))
        self.gated = bool(p.get("gated", True))
        self.routing = p.get("routing", "softmax_top")
        if self.routing not in ("softmax_top", "softmax_all"):
            raise ValueError(f"moe: unknown routing {self.routing!r} (softmax_top or softmax_all)")
        if not self.gated and (p.get("shared") or p.get("limit") is not None):
            raise ValueError("moe: experts without a gate take no clamp and no shared expert")
        shared = p.get("shared")
        self.shared_ff = int(shared["ff"]) if shared else 0
        self.shared_limit = (float(shared["limit"]) if shared.get("limit") is not None else float("inf")) if shared else 0.0
        self.shared_gated = bool(shared.get("gate", True)) if shared else False
        if not 1 <= self.top <= min(self.experts, 32):
            raise ValueError(f"moe: top {self.top} of {self.experts} experts is not supported (1 to 32, at most all)")
        self.router = self.bias = self.gate_up = self.down = None
        self.shared_gate_up = self.shared_down = None

    def wants(self):
        h, f = self.hidden_size, self.ff
        w = {"router": TensorWant((self.experts, h))}
        if self.router_bias:
            w["router_bias"] = TensorWant((self.experts,), "vector")
        for e in range(self.experts):
            if self.gated:
                w[f"e{e}.gate"] = TensorWant((f, h))
            w[f"e{e}.up"] = TensorWant((f, h))
            w[f"e{e}.down"] = TensorWant((h, f))
        if self.shared_ff:
            fs = self.shared_ff
            w.update({"shared.gate": TensorWant((fs, h)), "shared.up": TensorWant((fs, h)),
                      "shared.down": TensorWant((h, fs))})
            if self.shared_gated:
                w["shared.sg"] = TensorWant((1, h))
        return w

    def load(self, t):
        gate_row = [t["shared.sg"].reshape(1, -1)] if self.shared_ff and self.shared_gated else []
        # the router's logits and the shared expert's gate logit are one product, written in float32
        self.router = Linear(torch.cat([t["router"]] + gate_row, dim=0))
        self.bias = t["router_bias"].contiguous() if self.router_bias else None
        if self.gated:
            self.gate_up = torch.stack([torch.cat([t[f"e{e}.gate"], t[f"e{e}.up"]], dim=0) for e in range(self.experts)])
        else:
            self.gate_up = torch.stack([t[f"e{e}.up"] for e in range(self.experts)])      # [experts, ff, hidden]
        self.down = torch.stack([t[f"e{e}.down"] for e in range(self.experts)])
        if self.shared_ff:
            self.shared_gate_up = torch.cat([t["shared.gate"], t["shared.up"]], dim=0).contiguous()
            self.shared_down = t["shared.down"].contiguous()

    def kernel_units(self):
        if self.compute == "float32":
            return [("moe", ())] + kernels.gemm_units(self.compute)
        return [("moe", ()), ("grouped_gemm", ())] + kernels.gemm_units(self.compute)

    def _route(self, h):
        z = self.router(h, out_dtype=torch.float32)
        return kernels.moe_topk(z, self.bias, self.experts, self.top, has_gate=bool(self.shared_ff and self.shared_gated),
                                all_softmax=self.routing == "softmax_all")

    def weight_bytes(self):
        """What a decode step of one token reads: the router, ``top`` experts, the shared expert."""
        per = self.gate_up.element_size()
        one = (3 if self.gated else 2) * self.ff * self.hidden_size * per
        shared = 3 * self.shared_ff * self.hidden_size * per
        return self.router.bytes() + self.top * one + shared

    def decode_bytes(self, batch: int) -> int:
        """What a decode step of ``batch`` tokens has to read at least: the router, the shared expert,
        and every expert that some token chose, once; with choices spread evenly that is
        experts * (1 - (1 - top / experts) ** batch) experts on average."""
        per = self.gate_up.element_size()
        one = (3 if self.gated else 2) * self.ff * self.hidden_size * per
        distinct = self.experts * (1.0 - (1.0 - self.top / self.experts) ** max(batch, 1))
        return int(self.router.bytes() + distinct * one + 3 * self.shared_ff * self.hidden_size * per)

    def forward(self, ctx, h, residual):
        idx, wts, sg = self._route(h)
        if not self.gated:
            if kernels.moe_tc_usable(h, self.gate_up, self.down):
                run = kernels.moe_experts_plain_tc
            elif kernels.moe_grouped_usable(h, self.gate_up, self.down):
                run = kernels.moe_experts_plain_grouped
            else:
                run = kernels.moe_experts_plain
            run(h, idx, wts, self.gate_up, self.down, residual)
            return
        if self.shared_ff and sg is None:
            sg = torch.ones((h.shape[0],), dtype=torch.float32, device=h.device)
        if kernels.moe_tc_usable(h, self.gate_up, self.down):
            run = kernels.moe_experts_tc
        elif kernels.moe_grouped_usable(h, self.gate_up, self.down):
            run = kernels.moe_experts_grouped
        else:
            run = kernels.moe_experts
        run(h, idx, wts, sg, self.gate_up, self.down, self.shared_gate_up, self.shared_down, residual,
                            self.limit, self.shared_limit, self.alpha, self.shift)


register_part("ffn", "moe", RoutedExperts)
