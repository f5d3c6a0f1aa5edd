"""Rotary position encoding over the first ``rotary_dim`` dims of each head.

inv_freq[i] = float32(1 / theta^(2i / rotary_dim)), computed in float64 (src/qwen.rs:529-533);
angle = float32(position) * inv_freq[i] in float32 (src/kernels.rs:1525-1531);
the pair (a, b) -> (a cos - b sin, b cos + a sin) (src/kernels.rs:1538-1548).  Which dims make
pair i is the ``layout``: "half" pairs v[i] with v[i + rotary_dim / 2] (the default), "interleaved"
pairs v[2i] with v[2i + 1].

``scaling`` (default none) stretches the long wavelengths for contexts beyond the trained one,
{"factor", "low", "high", "original"}: with l = 2 pi / f the wavelength of a frequency f, f stays
where l < original / high, becomes f / factor where l > original / low, and in between is the
blend (1 - s) f / factor + s f with s = (original / l - low) / (high - low).  The table is made
once, in float64, and rounded to float32.

A second form of ``scaling``, {"factor", "original", "fast", "slow"}, blends along the index
instead of the wavelength: with d(t) = rotary_dim ln(original / (2 pi t)) / (2 ln theta) the
index whose wavelength makes t turns over ``original`` positions, lo = max(floor(d(fast)), 0) and
hi = min(ceil(d(slow)), rotary_dim - 1), the frequency is f / factor * r + f (1 - r) with
r = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), and the cosines and sines are multiplied by
``magnitude`` = 0.1 ln(factor) + 1 (1 without this form).  Only kernels that take a magnitude can
use such a part (``capped_attention`` does; the fused kernels of ``attention`` do not).

The attention part fuses the "half" rotation into its q/k kernel when its position encoding is
this class, and the latent attention part the "interleaved" one into the kernel that writes its
cache rows; ``apply`` is the stand-alone form of either."""
from __future__ import annotations

import math

import torch

from .. import kernels
from .base import Part, register_part


class Rotary(Part):
    category = "position"

    def __init__(self, spec, compute):
        super().__init__(spec, compute)
        self.head_dim = int(spec.params["head_dim"])
        self.rotary_dim = int(spec.params.get("rotary_dim", self.head_dim))
        self.theta = float(spec.params["theta"])
        self.layout = spec.params.get("layout", "half")
        if self.layout not in ("half", "interleaved"):
            raise ValueError(f"rotary: unknown layout {self.layout!r} (half or interleaved)")
        if self.rotary_dim % 2 or not 0 <= self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary: cannot rotate {self.rotary_dim} of {self.head_dim} dimensions")
        i = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        freq = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float64), 2.0 * i / max(self.rotary_dim, 1))
        self.scaling = spec.params.get("scaling")
        self.magnitude = 1.0
        if self.scaling and ("fast" in self.scaling or "slow" in self.scaling):
            freq, self.magnitude = self.ramped(freq, self.scaling, self.rotary_dim, self.theta)
        elif self.scaling:
            freq = self.scaled(freq, self.scaling)
        self._inv_freq_host = freq.to(torch.float32)
        self._inv_freq = {}

    @staticmethod
    def scaled(freq: torch.Tensor, scaling: dict) -> torch.Tensor:
        """``freq`` (float64) with its long wavelengths stretched as ``scaling`` says."""
        try:
            factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        except (KeyError, TypeError, ValueError):
            raise ValueError(f"rotary: scaling needs the numbers factor, low, high and original, got {scaling!r}") from None
        if factor <= 0 or original <= 0 or high <= 0 or low <= 0:
            raise ValueError(f"rotary: scaling factor, low, high and original must be positive, got {scaling!r}")
        wavelength = 2.0 * math.pi / freq
        if high == low:
            blend = freq
        else:
            s = (original / wavelength - low) / (high - low)
            blend = (1.0 - s) * freq / factor + s * freq
        out = torch.where(wavelength > original / low, freq / factor, blend)
        return torch.where(wavelength < original / high, freq, out)

    @staticmethod
    def ramped(freq: torch.Tensor, scaling: dict, dims: int, theta: float):
        """(``freq`` (float64) blended towards freq / factor along the index, the magnitude)."""
        try:
            factor, original, fast, slow = (float(scaling[k]) for k in ("factor", "original", "fast", "slow"))
        except (KeyError, TypeError, ValueError):
            raise ValueError(f"rotary: scaling needs the numbers factor, original, fast and slow, got {scaling!r}") from None
        if factor <= 0 or original <= 0 or fast <= 0 or slow <= 0 or theta <= 1.0:
            raise ValueError(f"rotary: scaling factor, original, fast and slow must be positive, got {scaling!r}")

        def index_of(turns):
            return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

        lo = max(math.floor(index_of(fast)), 0)
        hi = min(math.ceil(index_of(slow)), dims - 1)
        i = torch.arange(freq.numel(), dtype=torch.float64)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0

    def inv_freq(self, device) -> torch.Tensor:
        t = self._inv_freq.get(device)
        if t is None:
            t = self._inv_freq[device] = self._inv_freq_host.to(device)
        return t

    def kernel_units(self):
        return [("elementwise", ())] if self.layout == "half" else [("latent_attention", ())]

    def table(self, ctx) -> torch.Tensor:
        """(cos, sin) of the step's packed tokens' angles, [tokens, rotary_dim / 2, 2] float32,
        computed once a step and shared by every layer with the same rotation."""
        assert self.layout == "half" and self.magnitude == 1.0
        key = ("rope_table", self.rotary_dim, self.theta, repr(self.scaling))
        t = ctx.extras.get(key)
        if t is None:
            t = ctx.extras[key] = kernels.rope_table(ctx.tok_pos, self.inv_freq(ctx.device))
        return t

    def apply(self, ctx, q, k):
        """Rotates q [T, nh, hd] and k [T, nkv, hd] (contiguous views) in place."""
        if self.magnitude != 1.0:
            raise ValueError("rotary: the stand-alone rotation takes no magnitude (use a mixer whose kernel does)")
        for x in (q, k):
            t, heads, hd = x.shape
            if self.layout == "interleaved":
                if self.rotary_dim:
                    kernels.rope_pairs(x, ctx.tok_pos, self.inv_freq(x.device), self.rotary_dim)
                continue
            flat = x.view(t, heads * hd)
            # all heads are treated as "q" heads of one tensor: rotate in place, scale 1
            kernels.head_norm_rope_cache(flat, heads, 0, hd, self.rotary_dim, None, None, 0.0,
                                         self.inv_freq(x.device), 1.0, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot,
                                         None, ctx.page_size, None, None,
                                         kernels.FLAG_ROPE | kernels.FLAG_INPLACE)


register_part("position", "rotary", Rotary)
