"""The arrangement of a layer's parts.

``prenorm`` (src/qwen.rs:682-696): x += mixer(norm(x)); x += ffn(norm(x)), the residual stream
``x`` in float32.  ``parallel``: x += mixer(norm(x)) + ffn(norm(x)) with one norm, or with a norm of its own for the feed-forward.  ``sandwich``:
a norm on both sides of each sublayer, x += post(mixer(pre(x))); x += post(ffn(pre(x))).  Another
arrangement (a third norm) is another class like these, registered under its own kind
and reading its own part names from the layer's spec."""
from __future__ import annotations

import torch

from .. import kernels
from .base import Block, register_part


class PreNormBlock(Block):
    def __init__(self, layer_spec, compute):
        super().__init__(layer_spec, compute)
        self.mixer_norm = self.need("mixer_norm", "norm")
        self.mixer = self.need("mixer", "mixer")
        self.ffn_norm = self.need("ffn_norm", "norm")
        self.ffn = self.need("ffn", "ffn")

    def parts(self):
        return {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "ffn_norm": self.ffn_norm, "ffn": self.ffn}

    #: forward takes ``h_in`` / ``next_norm`` and returns what its last product left for the next block's first norm
    chains_norms = True

    def first_norm(self):
        """The norm that reads the residual first: the block before may be asked to feed it."""
        return self.mixer_norm

    def forward(self, ctx, x, caches, writes_cache=True, h_in=None, next_norm=None):
        """Runs the layer on ``x`` in place.  In decode steps the RMSNorms are taken into the
        products around them where the parts can (kernels.UnscaledRows): ``h_in`` is what the block
        before left for this block's first norm (None: the norm runs by itself), ``next_norm`` the
        first norm of the block after; returns what the feed-forward's last product left for it."""
        mine = self.split_caches(caches)
        linking = (kernels.NORM_LINKS and self.compute == "bfloat16" and ctx.n_tokens <= kernels.LINK_MAX_TOKENS)
        h = h_in if h_in is not None else self.mixer_norm.forward(ctx, x)
        left = None
        if getattr(self.mixer, "links_norms", False):
            then = self.ffn_norm if linking and getattr(self.ffn_norm, "linkable", False) else None
            left = self.mixer.forward(ctx, h, x, mine["mixer"], writes_cache, then_norm=then)
        else:
            self.mixer.forward(ctx, _plain(h), x, mine["mixer"], writes_cache)
        h = left if left is not None else self.ffn_norm.forward(ctx, x)
        if getattr(self.ffn, "links_norms", False):
            then = next_norm if linking and getattr(next_norm, "linkable", False) else None
            return self.ffn.forward(ctx, h, x, then_norm=then)
        self.ffn.forward(ctx, _plain(h), x)
        return None


class ParallelBlock(Block):
    """``parallel``: h = norm(x); x += mixer(h) + ffn(h).  One norm, and both branches read its
    output; each branch adds its result into the float32 residual stream, the mixer first.  The
    layer's spec lists ``norm``, ``mixer`` and, when the layer has a feed-forward, ``ffn``.  With
    ``ffn_norm`` in the spec the feed-forward reads a norm of its own of the same x:
    x += mixer(norm(x)) + ffn(ffn_norm(x)), both norms taken before either branch changes x."""

    def __init__(self, layer_spec, compute):
        super().__init__(layer_spec, compute)
        self.norm = self.need("norm", "norm")
        self.mixer = self.need("mixer", "mixer")
        self.ffn = self.need("ffn", "ffn") if "ffn" in layer_spec.parts else None
        self.ffn_norm = self.need("ffn_norm", "norm") if self.ffn is not None and "ffn_norm" in layer_spec.parts else None

    def parts(self):
        out = {"norm": self.norm, "mixer": self.mixer}
        if self.ffn_norm is not None:
            out["ffn_norm"] = self.ffn_norm
        if self.ffn is not None:
            out["ffn"] = self.ffn
        return out

    def forward(self, ctx, x, caches, writes_cache=True):
        mine = self.split_caches(caches)
        # read by both branches before either changes x; two norms of the same x are one pass where they can be
        if self.ffn_norm is not None and hasattr(self.norm, "forward_with"):
            h, h_ffn = self.norm.forward_with(ctx, x, self.ffn_norm)
        else:
            h = self.norm.forward(ctx, x)
            h_ffn = self.ffn_norm.forward(ctx, x) if self.ffn_norm is not None else h
        self.mixer.forward(ctx, h, x, mine["mixer"], writes_cache)
        if self.ffn is not None:
            self.ffn.forward(ctx, h_ffn, x)


class SandwichBlock(Block):
    """``sandwich``: x += mixer_post_norm(mixer(mixer_norm(x))); x += ffn_post_norm(ffn(ffn_norm(x))).
    A sublayer adds its output into float32 rows of zeros instead of the residual stream; the norm
    after it reads those rows and adds the normed rows into the stream.  The layer's spec lists
    ``mixer_norm``, ``mixer``, ``mixer_post_norm`` and, when the layer has a feed-forward,
    ``ffn_norm``, ``ffn``, ``ffn_post_norm``."""

    def __init__(self, layer_spec, compute):
        super().__init__(layer_spec, compute)
        self.mixer_norm = self.need("mixer_norm", "norm")
        self.mixer = self.need("mixer", "mixer")
        self.mixer_post_norm = self.need("mixer_post_norm", "norm")
        self.ffn = self.need("ffn", "ffn") if "ffn" in layer_spec.parts else None
        self.ffn_norm = self.need("ffn_norm", "norm") if self.ffn is not None else None
        self.ffn_post_norm = self.need("ffn_post_norm", "norm") if self.ffn is not None else None

    def parts(self):
        out = {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "mixer_post_norm": self.mixer_post_norm}
        if self.ffn is not None:
            out.update({"ffn_norm": self.ffn_norm, "ffn": self.ffn, "ffn_post_norm": self.ffn_post_norm})
        return out

    def forward(self, ctx, x, caches, writes_cache=True):
        mine = self.split_caches(caches)
        y = torch.zeros_like(x)
        self.mixer.forward(ctx, self.mixer_norm.forward(ctx, x), y, mine["mixer"], writes_cache)
        if self.ffn is None:
            self.mixer_post_norm.add_normed(ctx, y, x)
            return
        # the norm after the mixer and the norm before the feed-forward read the same rows: one pass
        fused = isinstance(self.ffn_norm, type(self.mixer_post_norm)) and hasattr(self.ffn_norm, "weight")
        h = self.mixer_post_norm.add_normed(ctx, y, x, self.ffn_norm if fused else None)
        if h is None:
            h = self.ffn_norm.forward(ctx, x)
        y.zero_()
        self.ffn.forward(ctx, h, y)
        self.ffn_post_norm.add_normed(ctx, y, x)


def _plain(h):
    return h.materialize() if isinstance(h, kernels.UnscaledRows) else h


register_part("block", "prenorm", PreNormBlock)
register_part("block", "parallel", ParallelBlock)
register_part("block", "sandwich", SandwichBlock)
