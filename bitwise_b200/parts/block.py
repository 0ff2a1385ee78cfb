"""The arrangements of a layer: the pre-norm residual block, and the parallel block whose mixer
and feed-forward read the same input.

``x += mixer(norm1(x)); x += feed_forward(norm2(x))`` (src/model.cpp:281-305).  The
block owns nothing but its four parts and the sub-names under which their tensors are
found; which mixer and which feed-forward it holds is decided where the model is assembled,
layer by layer.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..weights.loader import ParamSpec
from .base import FeedForward, Mixer, Norm, Part, StepContext


class PreNormBlock(Part):
    graph_safe = True  # kernels only: a step through this part can be captured

    def __init__(self, width: int, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, ffn_norm: Norm,
                 names: Dict[str, str]):
        self.width = width
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.ffn_norm = mixer_norm, ffn_norm
        self.names = names  # keys: mixer_norm, mixer, ffn_norm, feed_forward

    def _children(self, prefix: str):
        return [(self.mixer_norm, f"{prefix}.{self.names['mixer_norm']}"),
                (self.mixer, f"{prefix}.{self.names['mixer']}"),
                (self.ffn_norm, f"{prefix}.{self.names['ffn_norm']}"),
                (self.feed_forward, f"{prefix}.{self.names['feed_forward']}")]

    def param_specs(self, prefix: str) -> List[ParamSpec]:
        return [s for part, p in self._children(prefix) for s in part.param_specs(p)]

    def load_params(self, state: Dict[str, torch.Tensor], prefix: str) -> None:
        for part, p in self._children(prefix):
            part.load_params(state, p)

    def param_bytes(self) -> int:
        return sum(part.param_bytes() for part, _ in self._children(""))

    def cache_need(self):
        return self.mixer.cache_need()

    def state_need(self):
        return self.mixer.state_need()

    def prepare(self, ops) -> None:
        for part, _ in self._children(""):
            part.prepare(ops)

    def forward(self, ctx: StepContext, x: torch.Tensor, cache) -> None:
        """Run the block on the float32 stream ``x`` in place."""
        xn = ctx.workspace.rows("normed", ctx.n, self.width, ctx.act_dtype)
        self.mixer_norm.forward(ctx, x, xn)
        self.mixer.forward(ctx, xn, x, cache)
        self.ffn_norm.forward(ctx, x, xn)
        self.feed_forward.forward(ctx, xn, x)


class ParallelBlock(PreNormBlock):
    """``x += mixer(norm1(x)) + feed_forward(norm2(x))``: both parts see the same x, their
    outputs are added to each other first and to the stream last.  The mixer writes into a
    float32 buffer, the feed-forward adds to it, and the sum goes into the stream; a feed-forward
    that has ``forward_sum`` does the last two in its own last kernel.  ``feed_forward`` None: the
    layer is its mixer alone."""

    def _children(self, prefix: str):
        kids = super()._children(prefix)
        return [(p, n) for p, n in kids if p is not None]

    def forward(self, ctx: StepContext, x: torch.Tensor, cache) -> None:
        xn = ctx.workspace.rows("normed", ctx.n, self.width, ctx.act_dtype)
        if self.feed_forward is None:
            self.mixer_norm.forward(ctx, x, xn)
            self.mixer.forward(ctx, xn, x, cache)
            return
        xn2 = ctx.workspace.rows("normed_b", ctx.n, self.width, ctx.act_dtype)
        pair = getattr(self.mixer_norm, "forward_pair", None)
        if pair is not None and type(self.ffn_norm) is type(self.mixer_norm):
            pair(ctx, x, xn, self.ffn_norm, xn2)
        else:
            self.mixer_norm.forward(ctx, x, xn)
            self.ffn_norm.forward(ctx, x, xn2)
        delta = ctx.workspace.rows("block_sum", ctx.n, self.width, torch.float32)
        self.mixer.forward(ctx, xn, delta, cache, accumulate=False)
        fused = getattr(self.feed_forward, "forward_sum", None)
        if fused is not None:
            fused(ctx, xn2, delta, x)
        else:
            self.feed_forward.forward(ctx, xn2, delta)
            ctx.ops.add_rows(x, delta)


class SandwichBlock(PreNormBlock):
    """A norm before and after each sublayer: ``x += norm1b(mixer(norm1(x)))``, then ``x +=
    norm2b(feed_forward(norm2(x)))``.  A sublayer writes its output into a float32 buffer; the
    norm after it reads that buffer and adds the normed rows to the stream in one kernel
    (``Norm.forward_residual``).  ``feed_forward`` None: the layer is its mixer alone, with the
    two norms around it.  ``names`` has the keys of :class:`PreNormBlock` plus ``mixer_post`` and
    ``ffn_post``."""

    def __init__(self, width: int, mixer: Mixer, feed_forward, mixer_norm: Norm, mixer_post: Norm, ffn_norm,
                 ffn_post, names: Dict[str, str]):
        super().__init__(width, mixer, feed_forward, mixer_norm, ffn_norm, names)
        self.mixer_post, self.ffn_post = mixer_post, ffn_post

    def _children(self, prefix: str):
        kids = super()._children(prefix) + [(self.mixer_post, f"{prefix}.{self.names['mixer_post']}"),
                                            (self.ffn_post, f"{prefix}.{self.names['ffn_post']}")]
        return [(p, n) for p, n in kids if p is not None]

    def forward(self, ctx: StepContext, x: torch.Tensor, cache) -> None:
        xn = ctx.workspace.rows("normed", ctx.n, self.width, ctx.act_dtype)
        out = ctx.workspace.rows("sublayer_out", ctx.n, self.width, torch.float32)
        self.mixer_norm.forward(ctx, x, xn)
        self.mixer.forward(ctx, xn, out, cache, accumulate=False)
        if self.feed_forward is None:
            self.mixer_post.forward_residual(ctx, out, x)
            return
        fused = getattr(self.mixer_post, "forward_residual_then", None)
        if fused is not None:  # the norm after the mixer and the one before the feed-forward in one kernel
            fused(ctx, out, x, self.ffn_norm, xn)
        else:
            self.mixer_post.forward_residual(ctx, out, x)
            self.ffn_norm.forward(ctx, x, xn)
        self.feed_forward.forward(ctx, xn, out, accumulate=False)
        self.ffn_post.forward_residual(ctx, out, x)
