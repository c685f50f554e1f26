"""Block arrangements: how a mixer and a feed-forward sit on the residual stream.

``pre_norm``: h = h + mixer(norm(h)); h = h + ffn(norm(h)), plain adds in fp32
(src/architectures/impl/qwen3/block.zig:21-41).  The parts add their output
into the stream themselves, so the last projection of each can carry the add.

``sublayer_norm``: h = h + norm(mixer(h)); h = h + norm(ffn(h)): the norm stands on the sublayer's *output*, the
sublayers read the stream itself.  The norm may carry a scale per coordinate of its own (``rms_norm`` with
``layer_scale``); norm, scale and the residual add are one kernel in fp32.

``sandwich_norm``: h = h + post1(mixer(pre1(h))); h = h + post2(ffn(pre2(h))): a norm on what a sublayer reads and
another on what it gives.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..registry import register_arrangement
from .base import FeedForward, LayerIO, Mixer, Norm, Part, StepContext


@register_arrangement("pre_norm")
class PreNormBlock(Part):
    def __init__(self, hidden_size: int, mixer: Mixer, feed_forward: FeedForward,
                 mixer_norm: Norm, feed_forward_norm: Norm):
        self.hidden = int(hidden_size)
        self.mixer, self.ffn = mixer, feed_forward
        self.mixer_norm, self.ffn_norm = mixer_norm, feed_forward_norm

    def children(self) -> Dict[str, Part]:
        return {"mixer": self.mixer, "feed_forward": self.ffn,
                "mixer_norm": self.mixer_norm, "feed_forward_norm": self.ffn_norm}

    @property
    def graph_safe(self) -> bool:      # type: ignore[override]
        return all(c.graph_safe for c in self.children().values())

    def prefers_plain_launches(self, rows: int) -> bool:
        return any(c.prefers_plain_launches(rows) for c in self.children().values())

    def step_key(self, ctx: StepContext):
        keys = tuple(k for k in (c.step_key(ctx) for c in self.children().values()) if k is not None)
        return keys or None

    def first_norm_weight(self):
        """The weight of the norm that reads the stream first in this block, if that norm is the kernel
        object's ``rmsnorm`` and nothing else (what the block before may tell its last product)."""
        n = self.mixer_norm
        return getattr(n, "weight", None) if n.reads_stream_by_kernel else None

    def forward(self, hidden: torch.Tensor, ctx: StepContext, io: LayerIO) -> None:
        rt = self.rt
        ctx.extras.pop("stream.rounded", None)         # (this block changes the stream: a rounded copy of it is no longer one)
        x = rt.ws.get("block.normed", hidden.shape, rt.dtype)
        # What the kernel object may make of knowing who follows whom (``CudaKernels.expect_norm``): the
        # norm after a part, so that the part's last product can prepare it, and whether a norm's
        # output goes to products alone.  A kernel object without these words is told nothing.
        expect = getattr(rt.k, "expect_norm", None)
        by_products = getattr(rt.k, "norm_output_read_by_products", None)
        if not self.mixer_norm.reads_stream_by_kernel:
            self.finish_products()
        if by_products is not None:
            by_products(self.mixer.reads_input_by_products)
        self.mixer_norm.forward(x, hidden)
        if expect is not None:
            after_mixer = (ctx.extras.get("norm_after_block") if getattr(self.ffn, "is_identity", False)
                           else getattr(self.ffn_norm, "weight", None) if self.ffn_norm.reads_stream_by_kernel else None)
            expect(after_mixer)
        self.mixer.forward(x, hidden, ctx, io)
        if getattr(self.ffn, "is_identity", False):        # a layer without a feed-forward
            if expect is not None:
                expect(None)
            return
        if not self.ffn_norm.reads_stream_by_kernel:
            self.finish_products()
        if by_products is not None:
            by_products(self.ffn.reads_input_by_products)
        self.ffn_norm.forward(x, hidden)
        if expect is not None:
            expect(ctx.extras.get("norm_after_block"))       # the model's word: the next block's first norm
        self.ffn.forward(x, hidden, ctx)
        if expect is not None:
            expect(None)


@register_arrangement("sublayer_norm")
class SublayerNormBlock(Part):
    """x <- x + norm1(mixer(x)), then x <- x + norm2(ffn(x)).  The parts still "add their result into the stream they
    are given": they are given a scratch row per token that counts as zeros (the kernel object's ``expect_blank``:
    the part's last product stores instead of adding), and the norm adds its result into the real stream
    (``Norm.add_into``).  In bfloat16 the sublayer's input is the stream rounded once per sublayer."""

    def __init__(self, hidden_size: int, mixer: Mixer, feed_forward: FeedForward,
                 mixer_norm: Norm, feed_forward_norm: Norm):
        self.hidden = int(hidden_size)
        self.mixer, self.ffn = mixer, feed_forward
        self.mixer_norm, self.ffn_norm = mixer_norm, feed_forward_norm

    children = PreNormBlock.children
    graph_safe = PreNormBlock.graph_safe
    prefers_plain_launches = PreNormBlock.prefers_plain_launches
    step_key = PreNormBlock.step_key

    def first_norm_weight(self):
        return None             # the block's first reader of the stream is not a norm

    def _sublayer(self, part, norm: Norm, hidden: torch.Tensor, run, ctx: StepContext) -> None:
        rt, k = self.rt, self.rt.k
        self.finish_products()          # (a block of another arrangement before this one may have left its last product)
        if rt.dtype == torch.float32:
            x = hidden
        else:
            x = rt.ws.get("block.input", hidden.shape, rt.dtype)
            # the norm that closed the sublayer before left the stream's rounded copy there (else: round it now)
            if ctx.extras.pop("stream.rounded", None) != x.data_ptr():
                k.cast_rows(x, hidden)
        y = rt.ws.get("block.sublayer_out", hidden.shape, torch.float32)
        blank = getattr(k, "expect_blank", None)
        if blank is not None:
            blank(y)
        else:
            y.zero_()
        run(x, y)
        if blank is not None:
            blank(None)
        if norm.add_into(hidden, y, x if x is not hidden else None):
            ctx.extras["stream.rounded"] = x.data_ptr()

    def forward(self, hidden: torch.Tensor, ctx: StepContext, io: LayerIO) -> None:
        for word in ("expect_norm", "norm_output_read_by_products"):
            say = getattr(self.rt.k, word, None)
            if say is not None:
                say(None if word == "expect_norm" else False)
        self._sublayer(self.mixer, self.mixer_norm, hidden, lambda x, y: self.mixer.forward(x, y, ctx, io), ctx)
        if not getattr(self.ffn, "is_identity", False):
            self._sublayer(self.ffn, self.ffn_norm, hidden, lambda x, y: self.ffn.forward(x, y, ctx), ctx)


@register_arrangement("sandwich_norm")
class SandwichNormBlock(Part):
    """x <- x + post1(mixer(pre1(x))), then x <- x + post2(ffn(pre2(x))).  The sublayer reads the normed rows (compute
    dtype) and "adds its result" into a scratch row per token that counts as zeros (``expect_blank``); the second norm
    norms that row and adds it into the fp32 stream in one kernel (``Norm.add_into``), and where the next reader of the
    stream is a norm of the same kind (the feed-forward's, or the next block's first) that kernel leaves its rows too
    (``add_into_then_norm``), so that a layer launches two norm kernels, not four."""

    def __init__(self, hidden_size: int, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, feed_forward_norm: Norm,
                 mixer_post_norm: Norm, feed_forward_post_norm: Optional[Norm] = None):
        self.hidden = int(hidden_size)
        self.mixer, self.ffn = mixer, feed_forward
        self.mixer_norm, self.ffn_norm = mixer_norm, feed_forward_norm
        self.mixer_post, self.ffn_post = mixer_post_norm, feed_forward_post_norm
        if self.ffn_post is None and not getattr(self.ffn, "is_identity", False):
            raise ValueError("sandwich_norm: a feed-forward without a norm on its output")

    def children(self) -> Dict[str, Part]:
        c = {"mixer": self.mixer, "feed_forward": self.ffn, "mixer_norm": self.mixer_norm,
             "feed_forward_norm": self.ffn_norm, "mixer_post_norm": self.mixer_post}
        if self.ffn_post is not None:
            c["feed_forward_post_norm"] = self.ffn_post
        return c

    graph_safe = PreNormBlock.graph_safe
    prefers_plain_launches = PreNormBlock.prefers_plain_launches
    step_key = PreNormBlock.step_key

    def first_norm_weight(self):
        return None             # (no product is told of this block's first norm: see ``first_norm``)

    def first_norm(self) -> Norm:
        """The norm that reads the stream first in this block: a block of this arrangement before it may run it together
        with its own closing norm."""
        return self.mixer_norm

    def _sublayer(self, pre: Norm, post: Norm, nxt, hidden: torch.Tensor, run, ctx: StepContext) -> None:
        rt, k = self.rt, self.rt.k
        self.finish_products()
        x = rt.ws.get("block.normed", hidden.shape, rt.dtype)
        # (the norm that closed the sublayer before may have left this norm's rows there)
        if ctx.extras.pop("stream.normed", None) != (x.data_ptr(), id(pre)):
            pre.forward(x, hidden)
        y = rt.ws.get("block.sublayer_out", hidden.shape, torch.float32)
        blank = getattr(k, "expect_blank", None)
        if blank is not None:
            blank(y)
        else:
            y.zero_()
        run(x, y)
        if blank is not None:
            blank(None)
        # the closing norm, the residual add and, where the next reader of the stream is a norm of the same kind, that
        # norm too (the sublayer is done with x: its rows may be written anew)
        fuse = getattr(post, "add_into_then_norm", None)
        if nxt is not None and fuse is not None and fuse(hidden, y, nxt, x):
            ctx.extras["stream.normed"] = (x.data_ptr(), id(nxt))
        else:
            post.add_into(hidden, y)

    def forward(self, hidden: torch.Tensor, ctx: StepContext, io: LayerIO) -> None:
        ctx.extras.pop("stream.rounded", None)
        for word in ("expect_norm", "norm_output_read_by_products"):
            say = getattr(self.rt.k, word, None)
            if say is not None:
                say(None if word == "expect_norm" else False)
        after = ctx.extras.get("first_norm_after_block")           # the model's word: the next block's first norm, if it has one to offer
        has_ffn = not getattr(self.ffn, "is_identity", False)
        self._sublayer(self.mixer_norm, self.mixer_post, self.ffn_norm if has_ffn else after, hidden,
                       lambda x, y: self.mixer.forward(x, y, ctx, io), ctx)
        if has_ffn:
            self._sublayer(self.ffn_norm, self.ffn_post, after, hidden, lambda x, y: self.ffn.forward(x, y, ctx), ctx)
