"""How a layer arranges its norms, mixer and feed-forward around the stream."""
from __future__ import annotations

from ..kernels import ops
from .base import Part
from .spec import PartSpec, build_part, register_part


class ResidualStream:
    """The float32 stream x [n, width] plus the last part's output that has
    not been added yet (`pending`): the next norm adds it while it normalises,
    so the add costs no pass of its own.  `pending_slabs` > 1 says that the
    output is a sum of that many float32 slabs (split-K shares of the part's last
    product, ctx.delta_slabs[0..k)), which the norm adds as well; 0 says that the
    part's last product has added its result to x itself (ctx.to_stream), so the
    norm has nothing to add.  `pending_norm` (a norm part, or None) says that the pending output passes through that
    norm before it joins the stream; whoever adds the pending output applies it (Norm.add_norm(delta_norm=...))."""

    def __init__(self, x, pending=None, pending_slabs: int = 1, pending_norm=None):
        self.x, self.pending, self.pending_slabs, self.pending_norm = x, pending, pending_slabs, pending_norm

    def settle(self, ctx) -> None:
        """Add what is pending to x now (through the pending norm's kernel, which then normalises nothing else), for
        a part that wants the whole stream rather than a normalised copy of it."""
        if self.pending is None or self.pending_slabs == 0:
            self.pending, self.pending_slabs, self.pending_norm = None, 0, None
            return
        if self.pending_norm is None:
            ops.add_slabs(self.x, self.pending, ctx.n_tokens, self.pending_slabs, ctx.delta_slabs.stride(0))
            self.pending, self.pending_slabs = None, 0
            return
        self.pending_norm.add_norm(ctx, self.x, self.pending, None, n_partials=self.pending_slabs,
                                   delta_norm=self.pending_norm)
        self.pending, self.pending_slabs, self.pending_norm = None, 0, None


class PreNormBlock(Part):
    """x = x + mixer(norm1(x)); x = x + feed_forward(norm2(x))
    (crates/models/qwen35-v2/src/model.rs:25-42).  `feed_forward` (with its norm) may be None: the layer then ends
    behind the mixer."""
    graph_safe = True
    category = "block"

    def __init__(self, runtime=None, prefix="", *, mixer: PartSpec, mixer_norm: PartSpec,
                 feed_forward: PartSpec | None = None, feed_forward_norm: PartSpec | None = None):
        super().__init__(runtime, prefix)
        self.mixer = build_part(mixer, runtime)
        self.mixer_norm = build_part(mixer_norm, runtime)
        self.feed_forward = self.feed_forward_norm = None
        if feed_forward is not None:
            if feed_forward_norm is None:
                raise ValueError("a feed-forward behind a norm needs that norm")
            self.feed_forward = build_part(feed_forward, runtime)
            self.feed_forward_norm = build_part(feed_forward_norm, runtime)

    def children(self):
        return [p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward) if p is not None]

    def forward(self, ctx, stream: ResidualStream, call) -> None:
        h, delta = ctx.normed, ctx.delta
        ctx.stream_x = stream.x
        self.mixer_norm.add_norm(ctx, stream.x, stream.pending, h, n_partials=stream.pending_slabs,
                                 delta_norm=stream.pending_norm)
        stream.pending_norm = None
        ctx.pending_slabs = 1                 # a part that leaves split-K shares in ctx.delta_slabs says how many
        self.mixer.forward(ctx, h, delta, call)
        stream.pending, stream.pending_slabs = delta, ctx.pending_slabs
        if self.feed_forward is not None:
            self.feed_forward_norm.add_norm(ctx, stream.x, stream.pending, h, n_partials=stream.pending_slabs)
            ctx.pending_slabs = 1
            self.feed_forward.forward(ctx, h, delta)
            stream.pending, stream.pending_slabs = delta, ctx.pending_slabs
        ctx.stream_x = None                   # another kind of block decides for itself whether parts may add to its stream


class SandwichNormBlock(Part):
    """A norm before and behind each sublayer:
        x = x + mixer_post_norm(mixer(mixer_norm(x)));  x = x + feed_forward_post_norm(feed_forward(feed_forward_norm(x)))
    `feed_forward` (with its two norms) may be None: the layer then ends behind the mixer.  A sublayer's output is
    left pending with its post norm; the next norm's kernel normalises it, adds it to the stream and normalises the
    stream for the next sublayer in one pass.  No product adds to the stream by itself here (ctx.stream_x stays
    None): what joins the stream is the normalised output, not the output."""
    graph_safe = True
    category = "block"

    def __init__(self, runtime=None, prefix="", *, mixer: PartSpec, mixer_norm: PartSpec, mixer_post_norm: PartSpec,
                 feed_forward: PartSpec | None = None, feed_forward_norm: PartSpec | None = None,
                 feed_forward_post_norm: PartSpec | None = None):
        super().__init__(runtime, prefix)
        self.mixer = build_part(mixer, runtime)
        self.mixer_norm = build_part(mixer_norm, runtime)
        self.mixer_post_norm = build_part(mixer_post_norm, runtime)
        self.feed_forward = self.feed_forward_norm = self.feed_forward_post_norm = None
        if feed_forward is not None:
            if feed_forward_norm is None or feed_forward_post_norm is None:
                raise ValueError("a feed-forward between two norms needs both of them")
            self.feed_forward = build_part(feed_forward, runtime)
            self.feed_forward_norm = build_part(feed_forward_norm, runtime)
            self.feed_forward_post_norm = build_part(feed_forward_post_norm, runtime)

    def children(self):
        return [p for p in (self.mixer_norm, self.mixer, self.mixer_post_norm, self.feed_forward_norm,
                            self.feed_forward, self.feed_forward_post_norm) if p is not None]

    def forward(self, ctx, stream: ResidualStream, call) -> None:
        h, delta = ctx.normed, ctx.delta
        ctx.stream_x = None
        self.mixer_norm.add_norm(ctx, stream.x, stream.pending, h, n_partials=stream.pending_slabs,
                                 delta_norm=stream.pending_norm)
        ctx.pending_slabs = 1
        self.mixer.forward(ctx, h, delta, call)
        stream.pending, stream.pending_slabs, stream.pending_norm = delta, ctx.pending_slabs, self.mixer_post_norm
        if self.feed_forward is None:
            return
        self.feed_forward_norm.add_norm(ctx, stream.x, stream.pending, h, n_partials=stream.pending_slabs,
                                        delta_norm=stream.pending_norm)
        ctx.pending_slabs = 1
        self.feed_forward.forward(ctx, h, delta)
        stream.pending, stream.pending_slabs, stream.pending_norm = delta, ctx.pending_slabs, self.feed_forward_post_norm


register_part("block", "pre_norm", PreNormBlock)
register_part("block", "sandwich_norm", SandwichNormBlock)
