"""Arrangements of a layer's parts around the residual stream."""

from __future__ import annotations

from .base import Block, NormedDelta, ScaledSum, register_block, split_pending


class PreNormBlock(Block):
    """``h = h + mixer(norm(h)); h = h + ffn(norm(h))`` (fastgen/forward.py:412-499).

    The residual stream is float32.  Each sum is fused into the norm that
    follows it, so the feed-forward's output is handed on as ``pending`` and
    added by the next layer's first norm (or by the model's final norm).
    """

    def forward(self, h, pending, ctx, memory):
        delta, delta_norm = split_pending(pending)
        a = self.mixer_norm.add_forward(h, delta, delta_norm=delta_norm)
        m = self.mixer.forward(a, ctx, memory)
        if self.ffn is None:  # a layer of one sub-layer
            return h, m
        f = self.ffn_norm.add_forward(h, m)
        return h, self.ffn.forward(f, ctx)


class SandwichBlock(Block):
    """Norms before and after each sub-layer:
    ``h = h + post_mixer_norm(mixer(norm(h))); h = h + post_ffn_norm(ffn(norm(h)))``.

    The two closing norms are the extra parts ``post_mixer_norm`` and ``post_ffn_norm``.  A
    sub-layer's output is handed on together with its closing norm, so that a norm which can
    (Dynamic Tanh) applies the closing norm, adds to the residual stream and norms the sum in
    one kernel.  A layer without a feed-forward (``ffn`` is ``None``) ends after the mixer.
    """

    def forward(self, h, pending, ctx, memory):
        delta, delta_norm = split_pending(pending)
        a = self.mixer_norm.add_forward(h, delta, delta_norm=delta_norm)
        m = self.mixer.forward(a, ctx, memory)
        post_mixer = self.extra.get("post_mixer_norm")
        if self.ffn is None:
            return h, NormedDelta(m, post_mixer)
        f = self.ffn_norm.add_forward(h, m, delta_norm=post_mixer)
        return h, NormedDelta(self.ffn.forward(f, ctx), self.extra.get("post_ffn_norm"))


class StreamsBlock(Block):
    """Pre-norm sub-layers on several residual streams: ``h`` is [T, streams, dim] and every
    sub-layer reads and writes it through a connection of its own, the extra parts
    ``mixer_connection`` and ``ffn_connection``.  What a sub-layer writes stays pending until the
    next read, whose kernel applies it.  A layer without a feed-forward ends after the mixer."""

    def forward(self, h, pending, ctx, memory):
        c = self.extra["mixer_connection"]
        m = self.mixer.forward(c.read(h, pending, self.mixer_norm), ctx, memory)
        pending = c.write(m)
        if self.ffn is None:
            return h, pending
        c = self.extra["ffn_connection"]
        return h, c.write(self.ffn.forward(c.read(h, pending, self.ffn_norm), ctx))


class ParallelBlock(Block):
    """One norm, read by every sub-layer: ``h = h + m * (mixer(norm(h)) + ffn(norm(h)))`` with ``m``
    the ``residual_mult`` of the block's parameters.  The sub-layers' outputs stay apart (a
    :class:`ScaledSum`) until the next norm, whose kernel multiplies each by its factor in float32,
    adds them to the residual stream and norms the result.  A layer without a feed-forward adds the
    mixer alone."""

    def forward(self, h, pending, ctx, memory):
        mult = self.params.residual_mult if self.params is not None else 1.0
        delta, delta_norm = split_pending(pending)
        a = self.mixer_norm.add_forward(h, delta, delta_norm=delta_norm)
        out = ScaledSum.of(self.mixer.forward(a, ctx, memory), mult)
        if self.ffn is not None:
            out = out.plus(ScaledSum.of(self.ffn.forward(a, ctx), mult))
        return h, out


register_block("prenorm", PreNormBlock)
register_block("parallel", ParallelBlock)
register_block("streams", StreamsBlock)
register_block("sandwich", SandwichBlock)
