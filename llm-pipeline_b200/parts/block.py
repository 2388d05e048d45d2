"""Arrangements of a mixer, a feed-forward and their norms around the residual stream.

``pre_norm_residual`` is the decoder layer of
src/llm_pipeline/models/qwen3/custom_builder.py:222-255: ``x += mixer(norm1(x))`` then
``x += feed_forward(norm2(x))``. The sums are not taken here: each part's output is left pending
on the stream and the next norm kernel adds it into the float32 residual."""

from __future__ import annotations

from .base import Block, LayerCache, ResidualStream
from .registry import register_block


@register_block("pre_norm_residual")
class PreNormResidualBlock(Block):
    NORMS = ("mixer", "feed_forward")

    def forward(self, stream: ResidualStream, ctx, cache: LayerCache) -> None:
        h = self._norm(self.mixer_norm, self.mixer, stream, ctx)
        out, bias = getattr(self.mixer, "forward_deferred", self.mixer.forward)(h, ctx, cache)
        stream.add(out, bias)
        h = self._norm(self.feed_forward_norm, self.feed_forward, stream, ctx)
        out, bias = getattr(self.feed_forward, "forward_deferred", self.feed_forward.forward)(h, ctx)
        stream.add(out, bias)

    @staticmethod
    def _norm(norm, consumer, stream: ResidualStream, ctx):
        """The norm's rows for ``consumer``: with their factors still to be applied where the norm can leave them so
        and the consumer takes them so."""
        deferred = getattr(norm, "add_norm_deferred", None)
        if deferred is not None and getattr(consumer, "takes_scaled_rows", False):
            return deferred(stream, ctx)
        return norm.add_norm(stream, ctx)


@register_block("sandwich_norm_residual")
class SandwichNormResidualBlock(Block):
    """A norm before and after each sublayer: ``x += norm_out(mixer(norm_in(x)))``, then the same around the
    feed-forward if the layer has one. Neither the outer norms nor the sums are taken here: a sublayer's output is left
    pending on the stream together with the norm it has to pass, and the next norm kernel norms it, adds it into the
    float32 residual and norms the sum for its own reader in one pass. A layer with a depth mix asks the stream for it
    at its end (``ResidualStream.mix``), which the same kernel does."""

    NORMS = ("mixer", "mixer_out", "feed_forward", "feed_forward_out")

    def needed_norms(self):
        return self.NORMS if self.feed_forward is not None else ("mixer", "mixer_out")

    def forward(self, stream: ResidualStream, ctx, cache: LayerCache) -> None:
        h = self.norms["mixer"].add_norm(stream, ctx)
        out, bias = self.mixer.forward(h, ctx, cache)
        stream.add(out, bias, norm=self.norms["mixer_out"])
        if self.feed_forward is not None:
            h = self.norms["feed_forward"].add_norm(stream, ctx)
            out, bias = self.feed_forward.forward(h, ctx)
            stream.add(out, bias, norm=self.norms["feed_forward_out"])
        if self.depth_mix is not None:
            stream.mix(self.depth_mix.weights, self.depth_mix.index)


@register_block("parallel_residual")
class ParallelResidualBlock(Block):
    """One norm, and both sublayers read its output: ``x += mixer(norm(x)) + feed_forward(norm(x))`` (a layer without a
    feed-forward adds the mixer's output alone). Neither sum is taken here: the two outputs are left pending on the
    stream side by side, and the next norm kernel adds both into the float32 residual before it norms the row."""

    NORMS = ("mixer",)

    def forward(self, stream: ResidualStream, ctx, cache: LayerCache) -> None:
        h = self.norms["mixer"].add_norm(stream, ctx)
        out, bias = self.mixer.forward(h, ctx, cache)
        stream.add(out, bias)
        if self.feed_forward is not None:
            out, bias = self.feed_forward.forward(h, ctx)
            if bias is not None:
                out = out.float() + bias.float()
            stream.add_beside(out)
