"""How a layer's parts are arranged: the pre-norm residual block, and the block with both branches side by side.

``h += mixer(norm1(h)); h += feed_forward(norm2(h))`` as in
``src/turboserve/engine/model/layers.py:469-487``. The residual stream ``h`` is fp32; a part's
output is not added at once but handed on as ``pending`` and added by the next norm's kernel
(the fused residual-add + norm), so each sum is computed in 32-bit and read once.
"""

from __future__ import annotations

import torch

from .base import FeedForward, Mixer, Norm, NormedUpdate, ScaledUpdates, pending_updates, register_block, settle_pending


class PreNormBlock:
    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, feed_forward_norm: Norm) -> None:
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm

    def forward(self, residual: torch.Tensor, pending: torch.Tensor | None, ctx, cache) -> torch.Tensor:
        """Run the layer; returns the new pending update (the feed-forward's output)."""
        n, hidden = ctx.batch.num_tokens, residual.shape[-1]
        normed = ctx.buffer("block.normed", (n, hidden))
        self.mixer_norm.forward(residual, pending, normed, ctx)
        mixed = self.mixer.forward(normed, ctx, cache)
        self.feed_forward_norm.forward(residual, mixed, normed, ctx)
        return self.feed_forward.forward(normed, ctx)


class ParallelBlock:
    """Mixer and feed-forward side by side on the same input: ``h += mixer(norm1(h)) + ff(norm2(h))``.

    Both branches' outputs are handed on as a pair of pending updates; the next norm's kernel adds
    both into the fp32 residual (and a stream shift, if the next run brings one) and, when both
    norms are RMS norms with one ``eps``, writes both normed inputs in the same pass. A layer
    without a feed-forward has one branch. With ``residual_mult`` ``m`` other than 1 the layer is
    ``h += m * (mixer(norm1(h)) + ff(norm2(h)))``: the factor travels with the pending updates.
    """

    takes_shift = True

    def __init__(self, mixer: Mixer, feed_forward: FeedForward | None, mixer_norm: Norm, feed_forward_norm: Norm | None,
                 residual_mult: float = 1.0) -> None:
        self.residual_mult = float(residual_mult)
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm
        if (feed_forward is None) != (feed_forward_norm is None):
            raise ValueError("a feed-forward and its norm go together")

    def forward(self, residual: torch.Tensor, pending, ctx, cache, shift: torch.Tensor | None = None):
        n, hidden = ctx.batch.num_tokens, residual.shape[-1]
        for_mixer = ctx.buffer("block.normed", (n, hidden))
        if self.feed_forward is None:
            self.mixer_norm.forward(residual, pending, for_mixer, ctx, shift=shift)
            return self._scaled((self.mixer.forward(for_mixer, ctx, cache),))
        for_ff = ctx.buffer("block.normed_ff", (n, hidden))
        pair = getattr(self.mixer_norm, "forward_pair", None)
        if pair is not None and getattr(self.feed_forward_norm, "eps", None) == getattr(self.mixer_norm, "eps", 0):
            pair(residual, pending, self.feed_forward_norm, for_mixer, for_ff, ctx, shift=shift)
        else:
            self.mixer_norm.forward(residual, pending, for_mixer, ctx, shift=shift)
            self.feed_forward_norm.forward(residual, None, for_ff, ctx)
        mixed = self.mixer.forward(for_mixer, ctx, cache)
        return self._scaled((mixed, self.feed_forward.forward(for_ff, ctx)))

    def _scaled(self, updates: tuple):
        if self.residual_mult == 1.0:
            return updates if len(updates) > 1 else updates[0]
        return ScaledUpdates(updates, self.residual_mult)


class OutputNormBlock:
    """Norms behind the sublayers, which read the stream itself:
    ``h += mult * norm1(mixer(h)); h += mult * norm2(feed_forward(h))``.

    Each sum is one kernel: it norms the sublayer's output (statistics over the output alone, fp32), scales
    it, adds it to the fp32 stream and writes the stream in the activation type, which is what the next
    sublayer reads (in float32 the sublayers read the stream directly). Nothing is left pending. The copy a
    block's last sum writes is the next block's input; ``ctx.stream_copy`` says which run it is for.
    ``residual_mult`` is the factor ``mult``. A layer without a feed-forward has one sum.
    """

    def __init__(self, mixer: Mixer, feed_forward: FeedForward | None, mixer_norm: Norm, feed_forward_norm: Norm | None,
                 residual_mult: float = 1.0) -> None:
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm
        self.residual_mult = float(residual_mult)
        if (feed_forward is None) != (feed_forward_norm is None):
            raise ValueError("a feed-forward and its norm go together")
        for norm in (mixer_norm, feed_forward_norm):
            if norm is not None and not hasattr(norm, "forward_output"):
                raise ValueError("this block needs norms that can norm a sublayer's output (forward_output)")

    def forward(self, residual: torch.Tensor, pending, ctx, cache):
        from ..ops import kernels

        n, hidden = ctx.batch.num_tokens, residual.shape[-1]
        if pending is not None:  # what a block of another kind before this one left to be added
            settle_pending(residual, pending, n, ctx.dtype)
            ctx.stream_copy = None
        if ctx.dtype == torch.float32:
            x = copy = None
        else:
            copy = ctx.buffer("block.stream", (n, hidden))
            left = ctx.stream_copy
            if left is None or left[1] != ctx.run_index or left[0].data_ptr() != copy.data_ptr():
                kernels.norm_add(residual, None, None, copy, 0.0, 0.0, n)
        x = residual if copy is None else copy
        mixed = self.mixer.forward(x, ctx, cache)
        self.mixer_norm.forward_output(residual, mixed, self.residual_mult, copy, ctx)
        if self.feed_forward is not None:
            moved = self.feed_forward.forward(x, ctx)
            self.feed_forward_norm.forward_output(residual, moved, self.residual_mult, copy, ctx)
        ctx.stream_copy = None if copy is None else (copy, ctx.run_index + 1)
        return None


class BothSidesNormBlock:
    """Norms before and behind each sublayer: ``h += post1(mixer(pre1(h))); h += post2(feed_forward(pre2(h)))``.

    What stands between two sublayers is one kernel: the norm behind the sublayer that ran (statistics over its output
    alone), the sum into the fp32 stream, and the norm before the sublayer that runs next. The feed-forward's output is
    therefore left pending with its norm (:class:`~turboserve_b200.parts.base.NormedUpdate`) and enters the stream in
    the next block's first kernel, or in the final norm's. ``rows_added`` is a float32 matrix, a row a token, added to
    the stream right before the layer (a repeated stretch of layers adds the embedding's output before each pass but
    the first). A layer without a feed-forward has one sublayer.
    """

    takes_shift = True
    takes_rows = True

    def __init__(self, mixer: Mixer, feed_forward: FeedForward | None, mixer_norm: Norm, feed_forward_norm: Norm | None,
                 mixer_output_norm: Norm | None = None, feed_forward_output_norm: Norm | None = None) -> None:
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm
        self.mixer_output_norm = mixer_output_norm
        self.feed_forward_output_norm = feed_forward_output_norm
        if mixer_output_norm is None or not hasattr(mixer_output_norm, "normed"):
            raise ValueError("this block needs a norm behind its mixer that can travel with a pending update (normed)")
        if (feed_forward is None) != (feed_forward_norm is None) or (feed_forward is None) != (feed_forward_output_norm is None):
            raise ValueError("a feed-forward and its two norms go together")
        if feed_forward_output_norm is not None and not hasattr(feed_forward_output_norm, "normed"):
            raise ValueError("this block needs a norm behind its feed-forward that can travel with a pending update (normed)")

    def forward(self, residual: torch.Tensor, pending, ctx, cache, shift: torch.Tensor | None = None,
                rows_added: torch.Tensor | None = None):
        n, hidden = ctx.batch.num_tokens, residual.shape[-1]
        normed = ctx.buffer("block.normed", (n, hidden))
        if rows_added is None:
            self.mixer_norm.forward(residual, pending, normed, ctx, shift=shift)
        else:
            self.mixer_norm.forward(residual, pending, normed, ctx, shift=shift, rows_added=rows_added)
        mixed = self.mixer_output_norm.normed(self.mixer.forward(normed, ctx, cache))
        if self.feed_forward is None:
            return mixed
        self.feed_forward_norm.forward(residual, mixed, normed, ctx)
        return self.feed_forward_output_norm.normed(self.feed_forward.forward(normed, ctx))


register_block("pre_norm", PreNormBlock)
register_block("both_sides_norm", BothSidesNormBlock)
register_block("output_norm", OutputNormBlock)
register_block("parallel", ParallelBlock)
