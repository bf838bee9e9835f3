"""Pre-norm residual arrangement (reference src/qwen25vl_lite/text.py:196-206):
``x += mixer(norm1(x)); x += ffn(norm2(x))``.

The additions never run as kernels of their own.  A part that says ``accepts_residual``
adds its result into the float32 stream in the epilogue of its last product; otherwise the
result is carried as a pending update into the next norm kernel, which adds it before
normalising.  A part that says ``accepts_deferred_norm`` may be handed a norm that has not
run yet, to be computed inside its first product."""

from __future__ import annotations

from .base import Block, PendingUpdate, register_block


@register_block("prenorm_residual")
class PreNormResidualBlock(Block):
    def forward(self, ctx, x, pending, stop):
        mixer, ffn = self.mixer, self.feed_forward
        h = self.norms[0].forward(ctx, x, pending, defer=mixer.accepts_deferred_norm)
        if mixer.accepts_residual:
            mixed = mixer.forward(ctx, h, stop, residual=x)
        else:
            mixed = mixer.forward(ctx, h, stop)
        if ffn is None:                  # a layer of a mixer alone: its update is added by whoever normalises next
            return mixed
        h = self.norms[1].forward(ctx, x, mixed, defer=ffn.accepts_deferred_norm)
        if ffn.accepts_residual:
            return ffn.forward(ctx, h, residual=x)
        return ffn.forward(ctx, h)


@register_block("sandwich_residual")
class SandwichResidualBlock(Block):
    """Every sublayer is normalised before and after: ``x += norm1b(mixer(norm1(x)))``, then
    ``x += norm2b(ffn(norm2(x)))``; the norms come in that order (norm1, norm1b, norm2, norm2b).  A
    layer without a feed-forward has the mixer's two norms only.  The norm after a sublayer runs
    inside the kernel that adds the sublayer's result and normalises for the next one: the block
    hands its last result on as a ``PendingUpdate``."""

    def forward(self, ctx, x, pending, stop):
        h = self.norms[0].forward(ctx, x, pending)
        mixed = PendingUpdate(self.mixer.forward(ctx, h, stop), self.norms[1])
        if self.feed_forward is None:
            return mixed
        h = self.norms[2].forward(ctx, x, mixed)
        return PendingUpdate(self.feed_forward.forward(ctx, h), self.norms[3])
