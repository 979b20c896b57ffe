"""Block arrangements.  `parallel`: h = norm(x); x += mult * (mixer(h) + ff(h)) - one norm, both sublayers
read its output, their sum is scaled into the stream (the feed-forward may be absent).  `pre_norm`: x += mixer(norm1(x)); x += ff(norm2(x))
(crates/llm/src/model/gpt2.rs:6-9, 229-266).  The residual stream stays in
32-bit; the parts add into it.
"""
from __future__ import annotations

from .base import Block, PartSpec, build_part, register_part


class PreNormBlock(Block):
    graph_safe = True

    def __init__(self, prefix: str, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec, feed_forward: PartSpec,
                 norm1_name: str = "norm1.", mixer_name: str = "mixer.", norm2_name: str = "norm2.",
                 feed_forward_name: str = "ff."):
        super().__init__(prefix)
        self.norm1 = build_part("norm", norm1, prefix + norm1_name)
        self.mixer = build_part("mixer", mixer, prefix + mixer_name)
        self.norm2 = build_part("norm", norm2, prefix + norm2_name)
        self.feed_forward = build_part("feed_forward", feed_forward, prefix + feed_forward_name)

    def children(self):
        return [self.norm1, self.mixer, self.norm2, self.feed_forward]

    def forward(self, ctx, x, call):
        h = self.norm1.forward(ctx, x, n_rows=ctx.n_rows)
        self.mixer.forward(ctx, h, x, call)
        h = self.norm2.forward(ctx, x, n_rows=ctx.n_rows)
        self.feed_forward.forward(ctx, h, x)


class ParallelBlock(Block):
    """The sublayers add into a 32-bit sum of the stream's shape (their products' residual epilogues), not into
    the stream; the scaled sum is left in `ctx.shared["deferred_residual"]` for the next reader of the
    stream - the next block's norm or the head's, which folds `x += mult * sum` (and the clearing of the sum)
    into its own pass over the rows; a reader that cannot is served by `flush_deferred` first."""
    graph_safe = True
    kernel_families = ("norm_rotary",)

    def __init__(self, prefix: str, norm: PartSpec, mixer: PartSpec, feed_forward=None, residual_mult: float = 1.0,
                 norm_name: str = "norm1", mixer_name: str = "mix.", feed_forward_name: str = "mlp."):
        super().__init__(prefix)
        self.norm = build_part("norm", norm, prefix + norm_name)
        self.mixer = build_part("mixer", mixer, prefix + mixer_name)
        self.feed_forward = build_part("feed_forward", feed_forward, prefix + feed_forward_name) if feed_forward is not None else None
        self.residual_mult = float(residual_mult)

    def children(self):
        return [self.norm, self.mixer] + ([self.feed_forward] if self.feed_forward is not None else [])

    def forward(self, ctx, x, call):
        pending = ctx.shared.get("deferred_residual")
        if pending is not None and not (getattr(self.norm, "takes_deferred", False) and pending[0] is x):
            flush_deferred(ctx)
            pending = None
        if pending is not None:
            delta = pending[1]
        else:
            delta = ctx.shared.get("residual_sum")
            if delta is None or delta.shape != x.shape:
                delta = ctx.shared["residual_sum"] = ctx.buffer(tuple(x.shape), x.dtype)
                ctx.ops.zero(delta)
        h = self.norm.forward(ctx, x, n_rows=ctx.n_rows)          # (takes up what the block before left)
        self.mixer.forward(ctx, h, delta, call)
        if self.feed_forward is not None:
            self.feed_forward.forward(ctx, h, delta)
        ctx.shared["deferred_residual"] = (x, delta, self.residual_mult)


def flush_deferred(ctx) -> None:
    """x += mult * sum for a scaled sum a block has left, for readers of the stream that do not fold it in."""
    pending = ctx.shared.pop("deferred_residual", None)
    if pending is not None:
        x, delta, mult = pending
        ctx.ops.scale_add(x, delta, mult)


register_part("block", "pre_norm", PreNormBlock)
register_part("block", "parallel", ParallelBlock)
