"""Block arrangements.  `parallel`: h = norm(x); x += mult * (mixer(h) + ff(h)) - one norm, both sublayers
read its output, their sum is scaled into the stream (the feed-forward may be absent).  `pre_norm`: x += mixer(norm1(x)); x += ff(norm2(x))
(crates/llm/src/model/gpt2.rs:6-9, 229-266).  `sandwich`: a norm before AND after each sublayer,
x += scale1 * norm1b(mixer(conv(norm1(x)))); x += scale2 * norm2b(ff(norm2(x))), with a gain per channel
(`scale*`, may be absent), an optional short causal convolution that is added to the mixer's input
(`input_conv`), and an optional feed-forward; with `pre_norm` a `stream_copy` the sublayers read the stream itself and
only their results are normed, x += norm1(mixer(x)); x += norm2(ff(x)).  `stream_mix`: no sublayers - the stream is mixed with the
embedding output, x <- W [x; x0] + v[turn], which is how a repeated range of layers starts each of its
passes.  The residual stream stays in 32-bit; the parts add into it.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..cache.layout import StateNeed
from ..weights.source import TensorRequest
from .base import Block, Part, PartSpec, build_part, register_part
from .norms import PostNorm


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
    """x += mult * sum (or x += gain * norm(sum)) for a sum a block has left, for readers of the stream that do not
    fold it in."""
    pending = ctx.shared.pop("deferred_residual", None)
    if pending is not None:
        x, delta, mult = pending
        if isinstance(mult, PostNorm):
            ctx.ops.postnorm_rmsnorm(x[:ctx.n_rows], delta[:ctx.n_rows], mult.gain, mult.eps)
        else:
            ctx.ops.scale_add(x, delta, mult)


class InputConvolution(Part):
    """h <- h + conv(h): a causal convolution over time on each channel (`taps` taps, the last one on the row itself,
    zeros before a sequence's start, no bias), added to its own input.  A sequence keeps its last `taps` - 1 inputs
    (32-bit) in a cache entry of its own."""
    graph_safe = True
    kernel_families = ("channel_recurrence",)

    def __init__(self, prefix: str, width: int, taps: int, name: str = "canon1"):
        super().__init__(prefix)
        self.width, self.taps, self.name = int(width), int(taps), name
        if not (1 <= self.taps <= 16):
            raise ValueError("input convolution: 1 to 16 taps")
        self.weight = None

    def own_requests(self):
        return [TensorRequest(self.prefix + self.name, (self.width, self.taps))]

    def load_own(self, fetch):
        self.weight = fetch(self.prefix + self.name).contiguous()

    def own_tensors(self):
        return [self.weight] if self.weight is not None else []

    def cache_need(self):
        return StateNeed((max(1, (self.taps - 1) * self.width),), torch.float32)

    def forward(self, ctx, h, entry: int):
        state, ops = ctx.state(entry), ctx.ops
        out = ctx.buffer(tuple(h.shape))
        one_each = ctx.batch.is_decode          # every sequence brings one row: the kept inputs move on in the same launch
        ops.residual_conv(h, self.weight, out, state, 0, ctx.row_seq, ctx.row_pos, ctx.seq_starts, ctx.seq_slots, shift=one_each)
        if not one_each:
            ops.conv_keep(h, self.taps, state, 0, ctx.seq_starts, ctx.seq_slots, ctx.n_seqs)
        return out


class SandwichBlock(Block):
    """Both sublayers add into a cleared 32-bit sum of the stream's shape; how that sum enters the stream (normed,
    times the gain) is left in `ctx.shared["deferred_residual"]` for the next norm that reads the stream, which does
    x += gain * norm(sum), clears the sum and normalises x in one pass over the rows."""
    graph_safe = True
    kernel_families = ("norm_rotary",)

    def __init__(self, prefix: str, norm: PartSpec, mixer: PartSpec, feed_forward=None, input_conv: Optional[dict] = None,
                 scaled: bool = True, pre_norm: Optional[PartSpec] = None, norm1_name: str = "norm1", norm1b_name: str = "norm1b", norm2_name: str = "norm2",
                 norm2b_name: str = "norm2b", scale1_name: str = "ls1", scale2_name: str = "ls2", mixer_name: str = "mix.",
                 feed_forward_name: str = "mlp."):
        super().__init__(prefix)
        # `pre_norm`: what the sublayers read the stream through, if not `norm` (the norm of the results keeps `norm`'s width and eps)
        before = pre_norm if pre_norm is not None else norm
        self.norm1 = build_part("norm", before, prefix + norm1_name)
        self.mixer = build_part("mixer", mixer, prefix + mixer_name)
        self.conv = InputConvolution(prefix, **input_conv) if input_conv else None
        self.feed_forward = build_part("feed_forward", feed_forward, prefix + feed_forward_name) if feed_forward is not None else None
        self.norm2 = build_part("norm", before, prefix + norm2_name) if self.feed_forward is not None else None
        self.width, self.eps = int(norm.params["width"]), float(norm.params["eps"])
        self.scaled = bool(scaled)
        self.names = [(norm1b_name, scale1_name)] + ([(norm2b_name, scale2_name)] if self.feed_forward is not None else [])
        self.post: list = []

    def children(self):
        return [p for p in (self.norm1, self.conv, self.mixer, self.norm2, self.feed_forward) if p is not None]

    def cache_need(self):
        return self.conv.cache_need() if self.conv is not None else None

    def own_requests(self):
        out = []
        if self.conv is not None and getattr(self.mixer, "extra_cache_need", None) is not None and self.mixer.extra_cache_need() is not None:
            raise ValueError("sandwich: the input convolution and the mixer both want the call's `aux` cache entry")
        for norm_name, scale_name in self.names:
            out.append(TensorRequest(self.prefix + norm_name, (self.width,)))
            if self.scaled:
                out.append(TensorRequest(self.prefix + scale_name, (self.width,)))
        return out

    def load_own(self, fetch):
        self.post = []
        for norm_name, scale_name in self.names:
            gain = fetch(self.prefix + norm_name, keep_f32=True).float()
            if self.scaled:
                gain = gain * fetch(self.prefix + scale_name, keep_f32=True).float()
            self.post.append(PostNorm(gain.contiguous(), self.eps))

    def own_tensors(self):
        return [p.gain for p in self.post]

    def forward(self, ctx, x, call):
        pending = ctx.shared.get("deferred_residual")
        if pending is not None and not (getattr(self.norm1, "takes_deferred", False) and pending[0] is x):
            flush_deferred(ctx)
            pending = None
        if pending is not None:
            delta = pending[1]
        else:
            delta = ctx.shared.get("residual_sum")
            if delta is None or delta.shape != x.shape:
                delta = ctx.shared["residual_sum"] = ctx.buffer(tuple(x.shape), x.dtype)
                ctx.ops.zero(delta)
        h = self.norm1.forward(ctx, x, n_rows=ctx.n_rows)          # (takes up what the block before left)
        if self.conv is not None:
            h = self.conv.forward(ctx, h, call.aux)
        self.mixer.forward(ctx, h, delta, call)
        ctx.shared["deferred_residual"] = (x, delta, self.post[0])
        if self.feed_forward is not None:
            if not getattr(self.norm2, "takes_deferred", False):
                flush_deferred(ctx)
            h = self.norm2.forward(ctx, x, n_rows=ctx.n_rows)
            self.feed_forward.forward(ctx, h, delta)
            ctx.shared["deferred_residual"] = (x, delta, self.post[1])


class StreamMixBlock(Block):
    """x <- W [x; x0] + v[call.turn]: the stream and the embedding output (left in `ctx.shared["embedding_output"]` by
    an embedding told to keep it) side by side through one product `[width, 2 width]`, plus row `turn` of a table
    `[turns, width]`.  No mixer, nothing kept."""
    graph_safe = True
    kernel_families = ("norm_rotary",)
    mixer = None

    def __init__(self, prefix: str, width: int, turns: int, in_name: str = "in", step_name: str = "step"):
        super().__init__(prefix)
        self.width, self.turns, self.in_name, self.step_name = int(width), int(turns), in_name, step_name
        self.weight = self.steps = None

    def own_requests(self):
        return [TensorRequest(self.prefix + self.in_name, (self.width, 2 * self.width)),
                TensorRequest(self.prefix + self.step_name, (self.turns, self.width))]

    def load_own(self, fetch):
        self.weight = fetch(self.prefix + self.in_name).contiguous()
        self.steps = fetch(self.prefix + self.step_name, keep_f32=True).float().contiguous()

    def own_tensors(self):
        return [self.weight, self.steps]

    def forward(self, ctx, x, call):
        flush_deferred(ctx)
        x0 = ctx.shared.get("embedding_output")
        if x0 is None or x0.shape != x.shape:
            raise ValueError("stream_mix: the embedding has not kept its output for this step")
        if not (0 <= call.turn < self.turns):
            raise ValueError(f"stream_mix: pass {call.turn} of {self.turns}")
        both = ctx.buffer((x.shape[0], 2 * self.width))
        ctx.ops.stream_concat(x, x0, both)
        ctx.ops.linear(both, self.weight, self.steps[call.turn], x, "store_f32")


register_part("block", "pre_norm", PreNormBlock)
register_part("block", "parallel", ParallelBlock)
register_part("block", "sandwich", SandwichBlock)
register_part("block", "stream_mix", StreamMixBlock)
