"""Norms.  `rmsnorm`: x / sqrt(mean(x^2) + eps) times a weight, which may be stored around zero
(`unit_offset`: 1 is added) or be absent; it also takes up a scaled sum that a block before it still
owes to the residual stream (see `ParallelBlock`).  `layernorm`: centre, scale to unit variance (biased, eps inside the
root), then gain and bias - bisand/kvad's `layer_norm`
(crates/llm/src/tensor.rs:245-255).  Computed in 32-bit from the 32-bit
residual stream; gain and bias stay in 32-bit if the checkpoint stores them so.
"""
from __future__ import annotations

import torch

from ..weights.source import TensorRequest
from .base import Norm, register_part


class PostNorm:
    """How a sublayer's result enters the stream where it is normed first: x += gain * result / rms(result); `gain` is
    the norm's weight (times a block's gain per channel, if it has one), 32-bit.  Stands in the place of the
    multiplier in `ctx.shared["deferred_residual"]`."""

    def __init__(self, gain: torch.Tensor, eps: float):
        self.gain, self.eps = gain, float(eps)


class LayerNorm(Norm):
    graph_safe = True

    def __init__(self, prefix: str, width: int, eps: float, bias: bool = True):
        super().__init__(prefix)
        self.width, self.eps, self.has_bias = int(width), float(eps), bias
        self.gain = None
        self.bias = None

    def own_requests(self):
        out = [TensorRequest(self.prefix + "weight", (self.width,))]
        if self.has_bias:
            out.append(TensorRequest(self.prefix + "bias", (self.width,)))
        return out

    def load_own(self, fetch):
        self.gain = fetch(self.prefix + "weight", keep_f32=True)
        if self.has_bias:
            self.bias = fetch(self.prefix + "bias", keep_f32=True)
            if self.bias.dtype != self.gain.dtype:      # one dtype for the pair
                self.bias = self.bias.float()
                self.gain = self.gain.float()

    def own_tensors(self):
        return [t for t in (self.gain, self.bias) if t is not None]

    def forward(self, ctx, x, rows=None, n_rows=None):
        n = n_rows if n_rows is not None else (x.shape[0] if rows is None else rows.numel())
        out = ctx.buffer((n, self.width))
        ctx.ops.layernorm(x, self.gain, self.bias, self.eps, out, rows)
        return out


class RMSNorm(Norm):
    graph_safe = True
    kernel_families = ("norm_rotary",)
    #: a scaled sum that a block has left in `ctx.shared["deferred_residual"]` is folded in by this norm
    takes_deferred = True

    def __init__(self, prefix: str, width: int, eps: float, unit_offset: bool = False, name: str = "weight",
                 has_weight: bool = True):
        super().__init__(prefix)
        self.width, self.eps, self.unit_offset = int(width), float(eps), bool(unit_offset)
        self.name, self.has_weight = name, bool(has_weight)
        self.weight = None

    def own_requests(self):
        return [TensorRequest(self.prefix + self.name, (self.width,))] if self.has_weight else []

    def load_own(self, fetch):
        if self.has_weight:
            self.weight = fetch(self.prefix + self.name, keep_f32=True)

    def own_tensors(self):
        return [self.weight] if self.weight is not None else []

    def forward(self, ctx, x, rows=None, n_rows=None, out=None):
        """`out`: where to write (None: a new buffer of the compute dtype; a 32-bit one keeps a 32-bit input's precision)."""
        n = n_rows if n_rows is not None else (x.shape[0] if rows is None else rows.numel())
        if out is None:
            out = ctx.buffer((n, self.width))
        deferred = ctx.shared.get("deferred_residual") if x.dtype == torch.float32 else None
        if deferred is not None and deferred[0] is not x:
            deferred = None
        if deferred is not None:
            _, delta, mult = deferred
            if isinstance(mult, PostNorm):
                ctx.ops.postnorm_rmsnorm(x[:ctx.n_rows], delta[:ctx.n_rows], mult.gain, mult.eps, out, self.weight, self.eps,
                                         unit_offset=self.unit_offset, rows=rows)
            else:
                ctx.ops.rmsnorm(x[:ctx.n_rows], self.weight, self.eps, out, unit_offset=self.unit_offset, rows=rows,
                                deferred=(delta, mult))
            if rows is None:                      # the sum is in the stream now
                ctx.shared.pop("deferred_residual")
        else:
            ctx.ops.rmsnorm(x, self.weight, self.eps, out, unit_offset=self.unit_offset, rows=rows)
        return out


class StreamCopy(Norm):
    """No norm at all: the rows of the stream as they are, in the compute dtype - for sublayers that read the stream
    itself and whose RESULTS are normed (`PostNorm`).  Like `rmsnorm` it takes up a sum that a block before it still
    owes to the stream, in the same pass over the rows.  In the 32-bit engine the stream itself is handed on."""
    graph_safe = True
    kernel_families = ("norm_rotary",)
    takes_deferred = True

    def __init__(self, prefix: str, width: int):
        super().__init__(prefix)
        self.width = int(width)

    def forward(self, ctx, x, rows=None, n_rows=None, out=None):
        n = n_rows if n_rows is not None else (x.shape[0] if rows is None else rows.numel())
        deferred = ctx.shared.get("deferred_residual") if x.dtype == torch.float32 else None
        if deferred is not None and deferred[0] is not x:
            deferred = None
        same = ctx.dtype == torch.float32 and rows is None and out is None       # (the reader can take the stream itself)
        if deferred is not None and not isinstance(deferred[2], PostNorm):
            if rows is not None:
                raise ValueError("stream_copy: a scaled sum is taken up with all rows")
            from .block import flush_deferred
            flush_deferred(ctx)
            deferred = None
        if deferred is not None:
            _, delta, post = deferred
            if same:
                ctx.ops.postnorm_rmsnorm(x[:ctx.n_rows], delta[:ctx.n_rows], post.gain, post.eps)
            else:
                out = ctx.buffer((n, self.width)) if out is None else out
                ctx.ops.postnorm_rmsnorm(x[:ctx.n_rows], delta[:ctx.n_rows], post.gain, post.eps, out, rows=rows, plain_out=True)
            if rows is None:
                ctx.shared.pop("deferred_residual")
            return x[:n] if same else out
        if same:
            return x[:n]
        out = ctx.buffer((n, self.width)) if out is None else out
        ctx.ops.cast_rows(x, out, rows)
        return out


register_part("norm", "stream_copy", StreamCopy)
register_part("norm", "layernorm", LayerNorm)
register_part("norm", "rmsnorm", RMSNorm)
