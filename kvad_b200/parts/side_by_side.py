"""Two mixers side by side, as one mixer.

Both read the same rows; each one's result is RMS-normed over the model width with a plain weight of its own, and the
mixer's result is `mult` times their sum (1/2: the mean):

    y = mult * (w_l * left(h) / rms(left(h)) + w_r * right(h) / rms(right(h)))

Each side is a mixer of any registered kind and keeps what it keeps: the left one in the call's cache entry, the right
one in the call's `aux` entry (`extra_cache_need`).  The sides' output products add into two cleared 32-bit buffers of the
stream's shape (their ordinary residual epilogues); one kernel norms both, adds the mean to the block's sum and clears
the buffers again.
"""
from __future__ import annotations

import dataclasses

import torch

from ..weights.source import TensorRequest
from .base import Mixer, PartSpec, build_part, register_part


class SideBySide(Mixer):
    graph_safe = True
    kernel_families = ("norm_rotary",)

    def __init__(self, prefix: str, width: int, left: PartSpec, right: PartSpec, eps: float, mult: float = 0.5,
                 left_name: str = "left.", right_name: str = "right.", left_norm_name: str = "left.out", right_norm_name: str = "right.out"):
        super().__init__(prefix)
        self.width, self.eps, self.mult = int(width), float(eps), float(mult)
        self.left = build_part("mixer", left, prefix + left_name)
        self.right = build_part("mixer", right, prefix + right_name)
        self.norm_names = (left_norm_name, right_norm_name)
        self.gains = [None, None]

    def children(self):
        return [self.left, self.right]

    def own_requests(self):
        return [TensorRequest(self.prefix + n, (self.width,)) for n in self.norm_names]

    def load_own(self, fetch):
        self.gains = [fetch(self.prefix + n, keep_f32=True).float().contiguous() for n in self.norm_names]

    def own_tensors(self):
        return [g for g in self.gains if g is not None]

    def cache_need(self):
        return self.left.cache_need()

    def extra_cache_need(self):
        """What the right-hand mixer keeps per sequence: the call's `aux` entry."""
        return self.right.cache_need()

    def forward(self, ctx, h, residual, call):
        sums = ctx.shared.get("side_sums")
        if sums is None or sums[0].shape != residual.shape:
            sums = ctx.shared["side_sums"] = (ctx.buffer(tuple(residual.shape), torch.float32), ctx.buffer(tuple(residual.shape), torch.float32))
            ctx.ops.zero(sums[0])
            ctx.ops.zero(sums[1])
        self.left.forward(ctx, h, sums[0], call)
        if self.right.cache_need() is not None and call.aux is None:
            raise ValueError("side_by_side: the right-hand mixer keeps something: the call needs an `aux` cache entry")
        self.right.forward(ctx, h, sums[1], dataclasses.replace(call, cache=call.aux if call.aux is not None else call.cache, aux=None))
        ctx.ops.pair_norm_sum(sums[0], sums[1], self.gains[0], self.gains[1], residual, self.eps, self.mult)


register_part("mixer", "side_by_side", SideBySide)
