"""minGRU as a mixer: a gated recurrence, element by element, whose gates read only the current token.

    z = sigmoid(W_z h + b_z),  u = W_x h + b_x,  c = u + 1/2 where u >= 0, sigmoid(u) where u < 0
    S_t = (1 - z_t) S_(t-1) + z_t c_t                      (S_0 = 0; one number per channel, `inner` channels)
    out = W_o (S_t * silu(W_g h))

A sequence keeps S in its cache slot, in 32-bit.  The three projections of h run as one product that leaves 32-bit
sums; the gates, the candidate, the state and the read-out are 32-bit, one kernel (`csrc/channel_recurrence.cu`)
that walks a prompt's rows in chunks side by side, since the recurrence is linear in S.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..cache.layout import StateNeed
from .base import Mixer, register_part
from .linear import FusedLinear, Linear


class MinGRU(Mixer):
    graph_safe = True
    kernel_families = ("channel_recurrence",)

    def __init__(self, prefix: str, width: int, inner: int, z_name: str = "z", x_name: str = "x", gate_name: str = "g",
                 out_name: str = "o", bias_suffix: Optional[str] = ".b"):
        super().__init__(prefix)
        self.width, self.inner = int(width), int(inner)
        self.proj = FusedLinear(prefix, self.width, [(z_name, self.inner), (x_name, self.inner), (gate_name, self.inner)],
                                bias_suffix=bias_suffix, biased=(z_name, x_name))
        self.out = Linear(prefix + out_name, self.inner, self.width, bias=False, weight_name="")

    def children(self):
        return [self.proj, self.out]

    def cache_need(self):
        return StateNeed((self.inner,), torch.float32)

    def forward(self, ctx, h, residual, call):
        n = h.shape[0]
        sums = ctx.buffer((n, 3 * self.inner), torch.float32)
        self.proj.forward(ctx, h, sums, "store_f32")
        mixed = ctx.buffer((n, self.inner))
        ctx.ops.min_gru(sums, self.inner, mixed, ctx.state(call.cache), ctx.seq_starts, ctx.seq_slots, ctx.n_seqs, ctx.batch.max_new)
        self.out.forward(ctx, mixed, residual, "residual")


register_part("mixer", "min_gru", MinGRU)
