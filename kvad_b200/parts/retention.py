"""Retention as a mixer: linear attention with a fixed decay per head, no softmax and no denominator.

    q = W_q h, k = W_k h (heads x key_dim), v = W_v h (heads x value_dim), turned by position (`position`,
    a rotary encoding over the heads' first entries), k scaled by `key_scale` afterwards;
    S_t = decay_h S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t           per sequence and head;
    each head's o over its root mean square (`unit_norm`), the heads side by side times silu(W_g h) (`gate`),
    then the output projection.

`activation="silu"`: q, k and v pass a silu first (linear attention behind silu, "lightning attention").  `row_norm`
{name, eps}: instead of the per-head unit norm, all heads of a row are RMS-normed together with a weight as long as
the row, and the gate is sigmoid(W_g h).

What a sequence keeps is one 32-bit state `[heads, key_dim, value_dim]` in its cache slot, zero at the
start and carried from row to row and from step to step.  The four projections run as one product; the
turning, the recurrence, the norm and the gate are one kernel (`csrc/retention.cu`), everything in it 32-bit.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..cache.layout import StateNeed
from .base import Mixer, PartSpec, build_part, register_part
from .linear import FusedLinear, Linear


class Retention(Mixer):
    graph_safe = True
    kernel_families = ("retention", "norm_rotary")

    def __init__(self, prefix: str, width: int, n_heads: int, key_dim: int, decay: Sequence[float],
                 value_dim: Optional[int] = None, key_scale: Optional[float] = None, position: Optional[PartSpec] = None,
                 unit_norm_eps: Optional[float] = None, gate: bool = True, q_name: str = "q", k_name: str = "k",
                 v_name: str = "v", gate_name: str = "g", out_name: str = "o", activation: Optional[str] = None,
                 row_norm: Optional[dict] = None):
        super().__init__(prefix)
        self.width, self.n_heads, self.key_dim = int(width), int(n_heads), int(key_dim)
        self.value_dim = int(value_dim) if value_dim else self.key_dim
        if len(decay) != self.n_heads:
            raise ValueError(f"retention: {len(decay)} decays for {self.n_heads} heads")
        self.decay_values = [float(d) for d in decay]
        self.key_scale = float(key_scale) if key_scale is not None else 1.0
        self.unit_norm_eps = None if unit_norm_eps is None else float(unit_norm_eps)
        self.gated = bool(gate)
        if activation not in (None, "silu"):
            raise ValueError("retention: q, k and v pass no activation or `silu`")
        self.silu_inputs = activation == "silu"
        self.row_norm = dict(row_norm) if row_norm else None
        if self.row_norm is not None and self.unit_norm_eps is not None:
            raise ValueError("retention: a norm per head or one over the row, not both")
        self.row_weight = None
        self.qk_width, self.v_width = self.n_heads * self.key_dim, self.n_heads * self.value_dim
        maps = [(q_name, self.qk_width), (k_name, self.qk_width), (v_name, self.v_width)]
        if self.gated:
            maps.append((gate_name, self.v_width))
        self.proj = FusedLinear(prefix, self.width, maps)
        self.out = Linear(prefix + out_name, self.v_width, self.width, bias=False, weight_name="")
        self.position = build_part("position", position, prefix) if position is not None else None
        if self.position is not None and getattr(self.position, "dims", 0) > self.key_dim:
            raise ValueError("retention: more rotated entries than a head has")
        self.decay = None

    def children(self):
        return [self.proj, self.out] + ([self.position] if self.position is not None else [])

    def own_requests(self):
        from ..weights.source import TensorRequest
        return [TensorRequest(self.prefix + self.row_norm.get("name", "norm"), (self.v_width,))] if self.row_norm else []

    def own_tensors(self):
        return [self.row_weight] if self.row_weight is not None else []

    def load_own(self, fetch):
        if self.row_norm:
            self.row_weight = fetch(self.prefix + self.row_norm.get("name", "norm"), keep_f32=True).float().contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=getattr(fetch, "device", "cuda"))

    def cache_need(self):
        return StateNeed((self.n_heads, self.key_dim, self.value_dim), torch.float32)

    def forward(self, ctx, h, residual, call):
        n = h.shape[0]
        buf = ctx.buffer((n, self.proj.out_features))
        self.proj.forward(ctx, h, buf)
        q, k, v = (buf[:, self.proj.columns(i)] for i in range(3))
        gate = buf[:, self.proj.columns(3)] if self.gated else None
        mixed = ctx.buffer((n, self.v_width))
        pos = self.position
        if self.row_norm is not None:      # the raw 32-bit read-outs of all heads, then one norm over the row and the sigmoid gate
            raw = ctx.buffer((n, self.v_width), torch.float32)
            ctx.ops.retention(q, k, v, None, ctx.state(call.cache), ctx.seq_starts, ctx.kv_lens, ctx.seq_slots, ctx.n_seqs,
                              self.decay, self.n_heads, inv_freq=pos.inv_freq if pos is not None else None,
                              rot_dims=pos.dims if pos is not None else 0, interleaved=pos.interleaved if pos is not None else False,
                              k_scale=self.key_scale, raw=raw, silu_inputs=self.silu_inputs, raw_only=True)
            ctx.ops.row_norm_gate(raw, gate, self.row_weight, mixed, float(self.row_norm["eps"]))
            self.out.forward(ctx, mixed, residual, "residual")
            return
        raw = ctx.buffer((n, self.v_width), torch.float32) if ctx.ops.retention_needs_raw(self.key_dim, self.value_dim) else None
        ctx.ops.retention(q, k, v, mixed, ctx.state(call.cache), ctx.seq_starts, ctx.kv_lens, ctx.seq_slots, ctx.n_seqs,
                          self.decay, self.n_heads, inv_freq=pos.inv_freq if pos is not None else None,
                          rot_dims=pos.dims if pos is not None else 0, interleaved=pos.interleaved if pos is not None else False,
                          k_scale=self.key_scale, gate=gate, unit_norm_eps=self.unit_norm_eps, raw=raw, silu_inputs=self.silu_inputs)
        self.out.forward(ctx, mixed, residual, "residual")


register_part("mixer", "retention", Retention)
