"""Feed-forwards with clamped gates, alone or as a mixture of experts.

`clamped_glu_mlp`: g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit), y = g sigmoid(alpha g) (u + 1), out = W_down y;
no biases.  Gate and up run as one product, the activation as one row-wise kernel, the residual sum in the last
product's epilogue.

`routed_mlp`: `n_experts` such feed-forwards (`e0`, `e1`, ...), of which every row uses `top`: router logits
z = W_router h + b in 32-bit, the `top` largest are chosen, their weights are the softmax over the chosen logits only,
the output is the weighted sum of the chosen experts' outputs; an optional shared expert (`shared`, the same form with
sizes of its own) runs for every row and is added.  The (row, choice) pairs are grouped by expert on the device and
the experts' two products run as grouped products over those lists (`csrc/moe.cu`); how many tiles a step can need
follows from its shape alone, so the launches never depend on the routing.  The chosen experts' outputs are summed
choice by choice in a fixed order.

`score_routed_mlp`: experts of the plain form out = W_down act(W_up h), act = the square of relu, no biases, chosen by
scores: s = softmax(W_router h) over ALL router outputs (32-bit), the `top` largest of s + `correction` are chosen (the
correction only steers the choice), and the chosen weigh in with their s over the sum of the chosen s (+ 1e-20).  The
last `identity` router outputs are experts without matrices whose output is their input.  An optional shared expert of
the same form runs for every row, times sigmoid(w_sg . h), one number per row.  Same grouping, grouped products and
ordered sum as `routed_mlp`.

`input_scaled_routed_mlp`: gated experts out = W_down (act(W_gate x) * (W_up x)) (act = silu), no biases, chosen by the
`top` largest sigmoid scores s = sigmoid(W_router h) (32-bit), which are not renormalised and scale the expert's INPUT:
the output is the sum over the chosen of expert(s h).  Since the first two products are linear, s is applied to their
results where the gate is computed.  An optional shared expert (`gated_mlp` with the same activation) runs for every
row.  Same grouping, grouped products and ordered sum (with unit weights) as `routed_mlp`.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..weights.source import TensorRequest
from .base import FeedForward, register_part
from .linear import FusedLinear, Linear


class ClampedGluMLP(FeedForward):
    graph_safe = True
    kernel_families = ("moe",)

    def __init__(self, prefix: str, width: int, hidden: int, limit: float, alpha: float = 1.702, gate_name: str = "gate",
                 up_name: str = "up", down_name: str = "down"):
        super().__init__(prefix)
        self.width, self.hidden, self.limit, self.alpha = int(width), int(hidden), float(limit), float(alpha)
        self.gate_up = FusedLinear(prefix, self.width, [(gate_name, self.hidden, 8), (up_name, self.hidden, 8)], pad_to=8)
        self.down = Linear(prefix + down_name, self.hidden, self.width, bias=False, weight_name="")

    def children(self):
        return [self.gate_up, self.down]

    def forward(self, ctx, h, residual):
        n = h.shape[0]
        both = ctx.buffer((n, self.gate_up.out_features))
        self.gate_up.forward(ctx, h, both)
        hid = ctx.buffer((n, self.hidden))
        ctx.ops.clamped_glu(both[:, self.gate_up.columns(0)], both[:, self.gate_up.columns(1)], hid, self.limit, self.alpha)
        self.down.forward(ctx, hid, residual, "residual")


class RoutedMLP(FeedForward):
    graph_safe = True
    kernel_families = ("moe",)

    def __init__(self, prefix: str, width: int, n_experts: int, top: int, hidden: int, limit: float, alpha: float = 1.702,
                 shared: Optional[dict] = None, router_name: str = "router", router_bias_name: str = ".b", expert_name: str = "e{}.",
                 shared_name: str = "shared.", gate_name: str = "gate", up_name: str = "up", down_name: str = "down"):
        super().__init__(prefix)
        self.width, self.n_experts, self.top, self.hidden = int(width), int(n_experts), int(top), int(hidden)
        if not (1 <= self.top <= self.n_experts):
            raise ValueError(f"routed_mlp: every row uses {top} of {n_experts} experts")
        self.limit, self.alpha = float(limit), float(alpha)
        self.router = Linear(prefix + router_name, self.width, self.n_experts, bias=True, weight_name="", bias_name=router_bias_name)
        self.shared = ClampedGluMLP(prefix + shared_name, self.width, **shared) if shared else None
        self.names = dict(expert=expert_name, gate=gate_name, up=up_name, down=down_name)
        self.w_in = None           # [experts, 2 hidden, width]: every expert's gate rows, then its up rows
        self.w_out = None          # [experts, width, hidden]

    def children(self):
        return [self.router] + ([self.shared] if self.shared is not None else [])

    def _expert(self, e: int, which: str) -> str:
        return self.prefix + self.names["expert"].format(e) + self.names[which]

    def own_requests(self):
        out = []
        for e in range(self.n_experts):
            out += [TensorRequest(self._expert(e, "gate"), (self.hidden, self.width)), TensorRequest(self._expert(e, "up"), (self.hidden, self.width)),
                    TensorRequest(self._expert(e, "down"), (self.width, self.hidden))]
        return out

    def load_own(self, fetch):
        self.w_in = torch.stack([torch.cat([fetch(self._expert(e, "gate")), fetch(self._expert(e, "up"))], dim=0)
                                 for e in range(self.n_experts)]).contiguous()
        self.w_out = torch.stack([fetch(self._expert(e, "down")) for e in range(self.n_experts)]).contiguous()

    def own_tensors(self):
        return [t for t in (self.w_in, self.w_out) if t is not None]

    def forward(self, ctx, h, residual):
        n, ops, E, top, ff = h.shape[0], ctx.ops, self.n_experts, self.top, self.hidden
        logits = ctx.buffer((n, (E + 3) // 4 * 4), torch.float32)[:, :E]
        self.router.forward(ctx, h, logits, "store_f32")
        chosen, weight = ctx.buffer((n, top), torch.int32), ctx.buffer((n, top), torch.float32)
        tm = ops.moe_tile_rows(n, top, self.width % 8 == 0 and ff % 8 == 0)
        tiles = ops.moe_max_tiles(n, top, E, tm)
        tile_expert, slot_pos = ctx.buffer((tiles,), torch.int32), ctx.buffer((n * top,), torch.int32)
        pos_row, pos_slot = ctx.buffer((tiles * tm,), torch.int32), ctx.buffer((tiles * tm,), torch.int32)
        ops.moe_sort(chosen, E, tm, tile_expert, pos_row, pos_slot, slot_pos, logits=logits, weight=weight)       # (routes, then groups)
        both = ctx.buffer((tiles * tm, 2 * ff))
        few = n * top <= ops.MOE_FEW_SLOTS      # (by the step's shape only)
        if tm == ops.MOE_WIDE_TILE:            # many rows: whole tiles on the tensor cores, from a copy of the rows in position order
            rows = ctx.buffer((tiles * tm, self.width))
            ops.gather_rows(h, pos_row, rows)
            ops.grouped_linear(rows, self.w_in, both, tile_expert, pos_slot)
        else:
            ops.grouped_linear(h, self.w_in, both, tile_expert, pos_slot, in_rows=pos_row, few_rows=few)
        hid = ctx.buffer((tiles * tm, ff))
        ops.clamped_glu(both[:, :ff], both[:, ff:], hid, self.limit, self.alpha)
        outs = ctx.buffer((tiles * tm, self.width), torch.float32)
        ops.grouped_linear(hid, self.w_out, outs, tile_expert, pos_slot, few_rows=few)
        ops.moe_combine(residual, outs, slot_pos, weight)
        if self.shared is not None:
            self.shared.forward(ctx, h, residual)


class ScoreRoutedMLP(FeedForward):
    graph_safe = True
    kernel_families = ("moe",)

    def __init__(self, prefix: str, width: int, n_experts: int, top: int, hidden: int, identity: int = 0, shared: Optional[dict] = None,
                 router_name: str = "router", correction_name: Optional[str] = "correction", expert_name: str = "e{}.",
                 shared_name: str = "shared.", up_name: str = "up", down_name: str = "down", shared_gate_name: str = "sg"):
        super().__init__(prefix)
        self.width, self.n_experts, self.identity, self.top, self.hidden = int(width), int(n_experts), int(identity), int(top), int(hidden)
        self.n_routes = self.n_experts + self.identity
        if not (1 <= self.top <= self.n_routes) or self.n_experts < 0 or self.identity < 0:
            raise ValueError(f"score_routed_mlp: every row uses {top} of {self.n_routes} experts")
        self.router = Linear(prefix + router_name, self.width, self.n_routes, bias=False, weight_name="")
        self.names = dict(expert=expert_name, up=up_name, down=down_name, correction=correction_name)
        self.shared_hidden = int(shared["hidden"]) if shared else 0
        if shared:      # the shared expert's first product also gives its gate: one more row of the same matrix, on a 16-byte boundary
            self.shared_up = FusedLinear(prefix + shared_name, self.width, [(up_name, self.shared_hidden), (shared_gate_name, 1, 8)], pad_to=8)
            self.shared_down = Linear(prefix + shared_name + down_name, self.shared_hidden, self.width, bias=False, weight_name="")
        else:
            self.shared_up = self.shared_down = None
        self.w_in = self.w_out = self.correction = None          # [experts, hidden, width], [experts, width, hidden], [routes]

    def children(self):
        return [self.router] + ([self.shared_up, self.shared_down] if self.shared_up is not None else [])

    def _expert(self, e: int, which: str) -> str:
        return self.prefix + self.names["expert"].format(e) + self.names[which]

    def own_requests(self):
        out = []
        for e in range(self.n_experts):
            out += [TensorRequest(self._expert(e, "up"), (self.hidden, self.width)), TensorRequest(self._expert(e, "down"), (self.width, self.hidden))]
        if self.names["correction"]:
            out.append(TensorRequest(self.prefix + self.names["correction"], (self.n_routes,)))
        return out

    def load_own(self, fetch):
        if self.n_experts:
            self.w_in = torch.stack([fetch(self._expert(e, "up")) for e in range(self.n_experts)]).contiguous()
            self.w_out = torch.stack([fetch(self._expert(e, "down")) for e in range(self.n_experts)]).contiguous()
        if self.names["correction"]:
            self.correction = fetch(self.prefix + self.names["correction"], keep_f32=True).float().contiguous()

    def own_tensors(self):
        return [t for t in (self.w_in, self.w_out, self.correction) if t is not None]

    def forward(self, ctx, h, residual):
        n, ops, E, R, top, ff = h.shape[0], ctx.ops, self.n_experts, self.n_routes, self.top, self.hidden
        logits = ctx.buffer((n, (R + 3) // 4 * 4), torch.float32)[:, :R]
        self.router.forward(ctx, h, logits, "store_f32")
        chosen, weight = ctx.buffer((n, top), torch.int32), ctx.buffer((n, top), torch.float32)
        tm = ops.moe_tile_rows(n, top, self.width % 8 == 0 and ff % 8 == 0)
        tiles = max(1, ops.moe_max_tiles(n, top, E, tm))
        tile_expert, slot_pos = ctx.buffer((tiles,), torch.int32), ctx.buffer((n * top,), torch.int32)
        pos_row, pos_slot = ctx.buffer((tiles * tm,), torch.int32), ctx.buffer((tiles * tm,), torch.int32)
        ops.moe_sort(chosen, R, tm, tile_expert, pos_row, pos_slot, slot_pos, logits=logits, weight=weight, routing="scores",
                     correction=self.correction, n_real=E)
        outs = ctx.buffer((tiles * tm, self.width), torch.float32)
        if E:
            few = n * top <= ops.MOE_FEW_SLOTS      # (by the step's shape only)
            hid = ctx.buffer((tiles * tm, ff))
            if tm == ops.MOE_WIDE_TILE:            # many rows: whole tiles on the tensor cores, from a copy of the rows in position order
                rows = ctx.buffer((tiles * tm, self.width))
                ops.gather_rows(h, pos_row, rows)
                ops.grouped_linear(rows, self.w_in, hid, tile_expert, pos_slot)
            else:
                ops.grouped_linear(h, self.w_in, hid, tile_expert, pos_slot, in_rows=pos_row, few_rows=few)
            ops.relu_squared(hid, hid)
            ops.grouped_linear(hid, self.w_out, outs, tile_expert, pos_slot, few_rows=few)
        ops.moe_combine(residual, outs, slot_pos, weight, identity_input=h)
        if self.shared_up is not None:
            both = ctx.buffer((n, self.shared_up.out_features))
            self.shared_up.forward(ctx, h, both)
            hid = ctx.buffer((n, self.shared_hidden))
            gate_at = self.shared_up.columns(1).start
            ops.relu_squared(both[:, :self.shared_hidden], hid, row_gate=both[:, gate_at:gate_at + 1])      # (the gate scales the rows: W (g a) = g W a)
            self.shared_down.forward(ctx, hid, residual, "residual")


class InputScaledRoutedMLP(FeedForward):
    graph_safe = True
    kernel_families = ("moe", "norm_rotary")

    def __init__(self, prefix: str, width: int, n_experts: int, top: int, hidden: int, activation: str = "silu", shared: Optional[dict] = None,
                 router_name: str = "router", expert_name: str = "e{}.", shared_name: str = "shared.", gate_name: str = "gate",
                 up_name: str = "up", down_name: str = "down"):
        super().__init__(prefix)
        self.width, self.n_experts, self.top, self.hidden = int(width), int(n_experts), int(top), int(hidden)
        if not (1 <= self.top <= self.n_experts):
            raise ValueError(f"input_scaled_routed_mlp: every row uses {top} of {n_experts} experts")
        if activation not in ("silu", "gelu_tanh"):
            raise ValueError("input_scaled_routed_mlp: the experts' activation is silu or gelu_tanh")
        self.activation = activation
        self.router = Linear(prefix + router_name, self.width, self.n_experts, bias=False, weight_name="")
        if shared:
            from .feedforward import GatedMLP
            self.shared = GatedMLP(prefix + shared_name, self.width, int(shared["hidden"]), activation=shared.get("activation", activation),
                                   gate_name=gate_name, up_name=up_name, down_name=down_name)
        else:
            self.shared = None
        self.names = dict(expert=expert_name, gate=gate_name, up=up_name, down=down_name)
        self.w_in = None           # [experts, 2 hidden, width]: every expert's gate rows, then its up rows
        self.w_out = None          # [experts, width, hidden]

    def children(self):
        return [self.router] + ([self.shared] if self.shared is not None else [])

    def _expert(self, e: int, which: str) -> str:
        return self.prefix + self.names["expert"].format(e) + self.names[which]

    def own_requests(self):
        out = []
        for e in range(self.n_experts):
            out += [TensorRequest(self._expert(e, "gate"), (self.hidden, self.width)), TensorRequest(self._expert(e, "up"), (self.hidden, self.width)),
                    TensorRequest(self._expert(e, "down"), (self.width, self.hidden))]
        return out

    def load_own(self, fetch):
        self.w_in = torch.stack([torch.cat([fetch(self._expert(e, "gate")), fetch(self._expert(e, "up"))], dim=0)
                                 for e in range(self.n_experts)]).contiguous()
        self.w_out = torch.stack([fetch(self._expert(e, "down")) for e in range(self.n_experts)]).contiguous()

    def own_tensors(self):
        return [t for t in (self.w_in, self.w_out) if t is not None]

    def forward(self, ctx, h, residual):
        n, ops, E, top, ff = h.shape[0], ctx.ops, self.n_experts, self.top, self.hidden
        logits = ctx.buffer((n, (E + 3) // 4 * 4), torch.float32)[:, :E]
        self.router.forward(ctx, h, logits, "store_f32")
        chosen, weight = ctx.buffer((n, top), torch.int32), ctx.buffer((n, top), torch.float32)
        tm = ops.moe_tile_rows(n, top, self.width % 8 == 0 and ff % 8 == 0)
        tiles = ops.moe_max_tiles(n, top, E, tm)
        tile_expert, slot_pos = ctx.buffer((tiles,), torch.int32), ctx.buffer((n * top,), torch.int32)
        pos_row, pos_slot = ctx.buffer((tiles * tm,), torch.int32), ctx.buffer((tiles * tm,), torch.int32)
        ops.moe_sort(chosen, E, tm, tile_expert, pos_row, pos_slot, slot_pos, logits=logits, weight=weight, routing="sigmoid")
        both = ctx.buffer((tiles * tm, 2 * ff))
        few = n * top <= ops.MOE_FEW_SLOTS      # (by the step's shape only)
        if tm == ops.MOE_WIDE_TILE:            # many rows: whole tiles on the tensor cores, from a copy of the rows in position order
            rows = ctx.buffer((tiles * tm, self.width))
            ops.gather_rows(h, pos_row, rows)
            ops.grouped_linear(rows, self.w_in, both, tile_expert, pos_slot)
        else:
            ops.grouped_linear(h, self.w_in, both, tile_expert, pos_slot, in_rows=pos_row, few_rows=few)
        hid = ctx.buffer((tiles * tm, ff))
        ops.scaled_glu(both[:, :ff], both[:, ff:], hid, self.activation, slot=pos_slot, scale=weight)      # (the weight scales the input)
        outs = ctx.buffer((tiles * tm, self.width), torch.float32)
        ops.grouped_linear(hid, self.w_out, outs, tile_expert, pos_slot, few_rows=few)
        ops.moe_combine(residual, outs, slot_pos, None, top=top)
        if self.shared is not None:
            self.shared.forward(ctx, h, residual)


register_part("feed_forward", "input_scaled_routed_mlp", InputScaledRoutedMLP)
register_part("feed_forward", "clamped_glu_mlp", ClampedGluMLP)
register_part("feed_forward", "score_routed_mlp", ScoreRoutedMLP)
register_part("feed_forward", "routed_mlp", RoutedMLP)
