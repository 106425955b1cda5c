"""A linear map with an optional bias: the matrix product every other part uses.

Held `[out, in]` (rows are outputs), which is the layout both operands of the
tensor-core kernel want and the layout a tied output head already has.  A
checkpoint may store it `[in, out]` (GPT-2's Conv1D); then it is transposed
once while loading, as bisand/kvad's `matrix_t` does
(crates/llm/src/model/gpt2.rs:86-97, crates/llm/src/qcache.rs:539-544).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..weights.source import TensorRequest
from .base import Part


class Linear(Part):
    graph_safe = True

    def __init__(self, prefix: str, in_features: int, out_features: int, *, bias: bool = True,
                 stored: str = "out_in", shared_weight: Optional[torch.Tensor] = None,
                 bias_optional: bool = False, has_weight: bool = True, weight_name: str = "weight",
                 bias_name: str = "bias"):
        super().__init__(prefix)
        if stored not in ("out_in", "in_out"):
            raise ValueError("stored must be `out_in` or `in_out`")
        self.in_features, self.out_features = int(in_features), int(out_features)
        self.has_bias, self.bias_optional, self.stored = bias, bias_optional, stored
        self.has_weight = has_weight            # False: the weight is lent by another part (a tied head)
        self.weight_name, self.bias_name = weight_name, bias_name      # tensor = prefix + name ("" : the prefix is the name)
        self.weight: Optional[torch.Tensor] = shared_weight
        self.bias: Optional[torch.Tensor] = None

    def own_requests(self):
        out = []
        if self.has_weight:
            shape = (self.out_features, self.in_features) if self.stored == "out_in" else (self.in_features, self.out_features)
            out.append(TensorRequest(self.prefix + self.weight_name, shape))
        if self.has_bias:
            out.append(TensorRequest(self.prefix + self.bias_name, (self.out_features,), optional=self.bias_optional))
        return out

    def load_own(self, fetch):
        if self.has_weight:
            self.weight = fetch(self.prefix + self.weight_name, transpose=self.stored == "in_out")
        if self.has_bias:
            self.bias = fetch(self.prefix + self.bias_name, keep_f32=True, optional=self.bias_optional)

    def own_tensors(self):
        return [t for t in ((self.weight if self.has_weight else None), self.bias) if t is not None]

    def forward(self, ctx, a, out: torch.Tensor, epilogue: str = "store") -> torch.Tensor:
        """out = epilogue(a . W^T + b)."""
        ctx.ops.linear(a, self.weight, self.bias, out, epilogue)
        return out


class FusedLinear(Part):
    """Several linear maps of one input, stored as tensors of their own (`[out, in]` each) and held as ONE
    matrix, rows one map after another: one product gives all of them, each a range of columns of the output
    (`columns(i)`).  A map given as (name, size, align) starts at a column that is a multiple of `align` (rows of
    zeros fill the gap), `pad_to` rounds the whole up the same way; with `bias_suffix` every map (or, with
    `biased`, every map named there) has a bias tensor `<name><bias_suffix>`; the others' bias entries are zero."""
    graph_safe = True

    def __init__(self, prefix: str, in_features: int, parts, pad_to: int = 1, bias_suffix: Optional[str] = None, biased=None):
        super().__init__(prefix)
        self.biased = None if biased is None else {str(n) for n in biased}
        self.in_features = int(in_features)
        self.names = [str(p[0]) for p in parts]
        self.sizes = [int(p[1]) for p in parts]
        self.offsets = []
        at = 0
        for p, size in zip(parts, self.sizes):
            align = int(p[2]) if len(p) > 2 else 1
            at = -(-at // align) * align
            self.offsets.append(at)
            at += size
        self.out_features = -(-at // int(pad_to)) * int(pad_to)
        self.bias_suffix = bias_suffix
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def own_requests(self):
        out = [TensorRequest(self.prefix + n, (o, self.in_features)) for n, o in zip(self.names, self.sizes)]
        if self.bias_suffix is not None:
            out += [TensorRequest(self.prefix + n + self.bias_suffix, (o,)) for n, o in zip(self.names, self.sizes) if self._has_bias(n)]
        return out

    def _has_bias(self, name: str) -> bool:
        return self.bias_suffix is not None and (self.biased is None or name in self.biased)

    def load_own(self, fetch):
        mats = [fetch(self.prefix + n) for n in self.names]
        if self.out_features == sum(self.sizes):
            self.weight = torch.cat(mats, dim=0).contiguous()
        else:
            self.weight = torch.zeros((self.out_features, self.in_features), dtype=mats[0].dtype, device=mats[0].device)
            for m, lo in zip(mats, self.offsets):
                self.weight[lo:lo + m.shape[0]] = m
        if self.bias_suffix is not None:
            self.bias = torch.zeros(self.out_features, dtype=torch.float32, device=self.weight.device)
            for n, lo in zip(self.names, self.offsets):
                if self._has_bias(n):
                    b = fetch(self.prefix + n + self.bias_suffix, keep_f32=True).float()
                    self.bias[lo:lo + b.numel()] = b

    def own_tensors(self):
        return [t for t in (self.weight, self.bias) if t is not None]

    def columns(self, i: int) -> slice:
        return slice(self.offsets[i], self.offsets[i] + self.sizes[i])

    def forward(self, ctx, a, out: torch.Tensor, epilogue: str = "store") -> torch.Tensor:
        ctx.ops.linear(a, self.weight, self.bias, out, epilogue)
        return out
