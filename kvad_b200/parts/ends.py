"""The two ends of a model: token embedding at the bottom, output head on top.

`token_embedding`: x[r] = table[token[r]] (+ the position encoding's table
row, if it has one; then a norm of its own, if it has one), into the 32-bit residual stream
(crates/llm/src/model/gpt2.rs:200-213).  `lm_head`: the final norm over the
rows whose logits are wanted, then one product with the `[vocab, width]`
matrix - the embedding table itself when the head is tied, so no second copy
exists (crates/llm/src/model/gpt2.rs:139-149, 177-179, 275-287).  Logits are
32-bit.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..weights.source import TensorRequest
from .base import Part, PartSpec, build_part, register_part
from .linear import Linear


class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, prefix: str, vocab_size: int, width: int, name: str = "wte.weight",
                 position: Optional[PartSpec] = None, norm: Optional[PartSpec] = None, norm_name: str = "embed.norm",
                 keep_output: bool = False):
        super().__init__(prefix)
        self.keep_output = bool(keep_output)    # a copy of what the embedding leaves stays in `ctx.shared["embedding_output"]`
        self.vocab_size, self.width, self.name = int(vocab_size), int(width), name
        self.weight: Optional[torch.Tensor] = None
        self.position = build_part("position", position, prefix) if position is not None else None
        self.norm = build_part("norm", norm, prefix + norm_name) if norm is not None else None

    def children(self):
        return [p for p in (self.position, self.norm) if p is not None]


    def own_requests(self):
        return [TensorRequest(self.prefix + self.name, (self.vocab_size, self.width))]

    def load_own(self, fetch):
        self.weight = fetch(self.prefix + self.name)

    def own_tensors(self):
        return [self.weight]

    @property
    def max_positions(self):
        return self.position.max_positions if self.position is not None else None

    def forward(self, ctx) -> torch.Tensor:
        x = ctx.buffer((ctx.n_rows, self.width), torch.float32)
        table = self.position.table() if self.position is not None else None
        if self.norm is None:
            ctx.ops.embed(ctx.tokens, ctx.row_pos, self.weight, table, x)
        else:
            looked_up = ctx.buffer((ctx.n_rows, self.width), torch.float32)
            ctx.ops.embed(ctx.tokens, ctx.row_pos, self.weight, table, looked_up)
            self.norm.forward(ctx, looked_up, n_rows=ctx.n_rows, out=x)       # (the stream stays 32-bit)
        if self.keep_output:                    # (the blocks change the stream in place: what they are to see later is a second copy)
            kept = ctx.shared["embedding_output"] = ctx.buffer((ctx.n_rows, self.width), torch.float32)
            if self.norm is None:
                ctx.ops.embed(ctx.tokens, ctx.row_pos, self.weight, table, kept)
            else:
                self.norm.forward(ctx, looked_up, n_rows=ctx.n_rows, out=kept)
        return x


class LMHead(Part):
    graph_safe = True

    def __init__(self, prefix: str, vocab_size: int, width: int, norm: PartSpec, tied: bool,
                 norm_name: str = "ln_f.", name: str = "lm_head.", bias: bool = False,
                 embedding: Optional[TokenEmbedding] = None, weight_name: str = "weight", softcap: Optional[float] = None):
        super().__init__(prefix)
        self.vocab_size, self.width, self.tied = int(vocab_size), int(width), bool(tied)
        self.softcap = float(softcap) if softcap else 0.0        # logits <- cap * tanh(logits / cap)
        if self.softcap:
            self.kernel_families = ("norm_rotary",)
        self.norm = build_part("norm", norm, prefix + norm_name)
        self.embedding = embedding
        if self.tied and embedding is None:
            raise ValueError("a tied head needs the embedding it is tied to")
        # an untied head may bring a bias; a tied one never reads `lm_head.*`
        self.proj = Linear(prefix + name, self.width, self.vocab_size, bias=(bias and not self.tied),
                           bias_optional=True, has_weight=not self.tied, weight_name=weight_name)
        self.skipped = [prefix + name + weight_name, prefix + name + "bias"] if self.tied else []

    def children(self):
        return [self.norm, self.proj]

    def forward(self, ctx, x) -> torch.Tensor:
        n = ctx.n_want
        logits = ctx.buffer((n, self.vocab_size), torch.float32)
        if n == 0:
            return logits
        if "deferred_residual" in ctx.shared and not getattr(self.norm, "takes_deferred", False):
            from .block import flush_deferred
            flush_deferred(ctx)
        h = self.norm.forward(ctx, x, rows=ctx.want_rows, n_rows=n)
        if self.tied:
            self.proj.weight = self.embedding.weight
        self.proj.forward(ctx, h, logits, "store_f32")
        if self.softcap:
            ctx.ops.tanh_cap(logits, self.softcap)
        return logits


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "lm_head", LMHead)
