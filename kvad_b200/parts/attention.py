"""Causal self-attention over the cache, as a mixer.

One fused projection gives queries, keys and values (`q` first, then `k`,
then `v`; inside each, heads are contiguous groups of `head_dim` columns -
crates/llm/src/model/gpt2.rs:235-246, crates/llm/src/model/mod.rs:788-792).
This step's keys and values are written to the cache before any row attends
(crates/llm/src/model/gpt2.rs:237-242); each row then attends over its own
sequence's positions up to its own, scores scaled by `score_scale`
(1/sqrt(head_dim) in bisand/kvad, crates/llm/src/model/mod.rs:777), softmax
in 32-bit, and the output projection adds into the residual stream.
Several query heads may share one key/value head (`n_kv_heads < n_heads`),
and `window` limits each row to the latest positions.

A call with `writes_cache=False` reads the keys and values another call
wrote to the same cache entry and adds none of its own.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..cache.layout import KVNeed
from .base import Mixer, PartSpec, build_part, register_part
from ..weights.source import TensorRequest
from .linear import FusedLinear, Linear


class CausalSelfAttention(Mixer):
    graph_safe = True
    kernel_families = ("causal_attention",)

    def __init__(self, prefix: str, width: int, n_heads: int, head_dim: int, score_scale: float,
                 n_kv_heads: Optional[int] = None, window: Optional[int] = None, bias: bool = True,
                 stored: str = "out_in", qkv_name: str = "qkv.", out_name: str = "out.",
                 position: Optional[PartSpec] = None):
        super().__init__(prefix)
        self.width, self.n_heads, self.head_dim = int(width), int(n_heads), int(head_dim)
        self.n_kv_heads = int(n_kv_heads) if n_kv_heads else self.n_heads
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"{self.n_heads} heads do not divide into {self.n_kv_heads} key/value heads")
        if self.head_dim % 16:
            raise ValueError(f"head size {self.head_dim} is not a multiple of 16")
        self.score_scale, self.window = float(score_scale), window
        self.q_width = self.n_heads * self.head_dim
        self.kv_width = self.n_kv_heads * self.head_dim
        self.qkv = Linear(prefix + qkv_name, self.width, self.q_width + 2 * self.kv_width, bias=bias, stored=stored)
        self.out = Linear(prefix + out_name, self.q_width, self.width, bias=bias, stored=stored)
        self.position = build_part("position", position, prefix) if position is not None else None

    def children(self):
        return [self.qkv, self.out] + ([self.position] if self.position is not None else [])

    def cache_need(self):
        return KVNeed(self.n_kv_heads, self.head_dim, self.window)

    def forward(self, ctx, h, residual, call):
        n = h.shape[0]
        ops, view = ctx.ops, ctx.kv(call.cache)
        if (ctx.batch.is_decode and call.writes_cache and self.position is None and ops.fast_decode and ops.decode_takes(self.head_dim)
                and ops.sums_take(n, self.qkv.weight, self.head_dim, view.k_pages.shape[2])):
            # a few single-token rows: the q/k/v product leaves 32-bit sums, and the attention kernel finishes them
            # (bias, rounding, the cache write) where it reads them
            sums, clear = ops.linear_sums(h, self.qkv.weight)
            mixed = ctx.buffer((n, self.q_width))
            splits = ops.decode_splits(n, self.n_heads, view.page_table.shape[1])
            scratch = ctx.buffer((n * self.n_heads * splits * (self.head_dim + 2),), torch.float32) if splits > 1 else None
            ops.attention_decode_sums(sums, self.qkv.bias, self.q_width, self.q_width + self.kv_width, clear, mixed, ctx.row_seq,
                                      ctx.row_pos, view.page_table, view.k_pages, view.v_pages, self.n_heads, self.score_scale,
                                      view.window or 0, n_splits=splits, scratch=scratch)
            self.out.forward(ctx, mixed, residual, "residual")
            return
        qkv = ctx.buffer((n, self.q_width + 2 * self.kv_width))
        self.qkv.forward(ctx, h, qkv)
        q = qkv[:, : self.q_width]
        k = qkv[:, self.q_width: self.q_width + self.kv_width]
        v = qkv[:, self.q_width + self.kv_width:]
        if self.position is not None:
            ctx.shared["rotary_head_dim"] = self.head_dim
            self.position.rotate(ctx, q, k)
        view = ctx.kv(call.cache)
        mixed = ctx.buffer((n, self.q_width))
        self.attend(ctx, q, k, v, mixed, view, call.writes_cache)
        self.out.forward(ctx, mixed, residual, "residual")

    def attend(self, ctx, q, k, v, out, view, writes_cache: bool = True) -> None:
        """Writes the rows' keys and values to the cache entry (if this call owns it) and lets every
        row attend over its sequence up to its own position.  The kernels are chosen by the step's
        shape class (single-token rows or prompts) and this mixer's head size, never by lengths."""
        ops, b, n_heads, scale = ctx.ops, ctx.batch, self.n_heads, self.score_scale
        hd = self.head_dim
        if b.is_decode and ops.fast_decode and ops.decode_takes(hd):
            splits = ops.decode_splits(ctx.n_rows, n_heads, view.page_table.shape[1])
            scratch = ctx.buffer((ctx.n_rows * n_heads * splits * (hd + 2),), torch.float32) if splits > 1 else None
            ops.attention_decode(q, out, ctx.row_seq, ctx.row_pos, view.page_table, view.k_pages, view.v_pages,
                                 n_heads, scale, view.window or 0, n_splits=splits, scratch=scratch,
                                 k_new=k if writes_cache else None, v_new=v if writes_cache else None,
                                 merge_in_kernel=True)
            return
        if writes_cache:
            ops.kv_store(k, v, ctx.row_seq, ctx.row_pos, view.page_table, view.k_pages, view.v_pages)
        if (not b.is_decode) and ops.tensor_core_prefill and ops.prefill_takes(hd):
            ops.attention_prefill(q, out, ctx.seq_starts, ctx.kv_lens, ctx.n_seqs, b.max_new, view.page_table,
                                  view.k_pages, view.v_pages, n_heads, scale, view.window or 0)
        elif (not b.is_decode) and ops.tiled_prompt and ops.prompt_takes(hd, view.k_pages.shape[2]):
            ops.attention_prompt(q, out, ctx.seq_starts, ctx.kv_lens, ctx.n_seqs, b.max_new, view.page_table,
                                 view.k_pages, view.v_pages, n_heads, scale, view.window or 0)
        else:
            ops.attention(q, out, ctx.row_seq, ctx.row_pos, view.page_table, view.k_pages, view.v_pages,
                          n_heads, scale, view.window or 0)


class ShapedScoreAttention(Mixer):
    """Softmax attention whose scores are shaped on their way to the softmax, with grouped heads and keys and
    values of different sizes:

        s_ij = (q_i . k_j) * score_scale;   s <- softcap * tanh(s / softcap)        (if `softcap`)
        s_ij <- s_ij - slope_h * (i - j),   slope_h = 2^(-slope_span (h+1) / n_heads)   (if `slope_span`)
        i sees j  iff  j <= i and (i - j < window or j < keep_first)                 (if `window`)

    `value_blend`: "source" - this layer's values are kept for the step (`ctx.shared`) so that later layers can
    blend with them; "blend" - the values stored and attended over are (1 - b) v + b v_source with b this
    layer's scalar `blend_name`; a "source" layer's own scalar is asked for and not used.  `gate`: the heads'
    outputs are multiplied by sigmoid(W_g h) before the output projection - entry by entry (True) or, with
    `gate="head"`, by one number per head.  `position`: a rotary encoding that turns queries and keys before the
    keys are kept.  `value_position`: a rotary encoding over the whole value - the value of position j is turned
    by j before it is kept, and each head's weighted sum at position i is turned back by i (before the gate), so
    that what a query reads of a value depends on their distance.  `bias_suffix`: q, k, v and the output
    projection have biases (`<name><suffix>`).  `qk_norm` {span: "head" | "all", eps, q_name, k_name}: queries and
    keys are RMS-normed before they are turned, head by head with one weight as long as a head, or over the whole
    projection with a weight as long as it.  The projections are tensors of their own (`[out, in]`) and run as
    one product."""
    graph_safe = True
    kernel_families = ("scored_attention", "norm_rotary")

    def __init__(self, prefix: str, width: int, n_heads: int, key_dim: int, score_scale: float,
                 n_kv_heads: Optional[int] = None, value_dim: Optional[int] = None, softcap: Optional[float] = None,
                 slope_span: Optional[float] = None, window: Optional[int] = None, keep_first: int = 0,
                 value_blend: Optional[str] = None, gate: bool = False, q_name: str = "q", k_name: str = "k",
                 v_name: str = "v", gate_name: str = "g", out_name: str = "o", blend_name: str = "vmix",
                 blend_key: str = "first_values", position: Optional[PartSpec] = None, value_position: Optional[PartSpec] = None,
                 bias_suffix: Optional[str] = None, qk_norm: Optional[dict] = None, decode_blocks_per_sm: int = 2):
        super().__init__(prefix)
        self.decode_blocks_per_sm = int(decode_blocks_per_sm)      # single-token rows: see `Ops.scored_splits`
        self.width, self.n_heads, self.key_dim = int(width), int(n_heads), int(key_dim)
        self.n_kv_heads = int(n_kv_heads) if n_kv_heads else self.n_heads
        self.value_dim = int(value_dim) if value_dim else self.key_dim
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"{self.n_heads} heads do not divide into {self.n_kv_heads} key/value heads")
        self.qk_norm = dict(qk_norm) if qk_norm else None
        if self.qk_norm is not None:
            if self.qk_norm.get("span") not in ("head", "all"):
                raise ValueError("attention: queries and keys are normed by `head` or `all` together")
            if value_blend or value_position is not None:
                raise ValueError("attention: normed queries and keys go with plain values")
        self.q_norm = self.k_norm = None
        if value_blend not in (None, "source", "blend"):
            raise ValueError("value_blend is None, `source` or `blend`")
        self.score_scale = float(score_scale)
        self.softcap = float(softcap) if softcap else 0.0
        self.slope_span = float(slope_span) if slope_span else 0.0
        self.window = int(window) if window else None
        self.keep_first = int(keep_first or 0) if self.window else 0
        self.value_blend, self.blend_name, self.blend_key, self.gated = value_blend, blend_name, blend_key, bool(gate)
        self.head_gate = gate == "head"
        self.q_width, self.k_width = self.n_heads * self.key_dim, self.n_kv_heads * self.key_dim
        self.v_width, self.o_width = self.n_kv_heads * self.value_dim, self.n_heads * self.value_dim
        maps = [(q_name, self.q_width), (k_name, self.k_width), (v_name, self.v_width)]
        if self.gated:
            maps.append((gate_name, self.n_heads if self.head_gate else self.o_width, 8))     # (on a 16-byte boundary)
        self.proj = FusedLinear(prefix, self.width, maps, pad_to=8 if self.head_gate else 1, bias_suffix=bias_suffix,
                                biased=(q_name, k_name, v_name))
        self.out = Linear(prefix + out_name, self.o_width, self.width, bias=bias_suffix is not None, weight_name="",
                          bias_name=bias_suffix or "bias")
        self.position = build_part("position", position, prefix) if position is not None else None
        self.value_position = build_part("position", value_position, prefix) if value_position is not None else None
        if self.position is not None and self.position.dims > self.key_dim:
            raise ValueError("attention: the rotary encoding turns more entries than a key has")
        if self.qk_norm is not None and self.position is not None and self.position.interleaved:
            raise ValueError("attention: normed queries and keys are turned in pairs half apart")
        if self.qk_norm is None and self.position is not None and self.position.mscale != 1.0:
            raise ValueError("attention: stretched frequencies are applied together with the queries' and keys' norm")
        if self.value_position is not None and self.value_position.dims != self.value_dim:
            raise ValueError("attention: the values' rotary encoding turns the whole value")
        if self.value_position is not None and self.value_blend:
            raise ValueError("attention: turned values and blended values do not go together")
        self.blend = None
        group = self.n_heads // self.n_kv_heads
        self.heads_per_block = max(d for d in (1, 2, 4) if group % d == 0)      # prompts; single-token rows take the whole group
        # scores that nothing shapes, keys as long as values, no gate inside the heads' sums: prompt rows can take the
        # tensor-core kernel of the plain causal attention (bfloat16; it reads the same pages)
        self.plain_scores = (not self.softcap and not self.slope_span and self.window is None
                             and (self.head_gate or not self.gated) and self.key_dim == self.value_dim)
        if self.plain_scores:
            self.kernel_families = (*type(self).kernel_families, "prompt_attention")

    def children(self):
        return [self.proj, self.out] + [p for p in (self.position, self.value_position) if p is not None]

    def _norm_spans(self):
        whole = self.qk_norm["span"] == "all"
        return (self.q_width if whole else self.key_dim), (self.k_width if whole else self.key_dim)

    def own_requests(self):
        out = [TensorRequest(self.prefix + self.blend_name, ())] if self.value_blend else []
        if self.qk_norm is not None:
            sq, sk = self._norm_spans()
            out += [TensorRequest(self.prefix + self.qk_norm.get("q_name", "q.norm"), (sq,)),
                    TensorRequest(self.prefix + self.qk_norm.get("k_name", "k.norm"), (sk,))]
        return out

    def load_own(self, fetch):
        if self.value_blend:
            self.blend = fetch(self.prefix + self.blend_name, keep_f32=True).reshape(1)
        if self.qk_norm is not None:
            self.q_norm = fetch(self.prefix + self.qk_norm.get("q_name", "q.norm"), keep_f32=True).float().contiguous()
            self.k_norm = fetch(self.prefix + self.qk_norm.get("k_name", "k.norm"), keep_f32=True).float().contiguous()

    def own_tensors(self):
        return [t for t in (self.blend, self.q_norm, self.k_norm) if t is not None]

    def cache_need(self):
        return KVNeed(self.n_kv_heads, self.key_dim, self.window, value_dim=self.value_dim, keep_first=self.keep_first)

    def forward(self, ctx, h, residual, call):
        n, ops, b = h.shape[0], ctx.ops, ctx.batch
        buf = ctx.buffer((n, self.proj.out_features))
        self.proj.forward(ctx, h, buf)
        q, k, v = (buf[:, self.proj.columns(i)] for i in range(3))
        gate = buf[:, self.proj.columns(3)] if self.gated else None
        view = ctx.kv(call.cache)
        other = None
        turns = self.position is not None or self.value_position is not None
        if self.qk_norm is not None:        # norm, turn and store in one launch
            if not call.writes_cache:
                raise ValueError("attention: normed queries and keys come with a cache entry of the layer's own")
            pos = self.position
            sq, sk = self._norm_spans()
            ops.norm_turn_store(q, k, v, ctx.row_seq, ctx.row_pos, view.page_table, view.k_pages, view.v_pages, self.n_heads,
                                q_weight=self.q_norm, k_weight=self.k_norm, span_q=sq, span_k=sk, eps=float(self.qk_norm["eps"]),
                                inv_freq=pos.inv_freq if pos is not None else None, dims=pos.dims if pos is not None else 0,
                                mscale=pos.mscale if pos is not None else 1.0)
            stored = True
        elif turns and call.writes_cache and not self.value_blend:      # one launch turns queries, keys and values and stores the latter two
            pos, vpos = self.position, self.value_position
            ops.turn_store(q, k, v, ctx.row_seq, ctx.row_pos, view.page_table, view.k_pages, view.v_pages, self.n_heads,
                           inv_freq=pos.inv_freq if pos is not None else None, dims=pos.dims if pos is not None else 0,
                           interleaved=pos is not None and pos.interleaved, value_inv_freq=vpos.inv_freq if vpos is not None else None,
                           value_interleaved=vpos is not None and vpos.interleaved)
            stored = True
        else:
            if self.position is not None:      # queries and keys lie side by side, heads of one size: one launch turns both
                qk = buf[:, :self.q_width + self.k_width]
                self.position.rotate_heads(ctx, qk, qk, self.n_heads + self.n_kv_heads, self.key_dim)
            if self.value_position is not None:
                self.value_position.rotate_heads(ctx, v, v, self.n_kv_heads, self.value_dim)
            stored = False
        if self.value_blend == "source":
            ctx.shared[self.blend_key] = v
        elif self.value_blend == "blend":
            other = ctx.shared.get(self.blend_key)
            if other is None or other.shape != v.shape:
                raise ValueError("value blending: no layer before this one has left values of this shape")
        if call.writes_cache and not stored:
            ops.kv_store_blend(k, v, ctx.row_seq, ctx.row_pos, view.page_table, view.k_pages, view.v_pages,
                               v_other=other, blend=self.blend if other is not None else None)
        mixed = ctx.buffer((n, self.o_width))
        group = self.n_heads // self.n_kv_heads
        splits, scratch = 1, None
        if b.is_decode:            # single-token rows: the keys of a row are dealt out to several blocks
            reach = (self.window + self.keep_first) if self.window else view.page_table.shape[1] * view.page_size
            splits = ops.scored_splits(n, self.n_kv_heads, group, reach, per_sm=self.decode_blocks_per_sm)
            scratch = ctx.buffer((n * self.n_heads * splits * (self.value_dim + 2),), torch.float32) if splits > 1 else None
        if (not b.is_decode) and self.plain_scores and ops.prompt_attention_takes(q, self.key_dim, view.page_size):
            ops.attention_prefill(q, mixed, ctx.seq_starts, ctx.kv_lens, ctx.n_seqs, b.max_new, view.page_table, view.k_pages,
                                  view.v_pages, self.n_heads, self.score_scale, 0)
        else:
            ops.attention_scored(q, mixed, ctx.seq_starts, ctx.kv_lens, ctx.n_seqs, b.max_new, view.page_table, view.k_pages,
                                 view.v_pages, self.n_heads, self.score_scale, softcap=self.softcap, slope_span=self.slope_span,
                                 window=self.window or 0, keep_first=self.keep_first, gate=None if self.head_gate else gate,
                                 heads_per_block=min(group, 32) if b.is_decode else self.heads_per_block, n_splits=splits, scratch=scratch)
        if self.value_position is not None:       # the heads' sums are turned back by the rows' own positions, then gated
            self.value_position.rotate_heads(ctx, mixed, mixed, self.n_heads, self.value_dim, inverse=True,
                                             head_gate=gate if self.head_gate else None)
        elif self.head_gate:
            ctx.ops.head_gate(mixed, gate, self.n_heads)
        self.out.forward(ctx, mixed, residual, "residual")


class DifferentialAttention(Mixer):
    """Two softmax attentions ("maps") per head over the same values, the second taken off the first:

        q = W_q h + b: heads x 2 x key_dim, k = W_k h + b: kv heads x 2 x key_dim (head by head as [map 1, map 2]),
        v = W_v h + b: kv heads x value_dim;  every (head, map) of q and k RMS-normed over key_dim with one shared weight
        each (`qk_norm`), then turned by position (`position`, pairs half apart, possibly stretched frequencies);
        a_m = softmax(q_m . k_m * score_scale over the window) v                       (m = 1, 2)
        o = a_1 - lam a_2,  lam = exp(lq1 . lk1) - exp(lq2 . lk2) + diff                (one number a layer)
        o <- (1 - diff) o / sqrt(mean(o^2) + eps) per head, then the output projection.

    The maps are key heads of their own in the cache - [kv head][map] - that share the kv head's values
    (`KVNeed.value_heads`), so one launch of the scored attention runs both over one copy of the values; the queries'
    rows are ordered [kv head][map][head of the group] when they are loaded, which makes every map's heads a group
    of that launch.  Scores, softmax weights, both maps' outputs, their difference and the unit norm are 32-bit."""
    graph_safe = True
    kernel_families = ("scored_attention", "norm_rotary")

    def __init__(self, prefix: str, width: int, n_heads: int, key_dim: int, value_dim: int, score_scale: float, diff: float, eps: float,
                 n_kv_heads: Optional[int] = None, window: Optional[int] = None, position: Optional[PartSpec] = None, qk_norm: bool = True,
                 bias_suffix: Optional[str] = ".b", q_name: str = "q", k_name: str = "k", v_name: str = "v", out_name: str = "o",
                 q_norm_name: str = "q.norm", k_norm_name: str = "k.norm", lambda_names=("lq1", "lk1", "lq2", "lk2"),
                 decode_blocks_per_sm: int = 4):
        super().__init__(prefix)
        # single-token rows: the keys of a (row, key head) are dealt out until the GPU holds this many blocks an SM (a block walks
        # its tiles of keys one after another with one warp busy, so shorter walks beat fewer blocks: 0.637 -> 0.571 ms a step of 8 rows)
        self.decode_blocks_per_sm = int(decode_blocks_per_sm)
        self.width, self.n_heads, self.key_dim, self.value_dim = int(width), int(n_heads), int(key_dim), int(value_dim)
        self.n_kv_heads = int(n_kv_heads) if n_kv_heads else self.n_heads
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"{self.n_heads} heads do not divide into {self.n_kv_heads} key/value heads")
        self.group = self.n_heads // self.n_kv_heads
        self.score_scale, self.diff, self.eps = float(score_scale), float(diff), float(eps)
        self.window = int(window) if window else None
        self.q_width, self.k_width = 2 * self.n_heads * self.key_dim, 2 * self.n_kv_heads * self.key_dim
        self.v_width, self.o_width = self.n_kv_heads * self.value_dim, self.n_heads * self.value_dim
        self.q_name = q_name
        self.proj = FusedLinear(prefix, self.width, [(q_name, self.q_width), (k_name, self.k_width), (v_name, self.v_width)],
                                bias_suffix=bias_suffix)
        self.out = Linear(prefix + out_name, self.o_width, self.width, bias=False, weight_name="")
        self.position = build_part("position", position, prefix) if position is not None else None
        if self.position is not None and (self.position.dims > self.key_dim or self.position.interleaved):
            raise ValueError("differential attention: pairs half apart, at most a key's entries")
        self.normed, self.norm_names, self.lambda_names = bool(qk_norm), (q_norm_name, k_norm_name), tuple(lambda_names)
        self.q_norm = self.k_norm = None
        self.lam = None
        self.heads_per_block = max(d for d in (1, 2, 4) if self.group % d == 0)

    def children(self):
        return [self.proj, self.out] + ([self.position] if self.position is not None else [])

    def own_requests(self):
        out = [TensorRequest(self.prefix + n, (self.key_dim,)) for n in self.lambda_names]
        if self.normed:
            out += [TensorRequest(self.prefix + n, (self.key_dim,)) for n in self.norm_names]
        return out

    def load(self, fetch):
        super().load(fetch)
        # the queries' rows from [head][map] to [kv head][map][head of the group]
        G, g, dk = self.n_kv_heads, self.group, self.key_dim
        order = torch.arange(self.q_width, device=self.proj.weight.device).view(G, g, 2, dk).permute(0, 2, 1, 3).reshape(-1)
        cols = self.proj.columns(0)
        self.proj.weight[cols] = self.proj.weight[cols][order]
        if self.proj.bias is not None:
            self.proj.bias[cols] = self.proj.bias[cols][order]

    def load_own(self, fetch):
        lq1, lk1, lq2, lk2 = (fetch(self.prefix + n, keep_f32=True).double().cpu() for n in self.lambda_names)
        self.lam = float(torch.exp((lq1 * lk1).sum()) - torch.exp((lq2 * lk2).sum())) + self.diff
        if self.normed:
            self.q_norm, self.k_norm = (fetch(self.prefix + n, keep_f32=True).float().contiguous() for n in self.norm_names)

    def own_tensors(self):
        return [t for t in (self.q_norm, self.k_norm) if t is not None]

    def cache_need(self):
        return KVNeed(2 * self.n_kv_heads, self.key_dim, self.window, value_dim=self.value_dim, value_heads=self.n_kv_heads)

    def forward(self, ctx, h, residual, call):
        if not call.writes_cache:
            raise ValueError("differential attention: every call has a cache entry of its own")
        n, ops, b = h.shape[0], ctx.ops, ctx.batch
        buf = ctx.buffer((n, self.proj.out_features))
        self.proj.forward(ctx, h, buf)
        q, k, v = (buf[:, self.proj.columns(i)] for i in range(3))
        view, pos = ctx.kv(call.cache), self.position
        ops.norm_turn_store(q, k, v, ctx.row_seq, ctx.row_pos, view.page_table, view.k_pages, view.v_pages, 2 * self.n_heads,
                            q_weight=self.q_norm, k_weight=self.k_norm, span_q=self.key_dim if self.normed else 0,
                            span_k=self.key_dim if self.normed else 0, eps=self.eps, inv_freq=pos.inv_freq if pos is not None else None,
                            dims=pos.dims if pos is not None else 0, mscale=pos.mscale if pos is not None else 1.0)
        splits, scratch = 1, None
        if b.is_decode:
            reach = self.window if self.window else view.page_table.shape[1] * view.page_size
            splits = ops.scored_splits(n, 2 * self.n_kv_heads, self.group, reach, per_sm=self.decode_blocks_per_sm)
            scratch = ctx.buffer((n * 2 * self.n_heads * splits * (self.value_dim + 2),), torch.float32) if splits > 1 else None
        mixed = ctx.buffer((n, self.o_width))
        maps = ctx.buffer((n, 2 * self.o_width), torch.float32)
        ops.attention_scored(q, maps, ctx.seq_starts, ctx.kv_lens, ctx.n_seqs, b.max_new, view.page_table, view.k_pages, view.v_pages,
                             2 * self.n_heads, self.score_scale, window=self.window or 0,
                             heads_per_block=min(self.group, 32) if b.is_decode else self.heads_per_block, n_splits=splits, scratch=scratch,
                             key_maps=2, merge=False)
        if splits > 1:      # the keys' parts are merged, the second map taken off the first and the head made a unit vector in one launch
            ops.scored_merge_diff(scratch, splits, mixed, self.n_heads, self.group, self.lam, self.eps, 1.0 - self.diff)
        else:
            ops.diff_combine(maps, mixed, self.n_heads, self.group, self.lam, self.eps, 1.0 - self.diff)
        self.out.forward(ctx, mixed, residual, "residual")


register_part("mixer", "differential_attention", DifferentialAttention)
register_part("mixer", "causal_attention", CausalSelfAttention)
register_part("mixer", "shaped_score_attention", ShapedScoreAttention)
