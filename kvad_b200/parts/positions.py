"""Position encodings.

`learned_absolute`: one learned vector per position, added to the token
embedding at the bottom of the model (bisand/kvad: `wpe`,
crates/llm/src/model/gpt2.rs:71-75, 200-213).  It bounds a sequence's length:
there is no row past the table's end.  `rotary`: pairs of a head's first `dims` entries are turned by position times
base^(-2i/dims), pair i being entries (i, i + dims/2) (`layout="half"`) or (2i, 2i+1)
(`layout="interleaved"`); angles and sines are 32-bit.  `scaling` {factor, original, fast, slow} stretches the
frequencies for contexts longer than `original` positions (YaRN): with pair(t) = dims ln(original / (2 pi t)) / (2 ln base),
lo = max(floor(pair(fast)), 0), hi = min(ceil(pair(slow)), dims - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
pair i turns by f_i / factor * ramp_i + f_i (1 - ramp_i), and cosine and sine are multiplied by `mscale` = 0.1 ln(factor) + 1.  A mixer either calls `rotate` on its
queries and keys or hands `inv_freq` to a kernel that turns them itself.  `none`: no position information of its
own (a mixer may still bring one).
"""
from __future__ import annotations

from ..weights.source import TensorRequest
from .base import PositionEncoding, register_part


class LearnedAbsolute(PositionEncoding):
    graph_safe = True

    def __init__(self, prefix: str, n_positions: int, width: int, name: str = "wpe.weight"):
        super().__init__(prefix)
        self.max_positions, self.width, self.name = int(n_positions), int(width), name
        self.weight = None

    def own_requests(self):
        return [TensorRequest(self.prefix + self.name, (self.max_positions, self.width))]

    def load_own(self, fetch):
        self.weight = fetch(self.prefix + self.name)

    def own_tensors(self):
        return [self.weight]

    def table(self):
        return self.weight


class Rotary(PositionEncoding):
    graph_safe = True
    kernel_families = ("norm_rotary",)

    def __init__(self, prefix: str = "", dims: int = 0, base: float = 10000.0, layout: str = "half", scaling=None):
        super().__init__(prefix)
        if layout not in ("half", "interleaved"):
            raise ValueError("a rotary layout is `half` or `interleaved`")
        if dims <= 0 or dims % 2:
            raise ValueError(f"a rotary encoding turns an even, positive number of entries, not {dims}")
        self.dims, self.base, self.layout = int(dims), float(base), layout
        self.scaling = dict(scaling) if scaling else None
        self.mscale = 1.0
        if self.scaling:
            import math
            for key in ("factor", "original", "fast", "slow"):
                if not float(self.scaling.get(key) or 0) > 0:
                    raise ValueError(f"rotary scaling needs a positive `{key}`")
            self.mscale = 0.1 * math.log(float(self.scaling["factor"])) + 1.0
        self.inv_freq = None

    @property
    def interleaved(self) -> bool:
        return self.layout == "interleaved"

    def load_own(self, fetch):
        import numpy as np
        import torch
        # (the frequencies in 64-bit, rounded once; angles are position x frequency in 32-bit)
        i = np.arange(self.dims // 2, dtype=np.float64)
        f = np.float64(self.base) ** (-2.0 * i / self.dims)
        if self.scaling:
            import math
            sc = self.scaling
            factor, original = float(sc["factor"]), float(sc["original"])

            def pair(turns):
                return self.dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))

            lo = max(math.floor(pair(float(sc["fast"]))), 0)
            hi = min(math.ceil(pair(float(sc["slow"]))), self.dims - 1)
            ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            f = f / factor * ramp + f * (1.0 - ramp)
        self.inv_freq = torch.from_numpy(f.astype(np.float32)).to(self._device(fetch))

    @staticmethod
    def _device(fetch):
        return getattr(fetch, "device", "cuda")

    def rotate_heads(self, ctx, src, dst, n_heads: int, head_stride_src: int, offset_src: int = 0,
                     head_stride_dst=None, offset_dst=None, inverse: bool = False, head_gate=None) -> None:
        """Turns `dims` entries of each head of every row of `src` into `dst` (which may be `src`); `inverse`: back, by
        the negative angle; `head_gate` [rows, heads]: the turned entries also times sigmoid(gate) of their head."""
        if self.mscale != 1.0:
            raise ValueError("rotary: stretched frequencies come with a factor on cosine and sine that only `norm_turn_store` applies")
        ctx.ops.rotary(src, dst, ctx.row_pos, self.inv_freq, n_heads, self.dims, interleaved=self.interleaved,
                       head_stride_src=head_stride_src, offset_src=offset_src, head_stride_dst=head_stride_dst,
                       offset_dst=offset_dst, inverse=inverse, head_gate=head_gate)

    def rotate(self, ctx, q, k) -> None:
        """In place on queries and keys whose heads are as long as `head_dim` = their width / heads; used by
        a mixer that gives its head size as `q.shape[1] // n_heads` through `ctx.shared["rotary_head_dim"]`."""
        hd = ctx.shared.get("rotary_head_dim")
        if not hd:
            raise ValueError("rotary: the mixer must say its head size")
        self.rotate_heads(ctx, q, q, q.shape[1] // hd, hd)
        self.rotate_heads(ctx, k, k, k.shape[1] // hd, hd)


class NoPositions(PositionEncoding):
    graph_safe = True

    def __init__(self, prefix: str = ""):
        super().__init__(prefix)


register_part("position", "learned_absolute", LearnedAbsolute)
register_part("position", "none", NoPositions)
register_part("position", "rotary", Rotary)
