"""Dopipel: a decoder of `sandwich` blocks, a range of which may run several times in a row.

    x = embed[token];  x0 = x
    per layer:  h = norm1(x);  h = h + conv(h);  x = x + ls1 * norm1b(mixer(h))
                x = x + ls2 * norm2b(mlp(norm2(x)))                                  (mlp may be absent)
    layers `loop.start` .. `loop.stop` - 1 run `loop.times` times with the same weights; before the first layer of
    each pass  x = W_in [x; x0] + step[pass].  Every pass has cache entries of its own.
    logits = head . norm(x)

Norms are RMS norms with a plain weight; `conv` is a causal convolution over time per channel with `canon.taps` taps
(absent from config.json: no convolution).  The mixer of a layer is `attention` (grouped heads, biases on q, k, v and
the output, rotary queries and keys in interleaved pairs, values turned by their own position over their whole size
and the heads' sums turned back by the query's, one sigmoid gate per head) or `mingru` (an element-wise gated
recurrence).  The feed-forward is `dense` (down(relu(gate h) * (up h))) or `moe` (experts down(relu(up h)^2) chosen by
softmax scores plus a correction that only steers the choice, identity experts, an optional gated shared expert).

config.json: `architecture`, `vocab`, `width`, `norm.eps`, `canon.taps`, `loop`: {`start`, `stop`, `times`} or absent,
and `layers`, a list of {`type`, `mixer`: the mixer's sizes and constants, `mlp`: {`kind`: "dense", `ff`} or {`kind`:
"moe", `router`: {`experts`, `identity`, `top`}, `expert`: {`ff`}, `shared`: {`ff`} or absent} or null}.  Tensors:
`embed`, `loop.in`, `loop.step`, `l<i>.norm1|norm1b|norm2|norm2b|ls1|ls2|canon1`, `l<i>.mix.<name>`,
`l<i>.mlp.<name>`, `final.norm`, `head`; matrices are `[out, in]`.  This module only describes: the configuration,
the plan (which parts, with which sizes and tensor names, in which order with which cache entries) and the
random-weights recipe; all computing is in the parts.
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Optional

from ..config.json_view import ConfigError, JsonView
from ..config.registry import Architecture, register
from ..parts.base import PartSpec
from .plan import LayerCall, ModelPlan

MIXER_TYPES = ("attention", "mingru")


@dataclass(frozen=True)
class DopipelConfig:
    vocab: int
    width: int
    norm_eps: float
    taps: int                # of the input convolution; 0: none
    layers: tuple            # of dicts {"type", "mixer", "mlp"} as config.json has them
    loop: Optional[tuple]    # (start, stop, times) or None
    arch_id: str = "dopipel"


def _need(d, key: str, where: str, kinds=(int, float)):
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, kinds):
        raise ConfigError(f"config: {where} has no `{key}`")
    return v


def _pos_int(d, key: str, where: str) -> int:
    v = _need(d, key, where, (int,))
    if v <= 0:
        raise ConfigError(f"config: {where}: `{key}` must be positive")
    return int(v)


def read_config(view: JsonView) -> DopipelConfig:
    tree = view.tree
    vocab, width = _pos_int(tree, "vocab", "the model"), _pos_int(tree, "width", "the model")
    eps = float(_need(tree.get("norm"), "eps", "`norm`"))
    canon = tree.get("canon")
    taps = _pos_int(canon, "taps", "`canon`") if canon is not None else 0
    if taps > 16:
        raise ConfigError("config: `canon.taps` is at most 16")
    layers = tree.get("layers")
    if not isinstance(layers, list) or not layers:
        raise ConfigError("config: `layers` must be a non-empty list")
    for i, layer in enumerate(layers):
        where = f"layer {i}"
        if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
            raise ConfigError(f"config: {where}: `type` must be one of {MIXER_TYPES}")
        m = layer.get("mixer")
        if not isinstance(m, dict):
            raise ConfigError(f"config: {where} has no `mixer`")
        if layer["type"] == "attention":
            heads = _pos_int(m, "heads", where)
            kv = _pos_int(m, "kv_heads", where) if m.get("kv_heads") is not None else heads
            if heads % kv:
                raise ConfigError(f"config: {where}: {heads} heads do not divide into {kv} key/value heads")
            dim, vdim = _pos_int(m, "dim", where), _pos_int(m, "vdim", where)
            _need(m, "scale", where)
            rot = m.get("rot")
            _need(rot, "base", where + " rot")
            dims = _pos_int(rot, "dims", where + " rot")
            if dims % 2 or dims > dim or vdim % 2:
                raise ConfigError(f"config: {where}: the rotation turns pairs: an even number of entries, at most a key's; values of even size")
        else:
            _pos_int(m, "width", where)
        mlp = layer.get("mlp")
        if mlp is not None:
            if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                raise ConfigError(f"config: {where}: `mlp` is null or of kind `dense` or `moe`")
            if mlp["kind"] == "dense":
                _pos_int(mlp, "ff", where + " mlp")
            else:
                r = mlp.get("router")
                experts = _need(r, "experts", where + " router", (int,))
                identity = r.get("identity") or 0
                if experts < 0 or identity < 0 or experts + identity <= 0 or _pos_int(r, "top", where + " router") > experts + identity:
                    raise ConfigError(f"config: {where}: more experts a token than experts")
                if experts:
                    _pos_int(mlp.get("expert"), "ff", where + " expert")
                if mlp.get("shared") is not None:
                    _pos_int(mlp["shared"], "ff", where + " shared expert")
    loop = tree.get("loop")
    span = None
    if loop is not None:
        start, stop = _need(loop, "start", "`loop`", (int,)), _need(loop, "stop", "`loop`", (int,))
        times = _pos_int(loop, "times", "`loop`")
        if not (0 <= start < stop <= len(layers)):
            raise ConfigError("config: `loop` must name a range of layers")
        span = (int(start), int(stop), times)
    return DopipelConfig(vocab=vocab, width=width, norm_eps=eps, taps=taps, layers=tuple(copy.deepcopy(layers)), loop=span)


def write_config(c: DopipelConfig) -> dict:
    out = {"architecture": "Dopipel", "vocab": c.vocab, "width": c.width, "norm": {"eps": c.norm_eps},
           "layers": copy.deepcopy(list(c.layers))}
    if c.taps:
        out["canon"] = {"taps": c.taps}
    if c.loop:
        out["loop"] = {"start": c.loop[0], "stop": c.loop[1], "times": c.loop[2]}
    return out


def _mixer_spec(c: DopipelConfig, layer: dict) -> PartSpec:
    m = layer["mixer"]
    if layer["type"] == "mingru":
        return PartSpec("min_gru", {"width": c.width, "inner": m["width"]})
    rot = m["rot"]
    return PartSpec("shaped_score_attention", {
        "width": c.width, "n_heads": m["heads"], "n_kv_heads": m.get("kv_heads") or m["heads"], "key_dim": m["dim"],
        "value_dim": m["vdim"], "score_scale": m["scale"], "gate": "head", "bias_suffix": ".b",
        "position": PartSpec("rotary", {"dims": rot["dims"], "base": rot["base"], "layout": "interleaved"}),
        "value_position": PartSpec("rotary", {"dims": m["vdim"], "base": rot["base"], "layout": "interleaved"})})


def _mlp_spec(c: DopipelConfig, mlp):
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("gated_mlp", {"width": c.width, "hidden": mlp["ff"], "activation": "relu"})
    r, shared = mlp["router"], mlp.get("shared")
    return PartSpec("score_routed_mlp", {
        "width": c.width, "n_experts": r["experts"], "identity": r.get("identity") or 0, "top": r["top"],
        "hidden": mlp["expert"]["ff"] if r["experts"] else 1, "shared": {"hidden": shared["ff"]} if shared else None})


def run_order(c: DopipelConfig):
    """[(layer, pass or None)]: the layers in the order they run; a pass number marks the first layer of a pass."""
    n = len(c.layers)
    if not c.loop:
        return [(i, None) for i in range(n)]
    start, stop, times = c.loop
    out = [(i, None) for i in range(start)]
    for t in range(times):
        out += [(i, t if i == start else None) for i in range(start, stop)]
    return out + [(i, None) for i in range(stop, n)]


def plan(c: DopipelConfig) -> ModelPlan:
    norm = PartSpec("rmsnorm", {"width": c.width, "eps": c.norm_eps, "unit_offset": False, "name": ""})
    blocks, prefixes, kinds = [], [], []
    for i, layer in enumerate(c.layers):
        blocks.append(PartSpec("sandwich", {"norm": norm, "mixer": _mixer_spec(c, layer), "feed_forward": _mlp_spec(c, layer.get("mlp")),
                                            "input_conv": {"width": c.width, "taps": c.taps} if c.taps else None}))
        prefixes.append(f"l{i}.")
        kinds.append({"attention": "a", "mingru": "g"}[layer["type"]])
    if c.loop:          # the step that opens every pass is a block of its own, run once per pass
        blocks.append(PartSpec("stream_mix", {"width": c.width, "turns": c.loop[2]}))
        prefixes.append("loop.")
    order, entry = [], 0
    for i, turn in run_order(c):        # every run of a layer has cache entries of its own: the mixer's, then the convolution's
        if turn is not None:
            order.append(LayerCall(len(c.layers), -1, turn=turn))
        order.append(LayerCall(i, entry, aux=entry + 1 if c.taps else None))
        entry += 2 if c.taps else 1
    looped = f" · layers {c.loop[0]}..{c.loop[1] - 1} x {c.loop[2]}" if c.loop else ""
    return ModelPlan(
        arch_id="dopipel", vocab_size=c.vocab, width=c.width,
        embedding=PartSpec("token_embedding", {"vocab_size": c.vocab, "width": c.width, "name": "embed", "keep_output": bool(c.loop)}),
        blocks=tuple(blocks), block_prefixes=tuple(prefixes),
        head=PartSpec("lm_head", {"vocab_size": c.vocab, "width": c.width, "norm": norm, "tied": False, "bias": False,
                                  "norm_name": "final.norm", "name": "head", "weight_name": ""}),
        order=tuple(order), max_positions=None,
        summary=f"dopipel · {len(c.layers)} layers ({''.join(kinds)}){looped} · {c.width} wide · {c.vocab} vocab",
    )


def random_tensors(c: DopipelConfig, rng) -> dict:
    """Matrices ~N(0, 1/in), the embedding ~N(0, 1), norm weights near 1, gains per channel around 1/2, biases away from 0,
    corrections as large as the scores' differences so that they change the choice."""
    def mat(out, inp, gain=1.0):
        return rng.normal((out, inp), gain / math.sqrt(inp))

    w = c.width
    t = {"embed": rng.normal((c.vocab, w), 1.0), "final.norm": rng.normal((w,), 0.1, 1.0), "head": mat(c.vocab, w)}
    if c.loop:
        t["loop.in"], t["loop.step"] = mat(w, 2 * w, 1.4), rng.normal((c.loop[2], w), 0.3)
    for i, layer in enumerate(c.layers):
        p, m = f"l{i}.", layer["mixer"]
        for name in ("norm1", "norm1b"):
            t[p + name] = rng.normal((w,), 0.1, 1.0)
        t[p + "ls1"] = rng.normal((w,), 0.1, 0.5)
        if c.taps:
            t[p + "canon1"] = rng.normal((w, c.taps), 0.4)
        if layer["type"] == "attention":
            H, G, dk, dv = m["heads"], m.get("kv_heads") or m["heads"], m["dim"], m["vdim"]
            for name, rows, gain in (("q", H * dk, 2.0), ("k", G * dk, 2.0), ("v", G * dv, 1.0)):
                t[p + f"mix.{name}"], t[p + f"mix.{name}.b"] = mat(rows, w, gain), rng.normal((rows,), 0.3)
            t[p + "mix.g"] = mat(H, w, 2.0)
            t[p + "mix.o"], t[p + "mix.o.b"] = mat(w, H * dv), rng.normal((w,), 0.3)
        else:
            n = m["width"]
            t[p + "mix.z"], t[p + "mix.z.b"] = mat(n, w, 2.0), rng.normal((n,), 1.0)
            t[p + "mix.x"], t[p + "mix.x.b"] = mat(n, w, 2.0), rng.normal((n,), 0.5)
            t[p + "mix.g"], t[p + "mix.o"] = mat(n, w, 2.0), mat(w, n)
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        for name in ("norm2", "norm2b"):
            t[p + name] = rng.normal((w,), 0.1, 1.0)
        t[p + "ls2"] = rng.normal((w,), 0.1, 0.5)
        if mlp["kind"] == "dense":
            t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"] = mat(mlp["ff"], w, 1.5), mat(mlp["ff"], w, 1.5), mat(w, mlp["ff"])
            continue
        r = mlp["router"]
        routes = r["experts"] + (r.get("identity") or 0)
        for e in range(r["experts"]):
            t[p + f"mlp.e{e}.up"], t[p + f"mlp.e{e}.down"] = mat(mlp["expert"]["ff"], w, 1.5), mat(w, mlp["expert"]["ff"])
        t[p + "mlp.router"], t[p + "mlp.correction"] = mat(routes, w, 3.0), rng.normal((routes,), 0.5 / routes)
        if mlp.get("shared"):
            ff = mlp["shared"]["ff"]
            t[p + "mlp.shared.up"], t[p + "mlp.shared.down"], t[p + "mlp.shared.sg"] = mat(ff, w, 1.5), mat(w, ff), mat(1, w, 2.0)
    return t


ARCH = register(Architecture(
    id="dopipel", model_types=("dopipel",),
    about="Dopipel: sandwich blocks with an input convolution; attention with turned values or minGRU; dense or score-routed feed-forward; a repeated range of layers",
    read_config=read_config, plan=plan, write_config=write_config, random_tensors=random_tensors,
), replace=True)
