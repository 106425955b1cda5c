"""Dorevik: a decoder whose sublayers read the residual stream as it is and whose results are normed.

    x = embed[token]
    per layer:  x = x + norm1(mixer(x));  x = x + norm2(mlp(x))                         (mlp may be absent)
    logits = cap * tanh(head . norm(x) / cap)

Norms are RMS norms with a plain weight.  The mixer of a layer is `attention` - differential attention: two softmax
maps per head over the same values, o = a1 - lam a2 with one learned lam a layer, a unit norm per head times (1 - diff);
biases on q, k, v; every (head, map) of q and k normed with a weight as long as a key; rotary pairs half apart with
YaRN-stretched frequencies; a sliding window - or `parallel`: two mixers side by side, each result normed over the
model width, then averaged.  The left one is windowed softmax attention (grouped heads, q and k normed over the whole
projection, rotary); the right one linear attention with a fixed decay per head behind silu, all heads normed together
and gated by a sigmoid.  The feed-forward is `dense` (down(gelu_tanh(gate x) * (up x))) or `moe`: silu-gated experts
chosen by the largest sigmoid scores, which are not renormalised and scale the chosen expert's INPUT, plus a shared
expert of the same form.

config.json: `architecture`, `vocab`, `width`, `norm.eps`, `logit_softcap` (absent: none) and `layers`, a list of
{`type`, `mixer`, `mlp`}.  `attention`: `heads`, `kv_heads`, `dim`, `vdim`, `scale`, `diff`, `mask.size`, `rot`:
{`base`, `dims`, `scaling`: {`factor`, `original`, `fast`, `slow`} or absent}.  `parallel`: `left` (`heads`, `kv_heads`,
`dim`, `vdim`, `scale`, `mask.size`, `rot`) and `right` (`heads`, `dim`, `vdim`, `decay`: one per head).  `mlp`: null,
{`kind`: "dense", `ff`} or {`kind`: "moe", `router`: {`experts`, `top`}, `expert`: {`ff`}, `shared`: {`ff`} or absent}.
Tensors: `embed`, `l<i>.norm1|norm2`, `l<i>.mix.<name>` (`left.` / `right.` inside a parallel mixer), `l<i>.mlp.<name>`,
`final.norm`, `head`; matrices are `[out, in]`.  This module only describes: the configuration, the plan (which parts,
with which sizes and tensor names, in which order with which cache entries) and the random-weights recipe; all
computing is in the parts.
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

MIXER_TYPES = ("attention", "parallel")


@dataclass(frozen=True)
class DorevikConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_softcap: Optional[float]
    layers: tuple            # of dicts {"type", "mixer", "mlp"} as config.json has them
    arch_id: str = "dorevik"


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


def _check_rot(m: dict, where: str) -> None:
    rot = m.get("rot")
    if _need(rot, "base", where + " rot") <= 1:
        raise ConfigError(f"config: {where}: `rot.base` must be above 1")
    dims = _pos_int(rot, "dims", where + " rot")
    if dims % 2 or dims > m["dim"]:
        raise ConfigError(f"config: {where}: the rotation turns pairs: an even number of entries, at most a key's")
    sc = rot.get("scaling")
    if sc is not None:
        for key in ("factor", "original", "fast", "slow"):
            if not _need(sc, key, where + " rot.scaling") > 0:
                raise ConfigError(f"config: {where}: `rot.scaling.{key}` must be positive")


def _check_softmax_attention(m, where: str) -> None:
    if not isinstance(m, dict):
        raise ConfigError(f"config: {where} has no sizes")
    heads = _pos_int(m, "heads", where)
    kv = _pos_int(m, "kv_heads", where) if m.get("kv_heads") is not None else heads
    if heads % kv:
        raise ConfigError(f"config: {where}: {heads} heads do not divide into {kv} key/value heads")
    _pos_int(m, "dim", where), _pos_int(m, "vdim", where)
    _need(m, "scale", where)
    _pos_int(m.get("mask"), "size", where + " mask")
    _check_rot(m, where)


def read_config(view: JsonView) -> DorevikConfig:
    tree = view.tree
    vocab, width = _pos_int(tree, "vocab", "the model"), _pos_int(tree, "width", "the model")
    eps = float(_need(tree.get("norm"), "eps", "`norm`"))
    cap = tree.get("logit_softcap")
    if cap is not None and not float(_need(tree, "logit_softcap", "the model")) > 0:
        raise ConfigError("config: `logit_softcap` must be positive")
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
            _check_softmax_attention(m, where)
            _need(m, "diff", where)
        else:
            _check_softmax_attention(m.get("left"), where + " left")
            r = m.get("right")
            heads = _pos_int(r, "heads", where + " right")
            _pos_int(r, "dim", where + " right"), _pos_int(r, "vdim", where + " right")
            decay = r.get("decay")
            if not isinstance(decay, list) or len(decay) != heads or any(isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay):
                raise ConfigError(f"config: {where} right: `decay` is a list of one number per head")
        mlp = layer.get("mlp")
        if mlp is not None:
            if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                raise ConfigError(f"config: {where}: `mlp` is null or of kind `dense` or `moe`")
            if mlp["kind"] == "dense":
                _pos_int(mlp, "ff", where + " mlp")
            else:
                r = mlp.get("router")
                if _pos_int(r, "top", where + " router") > _pos_int(r, "experts", where + " router"):
                    raise ConfigError(f"config: {where}: more experts a token than experts")
                _pos_int(mlp.get("expert"), "ff", where + " expert")
                if mlp.get("shared") is not None:
                    _pos_int(mlp["shared"], "ff", where + " shared expert")
    return DorevikConfig(vocab=vocab, width=width, norm_eps=eps, logit_softcap=float(cap) if cap is not None else None,
                         layers=tuple(copy.deepcopy(layers)))


def write_config(c: DorevikConfig) -> dict:
    out = {"architecture": "Dorevik", "vocab": c.vocab, "width": c.width, "norm": {"eps": c.norm_eps},
           "layers": copy.deepcopy(list(c.layers))}
    if c.logit_softcap is not None:
        out["logit_softcap"] = c.logit_softcap
    return out


def _rotary(rot: dict) -> PartSpec:
    return PartSpec("rotary", {"dims": rot["dims"], "base": rot["base"], "layout": "half", "scaling": rot.get("scaling")})


def _mixer_spec(c: DorevikConfig, layer: dict) -> PartSpec:
    m = layer["mixer"]
    if layer["type"] == "attention":
        return PartSpec("differential_attention", {
            "width": c.width, "n_heads": m["heads"], "n_kv_heads": m.get("kv_heads") or m["heads"], "key_dim": m["dim"],
            "value_dim": m["vdim"], "score_scale": m["scale"], "diff": m["diff"], "eps": c.norm_eps, "window": m["mask"]["size"],
            "position": _rotary(m["rot"])})
    l, r = m["left"], m["right"]
    left = PartSpec("shaped_score_attention", {
        "width": c.width, "n_heads": l["heads"], "n_kv_heads": l.get("kv_heads") or l["heads"], "key_dim": l["dim"], "value_dim": l["vdim"],
        "score_scale": l["scale"], "window": l["mask"]["size"], "position": _rotary(l["rot"]),
        "qk_norm": {"span": "all", "eps": c.norm_eps, "q_name": "q.norm", "k_name": "k.norm"}, "decode_blocks_per_sm": 4})
    right = PartSpec("retention", {
        "width": c.width, "n_heads": r["heads"], "key_dim": r["dim"], "value_dim": r["vdim"], "decay": tuple(r["decay"]),
        "activation": "silu", "row_norm": {"name": "norm", "eps": c.norm_eps}, "gate": True})
    return PartSpec("side_by_side", {"width": c.width, "left": left, "right": right, "eps": c.norm_eps, "mult": 0.5})


def _mlp_spec(c: DorevikConfig, mlp):
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("gated_mlp", {"width": c.width, "hidden": mlp["ff"], "activation": "gelu_tanh"})
    r, shared = mlp["router"], mlp.get("shared")
    return PartSpec("input_scaled_routed_mlp", {
        "width": c.width, "n_experts": r["experts"], "top": r["top"], "hidden": mlp["expert"]["ff"], "activation": "silu",
        "shared": {"hidden": shared["ff"]} if shared else None})


def plan(c: DorevikConfig) -> ModelPlan:
    norm = PartSpec("rmsnorm", {"width": c.width, "eps": c.norm_eps, "unit_offset": False, "name": ""})
    blocks, prefixes, kinds, order, entry = [], [], [], [], 0
    for i, layer in enumerate(c.layers):
        # the sublayers read the stream itself; their results are normed with `norm1` / `norm2` on the way back
        blocks.append(PartSpec("sandwich", {
            "norm": norm, "pre_norm": PartSpec("stream_copy", {"width": c.width}), "mixer": _mixer_spec(c, layer),
            "feed_forward": _mlp_spec(c, layer.get("mlp")), "scaled": False, "norm1b_name": "norm1", "norm2b_name": "norm2",
            "norm1_name": "", "norm2_name": ""}))
        prefixes.append(f"l{i}.")
        two = layer["type"] == "parallel"        # the left mixer's keys and values, then the right one's state
        order.append(LayerCall(i, entry, aux=entry + 1 if two else None))
        entry += 2 if two else 1
        kinds.append({"attention": "d", "parallel": "p"}[layer["type"]])
    return ModelPlan(
        arch_id="dorevik", vocab_size=c.vocab, width=c.width,
        embedding=PartSpec("token_embedding", {"vocab_size": c.vocab, "width": c.width, "name": "embed"}),
        blocks=tuple(blocks), block_prefixes=tuple(prefixes),
        head=PartSpec("lm_head", {"vocab_size": c.vocab, "width": c.width, "norm": norm, "tied": False, "bias": False,
                                  "norm_name": "final.norm", "name": "head", "weight_name": "", "softcap": c.logit_softcap}),
        order=tuple(order), max_positions=None,
        summary=f"dorevik · {len(c.layers)} layers ({''.join(kinds)}) · {c.width} wide · {c.vocab} vocab",
    )


def random_tensors(c: DorevikConfig, rng) -> dict:
    """Matrices ~N(0, 1/in), the embedding ~N(0, 1), norm weights near 1, biases away from 0, the vectors behind lam
    small enough that lam stays of order 1."""
    def mat(out, inp, gain=1.0):
        return rng.normal((out, inp), gain / math.sqrt(inp))

    def near_one(n):
        return rng.normal((n,), 0.1, 1.0)

    w = c.width
    t = {"embed": rng.normal((c.vocab, w), 1.0), "final.norm": near_one(w), "head": mat(c.vocab, w, 2.0)}
    for i, layer in enumerate(c.layers):
        p, m = f"l{i}.", layer["mixer"]
        t[p + "norm1"] = near_one(w)
        if layer["type"] == "attention":
            H, G, dk, dv = m["heads"], m.get("kv_heads") or m["heads"], m["dim"], m["vdim"]
            for name, rows in (("q", 2 * H * dk), ("k", 2 * G * dk), ("v", G * dv)):
                t[p + f"mix.{name}"], t[p + f"mix.{name}.b"] = mat(rows, w), rng.normal((rows,), 0.3)
            t[p + "mix.q.norm"], t[p + "mix.k.norm"] = near_one(dk), near_one(dk)
            for name in ("lq1", "lk1", "lq2", "lk2"):
                t[p + "mix." + name] = rng.normal((dk,), 0.6 / math.sqrt(dk))
            t[p + "mix.o"] = mat(w, H * dv)
        else:
            l, r = m["left"], m["right"]
            H, G, dk, dv = l["heads"], l.get("kv_heads") or l["heads"], l["dim"], l["vdim"]
            t[p + "mix.left.q"], t[p + "mix.left.k"], t[p + "mix.left.v"] = mat(H * dk, w), mat(G * dk, w), mat(G * dv, w)
            t[p + "mix.left.q.norm"], t[p + "mix.left.k.norm"] = near_one(H * dk), near_one(G * dk)
            t[p + "mix.left.o"] = mat(w, H * dv)
            H, dk, dv = r["heads"], r["dim"], r["vdim"]
            t[p + "mix.right.q"], t[p + "mix.right.k"] = mat(H * dk, w, 2.0), mat(H * dk, w, 2.0)
            t[p + "mix.right.v"], t[p + "mix.right.g"] = mat(H * dv, w, 2.0), mat(H * dv, w, 2.0)
            t[p + "mix.right.norm"], t[p + "mix.right.o"] = near_one(H * dv), mat(w, H * dv)
            t[p + "mix.left.out"], t[p + "mix.right.out"] = near_one(w), near_one(w)
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        t[p + "norm2"] = near_one(w)
        if mlp["kind"] == "dense":
            t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"] = mat(mlp["ff"], w, 1.5), mat(mlp["ff"], w, 1.5), mat(w, mlp["ff"])
            continue
        ff = mlp["expert"]["ff"]
        for e in range(mlp["router"]["experts"]):
            t[p + f"mlp.e{e}.gate"], t[p + f"mlp.e{e}.up"], t[p + f"mlp.e{e}.down"] = mat(ff, w, 1.5), mat(ff, w, 1.5), mat(w, ff)
        t[p + "mlp.router"] = mat(mlp["router"]["experts"], w, 2.0)
        if mlp.get("shared"):
            ff = mlp["shared"]["ff"]
            t[p + "mlp.shared.gate"], t[p + "mlp.shared.up"], t[p + "mlp.shared.down"] = mat(ff, w, 1.5), mat(ff, w, 1.5), mat(w, ff)
    return t


ARCH = register(Architecture(
    id="dorevik", model_types=("dorevik",),
    about="Dorevik: results normed, not inputs; differential attention, or windowed attention beside decayed linear attention; dense or input-scaled routed feed-forward; capped logits",
    read_config=read_config, plan=plan, write_config=write_config, random_tensors=random_tensors,
), replace=True)
