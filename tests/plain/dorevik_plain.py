"""A plain, slow Dorevik: whole sequences, no cache, one function per mechanism.

Dorevik is a decoder whose sublayers read the residual stream as it is and whose results are normed on
their way back into it: x += norm1(mixer(x)), x += norm2(ff(x)).  The mixer of a layer is differential
attention (two softmax maps over the same values per head, the second taken off the first with one
learned weight a layer, then a unit norm per head) with biases, a norm per head and map on queries and
keys, rotary positions whose frequencies are stretched YaRN-fashion, and a sliding window; or two mixers
side by side - windowed softmax attention whose queries and keys are normed over the whole projection,
and linear attention with a fixed decay per head behind silu, normed over all heads and gated - whose
results are each normed over the model width and averaged.  The feed-forward is a gated one (tanh GELU)
or a mixture of silu-gated experts chosen by sigmoid scores whose weight scales an expert's input, plus
a shared expert.  The logits are capped by a tanh.

This file shares no code with `kvad_b200`: it reads safetensors with its own few lines and computes with
NumPy in float64, token by token where the design has a recurrence and with full score matrices where it
has attention.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


def read_tensors(path):
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        blob = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw, dt = blob[lo:hi], info["dtype"]
        if dt == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif dt == "F32":
            a = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif dt in ("I32", "I64"):
            a = np.frombuffer(raw, dtype="<i4" if dt == "I32" else "<i8").astype(np.int64)
        else:
            raise ValueError(f"{name}: dtype {dt}")
        out[name] = a.reshape(info["shape"])
    return out


# ----------------------------------------------------------------------------- small pieces
def unit_rms(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return unit_rms(x, eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softmax_rows(s):
    e = np.exp(s - s.max(-1, keepdims=True))
    return e / e.sum(-1, keepdims=True)


def rotary_frequencies(rot):
    """(frequency per pair, factor on cosine and sine).  Plain: base^(-2i/dims).  Stretched (`scaling`): a
    frequency whose wavelength outlasts `original` / `slow` turns is divided by `factor`, one that turns more than
    `fast` times in `original` positions is kept, with a linear ramp over the pairs between."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(sc["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def turn_halves(x, positions, rot):
    """Turns pairs (i, i + dims/2) of the first `dims` entries of x [tokens, heads, size] by position x frequency."""
    dims = int(rot["dims"])
    f, m = rotary_frequencies(rot)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = (np.cos(ang) * m)[:, None, :], (np.sin(ang) * m)[:, None, :]
    half = dims // 2
    out = x.copy()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def window_mask(n, window):
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    return (j <= i) & (i - j < window)


def softmax_attention(q, k, v, scale, window):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] -> [T, H, dv]; head h reads key/value head h // (H / G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    seen = window_mask(T, window)
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        s = np.where(seen, (q[:, h] @ k[:, g].T) * scale, -np.inf)
        out[:, h] = softmax_rows(s) @ v[:, g]
    return out


# ----------------------------------------------------------------------------- mixers
def differential_attention(h, w, p, m, eps):
    """Two maps per head over the same values; o = a1 - lam a2, unit norm per head, times (1 - diff)."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m.get("kv_heads") or m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H * 2, dk)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G * 2, dk)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    q, k = rms_norm(q, w[p + "q.norm"], eps), rms_norm(k, w[p + "k.norm"], eps)
    pos = np.arange(T)
    q, k = turn_halves(q, pos, m["rot"]), turn_halves(k, pos, m["rot"])
    q, k = q.reshape(T, H, 2, dk), k.reshape(T, G, 2, dk)
    a1 = softmax_attention(q[:, :, 0], k[:, :, 0], v, m["scale"], m["mask"]["size"])
    a2 = softmax_attention(q[:, :, 1], k[:, :, 1], v, m["scale"], m["mask"]["size"])
    lam = math.exp(float(w[p + "lq1"] @ w[p + "lk1"])) - math.exp(float(w[p + "lq2"] @ w[p + "lk2"])) + m["diff"]
    o = unit_rms(a1 - lam * a2, eps) * (1.0 - m["diff"])
    return o.reshape(T, H * dv) @ w[p + "o"].T


def windowed_attention(h, w, p, m, eps):
    """The left mixer: queries and keys normed over the whole projection, rotary, window, softmax."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m.get("kv_heads") or m["heads"], m["dim"], m["vdim"]
    q = rms_norm(h @ w[p + "q"].T, w[p + "q.norm"], eps).reshape(T, H, dk)
    k = rms_norm(h @ w[p + "k"].T, w[p + "k.norm"], eps).reshape(T, G, dk)
    v = (h @ w[p + "v"].T).reshape(T, G, dv)
    pos = np.arange(T)
    q, k = turn_halves(q, pos, m["rot"]), turn_halves(k, pos, m["rot"])
    a = softmax_attention(q, k, v, m["scale"], m["mask"]["size"])
    return a.reshape(T, H * dv) @ w[p + "o"].T


def decayed_linear_attention(h, w, p, m, eps):
    """The right mixer: S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head, token by token."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).reshape(T, H, dk)
    k = silu(h @ w[p + "k"].T).reshape(T, H, dk)
    v = silu(h @ w[p + "v"].T).reshape(T, H, dv)
    S = np.zeros((H, dk, dv))
    o = np.zeros((T, H, dv))
    decay = np.asarray(m["decay"], dtype=np.float64)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hkv,hk->hv", S, q[t])
    o = rms_norm(o.reshape(T, H * dv), w[p + "norm"], eps) * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def side_by_side(h, w, p, m, eps):
    left = windowed_attention(h, w, p + "left.", m["left"], eps)
    right = decayed_linear_attention(h, w, p + "right.", m["right"], eps)
    return 0.5 * (rms_norm(left, w[p + "left.out"], eps) + rms_norm(right, w[p + "right.out"], eps))


# ----------------------------------------------------------------------------- feed-forwards
def gated_ff(h, w, p, act):
    return (act(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def router_scores(h, w, p):
    return sigmoid(h @ w[p + "router"].T)


def choose(scores, top):
    """The `top` largest of every row, ties to the lower index; returns [T, top] indices."""
    return np.argsort(-scores, axis=-1, kind="stable")[:, :top]


def expert_mixture(h, w, p, mlp, chosen=None):
    s = router_scores(h, w, p)
    if chosen is None:
        chosen = choose(s, mlp["router"]["top"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e in chosen[t]:
            out[t] += gated_ff(s[t, e] * h[t:t + 1], w, f"{p}e{int(e)}.", silu)[0]
    if mlp.get("shared"):
        out += gated_ff(h, w, p + "shared.", silu)
    return out, s, chosen


# ----------------------------------------------------------------------------- the model
class Dorevik:
    def __init__(self, config: dict, tensors: dict):
        self.c, self.w = config, tensors
        self.eps = float(config["norm"]["eps"])

    @classmethod
    def from_folder(cls, folder):
        with open(os.path.join(folder, "config.json")) as f:
            return cls(json.load(f), read_tensors(os.path.join(folder, "model.safetensors")))

    def forward(self, tokens, choices=None, trace=None):
        """Logits [T, vocab] of one whole sequence.  `choices`: {layer: [T, top] experts} to use instead of the
        router's own; `trace`: a dict that receives the stream after every layer, the routers' scores and choices."""
        w, eps = self.w, self.eps
        x = w["embed"][np.asarray(tokens)]
        streams, routed = [], {}
        for i, layer in enumerate(self.c["layers"]):
            p = f"l{i}."
            if layer["type"] == "attention":
                y = differential_attention(x, w, p + "mix.", layer["mixer"], eps)
            elif layer["type"] == "parallel":
                y = side_by_side(x, w, p + "mix.", layer["mixer"], eps)
            else:
                raise ValueError(layer["type"])
            x = x + rms_norm(y, w[p + "norm1"], eps)
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp["kind"] == "dense":
                    y = gated_ff(x, w, p + "mlp.", gelu_tanh)
                else:
                    y, s, ch = expert_mixture(x, w, p + "mlp.", mlp, None if choices is None else choices.get(i))
                    routed[i] = (s, ch)
                x = x + rms_norm(y, w[p + "norm2"], eps)
            streams.append(x.copy())
        z = rms_norm(x, w["final.norm"], eps) @ w["head"].T
        cap = self.c.get("logit_softcap")
        if cap:
            z = cap * np.tanh(z / cap)
        if trace is not None:
            trace["streams"], trace["routed"] = streams, routed
        return z

    def greedy(self, prompt, n):
        """`n` tokens after `prompt`, each the largest logit's (the first of equals)."""
        toks = list(prompt)
        for _ in range(n):
            toks.append(int(np.argmax(self.forward(toks)[-1])))
        return toks[len(prompt):]
