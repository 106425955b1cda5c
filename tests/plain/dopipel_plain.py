"""A plain, slow Dopipel: whole sequences, no cache, one function per mechanism.

Dopipel is a decoder of sandwich blocks - a norm before AND after each sublayer, the normed result scaled
channel by channel into the residual stream - whose mixer reads its input through a short causal
convolution added to the input itself.  The mixer of a layer is softmax attention (grouped heads, biases,
rotary queries and keys, values that are turned by their position before they are kept and whose weighted
sum is turned back by the query's position, one sigmoid gate per head) or a minGRU (an element-wise gated
recurrence whose gates read the current token only).  The feed-forward is dense (relu gate) or a mixture of
squared-relu experts with identity experts, a bias that only the choice sees, and a gated shared expert.
A range of layers may run several times in a row with the same weights, each pass mixing the embedding
output back in and adding a vector of its own.

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
def rms_norm(x, w, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softmax_rows(s):
    e = np.exp(s - s.max(-1, keepdims=True))
    return e / e.sum(-1, keepdims=True)


def turn_pairs(x, positions, base, dims, sign=1.0):
    """Turns neighbouring pairs (2i, 2i+1) of the first `dims` entries of x [tokens, heads, size] by
    sign * position * base^(-2i/dims)."""
    out = x.copy()
    i = np.arange(dims // 2)
    ang = sign * np.asarray(positions, dtype=np.float64)[:, None] * (float(base) ** (-2.0 * i / dims))[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def input_convolution(h, taps_w):
    """h + conv(h): per channel, tap j of `taps_w` [width, taps] meets the input taps - 1 - j rows back."""
    T, taps = h.shape[0], taps_w.shape[1]
    out = h.copy()
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += taps_w[:, j] * h[s]
    return out


# ----------------------------------------------------------------------------- mixers
def rotated_value_attention(h, W, p, m):
    """Softmax attention; queries and keys turned on their first rot.dims entries, values turned over all of
    theirs by their own position and the heads' sums turned back by the query's; a sigmoid gate per head."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m.get("kv_heads") or m["heads"], m["dim"], m["vdim"]
    base, rd = m["rot"]["base"], m["rot"]["dims"]
    pos = np.arange(T)
    q = (h @ W[p + "q"].T + W[p + "q.b"]).reshape(T, H, dk)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).reshape(T, G, dk)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).reshape(T, G, dv)
    q, k = turn_pairs(q, pos, base, rd), turn_pairs(k, pos, base, rd)
    v = turn_pairs(v, pos, base, dv)
    gate = sigmoid(h @ W[p + "g"].T)                    # [T, H]
    out = np.zeros((T, H, dv))
    seen = np.tril(np.ones((T, T), dtype=bool))
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * m["scale"]
        s = np.where(seen, s, -np.inf)
        out[:, a] = softmax_rows(s) @ v[:, g]
    out = turn_pairs(out, pos, base, dv, sign=-1.0) * gate[:, :, None]
    return out.reshape(T, H * dv) @ W[p + "o"].T + W[p + "o.b"]


def min_gru(h, W, p, state=None):
    """S_t = (1 - z) S_(t-1) + z c, z = sigmoid(W_z h + b), c = u + 1/2 (u >= 0) or sigmoid(u) (u < 0), u = W_x h + b;
    out = W_o (S_t * silu(W_g h)).  Returns (output, last state)."""
    T = h.shape[0]
    z = sigmoid(h @ W[p + "z"].T + W[p + "z.b"])
    u = h @ W[p + "x"].T + W[p + "x.b"]
    c = np.where(u >= 0, u + 0.5, sigmoid(u))
    S = np.zeros(z.shape[1]) if state is None else state.copy()
    outs = np.zeros_like(z)
    for t in range(T):
        S = (1.0 - z[t]) * S + z[t] * c[t]
        outs[t] = S
    return (outs * silu(h @ W[p + "g"].T)) @ W[p + "o"].T, S


# ----------------------------------------------------------------------------- feed-forwards
def relu_glu(h, W, p):
    return (np.maximum(h @ W[p + "gate"].T, 0.0) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def squared_relu_expert(h, W, p):
    return (np.maximum(h @ W[p + "up"].T, 0.0) ** 2) @ W[p + "down"].T


def route(h, W, p, top):
    """(chosen [T, top], weights [T, top], scores [T, all], choice scores [T, all])."""
    s = softmax_rows(h @ W[p + "router"].T)
    pick = s + W[p + "correction"]
    chosen = np.argsort(-pick, axis=-1, kind="stable")[:, :top]
    w = np.take_along_axis(s, chosen, -1)
    return chosen, w / (w.sum(-1, keepdims=True) + 1e-20), s, pick


def mixture(h, W, p, mlp, chosen=None, margins=None, own_out=None):
    """`chosen`: take these experts instead of the router's own choice (the weights are still the scores').  `margins`
    receives, row by row, how far the last chosen choice score is above the first one left out; `own_out` the router's
    own choice."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    own, w, s, pick = route(h, W, p, top)
    if margins is not None:
        ranked = -np.sort(-pick, axis=-1)
        margins.append(ranked[:, top - 1] - ranked[:, top] if pick.shape[1] > top else np.full(h.shape[0], np.inf))
    if own_out is not None:
        own_out.append(own)
    if chosen is not None:
        w = np.take_along_axis(s, chosen, -1)
        w = w / (w.sum(-1, keepdims=True) + 1e-20)
    else:
        chosen = own
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t], w[t]):
            if e >= E:
                out[t] += wt * h[t]
            else:
                out[t] += wt * squared_relu_expert(h[t:t + 1], W, p + f"e{e}.")[0]
    if mlp.get("shared"):
        out += sigmoid(h @ W[p + "shared.sg"].T) * squared_relu_expert(h, W, p + "shared.")
    return out


# ----------------------------------------------------------------------------- the model
def run_order(cfg):
    """[(layer, pass number or None, first of its pass)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    out = [(i, None, False) for i in range(loop["start"])]
    for t in range(loop["times"]):
        out += [(i, t, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    out += [(i, None, False) for i in range(loop["stop"], n)]
    return out


def layer(x, W, cfg, i, forced=None, margins=None, own=None):
    """`forced`: an iterator over the experts to take, one array [T, top] per routed feed-forward in run order."""
    L, p, eps = cfg["layers"][i], f"l{i}.", cfg["norm"]["eps"]
    h = rms_norm(x, W[p + "norm1"], eps)
    if cfg.get("canon"):
        h = input_convolution(h, W[p + "canon1"])
    if L["type"] == "attention":
        y = rotated_value_attention(h, W, p + "mix.", L["mixer"])
    else:
        y, _ = min_gru(h, W, p + "mix.")
    x = x + rms_norm(y, W[p + "norm1b"], eps) * W[p + "ls1"]
    mlp = L.get("mlp")
    if mlp is None:
        return x
    h = rms_norm(x, W[p + "norm2"], eps)
    if mlp["kind"] == "dense":
        y = relu_glu(h, W, p + "mlp.")
    else:
        y = mixture(h, W, p + "mlp.", mlp, None if forced is None else next(forced), margins, own)
    return x + rms_norm(y, W[p + "norm2b"], eps) * W[p + "ls2"]


def forward(cfg, W, tokens, forced=None, streams=None, margins=None, own=None):
    """Logits [tokens, vocab] of one whole sequence.  `forced`: the experts to take instead of the routers' own
    choices, one array [T, top] per routed feed-forward in the order they run; `streams`: a list that receives the
    stream after every layer run; `margins`, `own`: see `mixture`."""
    x = W["embed"][np.asarray(tokens)]
    x0 = x.copy()
    forced = iter(forced) if forced is not None else None
    for i, t, first in run_order(cfg):
        if first:
            x = np.concatenate([x, x0], axis=-1) @ W["loop.in"].T + W["loop.step"][t]
        x = layer(x, W, cfg, i, forced, margins, own)
        if streams is not None:
            streams.append(x.copy())
    return rms_norm(x, W["final.norm"], cfg["norm"]["eps"]) @ W["head"].T


def greedy(cfg, W, prompt, n):
    toks, out = list(prompt), []
    for _ in range(n):
        out.append(int(forward(cfg, W, toks)[-1].argmax()))
        toks.append(out[-1])
    return out


def load(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_tensors(os.path.join(model_dir, "model.safetensors"))
