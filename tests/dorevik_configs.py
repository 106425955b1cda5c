"""Small Dorevik configurations for the tests: each differs from the others in every size, in the order of its layers
and in which options it has (a first layer of each kind; one key/value head for several heads, or one each, or the key
left out of config.json; keys and values of different sizes; a rotation over part of a key or all of it, with and without
stretched frequencies, also beside the linear attention; windows of 1, 3 and 7 positions, of exactly a page, of a page and
one, and wider than any prompt; one decay or several, a decay of 1; a router that takes one expert or all of them, with
and without a shared expert; a layer without a feed-forward; capped and uncapped logits; sizes that allow no 16-byte
pieces)."""


def rot(dims, base=10000.0, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling:
        out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return out


def attention(heads, kv_heads, dim, vdim, window, rotation, diff=0.3, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5, "diff": diff,
         "mask": {"size": window}, "rot": rotation}
    if kv_heads is None:
        del m["kv_heads"]
    return {"type": "attention", "mixer": m}


def parallel(left, right):
    heads, kv_heads, dim, vdim, window, rotation = left
    l = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5, "mask": {"size": window}, "rot": rotation}
    heads, dim, vdim, decay = right
    return {"type": "parallel", "mixer": {"left": l, "right": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def model(width, vocab, layers, mlps, cap=None, eps=1e-5):
    out = {"architecture": "Dorevik", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "layers": [{**layer, "mlp": mlp} for layer, mlp in zip(layers, mlps)]}
    if cap:
        out["logit_softcap"] = cap
    return out


CONFIGS = {
    # the two mixers side by side first, a window of 7 beside three decays; differential heads with a key/value head each; no
    # feed-forward in the last layer
    "A": model(64, 257,
               [parallel((4, 2, 16, 8, 7, rot(8, 500.0, (4.0, 32, 8.0, 1.0))), (3, 8, 12, (0.5, 0.9, 0.99))),
                attention(2, 2, 8, 16, 33, rot(8, 100.0)), attention(4, 2, 8, 8, 5, rot(4, 100.0, (2.0, 16, 4.0, 0.5)), diff=0.6)],
               [moe(5, 2, 24, shared=16), dense(96), None], cap=30.0),
    # a window of exactly a page, then one of a page and one, then one wider than any prompt; stretched frequencies in the
    # differential layers; a router that takes one expert, another that takes all; no cap on the logits
    "B": model(96, 500,
               [attention(6, 2, 16, 24, 64, rot(4, 1e4, (8.0, 64, 16.0, 2.0)), diff=0.5),
                parallel((3, 3, 32, 32, 65, rot(32, 1e6)), (1, 64, 96, (0.97,))),
                attention(4, 1, 12, 20, 200, rot(12, 300.0, (3.0, 40, 10.0, 1.0)), diff=0.1, scale=0.2)],
               [moe(8, 1, 40), moe(3, 3, 16, shared=24), dense(64)], eps=1e-6),
    # sizes that are multiples of two at most: no product on the tensor cores, no 16-byte pieces anywhere; windows of 3 and of 1
    # (a row sees itself only); a decay of 1; `kv_heads` left out
    "C": model(54, 131,
               [attention(3, None, 6, 10, 3, rot(2, 50.0), diff=0.2),
                parallel((2, 1, 10, 14, 1, rot(10, 50.0)), (2, 6, 10, (0.8, 1.0)))],
               [dense(30), moe(7, 3, 18, shared=10)], cap=5.0),
    # larger: keys of 64 and 128, values of 64 and 128, many small experts (their products on the tensor cores for long prompts
    # in bfloat16), windows that several pages pass through
    "D": model(256, 1000,
               [parallel((4, 2, 64, 64, 128, rot(32, 1e6)), (4, 64, 64, (0.7, 0.9, 0.97, 0.999))),
                attention(4, 2, 64, 128, 100, rot(64, 3e4, (2.0, 256, 24.0, 1.5))),
                attention(8, 8, 32, 32, 513, rot(16, 1e5), diff=0.4),
                parallel((2, 1, 128, 128, 70, rot(64, 1e4, (4.0, 128, 16.0, 1.0))), (2, 128, 128, (0.95, 0.995)))],
               [moe(16, 2, 64, shared=128), dense(512), moe(32, 4, 64), None], cap=20.0),
}
SEEDS = {"A": 131, "B": 232, "C": 333, "D": 434}
#: the configurations every test of the engine runs on; "D" has tests of its own
SMALL = ("A", "B", "C")
