"""Small Dopipel configurations for the tests: each differs from the others in every size, in the order of its
layers and in which options it has (a first layer of each kind; one key/value head for several heads, or one
each; keys and values of different sizes; a rotation over part of a key or all of it; one to five taps or no
convolution; a repeated range at the start, in the middle, of one layer, run once, or none; a router that takes
one route or all of them, identity experts only, none at all, experts without a shared one; a layer without a
feed-forward; sizes that allow no 16-byte pieces)."""


def attention(heads, kv_heads, dim, vdim, rot_dims, base=10000.0, scale=None):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5,
                                           "rot": {"base": base, "dims": rot_dims}}}


def mingru(width):
    return {"type": "mingru", "mixer": {"width": width}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, identity, top, ff, shared=None):
    m = {"kind": "moe", "router": {"experts": experts, "identity": identity, "top": top}, "expert": {"ff": ff}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def model(width, vocab, layers, mlps, taps=3, loop=None, eps=1e-5):
    out = {"architecture": "Dopipel", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "layers": [{**layer, "mlp": mlp} for layer, mlp in zip(layers, mlps)]}
    if taps:
        out["canon"] = {"taps": taps}
    if loop:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


CONFIGS = {
    # a minGRU first, narrower than the stream; the middle two layers three times; two taps; a router that takes all its routes
    "A": model(64, 257,
               [mingru(48), attention(3, 3, 12, 20, 8, base=500.0), mingru(80), attention(4, 1, 16, 8, 16, base=500.0, scale=0.3)],
               [dense(96), moe(3, 2, 2, 40, shared=24), None, moe(2, 1, 3, 16)],
               taps=2, loop=(1, 3, 3)),
    # attention first; no repeated range; four taps; a router that takes one route; identity experts only; no shared expert
    "B": model(96, 500,
               [attention(6, 2, 16, 24, 4, base=1e6), mingru(96), attention(2, 2, 24, 40, 24), attention(4, 2, 8, 16, 2, base=1e6)],
               [moe(5, 0, 1, 32), dense(64), moe(0, 3, 2, 8, shared=48), dense(200)],
               taps=4, loop=None, eps=1e-6),
    # long heads; the whole model is the repeated range, twice; one tap (the convolution sees the row itself only)
    "C": model(128, 300,
               [attention(2, 1, 136, 16, 64), mingru(200), attention(8, 4, 32, 32, 32, base=100.0)],
               [dense(128), moe(16, 2, 2, 64, shared=64), moe(2, 6, 3, 96)],
               taps=1, loop=(0, 3, 2)),
    # sizes that are multiples of two at most: no product on the tensor cores, no 16-byte pieces anywhere; no convolution;
    # a range of one layer, run once
    "D": model(54, 131,
               [mingru(30), attention(3, 3, 6, 10, 2, base=100.0), attention(2, 1, 10, 14, 10, base=100.0), mingru(54)],
               [moe(7, 1, 3, 18, shared=10), dense(30), moe(3, 0, 3, 14), None],
               taps=0, loop=(2, 3, 1)),
    # larger and deeper: five taps, the last layers repeated, many small experts (their products on the tensor cores for
    # long prompts in bfloat16), keys of 64 and values of 128
    "E": model(320, 1000,
               [attention(4, 4, 48, 40, 16, base=1e5), mingru(320), attention(5, 1, 64, 128, 64, base=3e4), mingru(512), attention(8, 2, 32, 32, 8, base=1e5)],
               [moe(32, 2, 4, 64, shared=192), dense(512), moe(12, 4, 3, 96), dense(384), moe(32, 0, 4, 64, shared=64)],
               taps=5, loop=(3, 5, 2)),
    # keys as long as values, 64 and 128 of them: in bfloat16 prompt rows attend on the tensor cores, single rows do not
    "F": model(192, 777,
               [attention(6, 3, 64, 64, 32, base=2e4, scale=0.11), mingru(128), attention(4, 1, 128, 128, 128, base=700.0, scale=0.07)],
               [dense(256), moe(4, 1, 2, 64, shared=32), None],
               taps=3, loop=(1, 3, 2)),
}
SEEDS = {"A": 111, "B": 212, "C": 313, "D": 414, "E": 515, "F": 616}
#: the configurations every test of the engine runs on; "E" and "F" have tests of their own
SMALL = ("A", "B", "C", "D")
