"""The kernels behind Dopipel's mechanisms, each alone against the plain function of the same mechanism
(tests/plain/dopipel_plain.py, float64), at sizes of their own, over several sequences packed into one step with
shuffled slots, in portions down to one row, and with inputs made so that a fault shows: a key hundreds of rows back
whose score stands out and whose value must come back turned by exactly that distance, a gate that stays shut for
hundreds of rows over a state written by the first, scores that tie, a correction that overturns the scores' order,
rows that choose identity experts only."""
import numpy as np
import pytest
import torch

from kvad_b200.ops import Ops
from tests.plain import dopipel_plain as pl

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
KTOL = {"float32": 3e-6, "bfloat16": 1.5e-2}
PAGE = 64


def dev(a, dtype=None):
    t = torch.as_tensor(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.to("cuda")


def i32(a):
    return dev(np.asarray(a, dtype=np.int32))


def rel(got, ref):
    got, ref = np.asarray(got.detach().double().cpu()), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape and np.isfinite(got).all()
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


def stored(a, dtype):
    """The values a tensor of the given dtype holds, as float64."""
    return torch.as_tensor(np.asarray(a)).to(DT[dtype]).double().numpy()


def angle_tol(dtype, far):
    """Angles are position x frequency in 32-bit: at position p they are rounded to about p x 2^-23 of a radian."""
    return KTOL[dtype] + 2.0 * far * 2.0 ** -23


def inv_freq(base, dims):
    return dev((np.float64(base) ** (-2.0 * np.arange(dims // 2) / dims)).astype(np.float32))


# ----------------------------------------------------------------------------- turns
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,size,dims", [(3, 10, 10), (2, 64, 64), (5, 24, 6)])
def test_pairs_turned_forth_back_and_gated_head_by_head(dtype, H, size, dims):
    rng, ops, base, n = np.random.default_rng(size), Ops(DT[dtype]), 300.0, 40
    pos = rng.integers(0, 3000, n)
    x = stored(rng.standard_normal((n, H * size + 3)), dtype)          # (three columns that are no head's stay as they are)
    f = inv_freq(base, dims)
    heads = x[:, :H * size].reshape(n, H, size)
    tol = angle_tol(dtype, 3000)
    t = dev(x, DT[dtype])
    ops.rotary(t, t, i32(pos), f, H, dims, interleaved=True, head_stride_src=size)
    want = np.concatenate([pl.turn_pairs(heads, pos, base, dims).reshape(n, -1), x[:, H * size:]], axis=1)
    assert rel(t, want) < tol
    back = dev(x, DT[dtype])
    ops.rotary(back, back, i32(pos), f, H, dims, interleaved=True, head_stride_src=size, inverse=True)
    want = np.concatenate([pl.turn_pairs(heads, pos, base, dims, sign=-1.0).reshape(n, -1), x[:, H * size:]], axis=1)
    assert rel(back, want) < tol
    if dims == size:          # whole heads: the gate of a head goes with the turn back
        gate = stored(rng.standard_normal((n, H)) * 2, dtype)
        g = dev(x, DT[dtype])
        ops.rotary(g, g, i32(pos), f, H, dims, interleaved=True, head_stride_src=size, inverse=True, head_gate=dev(gate, DT[dtype]))
        want[:, :H * size] = (pl.turn_pairs(heads, pos, base, dims, sign=-1.0) * pl.sigmoid(gate)[:, :, None]).reshape(n, -1)
        assert rel(g, want) < tol
    plain_gate = stored(rng.standard_normal((n, H)) * 2, dtype)
    y = dev(x[:, :H * size], DT[dtype])
    ops.head_gate(y, dev(plain_gate, DT[dtype]), H)
    assert rel(y, (heads * pl.sigmoid(plain_gate)[:, :, None]).reshape(n, -1)) < KTOL[dtype]


# ----------------------------------------------------------------------------- attention with turned values
def selection_weights(H, G, dk, dv):
    """Matrices that make the plain mixer read its input as q | k | v | gate logits and return the gated heads as they are."""
    w = H * dk + G * dk + G * dv + H
    W, at = {}, 0
    for name, rows in (("q", H * dk), ("k", G * dk), ("v", G * dv), ("g", H)):
        W[name] = np.zeros((rows, w))
        W[name][np.arange(rows), at + np.arange(rows)] = 1.0
        if name != "g":
            W[name + ".b"] = np.zeros(rows)
        at += rows
    W["o"], W["o.b"] = np.eye(H * dv), np.zeros(H * dv)
    return W


class Paged:
    """Keys and values of a few sequences in shuffled pages, as the cache lays them out."""

    def __init__(self, lens, G, dk, dv, dtype, seed):
        rng = np.random.default_rng(seed)
        n_pages = sum(-(-n // PAGE) for n in lens) + 3
        order = rng.permutation(n_pages)
        self.table = np.full((len(lens), max(-(-n // PAGE) for n in lens) + 1), -1, np.int32)
        at = 0
        for s, n in enumerate(lens):
            for j in range(-(-n // PAGE)):
                self.table[s, j] = order[at]
                at += 1
        self.k_pages = torch.full((n_pages, G, PAGE, dk), float("nan"), device="cuda", dtype=DT[dtype])
        self.v_pages = torch.full((n_pages, G, PAGE, dv), float("nan"), device="cuda", dtype=DT[dtype])


def attend(ops, dtype, cache, data, spans, m, hp, fused=True, tensor_cores=False):
    """Rows [a, a + r) of every sequence as one step, the way the mixer strings the launches: turn queries, keys and
    values and store the latter two (`fused`: in one launch; else in three), attend (`tensor_cores`: through the prompt
    kernel of the plain causal attention), turn the heads' sums back and gate them."""
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    live = [s for s, (_, r) in enumerate(spans) if r]
    cat = dev(np.concatenate([data[s][a:a + r] for s, (a, r) in enumerate(spans) if r]), DT[dtype])
    seq = i32(np.concatenate([[j] * spans[s][1] for j, s in enumerate(live)]))
    pos = i32(np.concatenate([np.arange(spans[s][0], sum(spans[s])) for s in live]))
    nq, nk, nv = H * dk, G * dk, G * dv
    qk, v, gate = cat[:, :nq + nk], cat[:, nq + nk:nq + nk + nv], cat[:, nq + nk + nv:]
    fk, fv = inv_freq(m["rot"]["base"], m["rot"]["dims"]), inv_freq(m["rot"]["base"], dv)
    table = dev(cache.table[live])
    if fused:
        ops.turn_store(qk[:, :nq], qk[:, nq:], v, seq, pos, table, cache.k_pages, cache.v_pages, H, inv_freq=fk, dims=m["rot"]["dims"],
                       interleaved=True, value_inv_freq=fv, value_interleaved=True)
    else:
        ops.rotary(qk, qk, pos, fk, H + G, m["rot"]["dims"], interleaved=True, head_stride_src=dk)
        ops.rotary(v, v, pos, fv, G, dv, interleaved=True, head_stride_src=dv)
        ops.kv_store_blend(qk[:, nq:], v, seq, pos, table, cache.k_pages, cache.v_pages)
    out = torch.full((cat.shape[0], H * dv), float("nan"), device="cuda", dtype=DT[dtype])
    starts = i32(np.concatenate([[0], np.cumsum([spans[s][1] for s in live])]))
    if tensor_cores:
        qq = qk[:, :nq].contiguous()              # (the mixer's rows are padded to 16 bytes; these are not)
        assert ops.prompt_attention_takes(qq, dk, PAGE)
        ops.attention_prefill(qq, out, starts, i32([sum(spans[s]) for s in live]), len(live), max(r for _, r in spans), table,
                              cache.k_pages, cache.v_pages, H, m["scale"], 0)
    else:
        ops.attention_scored(qk[:, :nq], out, starts, i32([sum(spans[s]) for s in live]), len(live), max(r for _, r in spans), table,
                             cache.k_pages, cache.v_pages, H, m["scale"], heads_per_block=hp)
    ops.rotary(out, out, pos, fv, H, dv, interleaved=True, head_stride_src=dv, inverse=True, head_gate=gate)
    o, at, res = out.double().cpu().numpy(), 0, {}
    for s in live:
        res[s] = o[at:at + spans[s][1]]
        at += spans[s][1]
    return res


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,dk,dv,rd", [(4, 2, 16, 24, 8), (3, 3, 6, 10, 2), (6, 1, 40, 8, 40), (8, 4, 64, 64, 32), (2, 1, 136, 16, 64), (5, 1, 64, 128, 64)])
def test_attention_with_turned_values_prompts_portions_and_single_rows(dtype, H, G, dk, dv, rd):
    rng, ops = np.random.default_rng(H * dk + dv), Ops(DT[dtype])
    m = {"heads": H, "kv_heads": G, "dim": dk, "vdim": dv, "scale": 0.3, "rot": {"base": 200.0, "dims": rd}}
    lens, W = [150, 9, 70], selection_weights(H, G, dk, dv)
    cache = Paged(lens, G, dk, dv, dtype, seed=dk)
    data = [stored(rng.standard_normal((n, H * dk + G * dk + G * dv + H)), dtype) for n in lens]
    want = [pl.rotated_value_attention(d, W, "", m) for d in data]
    tol = angle_tol(dtype, 150) * (3 if dtype == "bfloat16" else 1)            # (bfloat16: the values are rounded once more after their turn)
    group = H // G
    got = attend(ops, dtype, cache, data, [(0, n) for n in lens], m, hp=max(d for d in (1, 2, 4) if group % d == 0))
    for s in range(3):
        assert rel(torch.as_tensor(got[s]), want[s]) < tol, ("whole", s)
    # the same through portions (2 rows, an odd count, across a page edge), then single rows with a whole group a block
    cache.k_pages.fill_(float("nan")), cache.v_pages.fill_(float("nan"))
    cuts = [[(0, 2), (2, 61), (63, 2), (65, 60)], [(0, 3), (3, 2), (5, 2), (7, 1)], [(0, 64), (64, 1), (65, 2), (67, 2)]]
    for j in range(4):
        got = attend(ops, dtype, cache, data, [c[j] for c in cuts], m, hp=1 if j % 2 else max(d for d in (1, 2, 4) if group % d == 0), fused=j < 2)
        for s in range(3):
            a, r = cuts[s][j]
            assert rel(torch.as_tensor(got[s]), want[s][a:a + r]) < tol * max(1.0, np.abs(want[s]).max() / np.abs(want[s][a:a + r]).max()), ("portion", j, s)
    for p in range(125, 150):
        got = attend(ops, dtype, cache, data, [(p, 1), (0, 0), (0, 0)], m, hp=min(group, 32), fused=p % 2 == 0)
        assert rel(torch.as_tensor(got[0]), want[0][p:p + 1]) < tol * max(1.0, np.abs(want[0]).max() / np.abs(want[0][p]).max()), ("single", p)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,dk,dv,rd,layout,turn_v", [(4, 2, 16, 24, 8, "interleaved", True), (3, 1, 7, 10, 4, "half", True), (2, 2, 12, 5, 12, "half", False),
                                                        (5, 5, 6, 8, 0, "interleaved", True), (8, 2, 128, 64, 64, "interleaved", False)])
def test_one_launch_turns_and_stores_what_three_do(dtype, H, G, dk, dv, rd, layout, turn_v):
    """The fused launch against the single ones, bit for bit: queries in place, keys and values in their pages; a part of a
    key that does not turn, keys of odd size, values that turn or not, both layouts of pairs."""
    rng, ops, lens, inter = np.random.default_rng(dk + dv), Ops(DT[dtype]), [130, 5], layout == "interleaved"
    n = sum(lens)
    rows = dev(rng.standard_normal((n, H * dk + G * dk + G * dv + 3)), DT[dtype])
    seq, pos = i32(np.concatenate([[0] * lens[0], [1] * lens[1]])), i32(np.concatenate([np.arange(lens[0]), 700 + np.arange(lens[1])]))
    fk, fv = (inv_freq(300.0, rd) if rd else None), inv_freq(300.0, dv if dv % 2 == 0 else dv + 1)
    if dv % 2:
        turn_v = False
    caches = [Paged([lens[0], 700 + lens[1]], G, dk, dv, dtype, seed=3) for _ in range(2)]
    nq, nk = H * dk, G * dk
    a, b = rows.clone(), rows.clone()
    ops.turn_store(a[:, :nq], a[:, nq:nq + nk], a[:, nq + nk:nq + nk + G * dv], seq, pos, dev(caches[0].table), caches[0].k_pages, caches[0].v_pages, H,
                   inv_freq=fk, dims=rd, interleaved=inter, value_inv_freq=fv if turn_v else None, value_interleaved=inter)
    if rd:
        ops.rotary(b, b, pos, fk, H + G, rd, interleaved=inter, head_stride_src=dk)
    vb = b[:, nq + nk:nq + nk + G * dv]
    if turn_v:
        ops.rotary(vb, vb, pos, fv, G, dv, interleaved=inter, head_stride_src=dv)
    ops.kv_store_blend(b[:, nq:nq + nk], vb, seq, pos, dev(caches[1].table), caches[1].k_pages, caches[1].v_pages)
    assert torch.equal(a[:, :nq], b[:, :nq]) and torch.equal(a[:, nq:], rows[:, nq:])          # (the fused launch leaves keys and values as they came)
    for x, y in ((caches[0].k_pages, caches[1].k_pages), (caches[0].v_pages, caches[1].v_pages)):
        assert torch.equal(torch.isnan(x), torch.isnan(y)) and torch.equal(torch.nan_to_num(x), torch.nan_to_num(y))
    assert int((~torch.isnan(caches[0].k_pages)).sum()) == n * G * dk


@pytest.mark.parametrize("H,G,d,rd", [(6, 3, 64, 32), (4, 1, 128, 128), (8, 4, 32, 8), (2, 2, 48, 48)])
def test_prompt_rows_on_the_tensor_cores_with_turned_values(H, G, d, rd):
    """Keys as long as values, bfloat16: prompt rows go through the kernel of the plain causal attention (tcgen05 for
    heads of 64 and 128, mma.sync for the others) between the same turns; whole prompts, then portions over the pages
    the portions before them wrote."""
    from kvad_b200.ops import prefill_wait_timeouts
    rng, ops = np.random.default_rng(H * d), Ops(torch.bfloat16)
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": 0.2, "rot": {"base": 300.0, "dims": rd}}
    lens, W = [150, 9, 70], selection_weights(H, G, d, d)
    cache = Paged(lens, G, d, d, "bfloat16", seed=d)
    data = [stored(rng.standard_normal((n, H * d + 2 * G * d + H)), "bfloat16") for n in lens]
    want = [pl.rotated_value_attention(x, W, "", m) for x in data]
    tol = angle_tol("bfloat16", 150) * 3
    got = attend(ops, "bfloat16", cache, data, [(0, n) for n in lens], m, hp=1, tensor_cores=True)
    for s in range(3):
        assert rel(torch.as_tensor(got[s]), want[s]) < tol, ("whole", s)
    cache.k_pages.fill_(float("nan")), cache.v_pages.fill_(float("nan"))
    cuts = [[(0, 2), (2, 61), (63, 2), (65, 85)], [(0, 3), (3, 2), (5, 2), (7, 2)], [(0, 64), (64, 1), (65, 2), (67, 3)]]
    for j in range(4):
        got = attend(ops, "bfloat16", cache, data, [c[j] for c in cuts], m, hp=1, fused=j < 2, tensor_cores=True)
        for s in range(3):
            a, r = cuts[s][j]
            assert rel(torch.as_tensor(got[s]), want[s][a:a + r]) < tol * max(1.0, np.abs(want[s]).max() / np.abs(want[s][a:a + r]).max()), ("portion", j, s)
    assert prefill_wait_timeouts() == 0


@pytest.mark.parametrize("marked", [0, 63, 64, 333, 398, 399])
def test_a_far_value_comes_back_turned_on_the_tensor_cores(marked):
    """One key's score stands far above the rest; the last query of a prompt must read that key's value turned by the
    distance between them, through the tensor-core kernel (bfloat16, heads of 64)."""
    ops, n, d = Ops(torch.bfloat16), 400, 64
    m = {"heads": 2, "kv_heads": 1, "dim": d, "vdim": d, "scale": 1.0, "rot": {"base": 30.0, "dims": 2}}
    W = selection_weights(2, 1, d, d)
    x = np.zeros((n, 2 * d + d + d + 2))
    x[:, 2], x[:, d + 2] = 32.0, 32.0            # both heads ask along entry 2 (which no turn touches)
    x[:, 2 * d + 3] = 0.125
    x[marked, 2 * d + 2] = 1.0
    x[:, 3 * d:4 * d] = stored(np.random.default_rng(marked).standard_normal((n, d)) * 0.01, "bfloat16")
    x[marked, 3 * d:3 * d + 6] = [1.0, 0.0, 0.5, -0.5, 0.0, 2.0]
    x[:, 4 * d:] = 20.0                           # gates open
    want = pl.rotated_value_attention(x, W, "", m)[-1]
    turned = pl.turn_pairs(x[marked, 3 * d:4 * d].reshape(1, 1, d), [marked - (n - 1)], 30.0, d)[0, 0]
    assert np.allclose(want[:d], turned, atol=2e-3)
    if marked < n - 1:
        assert np.abs(turned - x[marked, 3 * d:4 * d]).max() > 0.3
    cache = Paged([n], 1, d, d, "bfloat16", seed=marked)
    got = attend(ops, "bfloat16", cache, [x], [(0, n)], m, hp=2, tensor_cores=True)[0][-1]
    assert np.abs(got - want).max() < 0.03


@pytest.mark.parametrize("mode", ["prompt", "single"])
@pytest.mark.parametrize("marked", [0, 5, 63, 64, 333, 399])
def test_a_far_value_comes_back_turned_by_its_distance(mode, marked):
    """All keys are alike but one, whose score is far above the rest; the last query must read that key's value turned
    by exactly the distance between them - not as stored, not as projected."""
    ops, n = Ops(torch.float32), 400
    m = {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 6, "scale": 1.0, "rot": {"base": 30.0, "dims": 2}}
    W = selection_weights(2, 1, 8, 6)
    d = np.zeros((n, 16 + 8 + 6 + 2))
    d[:, 2], d[:, 8 + 2] = 30.0, 30.0            # both heads ask along entry 2 (which no turn touches)
    d[:, 16 + 3] = 0.1
    d[marked, 16 + 2] = 1.0
    d[:, 24:30] = np.random.default_rng(marked).standard_normal((n, 6)) * 0.01
    d[marked, 24:30] = [1.0, 0.0, 0.5, -0.5, 0.0, 2.0]
    d[:, 30:] = 20.0                              # gates open
    want = pl.rotated_value_attention(d, W, "", m)[-1]
    turned = pl.turn_pairs(d[marked, 24:30].reshape(1, 1, 6), [marked - (n - 1)], 30.0, 6)[0, 0]
    assert np.allclose(want[:6], turned, atol=1e-3)
    if marked < n - 1:
        assert np.abs(turned - d[marked, 24:30]).max() > 0.3       # (the turn shows)
    cache = Paged([n], 1, 8, 6, "float32", seed=marked)
    if mode == "prompt":
        got = attend(ops, "float32", cache, [d], [(0, n)], m, hp=2)[0][-1]
    else:
        attend(ops, "float32", cache, [d], [(0, n - 1)], m, hp=2)
        got = attend(ops, "float32", cache, [d], [(n - 1, 1)], m, hp=2)[0][0]
    assert np.abs(got - want).max() < 2e-5


# ----------------------------------------------------------------------------- the input convolution
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("C,taps", [(24, 3), (54, 1), (100, 2), (600, 5), (16, 16)])
def test_input_convolution_in_portions_shorter_than_its_taps(dtype, C, taps):
    rng, ops = np.random.default_rng(C + taps), Ops(DT[dtype])
    lens, slots = [90, 7, 33], [4, 0, 2]
    w = stored(rng.standard_normal((C, taps)) * 0.5, dtype)
    x = [stored(rng.standard_normal((n, C)), dtype) for n in lens]
    want = [pl.input_convolution(a, w) for a in x]
    state = torch.zeros((6, 5 + max(1, (taps - 1) * C)), device="cuda")
    state[[1, 3, 5]] = 7.0
    done = [0, 0, 0]
    portions = [[40, 2, 30], [1, 1, 1], [2, 1, 0], [1, 1, 1], [3, 2, 0], [43, 0, 1]]
    for portion in portions:
        live = [s for s in range(3) if portion[s]]
        rows = np.concatenate([x[s][done[s]:done[s] + portion[s]] for s in live])
        starts = np.concatenate([[0], np.cumsum([portion[s] for s in live])])
        seq = np.concatenate([[j] * portion[s] for j, s in enumerate(live)])
        pos = np.concatenate([np.arange(done[s], done[s] + portion[s]) for s in live])
        out = torch.full(rows.shape, float("nan"), device="cuda", dtype=DT[dtype])
        one_each = all(portion[s] == 1 for s in live)
        xin = dev(rows, DT[dtype])
        ops.residual_conv(xin, dev(w, DT[dtype]), out, state, 5, i32(seq), i32(pos), i32(starts), i32([slots[s] for s in live]), shift=one_each)
        if not one_each:
            ops.conv_keep(xin, taps, state, 5, i32(starts), i32([slots[s] for s in live]), len(live))
        ref = np.concatenate([want[s][done[s]:done[s] + portion[s]] for s in live])
        assert rel(out, ref) < KTOL[dtype], portion
        for s in live:
            done[s] += portion[s]
    assert done == lens
    assert float((state[[1, 3, 5]] - 7.0).abs().max()) == 0.0 and float(state[:, :5].abs().max()) in (0.0, 7.0)      # slots of no sequence, and what lies before the offset


@pytest.mark.parametrize("C,taps", [(24, 3), (1000, 4), (64, 2), (520, 1), (512, 4)])
def test_input_convolution_of_prompt_rows_in_16_byte_pieces(C, taps):
    """Steps of 64 rows and more in bfloat16 with up to four taps: a thread walks four consecutive rows of 8 channels with
    the window in registers.  Sequences begin and end inside such a run, portions begin inside a sequence with fewer rows
    behind them than taps; the result has the bits of the row-by-row kernel (which a state offset of 5 numbers selects)."""
    rng, ops = np.random.default_rng(C + taps), Ops(torch.bfloat16)
    lens, slots = [150, 9, 70], [4, 0, 2]
    w = stored(rng.standard_normal((C, taps)) * 0.5, "bfloat16")
    x = [stored(rng.standard_normal((n, C)), "bfloat16") for n in lens]
    want = [pl.input_convolution(a, w) for a in x]
    states = {off: torch.zeros((6, off + max(1, (taps - 1) * C)), device="cuda") for off in (8, 5)}
    done = [0, 0, 0]
    for portion in ([61, 2, 30], [63, 5, 3], [26, 2, 37]):
        rows = np.concatenate([x[s][done[s]:done[s] + portion[s]] for s in range(3)])
        starts = np.concatenate([[0], np.cumsum(portion)])
        seq = np.concatenate([[s] * portion[s] for s in range(3)])
        pos = np.concatenate([np.arange(done[s], done[s] + portion[s]) for s in range(3)])
        xin, outs = dev(rows, torch.bfloat16), {}
        for off, state in states.items():
            outs[off] = torch.full(rows.shape, float("nan"), device="cuda", dtype=torch.bfloat16)
            ops.residual_conv(xin, dev(w, torch.bfloat16), outs[off], state, off, i32(seq), i32(pos), i32(starts), i32(slots), shift=False)
            ops.conv_keep(xin, taps, state, off, i32(starts), i32(slots), 3)
        ref = np.concatenate([want[s][done[s]:done[s] + portion[s]] for s in range(3)])
        assert rel(outs[8], ref) < KTOL["bfloat16"], portion
        assert torch.equal(outs[8], outs[5]), portion
        for s in range(3):
            done[s] += portion[s]
    assert done == lens


# ----------------------------------------------------------------------------- minGRU
def gru_weights(n):
    eye = np.eye(n)
    return {"z": np.concatenate([eye, 0 * eye, 0 * eye], 1), "z.b": np.zeros(n), "x": np.concatenate([0 * eye, eye, 0 * eye], 1), "x.b": np.zeros(n),
            "g": np.concatenate([0 * eye, 0 * eye, eye], 1), "o": eye}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n", [30, 48, 200, 1600])        # (1600 channels x 3 sequences: 32 channels a block; fewer: 16)
def test_min_gru_whole_in_portions_and_row_by_row(dtype, n):
    rng, ops = np.random.default_rng(n), Ops(DT[dtype])
    lens, slots, W = [700, 9, 130], [3, 0, 5], gru_weights(n)
    zug = [stored(rng.standard_normal((t, 3 * n)) * 2.0, "float32") for t in lens]
    want = [pl.min_gru(a, W, "")[0] for a in zug]
    state = torch.zeros((7, n + 2), device="cuda")
    done = [0, 0, 0]
    for portion in ([600, 5, 17], [1, 1, 1], [2, 1, 1], [15, 2, 16], [1, 0, 1], [81, 0, 94]):      # (600 rows: 32 chunks side by side; 17: one)
        live = [s for s in range(3) if portion[s]]
        rows = dev(np.concatenate([zug[s][done[s]:done[s] + portion[s]] for s in live]), torch.float32)
        starts = np.concatenate([[0], np.cumsum([portion[s] for s in live])])
        out = torch.full((rows.shape[0], n), float("nan"), device="cuda", dtype=DT[dtype])
        ops.min_gru(rows, n, out, state, i32(starts), i32([slots[s] for s in live]), len(live), max(portion), state_off=2)
        ref = np.concatenate([want[s][done[s]:done[s] + portion[s]] for s in live])
        assert rel(out, ref) < (1e-5 if dtype == "float32" else KTOL[dtype]), portion
        for s in live:
            done[s] += portion[s]
    assert done == lens
    for s in range(3):
        assert rel(state[slots[s], 2:], pl.min_gru(zug[s], W, "")[1]) < 1e-5
    assert float(state[[1, 2, 4, 6]].abs().max()) == 0.0 and float(state[:, :2].abs().max()) == 0.0


@pytest.mark.parametrize("cut", [None, 1, 100])
def test_min_gru_keeps_what_the_first_row_wrote_under_a_shut_gate(cut):
    """The first row opens the gate fully and writes a candidate; every later row keeps the gate shut: hundreds of rows
    on, the state is still the first row's, in a prompt and from step to step; both branches of the candidate show."""
    ops, n, T = Ops(torch.float32), 40, 500
    zug = np.zeros((T, 3 * n))
    zug[0, :n], zug[1:, :n] = 40.0, -40.0
    zug[:, n:2 * n] = np.random.default_rng(1).standard_normal((T, n)) * 3
    zug[0, n:2 * n] = np.linspace(-3, 3, n)
    zug[:, 2 * n:] = 1.0
    u = zug[0, n:2 * n]
    first = np.where(u >= 0, u + 0.5, pl.sigmoid(u))
    want = pl.min_gru(zug, gru_weights(n), "")[0]
    assert np.allclose(want[-1], first * pl.silu(1.0), atol=1e-9)
    state = torch.zeros((2, n), device="cuda")
    out = torch.zeros((T, n), device="cuda")
    z = dev(zug, torch.float32)
    if cut is None:
        ops.min_gru(z, n, out, state, i32([0, T]), i32([1]), 1, T)
    else:
        ops.min_gru(z[:cut], n, out[:cut], state, i32([0, cut]), i32([1]), 1, cut)
        for t in range(cut, T):
            ops.min_gru(z[t:t + 1], n, out[t:t + 1], state, i32([0, 1]), i32([1]), 1, 1)
    assert rel(out, want) < 1e-6 and rel(state[1], first) < 1e-6 and float(state[0].abs().max()) == 0.0


# ----------------------------------------------------------------------------- the router and the experts
def sort_buffers(ops, n, top, E, tm):
    tiles = max(1, ops.moe_max_tiles(n, top, E, tm))
    mk = lambda m: torch.full((m,), -7, device="cuda", dtype=torch.int32)
    return tiles, mk(tiles), mk(tiles * tm), mk(tiles * tm), mk(n * top)


@pytest.mark.parametrize("E,n_id,top", [(8, 3, 4), (3, 2, 2), (5, 0, 1), (0, 3, 2), (2, 1, 3), (32, 2, 4)])
def test_scores_choose_with_the_correction_and_weigh_without_it(E, n_id, top):
    rng, ops, n, R = np.random.default_rng(E + top), Ops(torch.float32), 300, E + n_id
    z = stored(rng.standard_normal((n, R)) * 2.0, "float32")
    z[0] = 0.0                                   # all level: the lowest indices are taken
    z[1, :] = 0.0
    z[1, R - 1] = 5.0                            # one clear winner ...
    corr = stored(rng.standard_normal(R) * 0.3, "float32")
    for c, what in ((corr, "steers"), (np.zeros(R), "none")):
        if what == "steers":
            z[2] = np.linspace(0.0, 1.0, R)      # ... and a row whose order the correction overturns
        W = {"router": np.eye(R), "correction": c}
        want_c, want_w, s, pick = pl.route(z, W, "", top)
        tm = ops.moe_tile_rows(n, top, False)
        tiles, tile_expert, pos_row, pos_slot, slot_pos = sort_buffers(ops, n, top, E, tm)
        chosen, weight = torch.zeros((n, top), device="cuda", dtype=torch.int32), torch.zeros((n, top), device="cuda")
        ops.moe_sort(chosen, R, tm, tile_expert, pos_row, pos_slot, slot_pos, logits=dev(z, torch.float32), weight=weight, routing="scores",
                     correction=dev(c, torch.float32) if what == "steers" else None, n_real=E)
        got_c, got_w = chosen.cpu().numpy(), weight.double().cpu().numpy()
        ranked = -np.sort(-pick, axis=-1)
        clear = (ranked[:, top - 1] - ranked[:, top] > 1e-5) if R > top else np.ones(n, bool)
        assert clear.sum() > n * 0.9
        for r in range(n):
            assert len(set(got_c[r].tolist())) == top
            if clear[r]:
                assert sorted(got_c[r].tolist()) == sorted(want_c[r].tolist()), (what, r)
                assert np.allclose(got_w[r], np.take_along_axis(s[r], got_c[r].astype(np.int64), -1) / np.take_along_axis(s[r], got_c[r].astype(np.int64), -1).sum(), rtol=2e-5)
        assert np.allclose(got_w.sum(-1), 1.0, atol=1e-5)
        if what == "none":
            assert got_c[0].tolist() == list(range(top)) and got_c[1, 0] == R - 1
        # the grouping: every slot of an expert with matrices has one place in a tile of its expert; the others have none
        sp, te, pr, ps = slot_pos.cpu().numpy(), tile_expert.cpu().numpy(), pos_row.cpu().numpy(), pos_slot.cpu().numpy()
        flat = got_c.reshape(-1)
        assert np.all(sp[flat >= E] == -1) and np.all(sp[flat < E] >= 0)
        placed = sp[flat < E]
        assert len(set(placed.tolist())) == len(placed)
        assert np.array_equal(te[placed // tm], flat[flat < E]) and np.array_equal(ps[placed], np.nonzero(flat < E)[0])
        assert np.array_equal(pr[placed], np.nonzero(flat < E)[0] // top)
        assert (ps >= 0).sum() == len(placed)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,E,n_id,top,ff,shared,n", [(64, 3, 2, 2, 40, 24, 70), (54, 7, 1, 3, 18, 10, 9), (96, 0, 3, 2, 8, 48, 33),
                                                          (128, 16, 2, 4, 64, 0, 1200), (40, 2, 6, 3, 24, 0, 5)])
def test_mixture_with_identity_experts_and_a_gated_shared_expert(dtype, width, E, n_id, top, ff, shared, n):
    """The launches the feed-forward strings together, from router logits to the sum in the stream, with the router's
    logits given so that both sides choose alike (their margins are kept clear)."""
    rng, ops, R = np.random.default_rng(width + E), Ops(DT[dtype]), E + n_id
    h = stored(rng.standard_normal((n, width)), dtype)
    W = {"router": np.zeros((R, width)), "correction": stored(rng.standard_normal(R) * 0.05, "float32")}
    z = stored(rng.permuted(np.tile(np.arange(R) * 0.7, (n, 1)), axis=1) + rng.standard_normal((n, R)) * 0.05, "float32")
    for e in range(E):
        W[f"e{e}.up"], W[f"e{e}.down"] = stored(rng.standard_normal((ff, width)) / width ** 0.5, dtype), stored(rng.standard_normal((width, ff)) / ff ** 0.5, dtype)
    mlp = {"router": {"experts": E, "identity": n_id, "top": top}}
    # (the plain mixture takes its logits from h; here they are given, so its router is asked for the choice only)
    chosen_ref, _, _, _ = pl.route(z, {"router": np.eye(R), "correction": W["correction"]}, "", top)
    s = pl.softmax_rows(z)
    wt = np.take_along_axis(s, chosen_ref, -1)
    wt = wt / (wt.sum(-1, keepdims=True) + 1e-20)
    want = np.zeros((n, width))
    for t in range(n):
        for e, a in zip(chosen_ref[t], wt[t]):
            want[t] += a * (h[t] if e >= E else pl.squared_relu_expert(h[t:t + 1], W, f"e{e}.")[0])
    if shared:
        W["shared.up"], W["shared.down"] = stored(rng.standard_normal((shared, width)) / width ** 0.5, dtype), stored(rng.standard_normal((width, shared)) / shared ** 0.5, dtype)
        W["shared.sg"] = stored(rng.standard_normal((1, width)) / width ** 0.5, dtype)
        want += pl.sigmoid(h @ W["shared.sg"].T) * pl.squared_relu_expert(h, W, "shared.")
    base = stored(rng.standard_normal((n, width)), "float32")
    residual = dev(base, torch.float32)
    hd = dev(h, DT[dtype])
    tm = ops.moe_tile_rows(n, top, width % 8 == 0 and ff % 8 == 0)
    tiles, tile_expert, pos_row, pos_slot, slot_pos = sort_buffers(ops, n, top, E, tm)
    chosen, weight = torch.zeros((n, top), device="cuda", dtype=torch.int32), torch.zeros((n, top), device="cuda")
    ops.moe_sort(chosen, R, tm, tile_expert, pos_row, pos_slot, slot_pos, logits=dev(z, torch.float32), weight=weight, routing="scores",
                 correction=dev(W["correction"], torch.float32), n_real=E)
    assert np.array_equal(np.sort(chosen.cpu().numpy(), -1), np.sort(chosen_ref, -1))
    outs = torch.full((tiles * tm, width), float("nan"), device="cuda")
    if E:
        w_in = dev(np.stack([W[f"e{e}.up"] for e in range(E)]), DT[dtype])
        w_out = dev(np.stack([W[f"e{e}.down"] for e in range(E)]), DT[dtype])
        few = n * top <= ops.MOE_FEW_SLOTS
        hid = torch.zeros((tiles * tm, ff), device="cuda", dtype=DT[dtype])
        if tm == ops.MOE_WIDE_TILE:
            rows = torch.zeros((tiles * tm, width), device="cuda", dtype=DT[dtype])
            ops.gather_rows(hd, pos_row, rows)
            ops.grouped_linear(rows, w_in, hid, tile_expert, pos_slot)
        else:
            ops.grouped_linear(hd, w_in, hid, tile_expert, pos_slot, in_rows=pos_row, few_rows=few)
        ops.relu_squared(hid, hid)
        ops.grouped_linear(hid, w_out, outs, tile_expert, pos_slot, few_rows=few)
    ops.moe_combine(residual, outs, slot_pos, weight, identity_input=hd)
    if shared:
        up = torch.zeros((n, shared + 1), device="cuda", dtype=DT[dtype])
        ops.linear(hd, dev(np.concatenate([W["shared.up"], W["shared.sg"]]), DT[dtype]), None, up, "store")
        hid = torch.zeros((n, shared), device="cuda", dtype=DT[dtype])
        ops.relu_squared(up[:, :shared], hid, row_gate=up[:, shared:shared + 1])
        ops.linear(hid, dev(W["shared.down"], DT[dtype]), None, residual, "residual")
    assert rel(residual - dev(base, torch.float32), want) < (2e-5 if dtype == "float32" else 3e-2)


# ----------------------------------------------------------------------------- the block's own steps
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,n", [(24, 37), (54, 37), (1000, 37), (1000, 700), (2100, 5)])      # (few rows of up to 2048 columns lie in registers)
def test_a_normed_sum_enters_the_stream_and_the_next_norm_reads_it(dtype, width, n):
    rng, ops, eps_post, eps = np.random.default_rng(width), Ops(DT[dtype]), 1e-5, 1e-6
    x, delta = stored(rng.standard_normal((n, width)), "float32"), stored(rng.standard_normal((n, width)) * 3, "float32")
    gain, weight = stored(rng.standard_normal(width), "float32"), stored(rng.standard_normal(width), "bfloat16")
    new_x = x + pl.rms_norm(delta, gain, eps_post)
    xs, ds = dev(x, torch.float32), dev(delta, torch.float32)
    out = torch.zeros((n, width), device="cuda", dtype=DT[dtype])
    ops.postnorm_rmsnorm(xs, ds, dev(gain, torch.float32), eps_post, out, dev(weight, torch.bfloat16), eps)
    assert rel(xs, new_x) < 3e-6 and float(ds.abs().max()) == 0.0
    assert rel(out, pl.rms_norm(new_x, weight, eps)) < KTOL[dtype]
    # without a norm after it (what a reader that folds nothing in asks for)
    xs, ds = dev(x, torch.float32), dev(delta, torch.float32)
    ops.postnorm_rmsnorm(xs, ds, dev(gain, torch.float32), eps_post)
    assert rel(xs, new_x) < 3e-6 and float(ds.abs().max()) == 0.0
    # some rows only (the head's rows): the output alone, the stream and the sum stay
    rows = [3, n - 1, 0]
    xs, ds = dev(x, torch.float32), dev(delta, torch.float32)
    out = torch.zeros((3, width), device="cuda", dtype=DT[dtype])
    ops.postnorm_rmsnorm(xs, ds, dev(gain, torch.float32), eps_post, out, dev(weight, torch.bfloat16), eps, rows=i32(rows))
    assert rel(out, pl.rms_norm(new_x[rows], weight, eps)) < KTOL[dtype]
    assert rel(xs, x) == 0.0 and rel(ds, delta) == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,n", [(24, 5), (54, 70), (256, 300)])
def test_the_stream_is_mixed_with_the_embedding_output(dtype, width, n):
    rng, ops = np.random.default_rng(width), Ops(DT[dtype])
    x, x0 = stored(rng.standard_normal((n, width)), "float32"), stored(rng.standard_normal((n, width)), "float32")
    w, step = stored(rng.standard_normal((width, 2 * width)) / width ** 0.5, dtype), stored(rng.standard_normal((3, width)), "float32")
    both = torch.zeros((n, 2 * width), device="cuda", dtype=DT[dtype])
    xs = dev(x, torch.float32)
    ops.stream_concat(xs, dev(x0, torch.float32), both)
    assert rel(both, np.concatenate([stored(x, dtype), stored(x0, dtype)], 1)) == 0.0
    ops.linear(both, dev(w, DT[dtype]), dev(step, torch.float32)[1], xs, "store_f32")
    want = np.concatenate([stored(x, dtype), stored(x0, dtype)], 1) @ w.T + step[1]
    assert rel(xs, want) < (3e-6 if dtype == "float32" else 1e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,width,pad", [(33, 50, 0), (70, 64, 7), (300, 704, 7)])      # (rows in eights with a padded gate: 16-byte pieces in bfloat16)
def test_squared_relu_alone_and_with_a_gate_per_row(dtype, n, width, pad):
    rng, ops = np.random.default_rng(5), Ops(DT[dtype])
    x, g = stored(rng.standard_normal((n, width)) * 2, dtype), stored(rng.standard_normal((n, 1)) * 2, dtype)
    out = torch.zeros((n, width), device="cuda", dtype=DT[dtype])
    ops.relu_squared(dev(x, DT[dtype]), out)
    assert rel(out, np.maximum(x, 0) ** 2) < KTOL[dtype]
    both = dev(np.concatenate([x, g, np.zeros((n, pad))], 1), DT[dtype])
    ops.relu_squared(both[:, :width], out, row_gate=both[:, width:width + 1])
    assert rel(out, np.maximum(x, 0) ** 2 * pl.sigmoid(g)) < KTOL[dtype]
