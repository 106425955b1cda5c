"""The kernels behind Dorevik's mechanisms, each alone against the plain function of the same mechanism
(tests/plain/dorevik_plain.py, float64), at sizes of their own, with inputs made so that a fault shows: one key whose
score stands out placed just inside and just outside a window, in a prompt and for a single row; a second map that
must be taken off the first with exactly lam; a far row that a decay of 0.999 still carries; a score that is level
with the next; shuffled pages."""
import math

import numpy as np
import pytest
import torch

from kvad_b200.ops import Ops
from tests.plain import dorevik_plain as pl
from tests.test_gpu_nifulix_ops import DT, KTOL, PAGE, Paged, dev, rel, stored

pytestmark = pytest.mark.gpu


def nan_like(shape, dtype):
    """A buffer that holds nothing a kernel may rely on: NaNs, or an absurd number where the type has none."""
    return torch.full(shape, float("nan") if dtype.is_floating_point else -12345, device="cuda", dtype=dtype)


# ----------------------------------------------------------------------------- row-wise pieces
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gate_mul_with_the_tanh_gelu(dtype):
    rng, ops = np.random.default_rng(5), Ops(DT[dtype])
    both = rng.standard_normal((6, 2 * 37)) * 3
    t, bs = dev(both, DT[dtype]), stored(both, dtype)
    out = nan_like((6, 37), DT[dtype])
    ops.gate_mul(t[:, :37], t[:, 37:], out, "gelu_tanh")
    assert rel(out, pl.gelu_tanh(bs[:, :37]) * bs[:, 37:]) < KTOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [24, 100, 1000, 2500])
def test_a_normed_result_enters_the_stream_and_the_stream_is_handed_on_as_it_is(dtype, width):
    """x += g * d / rms(d); d = 0; out = x in the compute dtype (no norm): what a sublayer that reads the stream itself gets."""
    rng, ops, eps = np.random.default_rng(width), Ops(DT[dtype]), 1e-5
    x, d, g = rng.standard_normal((9, width)) * 2, rng.standard_normal((9, width)) * 5, rng.standard_normal(width)
    xs, ds, gs = stored(x, "float32"), stored(d, "float32"), stored(g, "float32")
    want = xs + pl.rms_norm(ds, gs, eps)
    xd, dd = dev(x, torch.float32), dev(d, torch.float32)
    rows = dev([7, 0, 7], torch.int32)
    out = nan_like((3, width), DT[dtype])
    ops.postnorm_rmsnorm(xd, dd, dev(g, torch.float32), eps, out, rows=rows, plain_out=True)       # a row list writes nothing back
    assert rel(out, want[[7, 0, 7]]) < KTOL[dtype]
    assert torch.equal(xd.cpu(), torch.as_tensor(x).float()) and torch.equal(dd.cpu(), torch.as_tensor(d).float())
    out = nan_like((9, width), DT[dtype])
    ops.postnorm_rmsnorm(xd, dd, dev(g, torch.float32), eps, out, plain_out=True)
    assert rel(out, want) < KTOL[dtype] and rel(xd, want) < 2e-6 and float(dd.abs().max()) == 0.0
    out2 = nan_like((4, width), DT[dtype])
    ops.cast_rows(xd, out2, dev([8, 1, 1, 0], torch.int32))
    assert torch.equal(out2, out[[8, 1, 1, 0]])
    out3 = nan_like((9, width), DT[dtype])
    ops.cast_rows(xd, out3)
    assert torch.equal(out3, out)


@pytest.mark.parametrize("width", [6, 54, 256, 1030])
def test_two_results_normed_and_averaged_into_the_sum(width):
    rng, ops, eps = np.random.default_rng(width), Ops(torch.float32), 1e-6
    a, b, d = (rng.standard_normal((5, width)) * s for s in (3.0, 0.2, 1.0))
    ga, gb = rng.standard_normal(width), rng.standard_normal(width)
    want = stored(d, "float32") + 0.5 * (pl.rms_norm(stored(a, "float32"), stored(ga, "float32"), eps) + pl.rms_norm(stored(b, "float32"), stored(gb, "float32"), eps))
    ad, bd, dd = (dev(t, torch.float32) for t in (a, b, d))
    ops.pair_norm_sum(ad, bd, dev(ga, torch.float32), dev(gb, torch.float32), dd, eps, 0.5)
    assert rel(dd, want) < 2e-6
    assert float(ad.abs().max()) == 0.0 and float(bd.abs().max()) == 0.0


def test_capped_logits():
    ops = Ops(torch.float32)
    z = np.concatenate([np.linspace(-200, 200, 1001), [0.0, 1e-8, 1e4]])
    t = dev(z, torch.float32)
    ops.tanh_cap(t, 12.5)
    assert rel(t, 12.5 * np.tanh(stored(z, "float32") / 12.5)) < 2e-6
    assert float(t.abs().max()) <= 12.5


# ----------------------------------------------------------------------------- norm, turn and store
def plain_norm_turn(x, w, eps, span, rot, pos):
    """x [n, heads, dk] normed over `span` entries at a time of the flattened row (weight of that length), then turned."""
    n, H, dk = x.shape
    flat = x.reshape(n, -1, span)
    flat = pl.rms_norm(flat, w, eps) if w is not None else flat
    return pl.turn_halves(flat.reshape(n, H, dk), pos, rot) if rot else flat.reshape(n, H, dk)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,V,dk,dv,whole,rot", [
    (8, 4, 2, 48, 80, False, {"base": 3e4, "dims": 12, "scaling": {"factor": 6.0, "original": 512, "fast": 24.0, "slow": 2.0}}),
    (4, 2, 2, 128, 96, True, {"base": 5e5, "dims": 32}),
    (3, 3, 3, 6, 10, False, {"base": 50.0, "dims": 6}),
    (2, 1, 1, 10, 14, True, {"base": 50.0, "dims": 4, "scaling": {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 0.5}}),
    (4, 2, 1, 16, 8, False, None)])
def test_queries_and_keys_normed_turned_and_stored(dtype, H, G, V, dk, dv, whole, rot):
    """Head by head with one weight as long as a head, or over the whole projection; positions on both sides of a page's edge
    and far out; fewer value heads than key heads; shuffled pages."""
    rng, ops, eps = np.random.default_rng(H * dk + dv), Ops(DT[dtype]), 1e-5
    lens = [70, 3]
    pos = np.concatenate([np.arange(60, 70), np.arange(0, 3)])
    seq = np.array([0] * 10 + [1] * 3)
    n = len(pos)
    q, k, v = rng.standard_normal((n, H * dk)) * 2, rng.standard_normal((n, G * dk)) * 2, rng.standard_normal((n, V * dv))
    sq, sk = (H * dk, G * dk) if whole else (dk, dk)
    wq, wk = rng.standard_normal(sq) * 0.3 + 1, rng.standard_normal(sk) * 0.3 + 1
    want_q = plain_norm_turn(stored(q, dtype).reshape(n, H, dk), stored(wq, "float32"), eps, sq, rot, pos)
    want_k = plain_norm_turn(stored(k, dtype).reshape(n, G, dk), stored(wk, "float32"), eps, sk, rot, pos)
    cache = Paged(lens, G, dk, dv, dtype, seed=dk)
    cache.v_pages = nan_like((cache.k_pages.shape[0], V, PAGE, dv), DT[dtype])
    freq, mscale = (pl.rotary_frequencies(rot) if rot else (None, 1.0))
    qd = dev(q, DT[dtype])
    ops.norm_turn_store(qd, dev(k, DT[dtype]), dev(v, DT[dtype]), dev(seq, torch.int32), dev(pos, torch.int32), cache.table_dev, cache.k_pages,
                        cache.v_pages, H, q_weight=dev(wq, torch.float32), k_weight=dev(wk, torch.float32), span_q=sq, span_k=sk, eps=eps,
                        inv_freq=dev(freq, torch.float32) if rot else None, dims=rot["dims"] if rot else 0, mscale=mscale)
    assert rel(qd, want_q.reshape(n, -1)) < KTOL[dtype]
    kp, vp = cache.k_pages.double().cpu().numpy(), cache.v_pages.double().cpu().numpy()
    vs = stored(v, dtype).reshape(n, V, dv)
    for r in range(n):
        page = cache.table[seq[r], pos[r] // PAGE]
        assert np.abs(kp[page, :, pos[r] % PAGE] - want_k[r]).max() < KTOL[dtype] * np.abs(want_k).max()
        assert np.array_equal(vp[page, :, pos[r] % PAGE], vs[r])
    assert np.isnan(kp).sum() == kp.size - n * G * dk          # nothing else was written


# ----------------------------------------------------------------------------- differential attention
def plain_maps(q, k, v, H, G, scale, window, lam, eps, gain):
    """q [n, H, 2, dk], k [n, G, 2, dk], v [n, G, dv] of one whole sequence -> [n, H, dv]."""
    a1 = pl.softmax_attention(q[:, :, 0], k[:, :, 0], v, scale, window)
    a2 = pl.softmax_attention(q[:, :, 1], k[:, :, 1], v, scale, window)
    return pl.unit_rms(a1 - lam * a2, eps) * gain


def to_map_groups(q, H, G, dk):
    """Queries [n, H, 2, dk] as the attention wants them: [kv head][map][head of the group]."""
    n = q.shape[0]
    return q.reshape(n, G, H // G, 2, dk).transpose(0, 1, 3, 2, 4).reshape(n, -1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,dk,dv,window", [(4, 2, 40, 64, 75), (2, 2, 8, 16, 33), (6, 2, 16, 24, 64), (3, 3, 6, 10, 3), (4, 1, 12, 20, 500),
                                              (8, 2, 64, 128, 100)])
def test_two_maps_over_the_same_values_prompts_portions_and_single_rows(dtype, H, G, dk, dv, window):
    rng, ops, scale, lam, eps, gain = np.random.default_rng(H * dk + dv), Ops(DT[dtype]), 0.4, 0.37, 1e-5, 0.7
    lens = [150, 9, 70]
    cache = Paged(lens, 2 * G, dk, dv, dtype, seed=dk)
    cache.v_pages = nan_like((cache.k_pages.shape[0], G, PAGE, dv), DT[dtype])
    data = [[rng.standard_normal((n, w)) for w in (2 * H * dk, 2 * G * dk, G * dv)] for n in lens]
    want = [plain_maps(stored(q, dtype).reshape(n, H, 2, dk), stored(k, dtype).reshape(n, G, 2, dk), stored(v, dtype).reshape(n, G, dv), H, G, scale,
                       window, lam, eps, gain).reshape(n, -1) for n, (q, k, v) in zip(lens, data)]
    group = H // G

    def step(spans, single, fused=False):
        live = [s for s, (_, r) in enumerate(spans) if r]
        q = dev(np.concatenate([to_map_groups(data[s][0][a:a + r].reshape(r, H, 2, dk), H, G, dk) for s, (a, r) in enumerate(spans) if r]), DT[dtype])
        k, v = (dev(np.concatenate([data[s][i][a:a + r] for s, (a, r) in enumerate(spans) if r]), DT[dtype]) for i in (1, 2))
        seq = np.concatenate([[j] * spans[s][1] for j, s in enumerate(live)])
        pos = np.concatenate([np.arange(spans[s][0], sum(spans[s])) for s in live])
        table = dev(cache.table[live])
        ops.norm_turn_store(q, k, v, dev(seq, torch.int32), dev(pos, torch.int32), table, cache.k_pages, cache.v_pages, 2 * H)     # (no norm, no turn: a plain store)
        maps = nan_like((len(seq), 2 * H * dv), torch.float32)
        starts = dev(np.concatenate([[0], np.cumsum([spans[s][1] for s in live])]), torch.int32)
        splits = 3 if single else 1
        scratch = nan_like((len(seq) * 2 * H * splits * (dv + 2),), torch.float32) if single else None
        ops.attention_scored(q, maps, starts, dev([sum(spans[s]) for s in live], torch.int32), len(live), max(r for _, r in spans), table,
                             cache.k_pages, cache.v_pages, 2 * H, scale, window=window, key_maps=2, n_splits=splits, scratch=scratch,
                             heads_per_block=min(group, 32) if single else max(d for d in (1, 2, 4) if group % d == 0), merge=not fused)
        out = nan_like((len(seq), H * dv), DT[dtype])
        if fused:      # the parts' merge and the maps' difference in one launch
            ops.scored_merge_diff(scratch, splits, out, H, group, lam, eps, gain)
        else:
            ops.diff_combine(maps, out, H, group, lam, eps, gain)
        o, at, res = out.double().cpu().numpy(), 0, {}
        for s in live:
            res[s] = o[at:at + spans[s][1]]
            at += spans[s][1]
        return res

    tol = KTOL[dtype] * (4 if dtype == "bfloat16" else 1)      # (a difference of two sums, then a unit norm)
    got = step([(0, n) for n in lens], False)
    for s in range(3):
        assert rel(torch.as_tensor(got[s]), want[s]) < tol, ("whole", s)
    cache.k_pages.fill_(float("nan"))
    cache.v_pages.fill_(float("nan"))
    cuts = [[(0, 2), (2, 61), (63, 2), (65, 60)], [(0, 3), (3, 2), (5, 2), (7, 1)], [(0, 64), (64, 1), (65, 2), (67, 2)]]
    for j in range(4):
        got = step([c[j] for c in cuts], False)
        for s in range(3):
            a, r = cuts[s][j]
            assert rel(torch.as_tensor(got[s]), want[s][a:a + r]) < tol, ("portion", j, s)
    for p in range(125, 150):
        got = step([(p, 1), (0, 0), (0, 0)], True, fused=p % 2 == 0)
        assert rel(torch.as_tensor(got[0]), want[0][p:p + 1]) < tol, ("single", p)


@pytest.mark.parametrize("mode", ["prompt", "single"])
def test_the_second_map_is_taken_off_with_lam_and_windows_end_where_they_should(mode):
    """Map 1 of the query reads one marked key (a score far above the rest) with value e_2, map 2 another with value e_3; all
    other keys are alike with zero values.  The head's output before the unit norm must be e_2 - lam e_3 when both marked
    keys are inside the window, e_2 alone when the second is one position outside it, and -lam e_3 when the first is."""
    ops, dk, dv, n, window, lam = Ops(torch.float32), 8, 4, 300, 96, 0.25

    def run(mark1, mark2):
        cache = Paged([n], 2, dk, dv, "float32", seed=mark1)
        cache.v_pages = nan_like((cache.k_pages.shape[0], 1, PAGE, dv), torch.float32)
        q, k, v = np.zeros((n, 2, dk)), np.zeros((n, 2, dk)), np.zeros((n, dv))
        k[:, :, 1], q[:, :, 0] = 0.1, 40.0
        k[mark1, 0, 0], k[mark2, 1, 0] = 1.0, 1.0
        v[mark1, 2], v[mark2, 3] = 1.0, 1.0
        seq, pos = cache.rows_meta([(0, n)])
        qd = dev(q.reshape(n, -1), torch.float32)
        ops.norm_turn_store(qd, dev(k.reshape(n, -1), torch.float32), dev(v, torch.float32), seq, pos, cache.table_dev, cache.k_pages, cache.v_pages, 2)
        if mode == "prompt":
            maps = nan_like((n, 2 * dv), torch.float32)
            ops.attention_scored(qd, maps, dev([0, n], torch.int32), dev([n], torch.int32), 1, n, cache.table_dev, cache.k_pages, cache.v_pages,
                                 2, 1.0, window=window, key_maps=2)
            maps = maps[n - 1:]
        else:
            maps = nan_like((1, 2 * dv), torch.float32)
            scratch = nan_like((2 * 2 * (dv + 2),), torch.float32)
            ops.attention_scored(qd[n - 1:], maps, dev([0, 1], torch.int32), dev([n], torch.int32), 1, 1, cache.table_dev, cache.k_pages,
                                 cache.v_pages, 2, 1.0, window=window, key_maps=2, n_splits=2, scratch=scratch)
        out = nan_like((1, dv), torch.float32)
        ops.diff_combine(maps, out, 1, 1, lam, 1e-12, 1.0)
        o = out[0].double().cpu().numpy()
        return o * math.sqrt((np.array([1.0, lam]) ** 2).sum() / dv) if abs(o[2]) > 1e-3 and abs(o[3]) > 1e-3 else o      # (undo the unit norm where both are read)

    edge = n - window                                    # the oldest position the last row sees
    both = run(edge, n - 5)
    assert abs(both[2] - 1.0) < 1e-3 and abs(both[3] + lam) < 1e-3 and abs(both[0]) < 1e-6
    first_only = run(edge, edge - 1)                     # the second map's key is just outside: that map reads zeros
    assert first_only[2] > 1.9 and abs(first_only[3]) < 1e-6          # (a unit vector of 4 entries with one non-zero: 2)
    second_only = run(edge - 1, edge)
    assert abs(second_only[2]) < 1e-6 and second_only[3] < -1.9
    far = run(3, 7)                                      # hundreds of rows back: neither is seen
    assert np.abs(far).max() < 1e-6


# ----------------------------------------------------------------------------- linear attention with a decay, behind silu
def plain_decayed(q, k, v, g, decay, w, eps, S0=None):
    n, H, dk = q.shape
    dv = v.shape[2]
    q, k, v = pl.silu(q), pl.silu(k), pl.silu(v)
    S = np.zeros((H, dk, dv)) if S0 is None else S0.copy()
    o = np.zeros((n, H, dv))
    for t in range(n):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hkv,hk->hv", S, q[t])
    return pl.rms_norm(o.reshape(n, -1), w, eps) * pl.sigmoid(g), S


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,dk,dv", [(4, 24, 64), (3, 8, 12), (1, 64, 96), (2, 6, 10), (2, 128, 128)])
def test_decayed_linear_attention_whole_in_portions_and_token_by_token(dtype, H, dk, dv):
    rng, ops, eps = np.random.default_rng(dk * dv), Ops(DT[dtype]), 1e-6
    lens, slots = [37, 5, 70], [4, 0, 2]
    decay = np.linspace(0.6, 1.0, H) if H > 1 else np.array([0.97])
    w = rng.standard_normal(H * dv) * 0.3 + 1
    data = [[rng.standard_normal((n, H * d)) for d in (dk, dk, dv, dv)] for n in lens]
    want, want_S = [], []
    for n, (q, k, v, g) in zip(lens, data):
        o, S = plain_decayed(*(stored(a, dtype).reshape(n, H, -1) for a in (q, k, v)), stored(g, dtype), decay, stored(w, "float32"), eps)
        want.append(o)
        want_S.append(S)

    def run(state, cuts):
        got, done = [np.zeros((n, H * dv)) for n in lens], [0] * 3
        for j in range(max(len(c) for c in cuts)):
            live = [s for s in range(3) if j < len(cuts[s])]
            rows = [cuts[s][j] for s in live]
            q, k, v, g = (dev(np.concatenate([data[s][i][done[s]:done[s] + r] for s, r in zip(live, rows)]), DT[dtype]) for i in range(4))
            starts = dev(np.concatenate([[0], np.cumsum(rows)]), torch.int32)
            raw = nan_like((sum(rows), H * dv), torch.float32)
            ops.retention(q, k, v, None, state, starts, dev([done[s] + r for s, r in zip(live, rows)], torch.int32),
                          dev([slots[s] for s in live], torch.int32), len(live), dev(decay, torch.float32), H, raw=raw, silu_inputs=True, raw_only=True)
            out = nan_like((sum(rows), H * dv), DT[dtype])
            ops.row_norm_gate(raw, g, dev(w, torch.float32), out, eps)
            o, at = out.double().cpu().numpy(), 0
            for s, r in zip(live, rows):
                got[s][done[s]:done[s] + r] = o[at:at + r]
                at += r
                done[s] += r
        return got

    def check(cuts):
        state = torch.zeros((6, H, dk, dv), device="cuda")
        got = run(state, cuts)
        for s in range(3):
            assert rel(torch.as_tensor(got[s]), want[s]) < KTOL[dtype] * 4, (cuts, s)
            assert rel(state[slots[s]], want_S[s]) < 2e-5, (cuts, s)
        assert float(state[[1, 3, 5]].abs().max()) == 0.0                      # other slots untouched
        return got

    whole = check([[n] for n in lens])
    pieces = check([[16, 16, 5], [2, 3], [1, 2, 17, 33, 17]])
    single = check([[20] + [1] * 17, [1] * 5, [64] + [1] * 6])
    if dtype == "float32":                                                      # the same walk however it is cut: the same bits
        for s in range(3):
            assert np.array_equal(whole[s], pieces[s]) and np.array_equal(whole[s], single[s])


def test_a_far_row_is_still_read_through_a_slow_decay_and_gone_through_a_fast_one():
    ops, H, d, n = Ops(torch.float32), 2, 8, 640
    q, k, v = np.full((n, H, d), -30.0), np.full((n, H, d), -30.0), np.full((n, H, d), -30.0)      # (silu(-30) is nothing)
    k[3, :, 0], v[3, :, 1], q[-1, :, 0] = 50.0, 1.0, 1.0
    decay = np.array([0.999, 0.9])
    raw = torch.zeros((n, H * d), device="cuda")
    state = torch.zeros((1, H, d, d), device="cuda")
    args = [dev(a.reshape(n, -1), torch.float32) for a in (q, k, v)]
    ops.retention(*args, None, state, dev([0, n], torch.int32), dev([n], torch.int32), dev([0], torch.int32), 1, dev(decay, torch.float32), H,
                  raw=raw, silu_inputs=True, raw_only=True)
    got = raw.cpu().numpy().reshape(n, H, d)
    want = 50.0 * float(pl.silu(np.float64(1.0))) ** 2 * 0.999 ** (n - 4)
    assert abs(got[-1, 0, 1] - want) < 1e-3 * want and got[-1, 0, 1] > 5
    assert abs(got[-1, 1, 1]) < 1e-20


# ----------------------------------------------------------------------------- experts whose input the score scales
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,E,top,width,ff", [(40, 8, 1, 64, 24), (7, 3, 3, 54, 18), (300, 5, 2, 96, 40), (1, 7, 3, 32, 8), (600, 16, 2, 128, 64)])
def test_sigmoid_routing_and_experts_on_scaled_inputs(dtype, n, E, top, width, ff):
    """Through the part itself, with a context that only hands out buffers: routing, grouping, both grouped products, the
    gate with the score inside, the sum - against expert(s h) computed expert by expert."""
    from kvad_b200.parts.routed_mlp import InputScaledRoutedMLP
    rng, ops = np.random.default_rng(n + E), Ops(DT[dtype])
    part = InputScaledRoutedMLP("m.", width, E, top, ff, shared={"hidden": ff + 8})
    w = {"m.router": rng.standard_normal((E, width)) * 2 / math.sqrt(width)}
    for e in range(E):
        w[f"m.e{e}.gate"], w[f"m.e{e}.up"] = (rng.standard_normal((ff, width)) * 1.5 / math.sqrt(width) for _ in range(2))
        w[f"m.e{e}.down"] = rng.standard_normal((width, ff)) / math.sqrt(ff)
    w["m.shared.gate"], w["m.shared.up"] = (rng.standard_normal((ff + 8, width)) / math.sqrt(width) for _ in range(2))
    w["m.shared.down"] = rng.standard_normal((width, ff + 8)) / math.sqrt(ff + 8)
    part.load(lambda name, transpose=False, keep_f32=False, optional=False: dev(w[name], DT[dtype]))
    ws = {name: stored(a, dtype) for name, a in w.items()}
    h = rng.standard_normal((n, width))
    if n >= 4:      # a row whose scores are all level: the lower indices are taken
        h[3] = 0.0
    hs = stored(h, dtype)

    class Ctx:
        def __init__(self):
            self.ops, self.kept, self.dtype = ops, [], DT[dtype]

        def buffer(self, shape, dt=None):
            t = nan_like(tuple(shape), dt or DT[dtype])
            self.kept.append(t)
            return t

    ctx = Ctx()
    chosen = []
    inner = ops.moe_sort

    def sort(ch, *a, **kw):
        inner(ch, *a, **kw)
        chosen.append(ch.clone())
    ops.moe_sort = sort
    residual = torch.zeros((n, width), device="cuda")
    part.forward(ctx, dev(h, DT[dtype]), residual)
    mine = chosen[0].cpu().numpy()
    want, scores, _ = pl.expert_mixture(hs, ws, "m.", {"router": {"experts": E, "top": top}, "shared": {"ff": ff + 8}}, chosen=mine)
    assert rel(residual, want) < KTOL[dtype] * 3
    own = pl.choose(scores, top)
    ranked = -np.sort(-scores, axis=-1)
    for t in range(n):
        assert len(set(mine[t].tolist())) == top
        if top == E or ranked[t, top - 1] - ranked[t, top] > (1e-6 if dtype == "float32" else 0.02):
            assert sorted(mine[t].tolist()) == sorted(own[t].tolist()), t
    if n >= 4:
        assert mine[3].tolist() == list(range(top))          # level scores: the first experts
