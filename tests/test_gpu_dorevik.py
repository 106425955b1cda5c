"""Dorevik through the engine - its step function, cache, state and scheduler - against the plain implementation
(tests/plain/dorevik_plain.py, float64, whole sequences): whole prompts, token-by-token decoding from the first
token on, portions down to one and two tokens, unequal batches against each request alone, slots and pages that are
freed and used again, page borders and window edges passed while decoding, long decoding, and greedy generation
through the entry point.  The float32 engine is held to rounding of 32-bit sums against the oracle as it is.  In
bfloat16 a router whose last chosen score is nearly level with the next may choose the other way than the oracle, and
what that row then writes stays in the cache and state that later rows read; so the bfloat16 runs (and the largest
configuration's) record which experts the engine chose (a wrapper around the call that routes and groups, graphs
off), the oracle computes with those experts, and the choices themselves are compared with the oracle's own wherever
its margin is not small."""
import numpy as np
import pytest

from kvad_b200 import Engine, StepEntry, write_random_model
from tests.conftest import random_tokens, rel_err
from tests.dorevik_configs import CONFIGS, SEEDS, SMALL
from tests.plain import dorevik_plain as plain

pytestmark = pytest.mark.gpu
TOL = {"float32": 3e-5, "bfloat16": 0.1}
MARGIN = 0.05            # of router scores, which lie in 0 .. 1
CASES = [(n, d) for n in SMALL for d in ("float32", "bfloat16")]


def routed_layers(name):
    return [i for i, layer in enumerate(CONFIGS[name]["layers"]) if layer["mlp"] and layer["mlp"]["kind"] == "moe"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {n: write_random_model(str(tmp_path_factory.mktemp("dorevik" + n)), CONFIGS[n], SEEDS[n]) for n in CONFIGS}


@pytest.fixture(scope="module")
def loaded(folders):
    return {n: plain.Dorevik.from_folder(folders[n]) for n in CONFIGS}


@pytest.fixture(scope="module")
def oracle(loaded):
    cache = {}

    def get(name, tokens):
        key = (name, tuple(tokens))
        if key not in cache:
            cache[key] = loaded[name].forward(list(tokens))
        return cache[key]
    return get


@pytest.fixture(scope="module")
def engine(folders):
    cache = {}

    def get(name, dtype, max_tokens=2048):
        if (name, dtype) not in cache:
            e = cache[(name, dtype)] = Engine.from_pretrained(folders[name], dtype, max_tokens=max_tokens)
            assert e.use_graphs                           # every part's launches depend on the step's shape only
            e.routes = None
            if dtype == "bfloat16" or name == "D":
                e.use_graphs, e.routes, inner = False, [], e.ops.moe_sort

                def sort(chosen, *args, **kwargs):                    # (the launch that routes the rows and groups them)
                    inner(chosen, *args, **kwargs)
                    e.routes.append(chosen.clone())
                e.ops.moe_sort = sort
        return cache[(name, dtype)]
    return get


class Seq:
    """One request: its tokens, the rows the engine has answered, and (bfloat16) the experts it chose row by row, one
    array per routed feed-forward in the order they run."""

    def __init__(self, e, toks):
        self.e, self.toks, self.slot, self.at, self.got, self.routes = e, list(toks), e.open(), 0, {}, None

    def close(self):
        self.e.close(self.slot)


def step(e, parts):
    """One step of the engine: `parts` = [(seq, how many of its next tokens, wanted places among them)]."""
    if e.routes is not None:
        e.routes.clear()
    logits = e.step([StepEntry(q.slot, q.toks[q.at:q.at + n], list(want)) for q, n, want in parts]).cpu().numpy()
    row, first = 0, 0
    for q, n, want in parts:
        for wpos in want:
            q.got[q.at + wpos] = logits[row]
            row += 1
        if e.routes is not None:
            mine = [r[first:first + n].cpu().numpy() for r in e.routes]
            q.routes = mine if q.routes is None else [np.concatenate([a, b]) for a, b in zip(q.routes, mine)]
        first += n
        q.at += n


def verify(name, dtype, loaded, *seqs, scale=1.0):
    for q in seqs:
        toks = q.toks[:q.at]
        choices = None if q.routes is None else dict(zip(routed_layers(name), q.routes))
        ref = loaded[name].forward(toks, choices=choices)            # (None: the oracle's own choices)
        for p, row in q.got.items():
            e = rel_err(row, ref[p])
            assert e < TOL[dtype] * scale, (name, dtype, p, e)


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_prompts_from_one_token_to_several_pages(engine, loaded, name, dtype):
    e = engine(name, dtype)
    vocab = CONFIGS[name]["vocab"]
    for seed, n in ((1, 1), (2, 2), (3, 3), (4, 63), (5, 64), (6, 65), (7, 300)):
        q = Seq(e, random_tokens(seed, n, vocab))
        step(e, [(q, n, range(n))])
        q.close()
        verify(name, dtype, loaded, q)
    e.cache.book.check_all_free()


@pytest.mark.parametrize("name", SMALL)
def test_the_stream_after_every_layer(folders, loaded, name):
    """Layer by layer in 32-bit: what every block leaves in the residual stream (the sum it still owes taken up), for a
    prompt and for the token after it."""
    from kvad_b200.parts.block import flush_deferred
    e = Engine.from_pretrained(folders[name], "float32", max_tokens=512)
    e.use_graphs = False
    seen = []
    for blk in e.model.blocks:
        def wrap(inner):
            def forward(ctx, x, call):
                inner(ctx, x, call)
                flush_deferred(ctx)
                seen.append(x[:ctx.n_rows].cpu().numpy().copy())
            return forward
        blk.forward = wrap(blk.forward)
    toks = random_tokens(5, 75, CONFIGS[name]["vocab"])
    trace = {}
    loaded[name].forward(toks, trace=trace)
    s = e.open()
    e.step([StepEntry(s, toks[:74], [73])])
    e.step([StepEntry(s, toks[74:], [0])])
    e.close(s)
    n = len(CONFIGS[name]["layers"])
    assert len(seen) == 2 * n
    for i in range(n):
        assert rel_err(seen[i], trace["streams"][i][:74]) < TOL["float32"], (name, "prompt", i)
        assert rel_err(seen[n + i], trace["streams"][i][74:]) < TOL["float32"], (name, "token", i)


@pytest.mark.parametrize("name,dtype", CASES)
def test_prompt_then_token_by_token_across_pages_and_windows(engine, loaded, name, dtype):
    """Every window of the small configurations (1 to 200 positions) is passed while single tokens are decoded, pages
    fill up and are left behind."""
    e = engine(name, dtype)
    q = Seq(e, random_tokens(11, 290, CONFIGS[name]["vocab"]))
    step(e, [(q, 110, [0, 109])])
    for _ in range(110, 290):
        step(e, [(q, 1, [0])])
    q.close()
    verify(name, dtype, loaded, q)
    e.cache.book.check_all_free()


@pytest.mark.parametrize("name,dtype", CASES)
def test_decoding_from_the_first_token(engine, loaded, name, dtype):
    """No prompt to speak of: the state starts at zero, the first key is alone (both maps see one key: o = (1 - lam) v), and
    position 0 turns nothing; the windows fill up and start to drop keys token by token."""
    e = engine(name, dtype)
    q = Seq(e, random_tokens(12, 80, CONFIGS[name]["vocab"]))
    for _ in range(80):
        step(e, [(q, 1, [0])])
    q.close()
    verify(name, dtype, loaded, q)


@pytest.mark.parametrize("name,dtype", CASES)
@pytest.mark.parametrize("cuts", [[2, 2, 2, 58, 2, 3, 131], [64, 64, 64, 8], [1, 1, 126, 65, 7], [199, 1], [3, 1, 2, 1, 193]])
def test_portions_of_a_prompt(engine, loaded, name, dtype, cuts):
    e = engine(name, dtype)
    q = Seq(e, random_tokens(21, 200, CONFIGS[name]["vocab"]))
    for c in cuts:
        step(e, [(q, c, range(c))])
    q.close()
    verify(name, dtype, loaded, q)


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_batches_against_each_alone_and_slots_used_again(engine, loaded, name, dtype):
    e = engine(name, dtype)
    vocab = CONFIGS[name]["vocab"]
    lens = [1, 150, 37, 90]
    for rnd in range(2):                                   # the second round takes the slots and pages the first gave back
        seqs = [Seq(e, random_tokens(30 + i + 10 * rnd, n + 40, vocab)) for i, n in enumerate(lens)]
        step(e, [(q, n, [n - 1]) for q, n in zip(seqs, lens)])
        live = list(seqs)
        for j in range(40):
            if j == 10:                                    # a request ends early; the batch goes on without it
                seqs[2].close()
                live.remove(seqs[2])
            if j == 25:
                seqs[0].close()
                live.remove(seqs[0])
            step(e, [(q, 1, [0]) for q in live])
        for q in live:
            q.close()
        e.cache.book.check_all_free()
        verify(name, dtype, loaded, *seqs)


@pytest.mark.parametrize("name,dtype", CASES)
def test_batched_portions_of_unequal_prompts(engine, loaded, name, dtype):
    e = engine(name, dtype)
    vocab = CONFIGS[name]["vocab"]
    a, b = Seq(e, random_tokens(45, 180, vocab)), Seq(e, random_tokens(46, 100, vocab))
    for na, nb in ((70, 2), (2, 61), (58, 1), (1, 3), (40, 30)):
        step(e, [(a, na, [0, na - 1]), (b, nb, [nb - 1])])
    for _ in range(3):
        step(e, [(a, 1, [0]), (b, 1, [0])])
    a.close(), b.close()
    verify(name, dtype, loaded, a, b)
    e.cache.book.check_all_free()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_in_two_portions_then_a_batch_decoded_over_many_pages(engine, loaded, dtype):
    """The larger configuration: 1100 tokens (17 pages; the experts' products on the tensor cores in bfloat16) cut at a
    place that is no page's border, a second request joining for the decoding; windows of 70 to 513 positions that end
    hundreds of rows back, a decay of 0.999 that still carries the first rows."""
    e = engine("D", dtype, max_tokens=4096)
    vocab = CONFIGS["D"]["vocab"]
    a, b = Seq(e, random_tokens(95, 1140, vocab)), Seq(e, random_tokens(96, 240, vocab))
    step(e, [(a, 1000, [0, 1, 63, 64, 500, 999])])
    step(e, [(a, 100, [0, 27, 99]), (b, 200, [199])])
    for _ in range(40):
        step(e, [(a, 1, [0]), (b, 1, [0])])
    a.close(), b.close()
    verify("D", dtype, loaded, a, b, scale=3.0)      # (angles are 32-bit: a thousand positions on they are rounded to 1e-4 of a radian)
    e.cache.book.check_all_free()


@pytest.mark.parametrize("name", SMALL)
def test_the_routers_choices_are_the_oracles_where_its_margin_is_clear(engine, loaded, name):
    """bfloat16: with the engine's choices before it, the oracle chooses the same experts wherever the last chosen score is
    clear of the next one; the engine never takes an expert twice."""
    e = engine(name, "bfloat16")
    q = Seq(e, random_tokens(91, 150, CONFIGS[name]["vocab"]))
    step(e, [(q, 100, [])])
    for _ in range(50):
        step(e, [(q, 1, [])])
    q.close()
    layers = routed_layers(name)
    trace = {}
    loaded[name].forward(q.toks, choices=dict(zip(layers, q.routes)), trace=trace)
    assert len(q.routes) == len(layers) > 0
    seen = clear = 0
    for i, mine in zip(layers, q.routes):
        scores, _ = trace["routed"][i]
        top = mine.shape[1]
        own = plain.choose(scores, top)
        ranked = -np.sort(-scores, axis=-1)
        for t in range(len(q.toks)):
            seen += 1
            assert len(set(mine[t].tolist())) == top
            if top == scores.shape[1] or ranked[t, top - 1] - ranked[t, top] > MARGIN:
                clear += 1
                assert sorted(own[t].tolist()) == sorted(mine[t].tolist()), (i, t)
    assert clear > seen // 4


@pytest.mark.parametrize("name", SMALL)
def test_a_slot_used_again_starts_from_nothing(engine, oracle, name):
    """A sequence that takes the slot another one left must not see its state or its pages."""
    e = engine(name, "float32")
    vocab = CONFIGS[name]["vocab"]
    a, b = random_tokens(81, 90, vocab), random_tokens(82, 20, vocab)
    s = e.open()
    e.step([StepEntry(s, a, [])])
    e.close(s)
    s2 = e.open()
    assert s2 == s
    got = e.step([StepEntry(s2, b[:1], [0])]).cpu().numpy()          # one row first: the state must read as zeros
    got = np.concatenate([got, e.step([StepEntry(s2, b[1:], range(19))]).cpu().numpy()])
    e.close(s2)
    assert rel_err(got, oracle(name, b)) < TOL["float32"]


@pytest.mark.parametrize("name", SMALL)
def test_company_and_cutting_change_nothing_beyond_rounding_in_32_bit(engine, name):
    e = engine(name, "float32")
    vocab = CONFIGS[name]["vocab"]
    a, b = random_tokens(41, 140, vocab), random_tokens(42, 75, vocab)
    s = e.open()
    alone = e.step([StepEntry(s, a, [139])]).cpu().numpy()[0]
    e.close(s)
    sa, sb = e.open(), e.open()
    e.step([StepEntry(sa, a[:100], []), StepEntry(sb, b[:70], [])])
    e.step([StepEntry(sa, a[100:139], []), StepEntry(sb, b[70:74], [])])
    both = e.step([StepEntry(sa, [a[139]], [0]), StepEntry(sb, [b[74]], [0])]).cpu().numpy()[0]
    e.close(sa), e.close(sb)
    assert rel_err(both, alone) < 5e-6


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("C", "float32"), ("B", "bfloat16")])
def test_greedy_generation_through_the_entry_point(engine, loaded, name, dtype):
    e = engine(name, dtype)
    vocab = CONFIGS[name]["vocab"]
    prompts = [random_tokens(50, 9, vocab), random_tokens(51, 70, vocab), random_tokens(52, 1, vocab)]
    outs = e.generate(prompts, max_tokens=10, temperature=0.0, stop_token_ids=[])
    for p, o in zip(prompts, outs):
        assert len(o) == 10
        if dtype == "float32":
            ref = loaded[name].forward(list(p) + o)
            for j, tok in enumerate(o):                    # the chosen token is the oracle's, or ties with it to rounding
                row = ref[len(p) - 1 + j]
                assert row.max() - row[tok] <= 2 * TOL[dtype] * np.abs(row).max(), (j, tok, int(row.argmax()))
    if dtype == "float32":
        assert outs == [loaded[name].greedy(p, 10) for p in prompts]
        assert e.generate(prompts, max_tokens=10, temperature=0.0, stop_token_ids=[], batch_size=2) == outs
    e.cache.book.check_all_free()


def test_long_decoding_keeps_the_state_and_leaves_every_window_behind(engine, oracle):
    e = engine("A", "float32")
    toks = random_tokens(61, 600, CONFIGS["A"]["vocab"])
    ref = oracle("A", toks)
    s = e.open()
    e.step([StepEntry(s, toks[:5], [])])
    for p in range(5, 600):
        got = e.step([StepEntry(s, [toks[p]], [0])])
        if p % 50 == 0 or p > 590:
            assert rel_err(got.cpu().numpy()[0], ref[p]) < TOL["float32"], p
    e.close(s)
    e.cache.book.check_all_free()


def test_replay_runs_the_design_as_a_subprocess(folders, oracle, tmp_path):
    """bin/trace_run on a Dorevik folder: a batch of unequal prompts, then single tokens, one request ending early."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    vocab = CONFIGS["A"]["vocab"]
    a, b = random_tokens(71, 100, vocab), random_tokens(72, 30, vocab)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:90], "want": [0, 89]}, {"id": "b", "tokens": b[:25], "want": [24]}], "end": []}]
    for j in range(10):
        ents = [{"id": "a", "tokens": [a[90 + j]], "want": [0]}]
        if j < 5:
            ents.append({"id": "b", "tokens": [b[25 + j]], "want": [0]})
        steps.append({"step": j + 1, "entries": ents, "end": (["b"] if j == 4 else []) + (["a"] if j == 9 else [])})
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders["A"], "--dtype", "float32", "--out", str(out),
                           "--max-tokens", "130"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.split("\n") if l.startswith("done")] == [f"done {i}" for i in range(11)]
    ra, rb = oracle("A", a), oracle("A", b)
    first = np.fromfile(out / "0.f32", dtype="<f4").reshape(3, vocab)
    assert rel_err(first, np.stack([ra[0], ra[89], rb[24]])) < TOL["float32"]
    for j in range(10):
        got = np.fromfile(out / f"{j + 1}.f32", dtype="<f4").reshape(-1, vocab)
        assert rel_err(got[0], ra[90 + j]) < TOL["float32"]
        if j < 5:
            assert rel_err(got[1], rb[25 + j]) < TOL["float32"]


def test_command_line_writes_random_weights_and_generates(tmp_path):
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(CONFIGS["C"]))
    folder = tmp_path / "model"
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "kvad"), "run", "--model", str(folder), "--random-weights", str(cfg),
                           "--tokens", "5,17,3,99", "--max-tokens", "6", "--greedy", "--dtype", "f32", "--seed", "3"],
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = [int(t) for t in proc.stdout.strip().split(",")]
    assert got == plain.Dorevik.from_folder(str(folder)).greedy([5, 17, 3, 99], 6)
    assert "dorevik" in proc.stderr
