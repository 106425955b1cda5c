"""Dopipel without a GPU: its configuration, plan, tensor list, cache needs and run order (a repeated range of
layers has cache entries for every pass), random-weights mode, and the plain implementation's pieces against each other."""
import json

import numpy as np
import pytest
import torch

from kvad_b200 import write_random_model
from kvad_b200.cache import KVNeed, StateNeed
from kvad_b200.config import ConfigError, JsonView, load_config, resolve
from kvad_b200.models.plan import LayerCall, Model
from tests.dopipel_configs import CONFIGS, SEEDS
from tests.plain import dopipel_plain as pl


def build(folder):
    arch, cfg = load_config(folder)
    return cfg, Model(arch.plan(cfg))


def test_the_registry_finds_it_by_the_architecture_key():
    arch = resolve(JsonView(CONFIGS["A"]))
    assert arch.id == "dopipel"
    cfg = arch.read_config(JsonView(CONFIGS["A"]))
    assert (cfg.width, cfg.taps, cfg.loop) == (64, 2, (1, 3, 3))
    assert arch.read_config(JsonView(CONFIGS["D"])).taps == 0 and arch.read_config(JsonView(CONFIGS["B"])).loop is None


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_plan_asks_for_exactly_the_tensors_the_writer_writes(tmp_path, name):
    d = write_random_model(str(tmp_path), CONFIGS[name], SEEDS[name])
    cfg, model = build(d)
    stored = pl.read_tensors(str(tmp_path / "model.safetensors"))
    asked = {r.name: tuple(r.shape) for r in model.requests()}
    assert asked == {k: tuple(v.shape) for k, v in stored.items()}
    written = json.load(open(tmp_path / "config.json"))
    assert written["layers"] == CONFIGS[name]["layers"] and written.get("loop") == CONFIGS[name].get("loop")
    assert written.get("canon") == CONFIGS[name].get("canon")
    assert pl.forward(*pl.load(d), [1, 2, 3]).shape == (3, CONFIGS[name]["vocab"])


def test_every_pass_of_a_repeated_range_has_cache_entries_of_its_own(tmp_path):
    d = write_random_model(str(tmp_path), CONFIGS["A"], SEEDS["A"])
    _, model = build(d)
    # A: minGRU(48) | [attention(3 heads, 3 kv, 12, 20) | minGRU(80)] x 3 | attention(4 heads, 1 kv, 16, 8); two taps, 64 wide
    order = model.plan.order
    mix = len(CONFIGS["A"]["layers"])            # the step that opens a pass is the block after the layers
    assert [c.layer for c in order] == [0, mix, 1, 2, mix, 1, 2, mix, 1, 2, 3]
    assert [c.turn for c in order if c.layer == mix] == [0, 1, 2]
    runs = [c for c in order if c.layer != mix]
    assert [c.cache for c in runs] == list(range(0, 16, 2)) and [c.aux for c in runs] == list(range(1, 16, 2))
    needs = model.cache_layout.needs
    assert len(needs) == 16
    conv = StateNeed((64,), torch.float32)        # one kept input row
    assert needs[0] == StateNeed((48,), torch.float32) and all(n == conv for n in needs[1::2])
    for e in (2, 6, 10):
        assert needs[e] == KVNeed(3, 12, None, value_dim=20) and needs[e + 2] == StateNeed((80,), torch.float32)
    assert needs[14] == KVNeed(1, 16, None, value_dim=8)
    assert model.graph_safe and model.max_positions is None
    assert model.cache_layout.bytes_per_token(2) == 2 * (3 * 3 * (12 + 20) + 16 + 8)


def test_a_model_without_a_convolution_or_a_range_keeps_one_entry_a_layer(tmp_path):
    d = write_random_model(str(tmp_path), CONFIGS["D"], SEEDS["D"])
    _, model = build(d)
    # D: no taps; the range is layer 2 alone, run once: still opened by the mixing step
    assert [(c.layer, c.cache, c.aux) for c in model.plan.order] == [(0, 0, None), (1, 1, None), (4, -1, None), (2, 2, None), (3, 3, None)]
    d2 = write_random_model(str(tmp_path / "b"), CONFIGS["B"], SEEDS["B"])
    _, model = build(d2)
    assert [c.layer for c in model.plan.order] == [0, 1, 2, 3] and len(model.blocks) == 4


def test_libraries_are_those_of_the_models_parts():
    from kvad_b200.ops import libraries_for
    arch = resolve(JsonView(CONFIGS["A"]))
    fams = Model(arch.plan(arch.read_config(JsonView(CONFIGS["A"])))).kernel_families()
    libs = libraries_for(torch.bfloat16, fams)
    assert {"norm_rotary", "attention_scored", "channel_recurrence", "moe", "linear_tcgen05"} <= set(libs)
    assert not {"attention_prefill", "attention_decode", "attention_simt", "retention", "gated_recurrence"} & set(libs)
    # keys as long as values: bfloat16 prompts take the prompt kernel of the plain causal attention, 32-bit ones do not
    fams = Model(arch.plan(arch.read_config(JsonView(CONFIGS["F"])))).kernel_families()
    assert "attention_prefill" in libraries_for(torch.bfloat16, fams) and "attention_prefill" not in libraries_for(torch.float32, fams)
    assert not {"attention_decode", "attention_simt"} & set(libraries_for(torch.bfloat16, fams))


@pytest.mark.parametrize("change,what", [
    (lambda c: c["layers"][0].update(type="retention"), "type"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=2), "divide"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rotation"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=14), "rotation"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=5), "rotation"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"].pop("width"), "width"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=6), "experts"),
    (lambda c: c["layers"][0].update(mlp={"kind": "routed", "ff": 8}), "mlp"),
    (lambda c: c["loop"].update(stop=5), "range"),
    (lambda c: c["loop"].update(times=0), "times"),
    (lambda c: c["canon"].update(taps=40), "taps"),
    (lambda c: c.pop("norm"), "eps"),
])
def test_a_configuration_that_cannot_be_run_is_refused(change, what):
    cfg = json.loads(json.dumps(CONFIGS["A"]))
    change(cfg)
    arch = resolve(JsonView(cfg))
    with pytest.raises(ConfigError, match=what):
        arch.read_config(JsonView(cfg))


def test_plain_mechanisms_agree_with_each_other():
    """The oracle's own pieces, checked against each other where the design says two things are the same."""
    rng = np.random.default_rng(0)
    # a turn keeps lengths, position 0 turns nothing, what lies past `dims` passes, and turning back undoes it
    x = rng.standard_normal((5, 2, 8))
    y = pl.turn_pairs(x, np.arange(5), 100.0, 6)
    assert np.allclose((y ** 2).sum(-1), (x ** 2).sum(-1)) and np.array_equal(y[0], x[0]) and np.array_equal(y[..., 6:], x[..., 6:])
    assert np.allclose(pl.turn_pairs(y, np.arange(5), 100.0, 6, sign=-1.0), x)
    # neighbours are paired, the first pair turns by the position itself
    one = np.zeros((1, 1, 4))
    one[0, 0, 0] = 1.0
    assert np.allclose(pl.turn_pairs(one, [1], 100.0, 4)[0, 0], [np.cos(1.0), np.sin(1.0), 0.0, 0.0])
    # a convolution with one tap scales the row; with more, the last column meets the row itself and the first the oldest
    x, taps = rng.standard_normal((7, 3)), rng.standard_normal((3, 4))
    assert np.allclose(pl.input_convolution(x, taps[:, 3:]), x * (1 + taps[:, 3]))
    got = pl.input_convolution(x, taps)
    assert np.allclose(got[0], x[0] * (1 + taps[:, 3])) and np.allclose(got[1], x[1] * (1 + taps[:, 3]) + x[0] * taps[:, 2])
    assert np.allclose(got[5], x[5] + sum(taps[:, j] * x[5 - 3 + j] for j in range(4)))
    # the minGRU in two portions is the minGRU; a gate fully open takes the candidate, one shut keeps the state
    W = {"z": rng.standard_normal((6, 3)), "z.b": rng.standard_normal(6), "x": rng.standard_normal((6, 3)), "x.b": rng.standard_normal(6),
         "g": rng.standard_normal((6, 3)), "o": rng.standard_normal((3, 6))}
    whole, last = pl.min_gru(x, W, "")
    first, state = pl.min_gru(x[:3], W, "")
    rest, last2 = pl.min_gru(x[3:], W, "", state)
    assert np.allclose(np.concatenate([first, rest]), whole) and np.allclose(last, last2)
    shut = dict(W, **{"z": np.zeros((6, 3)), "z.b": np.full(6, -60.0)})
    assert np.allclose(pl.min_gru(x, shut, "", state)[1], state)
    wide = dict(W, **{"z": np.zeros((6, 3)), "z.b": np.full(6, 60.0), "x": np.zeros((6, 3)), "x.b": np.array([2.0, 0.0, -1.0, 3.0, -4.0, 0.5])})
    assert np.allclose(pl.min_gru(x, wide, "")[1], [2.5, 0.5, pl.sigmoid(-1.0), 3.5, pl.sigmoid(-4.0), 1.0])
    # attention over one row: position 0 turns nothing, the only weight is 1: the row's own values, gated head by head
    m = {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 6, "scale": 0.5, "rot": {"base": 50.0, "dims": 4}}
    A = {k: rng.standard_normal(s) for k, s in (("q", (8, 3)), ("q.b", 8), ("k", (4, 3)), ("k.b", 4), ("v", (6, 3)), ("v.b", 6), ("g", (2, 3)),
                                                ("o", (3, 12)), ("o.b", 3))}
    h = rng.standard_normal((6, 3))
    alone = pl.rotated_value_attention(h[:1], A, "", m)
    assert np.allclose(alone[0], (np.tile(h[0] @ A["v"].T + A["v.b"], 2) * np.repeat(pl.sigmoid(h[0] @ A["g"].T), 6)) @ A["o"].T + A["o.b"])
    # the router: weights sum to one; all routes chosen: the scores themselves; the correction moves the choice, not the weights
    R = {"router": rng.standard_normal((5, 3)), "correction": np.zeros(5)}
    c, w, s, _ = pl.route(h, R, "", 2)
    assert np.allclose(w.sum(-1), 1.0) and np.array_equal(c[:, 0], s.argmax(-1))
    c5, w5, _, _ = pl.route(h, R, "", 5)
    assert np.allclose(np.take_along_axis(s, c5, -1), w5)
    R2 = dict(R, correction=np.array([0.0, 0.0, 0.0, 0.0, 9.0]))
    c2, w2, s2, _ = pl.route(h, R2, "", 2)
    assert np.all(c2[:, 0] == 4) and np.allclose(s2, s) and np.allclose(w2[:, 0], s[:, 4] / (s[:, 4] + np.take_along_axis(s, c2[:, 1:], -1)[:, 0]))
    # identity experts alone with every route chosen: the mixture is its input
    mlp = {"router": {"experts": 0, "identity": 5, "top": 5}}
    assert np.allclose(pl.mixture(h, R, "", mlp), h)
    # the order in which a repeated range runs
    assert [(i, t) for i, t, _ in pl.run_order(CONFIGS["A"])] == [(0, None), (1, 0), (2, 0), (1, 1), (2, 1), (1, 2), (2, 2), (3, None)]
    assert [f for _, _, f in pl.run_order(CONFIGS["A"])] == [False, True, False, True, False, True, False, False]
