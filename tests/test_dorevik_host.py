"""Dorevik without a GPU: its configuration, plan, tensor list, cache needs and run order, refusals, the stretched
rotary frequencies of the part against the plain implementation's, random-weights mode, and the plain
implementation's pieces against each other."""
import copy
import json
import math

import numpy as np
import pytest
import torch

from kvad_b200 import write_random_model
from kvad_b200.cache import KVNeed, StateNeed
from kvad_b200.config import ConfigError, JsonView, load_config, resolve
from kvad_b200.models.plan import Model
from kvad_b200.parts.positions import Rotary
from tests.dorevik_configs import CONFIGS, SEEDS
from tests.plain import dorevik_plain as pl


def build(folder):
    arch, cfg = load_config(folder)
    return cfg, Model(arch.plan(cfg))


def test_the_registry_finds_it_by_the_architecture_key():
    arch = resolve(JsonView(CONFIGS["A"]))
    assert arch.id == "dorevik"
    cfg = arch.read_config(JsonView(CONFIGS["A"]))
    assert (cfg.width, cfg.vocab, cfg.logit_softcap, cfg.norm_eps) == (64, 257, 30.0, 1e-5)
    assert arch.read_config(JsonView(CONFIGS["B"])).logit_softcap is None


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_plan_asks_for_exactly_the_tensors_the_writer_writes(tmp_path, name):
    d = write_random_model(str(tmp_path), CONFIGS[name], SEEDS[name])
    cfg, model = build(d)
    stored = pl.read_tensors(str(tmp_path / "model.safetensors"))
    asked = {r.name: tuple(r.shape) for r in model.requests()}
    assert asked == {k: tuple(v.shape) for k, v in stored.items()}
    written = json.load(open(tmp_path / "config.json"))
    assert written["layers"] == CONFIGS[name]["layers"] and written.get("logit_softcap") == CONFIGS[name].get("logit_softcap")
    assert pl.Dorevik.from_folder(d).forward([1, 2, 3]).shape == (3, CONFIGS[name]["vocab"])


def test_two_mixers_side_by_side_have_a_cache_entry_each_and_maps_share_their_values():
    arch = resolve(JsonView(CONFIGS["A"]))
    model = Model(arch.plan(arch.read_config(JsonView(CONFIGS["A"]))))
    # A: [windowed attention (4 heads over 2, keys 16, values 8, window 7) | linear attention (3 heads, 8 x 12)], then two differential layers
    order = model.plan.order
    assert [(c.layer, c.cache, c.aux) for c in order] == [(0, 0, 1), (1, 2, None), (2, 3, None)]
    needs = model.cache_layout.needs
    assert needs[0] == KVNeed(2, 16, 7, value_dim=8) and needs[1] == StateNeed((3, 8, 12), torch.float32)
    assert needs[2] == KVNeed(4, 8, 33, value_dim=16, value_heads=2)          # two maps per key/value head, one copy of the values
    assert needs[3] == KVNeed(4, 8, 5, value_dim=8, value_heads=2)
    assert needs[2].v_heads == 2 and needs[0].v_heads == 2
    assert model.graph_safe and model.max_positions is None
    assert set(model.kernel_families()) == {"norm_rotary", "scored_attention", "retention", "moe"}
    # a key/value head per head where config.json leaves `kv_heads` out
    arch_c = resolve(JsonView(CONFIGS["C"]))
    assert Model(arch_c.plan(arch_c.read_config(JsonView(CONFIGS["C"])))).cache_layout.needs[0] == KVNeed(6, 6, 3, value_dim=10, value_heads=3)


def test_the_cache_counts_the_shared_values_once():
    arch = resolve(JsonView(CONFIGS["A"]))
    layout = Model(arch.plan(arch.read_config(JsonView(CONFIGS["A"])))).cache_layout
    assert layout.bytes_per_token(2) == 2 * ((2 * 16 + 2 * 8) + (4 * 8 + 2 * 16) + (4 * 8 + 2 * 8))
    with pytest.raises(ValueError):
        KVNeed(4, 8, None, value_heads=3)


@pytest.mark.parametrize("change,what", [
    (lambda c: c["layers"][0].update(type="mamba"), "type"),
    (lambda c: c["layers"][1]["mixer"].pop("diff"), "diff"),
    (lambda c: c["layers"][1]["mixer"]["mask"].pop("size"), "size"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=10), "rotation"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=3), "rotation"),
    (lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.5, 0.9]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "divide"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "experts"),
    (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "kind"),
    (lambda c: c.update(logit_softcap=-1.0), "logit_softcap"),
    (lambda c: c.pop("norm"), "eps"),
])
def test_configurations_that_are_refused_say_where(change, what):
    c = copy.deepcopy(CONFIGS["A"])
    change(c)
    arch = resolve(JsonView(c))
    with pytest.raises(ConfigError) as err:
        arch.read_config(JsonView(c))
    assert what in str(err.value)


@pytest.mark.parametrize("rot", [
    {"base": 3e4, "dims": 12, "scaling": {"factor": 6.0, "original": 512, "fast": 24.0, "slow": 2.0}},
    {"base": 1e4, "dims": 4, "scaling": {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}},
    {"base": 300.0, "dims": 12, "scaling": {"factor": 3.0, "original": 40, "fast": 10.0, "slow": 1.0}},
    {"base": 1e6, "dims": 64}])
def test_stretched_frequencies_of_the_part_are_the_plain_ones(rot):
    part = Rotary("", dims=rot["dims"], base=rot["base"], layout="half", scaling=rot.get("scaling"))

    def fetch(*a, **k):
        raise AssertionError("a rotary encoding reads no tensor")
    fetch.device = "cpu"
    part.load_own(fetch)
    f, m = pl.rotary_frequencies(rot)
    assert np.allclose(part.inv_freq.numpy(), f, rtol=2e-7, atol=0) and abs(part.mscale - m) < 1e-12
    if "scaling" in rot:
        plain = rot["base"] ** (-2.0 * np.arange(rot["dims"] // 2) / rot["dims"])
        assert np.all(f <= plain * (1 + 1e-12)) and np.all(f >= plain / rot["scaling"]["factor"] * (1 - 1e-12))
        assert f[-1] < plain[-1] or rot["dims"] <= 4          # the slowest pair is stretched
        assert m == 0.1 * math.log(rot["scaling"]["factor"]) + 1.0
    with pytest.raises(ValueError):
        Rotary("", dims=8, base=100.0, scaling={"factor": 2.0, "original": 16, "fast": 4.0})


def test_plain_pieces_agree_with_each_other():
    rng = np.random.default_rng(0)
    # a window as long as the sequence is no window; a window of 1 reads the row's own value
    q, k, v = rng.standard_normal((9, 4, 6)), rng.standard_normal((9, 2, 6)), rng.standard_normal((9, 2, 5))
    full = pl.softmax_attention(q, k, v, 0.4, 9)
    assert np.allclose(full, pl.softmax_attention(q, k, v, 0.4, 1000))
    own = pl.softmax_attention(q, k, v, 0.4, 1)
    assert np.allclose(own[:, 0], v[:, 0]) and np.allclose(own[:, 3], v[:, 1])
    assert pl.window_mask(5, 2).sum() == 9
    # turning by position 0 changes nothing but the factor; turning keeps the pairs' lengths (times the factor)
    rot = {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 0.5}}
    x = rng.standard_normal((3, 2, 6))
    t = pl.turn_halves(x, [0, 5, 9], rot)
    m = 0.1 * math.log(2.0) + 1.0
    assert np.allclose(t[0, :, :4], x[0, :, :4] * m) and np.allclose(t[..., 4:], x[..., 4:])
    assert np.allclose(t[..., 0] ** 2 + t[..., 2] ** 2, (x[..., 0] ** 2 + x[..., 2] ** 2) * m * m)
    # scores that depend on the distance only: q_i . k_j after turning equals q_0 . k_(j-i) turned
    plain_rot = {"base": 100.0, "dims": 6}
    a, b = rng.standard_normal((1, 1, 6)), rng.standard_normal((1, 1, 6))
    s1 = (pl.turn_halves(a, [7], plain_rot) * pl.turn_halves(b, [4], plain_rot)).sum()
    s2 = (pl.turn_halves(a, [3], plain_rot) * pl.turn_halves(b, [0], plain_rot)).sum()
    assert abs(s1 - s2) < 1e-12
    # an expert on a scaled input is not the scaled expert (the gate is not linear)
    w = {"e.gate": rng.standard_normal((5, 4)), "e.up": rng.standard_normal((5, 4)), "e.down": rng.standard_normal((4, 5))}
    h = rng.standard_normal((2, 4))
    assert not np.allclose(pl.gated_ff(0.3 * h, w, "e.", pl.silu), 0.3 * pl.gated_ff(h, w, "e.", pl.silu))
    assert pl.choose(np.array([[0.5, 0.7, 0.7, 0.1]]), 2).tolist() == [[1, 2]]
    assert abs(pl.gelu_tanh(np.float64(1.0)) - 0.8411919906082768) < 1e-12


def test_greedy_of_the_plain_implementation_follows_its_logits(tmp_path):
    d = write_random_model(str(tmp_path), CONFIGS["C"], SEEDS["C"])
    m = pl.Dorevik.from_folder(d)
    out = m.greedy([4, 9], 3)
    assert out[0] == int(np.argmax(m.forward([4, 9])[-1])) and len(out) == 3
    cap = CONFIGS["C"]["logit_softcap"]
    assert np.abs(m.forward([4, 9, 11])).max() < cap
