"""The Fudelorn design on the host: its configuration, its layout as parts, the stretch of rotary frequencies against the
plain implementation's, random tables, and the plain implementation's own mask and attention against brute force."""

from __future__ import annotations

import copy
import math

import numpy as np
import pytest

import plain_fudelorn as pf
from borrowed_compute_b200.config import ConfigError
from borrowed_compute_b200.config.fudelorn import DenseConfig, FudelornConfig, TableExpertsConfig
from borrowed_compute_b200.engine.model import model_for_config


def test_the_architecture_is_registered_and_declares_the_tensors_of_the_format():
    for name in "AB":
        cfg = pf.SMALL[name]
        typed, model = model_for_config(cfg)
        assert isinstance(typed, FudelornConfig)
        want = pf.make_weights(cfg, 1)
        have = model.expected_tensors()
        assert set(have) == set(want)
        assert all(tuple(have[n].shape) == want[n].shape for n in want)
        assert have["l1.mlp.table" if name == "A" else "l0.mlp.table"].role == "index"
    typed, model = model_for_config(pf.SMALL["A"])
    assert isinstance(typed.layers[0].mlp, DenseConfig) and isinstance(typed.layers[1].mlp, TableExpertsConfig) and typed.layers[3].mlp is None
    assert "l3.mix.dkv" not in model.expected_tensors() and "l3.norm2" not in model.expected_tensors()


def test_a_layer_that_reads_another_layers_cache_owns_none():
    _, model = model_for_config(pf.SMALL["A"])
    needs, states, memory_of = model.memory_needs()
    assert memory_of == [None, None, None, 1] and states == [None] * 4
    assert needs[1].planes == ((1, 72), (1, 8)) and needs[1].window == 0
    assert needs[0].planes == ((1, 48),) and needs[0].window == 5 and needs[2].window == 70


@pytest.mark.parametrize("change, match", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
    (lambda c: c["layers"][0].update(type="attention"), r"layers\[0\].type"),
    (lambda c: c["layers"][0]["mixer"].pop("mask"), r"layers\[0\].mixer.mask"),
    (lambda c: c["layers"][0]["mixer"].update(rot_dim=4), "without positions"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), r"layers\[1\].mixer.kv_rank"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=6), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].pop("fast"), "scaling.fast"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "router.top"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=0), "kv_rank, rot_dim and rotation"),
    (lambda c: c["layers"][3]["mixer"].update(kv_rank=64), "kv_rank, rot_dim and rotation"),
    (lambda c: c["layers"][2].update(mlp={"kind": "gated", "ff": 8}), r"layers\[2\].mlp.kind"),
])
def test_configuration_errors_name_the_key(change, match):
    cfg = copy.deepcopy(pf.SMALL["A"])
    change(cfg)
    with pytest.raises(ConfigError, match=match):
        model_for_config(cfg)


def test_defaults_of_keys_that_a_file_may_leave_out():
    cfg = copy.deepcopy(pf.SMALL["A"])
    for i in (0, 1):
        cfg["layers"][i]["mixer"].pop("scale")
        cfg["layers"][i]["mixer"].pop("vdim")
    cfg["layers"][1]["mixer"]["rot"].pop("scaling")
    cfg["layers"][3]["mixer"]["rot"].pop("scaling")
    typed, _ = model_for_config(cfg)
    assert typed.layers[0].mixer.scale == pytest.approx(16 ** -0.5) and typed.layers[0].mixer.vdim == 16
    assert typed.layers[1].mixer.scale == pytest.approx(40 ** -0.5) and typed.layers[1].mixer.stretch is None


@pytest.mark.parametrize("dims, base, scaling", [
    (16, 500000.0, {"factor": 8.0, "original": 512, "fast": 32.0, "slow": 1.0}),
    (8, 10000.0, {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}),
    (64, 10000.0, {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}),
    (4, 100.0, {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 0.5}),
    (6, 10000.0, {"factor": 3.0, "original": 8, "fast": 0.5, "slow": 0.25}),       # both edges clamp: lo = hi
    (8, 10000.0, None),
])
def test_the_stretched_frequencies_and_the_tables_factor(dims, base, scaling):
    from borrowed_compute_b200.parts.rope import inverse_frequencies, rotary_table, table_magnitude

    named = None if scaling is None else dict(scaling, type="yarn")
    f, m = pf.stretched_frequencies(dims, base, scaling)
    got = inverse_frequencies(dims, base, named).numpy()
    assert np.allclose(got, f, rtol=1e-6, atol=0)
    assert table_magnitude(named) == pytest.approx(m)
    if scaling is not None:
        ramp = (base ** (-2.0 * np.arange(dims // 2) / dims) - f) / (base ** (-2.0 * np.arange(dims // 2) / dims) * (1 - 1 / scaling["factor"]))
        assert (np.diff(ramp) >= -1e-12).all() and ramp.min() >= -1e-12 and ramp.max() <= 1 + 1e-12      # fast pairs keep, slow pairs stretch
    table = rotary_table(inverse_frequencies(dims, base, named), 40, table_magnitude(named)).numpy().astype(np.float64)
    a = np.arange(40)[:, None] * f[None, :]
    assert np.allclose(table[..., 0], np.cos(a) * m, atol=2e-5) and np.allclose(table[..., 1], np.sin(a) * m, atol=2e-5)


def test_an_unknown_stretch_is_refused_when_the_part_is_built():
    from borrowed_compute_b200.parts.rope import RotaryEncoding

    with pytest.raises(ValueError, match="not known"):
        RotaryEncoding(8, 10000.0, scaling={"type": "elastic", "factor": 2.0})
    with pytest.raises(ValueError, match="yarn"):
        RotaryEncoding(8, 10000.0, scaling={"type": "yarn", "factor": 2.0})


def test_random_tables_name_different_experts_in_every_row():
    from borrowed_compute_b200.weights.random_init import random_tensors

    for name in "AB":
        _, model = model_for_config(pf.SMALL[name])
        made = random_tensors(model.expected_tensors(), 5, __import__("torch").float32)
        for n, t in made.items():
            if n.endswith("mlp.table"):
                layer = pf.SMALL[name]["layers"][int(n[1:n.index(".")])]
                E = layer["mlp"]["router"]["experts"]
                rows = t.numpy()
                assert rows.min() >= 0 and rows.max() < E
                assert all(len(set(r)) == len(r) for r in rows.tolist())
                assert len(np.unique(rows[:, 0])) == E        # every expert is somebody's first


def test_the_plain_mask_and_attention_against_brute_force():
    rng = np.random.default_rng(3)
    assert pf.visible(4, 0).tolist() == [[j <= i for j in range(4)] for i in range(4)]
    assert pf.visible(5, 2).tolist() == [[0 <= i - j < 2 for j in range(5)] for i in range(5)]
    assert pf.visible(3, 1).tolist() == [[i == j for j in range(3)] for i in range(3)]
    # One head, by hand: keys and values from the latent, the rotated part shared, gate and output last.
    m = pf._rotated(1, 4, 3, 5, 6, 2, 100.0, {"factor": 2.0, "original": 4, "fast": 2.0, "slow": 0.5}, scale=0.7)
    E, T = 8, 6
    w = {"dq": rng.standard_normal((5, E)), "dq.norm": rng.uniform(0.5, 1.5, 5), "uq": rng.standard_normal((6, 5)), "dkv": rng.standard_normal((8, E)),
         "dkv.norm": rng.uniform(0.5, 1.5, 6), "uk": rng.standard_normal((4, 6)), "uv": rng.standard_normal((3, 6)), "g": rng.standard_normal((1, E)),
         "o": rng.standard_normal((E, 3))}
    h = rng.standard_normal((T, E))
    got, (c, kr) = pf.latent_attention(h, w, m, 1e-5)
    f, mag = pf.stretched_frequencies(2, 100.0, m["rot"]["scaling"])
    for i in range(T):
        zq = w["dq"] @ h[i]
        q = w["uq"] @ (zq / math.sqrt((zq ** 2).mean() + 1e-5) * w["dq.norm"])
        ai = i * f[0]
        qr = np.array([q[4] * math.cos(ai) - q[5] * math.sin(ai), q[5] * math.cos(ai) + q[4] * math.sin(ai)]) * mag
        scores = np.array([(q[:4] @ (w["uk"] @ c[j]) + qr @ kr[j]) * 0.7 for j in range(i + 1)])
        p = np.exp(scores - scores.max())
        p /= p.sum()
        o = sum(p[j] * (w["uv"] @ c[j]) for j in range(i + 1)) / (1.0 + math.exp(-(w["g"] @ h[i])[0]))
        assert np.allclose(got[i], w["o"] @ o, atol=1e-10)


def test_a_step_of_the_plain_model_does_not_depend_on_later_tokens():
    cfg = pf.SMALL["A"]
    w = pf.make_weights(cfg, 2)
    toks = [int(t) for t in np.random.default_rng(0).integers(0, cfg["vocab"], 12)]
    whole = pf.forward(cfg, w, toks)
    assert np.allclose(pf.forward(cfg, w, toks[:7]), whole[:7], atol=1e-10)
