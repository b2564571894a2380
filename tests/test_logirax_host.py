"""Logirax on the host: its configuration and the errors it names, the layout of parts against the tensors the plain
implementation expects, what the cache is asked for, and the slot table's pages when a window keeps a sequence's first positions."""

from __future__ import annotations

import copy

import pytest

import plain_logirax as pl
from borrowed_compute_b200.cache.slots import PAGE, GroupPlan, SlotTable
from borrowed_compute_b200.config import ConfigError, LogiraxConfig
from borrowed_compute_b200.engine.model import model_for_config


@pytest.mark.parametrize("name", ["A", "B"])
def test_the_layout_asks_for_exactly_the_tensors_of_the_plain_model(name):
    cfg = pl.SMALL[name]
    _, model = model_for_config(cfg)
    want = {n: s for n, s in model.expected_tensors().items() if not s.optional}
    shapes = pl.tensor_shapes(cfg)
    assert {n: tuple(s.shape) for n, s in want.items()} == {n: tuple(s) for n, s in shapes.items()}
    assert all(want[n].role == "vector" for n in want if n.endswith((".temp", ".talk", ".sink", ".shift", ".router", ".b")) or "norm" in n)


def test_every_size_and_constant_comes_from_the_file():
    typed = LogiraxConfig.from_dict(pl.SMALL["B"])
    assert (typed.vocab, typed.width, typed.norm_eps, typed.embedding_scale, typed.logit_scale) == (97, 40, 1e-6, 1.0, 3.0)
    lat, talk6, talk3 = (layer.mixer for layer in typed.layers)
    assert (lat.heads, lat.dim, lat.vdim, lat.q_rank, lat.kv_rank, lat.rot_dim) == (2, 8, 8, 16, 16, 0)
    assert (talk6.heads, talk6.kv_heads, talk6.dim, talk6.window, talk6.keep_first, talk6.rot_dims, talk6.softcap, talk6.rot_base) == (6, 6, 20, 70, 0, 20, 0.0, 300.0)
    assert (talk3.heads, talk3.kv_heads, talk3.window, talk3.keep_first, talk3.rot_dims, talk3.softcap) == (3, 1, 9, 70, 0, 4.0)
    moe3, dense, moe5 = (layer.mlp for layer in typed.layers)
    assert (moe3.experts, moe3.top, moe3.ff, moe3.shared_ff, moe3.weight_scale) == (3, 3, 8, 0, 1.0)
    assert (dense.ff, dense.limit) == (24, 0.5)
    assert (moe5.experts, moe5.top, moe5.shared_ff, moe5.weight_scale) == (5, 1, 8, 2.5)
    assert LogiraxConfig.from_dict(pl.SMALL["A"]).layers[2].mlp is None


def broken(change):
    cfg = copy.deepcopy(pl.SMALL["A"])
    change(cfg)
    return cfg


@pytest.mark.parametrize("change,names", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c.pop("norm"), "norm.eps"),
    (lambda c: c["layers"][0].update(type="convolution"), "layers[0].type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "layers[0].mixer.heads"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=24), "layers[0].mixer.vdim"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "layers[0].mixer.rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["mask"].pop("size"), "layers[0].mixer.mask.size"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=4), "layers[1].mixer.rot.dims"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "layers[1].mixer.kv_rank"),
    (lambda c: c["layers"][1]["mlp"].pop("limit"), "layers[1].mlp.limit"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "layers[0].mlp.router.top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "layers[0].mlp.kind"),
])
def test_a_wrong_configuration_is_refused_with_the_key_named(change, names):
    with pytest.raises(ConfigError) as e:
        LogiraxConfig.from_dict(broken(change))
    assert names in str(e.value)


def test_what_the_cache_is_asked_for():
    _, model = model_for_config(pl.SMALL["A"])
    needs, states, memory_of = model.memory_needs()
    assert [n.planes for n in needs] == [((2, 16), (2, 16)), ((1, 40), (1, 8)), ((2, 16), (2, 16)), ((1, 40), (1, 8))]
    assert [(n.window, n.keep_first) for n in needs] == [(24, 3), (0, 0), (24, 3), (0, 0)]
    assert states == [None] * 4 and memory_of == [None] * 4
    # every layer keeps the mixer's last input: the token shift's state
    assert [sorted(m) for m in model.more_state_needs()] == [["conv"]] * 4
    assert all(m["conv"].shape == (1, 64) for m in model.more_state_needs())


def test_the_token_shift_is_a_convolution_of_two_taps():
    import numpy as np
    import torch

    from borrowed_compute_b200.parts import CONVOLUTIONS, Runtime

    part = CONVOLUTIONS.get("token_shift")(width=5, tensor="shift")
    assert part.taps == 2 and part.tensors()["shift"].shape == (5,)
    s = torch.tensor([0.0, 1.0, 0.25, -0.5, 0.75])
    part.load({"shift": s}, Runtime(torch.device("cpu"), torch.float32))
    h = torch.tensor(np.random.default_rng(0).standard_normal((4, 5)), dtype=torch.float32)
    before = torch.cat([torch.zeros(1, 5), h[:-1]])
    taps = h + part.weight_t[0] * before + part.weight_t[1] * h
    assert torch.allclose(taps, h + (before - h) * s, atol=1e-6)


def pages_held(table, slot, g=0):
    return [i for i, p in enumerate(table.tables[g][slot]) if p >= 0]


@pytest.mark.parametrize("window,keep,want_kept", [(10, 4, [0]), (10, 64, [0]), (10, 65, [0, 1]), (10, 0, []), (200, 3, [0])])
def test_pages_of_the_first_positions_are_never_let_go(window, keep, want_kept):
    table = SlotTable(n_slots=2, n_pages=64, max_seq=64 * PAGE, groups=[GroupPlan(window=window, keep_first=keep), GroupPlan()])
    s = table.acquire()
    table.reserve(s, 300, rows=300)
    table.commit(s, 300)
    assert pages_held(table, s) == list(range(5)) and pages_held(table, s, 1) == list(range(5))
    for n in range(301, 1200):
        table.reserve(s, n, rows=1)
        table.commit(s, n)
        first = max(0, n - window) // PAGE
        assert pages_held(table, s) == sorted(set(want_kept) | set(range(first, (n - 1) // PAGE + 1))), n
        table.check()
    assert len(pages_held(table, s, 1)) == -(-1199 // PAGE)
    # a prompt step that jumps far ahead lets go of everything between the kept pages and its window at once
    t = table.acquire()
    table.reserve(t, 1000, rows=1000)
    table.commit(t, 1000)
    table.reserve(t, 1001, rows=1)
    assert pages_held(table, t) == sorted(set(want_kept) | set(range((1001 - window) // PAGE, 1000 // PAGE + 1)))
    table.release(s), table.release(t)
    table.check()
    assert table.pools[0].available == 64
