"""The Logirax decoder on the engine against the plain implementation (plain_logirax.py): each new mechanism alone through its
kernels, then whole models through the engine's step function, cache, scheduler and entry points: whole prompts, token-by-token
decoding, portions down to two tokens, unequal batches, slots and pages used again, keys at the edges of windows, of the kept
first positions and of pages, and far away, the first tokens, long decoding, drawn configurations, and greedy generation.

The attention whose heads talk is run on inputs and weights made so that ONE position's key wins every softmax that sees it: a
mask that is one position off then changes whole rows.

float32 engines are held to the float64 oracle tightly (1e-4 (1 + max|score|)), bfloat16 ones within 6e-2 (1 + max|score|)."""

from __future__ import annotations

import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_logirax as pl
from conftest import BF16_TOL, F32_TOL, ROOT

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]


def tol(dtype, ref):
    return (F32_TOL if dtype == "float32" else 2 * BF16_TOL) * (1.0 + float(np.abs(ref).max()))


def close(got, ref, dtype, what=""):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: {got.shape} against {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: not finite"
    worst = np.abs(got - ref).reshape(got.shape[0], -1).max(axis=-1)
    assert worst.max() <= tol(dtype, ref), f"{what}: row {int(worst.argmax())} differs by {worst.max():.4g} (allowed {tol(dtype, ref):.4g})"


def mostly_close(got, ref, dtype, what=""):
    """Whole bfloat16 models: a sublayer's result passes a norm before it joins the stream, which magnifies the rounding of a small
    result, and a router may choose another expert where two scores lie within rounding.  Nine rows in ten are held to the
    tolerance and the median row to a third of it; a wrong key, window or state moves every row that follows."""
    if dtype == "float32":
        return close(got, ref, dtype, what)
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape and np.isfinite(got).all(), f"{what}: shape or numbers"
    worst = np.abs(got - ref).reshape(got.shape[0], -1).max(axis=-1)
    assert np.quantile(worst, 0.9) <= tol(dtype, ref) and np.median(worst) <= tol(dtype, ref) / 3, \
        f"{what}: the 90th percentile of the rows differs by {np.quantile(worst, 0.9):.4g}, the median by {np.median(worst):.4g} (allowed {tol(dtype, ref):.4g})"


def tokens_for(cfg, w, n, seed=0):
    """n tokens on which the routers choose by the widest margin among a few draws."""
    draws = [[int(t) for t in np.random.default_rng(seed * 100 + i).integers(0, cfg["vocab"], n)] for i in range(6)]
    return max(draws, key=lambda toks: pl.router_margin(cfg, w, toks[: min(n, 48)]))


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    return t if dtype is None else t.to(dtype)


def engine_for(cfg, weights, dtype, **kw):
    from borrowed_compute_b200.engine import Engine

    kw.setdefault("max_tokens", 4096)
    kw.setdefault("max_slots", 6)
    kw.setdefault("max_seq", 1024)
    return Engine.from_tensors(cfg, {n: torch.from_numpy(np.ascontiguousarray(a)) for n, a in weights.items()}, dtype=dtype, **kw)


_made = {}


def small(name, dtype):
    key = (name, dtype)
    if key not in _made:
        cfg = pl.SMALL[name]
        w = pl.make_weights(cfg, seed=31 if name == "A" else 32)
        _made[key] = (engine_for(cfg, w, dtype), cfg, w)
    return _made[key]


def run_whole(eng, toks):
    from borrowed_compute_b200.engine import StepEntry

    s = eng.acquire()
    out = eng.step([StepEntry(s, toks, tuple(range(len(toks))))]).cpu().numpy()
    eng.release(s)
    return out


def run_cut(eng, toks, cuts):
    """The same tokens in portions of the given sizes (the rest one token at a time)."""
    from borrowed_compute_b200.engine import StepEntry

    s, at, rows = eng.acquire(), 0, []
    for n in list(cuts) + [1] * len(toks):
        if at >= len(toks):
            break
        part = toks[at:at + n]
        rows.append(eng.step([StepEntry(s, part, tuple(range(len(part))))]).cpu().numpy())
        at += len(part)
    eng.release(s)
    return np.concatenate(rows)


@pytest.fixture(autouse=True)
def _the_parts_choose_again():
    from borrowed_compute_b200.parts import latent_attention, talking_attention

    yield
    latent_attention.force = None
    talking_attention.force = None


# ------------------------------------------------------------------ each mechanism alone

def context(entries, starts):
    """A StepContext on the device for parts run outside an engine."""
    from borrowed_compute_b200.engine.batch import plan_step
    from borrowed_compute_b200.parts import StepContext

    p = plan_step(entries, starts)
    return StepContext(rows=p.rows, seqs=p.seqs, tokens=dev(p.tokens), row_pos=dev(p.row_pos), row_slot=dev(p.row_slot),
                       seq_rows=dev(p.seq_rows), seq_slot=dev(p.seq_slot), seq_start=dev(p.seq_start), max_new=p.max_new,
                       max_total=p.max_total, decode=p.decode, host_seq_rows=tuple(int(x) for x in p.seq_rows),
                       host_seq_slot=tuple(int(x) for x in p.seq_slot), host_seq_start=tuple(int(x) for x in p.seq_start))


def load_part(part, w, dtype, prefix=""):
    from borrowed_compute_b200.parts import Runtime

    rt = Runtime(torch.device(DEV), dtype, max_positions=1024)
    part.load({k: dev(w[prefix + k], torch.float32 if s.role == "vector" else dtype) for k, s in part.tensors().items()}, rt)
    return rt


def torch_type(dtype):
    return torch.float32 if dtype == "float32" else torch.bfloat16


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E", [8, 40, 250])
def test_norm_with_a_weight_stored_around_zero(dtype, E):
    from borrowed_compute_b200.parts import NORMS

    rng = np.random.default_rng(E)
    w = {"n": pl.to_bf16(0.3 * rng.standard_normal(E))}
    part = NORMS.get("rmsnorm")(size=E, eps=1e-3, tensor="n", offset=1.0)
    load_part(part, w, torch_type(dtype))
    x = rng.standard_normal((7, E)) * 3.0
    out = torch.empty((7, E), dtype=torch_type(dtype), device=DEV)
    part.forward(dev(x, torch.float32), out)
    close(out.float().cpu().numpy(), pl.offset_norm(x.astype(np.float32), w["n"], 1e-3), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E", [8, 36, 264])
def test_token_shift_keeps_the_last_input_of_every_sequence(dtype, E):
    """Portions of many sizes and single rows continue where the sequence stopped; a slot handed out anew starts from zeros."""
    from borrowed_compute_b200 import StepEntry
    from borrowed_compute_b200.parts import CONVOLUTIONS

    rng = np.random.default_rng(E)
    w = {"shift": pl.to_bf16(rng.uniform(-0.5, 1.5, E))}
    part = CONVOLUTIONS.get("token_shift")(width=E, tensor="shift")
    rt = load_part(part, w, torch_type(dtype))
    state = torch.zeros((3,) + part.state_need().shape, dtype=rt.dtype, device=DEV)
    for slot, T, portions in ((1, 40, [40]), (2, 40, [1, 2, 17, 1, 1, 3, 15]), (1, 9, [2, 2, 5])):
        state[slot].zero_()                           # what the cache does when it hands a slot out
        x = pl.to_bf16(rng.standard_normal((T, E)))
        ref, at, got = pl.token_shift(x, w["shift"]), 0, []
        for n in portions:
            out = torch.empty((n, E), dtype=rt.dtype, device=DEV)
            part.forward(dev(x[at:at + n], rt.dtype), out, context([StepEntry(slot, [0] * n)], [at]), state)
            got.append(out.float().cpu().numpy())
            at += n
        close(np.concatenate(got), ref, dtype, f"portions {portions}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,F,limit,rows", [(16, 24, 1.0, 5), (40, 52, 0.25, 70), (64, 128, 7.0, 300), (512, 1024, 1.5, 9), (264, 384, 2.0, 700)])
def test_feed_forward_with_a_clipped_gate(dtype, E, F, limit, rows):
    """Inputs large enough that the gate meets its bound from above and the up branch both of its bounds."""
    from borrowed_compute_b200.parts import FEED_FORWARDS

    rng = np.random.default_rng(F)
    w = {"gate": pl.to_bf16(rng.standard_normal((F, E)) / math.sqrt(E)), "up": pl.to_bf16(rng.standard_normal((F, E)) / math.sqrt(E)),
         "down": pl.to_bf16(rng.standard_normal((E, F)) / math.sqrt(F))}
    x = pl.to_bf16(rng.standard_normal((rows, E)) * 2.0 * limit)
    g, u = x @ w["gate"].T, x @ w["up"].T
    assert (g > limit).any() and (u > limit).any() and (u < -limit).any() and (np.abs(g) < limit).any()
    part = FEED_FORWARDS.get("clipped_glu")(hidden_size=E, intermediate_size=F, limit=limit)
    rt = load_part(part, w, torch_type(dtype))
    for fused in (True, False):          # in the tensor-core product's epilogue, and in the kernel of its own
        part.fused = fused
        out = torch.zeros((rows, E), dtype=torch.float32, device=DEV)
        part.forward(dev(x, rt.dtype), out, None)
        close(out.cpu().numpy(), pl.clipped_glu(x, {"limit": limit}, w, ""), dtype, f"fused {fused}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,n,top,ff,shared,factor,rows", [(32, 6, 2, 16, 8, 1.5, 50), (24, 3, 3, 8, 0, 1.0, 9), (40, 10, 4, 24, 16, 2.5, 200), (16, 1, 1, 8, 8, 0.5, 4)])
def test_routed_experts_with_weights_that_add_up_to_a_factor(dtype, E, n, top, ff, shared, factor, rows):
    from borrowed_compute_b200 import StepEntry
    from borrowed_compute_b200.parts import FEED_FORWARDS

    rng = np.random.default_rng(n * 10 + top)
    f = pl.moe(n, top, ff, shared, factor)
    cfg = pl.model(10, E, [(pl.latent_mixer(1, 8, 8, 8, 8, 0), f)])
    w = {k[len("l0.mlp."):]: v for k, v in pl.make_weights(cfg, n).items() if k.startswith("l0.mlp.")}
    # rows whose routers choose by a margin, so that rounding the input to bfloat16 chooses the same
    x = pl.to_bf16(rng.standard_normal((rows * 4, E)))
    s = np.sort(pl.sigmoid(x @ w["router"].T), axis=1)[:, ::-1]
    x = x[np.argsort(-(s[:, top - 1] - s[:, top]) if top < n else np.zeros(len(x)), kind="stable")[:rows]]
    ref, pick, _ = pl.experts(x, f, w, "")
    part = FEED_FORWARDS.get("routed_experts")(hidden_size=E, experts=n, top=top, intermediate_size=ff, shared_size=shared, score="sigmoid",
                                               renormalize=True, weight_on="output", weight_factor=factor)
    rt = load_part(part, w, torch_type(dtype))
    out = torch.zeros((rows, E), dtype=torch.float32, device=DEV)
    part.forward(dev(x, rt.dtype), out, context([StepEntry(0, [0] * rows)], [0]))
    close(out.cpu().numpy(), ref, dtype)


def talking_part(m, E, eps):
    from borrowed_compute_b200.parts import MIXERS

    rot = m.get("rot")
    position = {"kind": "none"} if not rot else {"kind": "rotary", "head_dim": rot["dims"], "theta": rot["base"], "pairing": "half", "max_positions": 1024}
    return MIXERS.get("talking_attention")(hidden_size=E, heads=m["heads"], kv_heads=m["kv_heads"], head_dim=m["dim"], norm_eps=eps, position=position,
                                           scale=m["scale"], softcap=m.get("softcap", 0.0), window=m["mask"]["size"] if m.get("mask") else 0,
                                           keep_first=m["mask"].get("keep_first", 0) if m.get("mask") else 0)


def latent_part(m, E, eps):
    from borrowed_compute_b200.parts import MIXERS

    rot = int(m.get("rot_dim", 0))
    position = {"kind": "none"} if not rot else {"kind": "rotary", "head_dim": rot, "theta": m["rot"]["base"], "pairing": "adjacent", "max_positions": 1024}
    return MIXERS.get("latent_attention")(hidden_size=E, heads=m["heads"], head_dim=m["dim"], value_dim=m["vdim"], q_rank=m["q_rank"], kv_rank=m["kv_rank"],
                                          norm_eps=eps, rot_dim=rot, position=position, scale=m["scale"], sink=True)


def run_part(part, rt, x, portions, E):
    """The mixer's output for one sequence's rows, fed in portions (then one row a step), from a cache of its own."""
    from borrowed_compute_b200 import StepEntry
    from borrowed_compute_b200.cache import PagedCache

    cache = PagedCache(rt, [part.cache_need()], [part.state_need()], [None], max_tokens=1024, n_slots=2, max_seq=1024)
    slot, at, got = cache.acquire(), 0, []
    for n in list(portions) + [1] * len(x):
        if at >= len(x):
            break
        rows = x[at:at + n]
        cache.slots.reserve(slot, at + len(rows), rows=len(rows))
        cache.sync_tables()
        residual = torch.zeros((len(rows), E), dtype=torch.float32, device=DEV)
        part.forward(dev(rows, rt.dtype), residual, context([StepEntry(slot, [0] * len(rows))], [at]), cache.memory(0))
        cache.slots.commit(slot, at + len(rows))
        got.append(residual.cpu().numpy())
        at += len(rows)
    cache.slots.check()
    cache.release(slot)
    return np.concatenate(got)


def planted_talk(rng, m, E, star, T):
    """Weights and inputs of one talking mixer in which position ``star``'s key wins every softmax that sees it: input channel 0 is
    zero but at ``star`` and alone drives every key head along one direction of the dimensions that do not turn; input channel 1
    (one everywhere) drives every query along the same direction.  The values being the keys, rows that see ``star`` return it."""
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    rot = m["rot"]["dims"] if m.get("rot") else 0
    mat = lambda r, c, s=1.0: rng.standard_normal((r, c)) * s / math.sqrt(c)                 # noqa: E731
    w = {"q": mat(H * D, E, 0.3), "q.b": 0.05 * rng.standard_normal(H * D), "k": mat(G * D, E), "k.b": 0.05 * rng.standard_normal(G * D),
         "g": mat(H * D, E, 2.0), "o": mat(E, H * D), "o.b": 0.3 * rng.standard_normal(E), "temp": rng.uniform(0.8, 1.25, H),
         "talk": np.eye(H) + 0.1 * rng.standard_normal((H, H)) / math.sqrt(H)}
    w["q"][:, 0], w["k"][:, 0] = 0.0, 0.0
    for h in range(H):
        u = np.zeros(D)
        u[rot:] = rng.choice([-1.0, 1.0], D - rot)
        w["q"][h * D:(h + 1) * D, 1] = 6.0 * u
        if h % (H // G) == 0:
            w["k"][(h // (H // G)) * D:(h // (H // G) + 1) * D, 0] = 2.0 * u
        else:
            w["q"][h * D:(h + 1) * D, 1] = w["q"][(h - h % (H // G)) * D:(h - h % (H // G) + 1) * D, 1]
    x = rng.standard_normal((T, E)) * 0.5
    x[:, 0], x[:, 1] = 0.0, 1.0
    x[star, 0] = 8.0
    return {k: pl.to_bf16(v) for k, v in w.items()}, pl.to_bf16(x)


TALK_PATHS = [("float32", "rows"), ("bfloat16", "rows"), ("bfloat16", "tiles")]


@pytest.mark.parametrize("dtype,path", TALK_PATHS)
@pytest.mark.parametrize("window,keep,star", [(9, 0, 5), (9, 0, 63), (1, 0, 64), (64, 0, 63), (64, 2, 64), (70, 0, 127), (9, 3, 2), (9, 3, 3), (40, 64, 63),
                                              (40, 65, 64), (33, 70, 69), (200, 4, 10), (129, 1, 0)])
def test_talking_attention_with_one_key_that_matters_at_every_edge(dtype, path, window, keep, star):
    """Rows that see the planted key return it, the row just past the window's edge does not, unless the key is one of the kept
    first positions: in a whole prompt, in portions of two and more rows whose borders fall beside the key, the edge and the pages'
    borders, and row by row."""
    from borrowed_compute_b200 import StepEntry
    from borrowed_compute_b200.parts import talking_attention

    E, T = 48, 300
    m = pl.talking_mixer(4, 2, 32, window, keep, 8, softcap=30.0, scale=14.0 / 32)
    w, x = planted_talk(np.random.default_rng(window * 7 + keep + star), m, E, star, T)
    ref = pl.talking_attention(x, m, w, "", 1e-5)
    edge = star + window
    if edge + 1 < T:
        # the planted key decides: a window one position longer changes the row at the edge, unless the key is kept for good
        longer = pl.talking_attention(x, dict(m, mask={"size": window + 1, "keep_first": keep}), w, "", 1e-5)
        assert (np.abs(longer[edge] - ref[edge]).max() > 0.05 * np.abs(ref).max()) == (star >= keep)
    part = talking_part(m, E, 1e-5)
    rt = load_part(part, w, torch_type(dtype))
    talking_attention.force = path
    if part.path(context([StepEntry(0, [0] * 20)], [0]), rt.dtype) != path:
        pytest.skip("these sizes do not take this path")
    for portions in ([T], [star + 1], [max(star, 1), 2, 2], [2, 61, 3, 62, 2, 9, 64]):
        close(run_part(part, rt, x, portions, E), ref, dtype, f"portions {portions}")


@pytest.mark.parametrize("dtype,path", TALK_PATHS)
@pytest.mark.parametrize("H,G,D,rot,window,keep,cap", [(1, 1, 8, 8, 0, 0, 0.0), (6, 2, 40, 20, 100, 5, 10.0), (40, 8, 16, 0, 50, 1, 50.0), (3, 3, 128, 64, 64, 64, 0.0),
                                                       (16, 4, 64, 32, 77, 0, 20.0), (5, 1, 12, 4, 300, 7, 3.0), (8, 8, 48, 48, 31, 2, 25.0),
                                                       (32, 8, 128, 64, 100, 4, 30.0), (24, 6, 32, 16, 40, 0, 0.0), (20, 5, 64, 64, 90, 33, 12.0)])
def test_talking_attention_in_other_sizes(dtype, path, H, G, D, rot, window, keep, cap):
    """One head; more heads than a block takes (two and four blocks a cluster share them out, or two heads a warp where the kv heads
    do not divide); heads that are no power of two; every dimension turning, or none; no window."""
    from borrowed_compute_b200 import StepEntry
    from borrowed_compute_b200.parts import talking_attention

    E, T = 40, 150
    m = pl.talking_mixer(H, G, D, window or 1, keep, rot, softcap=cap, scale=3.0 / D)
    if not window:
        del m["mask"]
    cfg = pl.model(10, E, [(m, None)])
    w = {k[len("l0.mix."):]: v for k, v in pl.make_weights(cfg, H + D).items() if k.startswith("l0.mix.")}
    x = pl.to_bf16(np.random.default_rng(D).standard_normal((T, E)))
    ref = pl.talking_attention(x, m, w, "", 1e-6)
    part = talking_part(m, E, 1e-6)
    rt = load_part(part, w, torch_type(dtype))
    talking_attention.force = path
    if part.path(context([StepEntry(0, [0] * 20)], [0]), rt.dtype) != path:
        pytest.skip("these sizes do not take this path")
    for portions in ([T], [70, 40, 2]):
        close(run_part(part, rt, x, portions, E), ref, dtype, f"portions {portions}")


LATENT_PATHS = [("float32", "rows"), ("bfloat16", "rows"), ("bfloat16", "split"), ("bfloat16", "expand")]


@pytest.mark.parametrize("dtype,path", LATENT_PATHS)
@pytest.mark.parametrize("H,D,DV,QR,R,rot,sink", [(3, 16, 24, 24, 40, 8, 2.0), (1, 8, 8, 8, 8, 0, 6.0), (17, 16, 8, 16, 24, 16, -3.0), (2, 64, 128, 40, 136, 32, 9.0),
                                                  (5, 40, 80, 32, 64, 24, 0.0)])
def test_latent_attention_with_a_sink_and_neighbouring_pairs(dtype, path, H, D, DV, QR, R, rot, sink):
    """A head's sink takes its share of every row's weights (a large one nearly all of it), and the rotated part turns pairs
    (2i, 2i + 1): on every way through the kernels, whole and in portions."""
    from borrowed_compute_b200 import StepEntry
    from borrowed_compute_b200.parts import latent_attention

    E, T = 48, 150
    m = pl.latent_mixer(H, D, DV, QR, R, rot, scale=0.3, base=500.0)
    cfg = pl.model(10, E, [(m, None)])
    w = {k[len("l0.mix."):]: v for k, v in pl.make_weights(cfg, H + D).items() if k.startswith("l0.mix.")}
    w["sink"] = pl.to_bf16(sink + np.arange(H) * 0.5)
    x = pl.to_bf16(np.random.default_rng(R).standard_normal((T, E)))
    ref = pl.latent_attention(x, m, w, "", 1e-6)
    without = pl.latent_attention(x, m, dict(w, sink=np.full(H, -60.0)), "", 1e-6)
    assert np.abs(ref - without).max() > 0.02 * np.abs(without).max()          # the sink matters
    part = latent_part(m, E, 1e-6)
    rt = load_part(part, w, torch_type(dtype))
    latent_attention.force = path
    if part.path(context([StepEntry(0, [0] * 20)], [0]), rt.dtype) != path:
        pytest.skip("these sizes do not take this path")
    for portions in ([T], [70, 40, 2], [1, 1, 2, 64]):
        close(run_part(part, rt, x, portions, E), ref, dtype, f"portions {portions}")


def planted_latent(rng, m, E, star, T, sink):
    """Weights and inputs of one latent mixer in which position ``star`` outweighs every other position and the sink: only input
    channel 0 feeds latent channel 0, and it is zero but at ``star``; every head's plain key reads latent channel 0 along a direction
    of its own, and every query has that direction, fed by input channel 1 (one everywhere) through query-latent channel 0."""
    H, D, DV, QR, R, rot = m["heads"], m["dim"], m["vdim"], m["q_rank"], m["kv_rank"], m["rot_dim"]
    mat = lambda r, c, f=1.0: rng.standard_normal((r, c)) * f / math.sqrt(c)                 # noqa: E731
    w = {"dq": mat(QR, E), "dq.norm": 1.0 + 0.2 * rng.uniform(-1, 1, QR), "uq": mat(H * (D + rot), QR), "dkv": mat(R + rot, E),
         "dkv.norm": 1.0 + 0.2 * rng.uniform(-1, 1, R), "uk": mat(H * D, R), "uv": mat(H * DV, R, 2.0), "g": mat(H, E, 2.0), "o": mat(E, H * DV),
         "sink": np.full(H, sink) + 0.25 * np.arange(H)}
    w["dkv"][:, 0] = 0.0
    w["dkv"][0, :] = 0.0
    w["dkv"][0, 0] = 4.0
    w["dq"][0, :] = 0.0
    w["dq"][0, 1] = 3.0
    for h in range(H):
        direction = rng.choice([-1.0, 1.0], D) * (3.0 / math.sqrt(D * m["scale"]))
        w["uq"][h * (D + rot):h * (D + rot) + D, 0] = direction
        w["uk"][h * D:(h + 1) * D, 0] = direction
    x = rng.standard_normal((T, E)) * 0.5
    x[:, 0], x[:, 1] = 0.0, 1.0
    x[star, 0] = 8.0
    return {k: pl.to_bf16(v) for k, v in w.items()}, pl.to_bf16(x)


@pytest.mark.parametrize("dtype,path", LATENT_PATHS)
@pytest.mark.parametrize("star,rot,sink", [(0, 8, 2.0), (5, 0, 2.0), (63, 8, -1.0), (64, 16, 4.0), (250, 8, 2.0)])
def test_latent_attention_with_one_far_key_and_a_sink(dtype, path, star, rot, sink):
    """Every later row returns the planted position's value, hundreds of positions on, less the sink's share: whole, in portions
    whose borders fall beside the key and the pages' borders, and row by row."""
    from borrowed_compute_b200 import StepEntry
    from borrowed_compute_b200.parts import latent_attention

    E, T = 64, 330
    m = pl.latent_mixer(3, 16, 24, 24, 40, rot, scale=0.25, base=10000.0)
    w, x = planted_latent(np.random.default_rng(star * 3 + rot), m, E, star, T, sink)
    ref = pl.latent_attention(x, m, w, "", 1e-5)
    lost = pl.latent_attention(np.concatenate([x[:star], 0.0 * x[star:star + 1], x[star + 1:]]), m, w, "", 1e-5)
    assert np.abs(ref[-1] - lost[-1]).max() > 0.05 * np.abs(ref).max()          # the far key decides the last row
    part = latent_part(m, E, 1e-5)
    rt = load_part(part, w, torch_type(dtype))
    latent_attention.force = path
    if part.path(context([StepEntry(0, [0] * 20)], [0]), rt.dtype) != path:
        pytest.skip("these sizes do not take this path")
    for portions in ([T], [star + 1], [max(star, 1), 2, 2], [2, 61, 3, 62, 2, 9, 64, 100]):
        close(run_part(part, rt, x, portions, E), ref, dtype, f"portions {portions}")


# ------------------------------------------------------------------------- whole models

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_prompts_and_the_stream_after_every_layer(name, dtype):
    eng, cfg, w = small(name, dtype)
    toks = tokens_for(cfg, w, 150, seed=1)
    streams, got = [], []
    ref = pl.forward(cfg, w, toks, streams)
    eng.model.after_run = lambda i, res: got.append(res.detach().float().cpu().numpy().copy())
    try:
        out = run_whole(eng, toks)
    finally:
        eng.model.after_run = None
    assert len(got) == len(streams)
    for i, (g, s) in enumerate(zip(got, streams)):
        mostly_close(g[: len(toks)], s, dtype, f"the stream after layer {i}")
    mostly_close(out, ref, dtype, "scores")
    for n in (1, 2, 3):            # the first tokens of a sequence, alone
        mostly_close(run_whole(eng, toks[:n]), ref[:n], dtype, f"a prompt of {n}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_prefill_against_token_by_token_and_portions(name, dtype):
    """The window passes over decoded tokens, the kept first positions stay, pages fill and are let go."""
    eng, cfg, w = small(name, dtype)
    toks = tokens_for(cfg, w, 200, seed=2)
    ref = pl.forward(cfg, w, toks)
    for cuts in ([], [120], [2, 2, 60, 3, 64, 1, 2, 40], [64, 64], [63, 2, 63], [199]):
        mostly_close(run_cut(eng, toks, cuts), ref, dtype, f"portions {cuts}")
    eng.cache.slots.check()


@pytest.mark.parametrize("name", ["A", "B"])
def test_cuts_and_batches_give_the_same_bits_in_float32(name):
    from borrowed_compute_b200.engine import StepEntry

    eng, cfg, w = small(name, "float32")
    toks = tokens_for(cfg, w, 140, seed=3)
    whole = run_whole(eng, toks)
    assert np.array_equal(run_cut(eng, toks, [70, 2, 30]), whole)
    others = [tokens_for(cfg, w, n, seed=4 + n) for n in (5, 90)]
    slots = [eng.acquire() for _ in range(3)]
    out = eng.step([StepEntry(slots[0], others[0], (4,)), StepEntry(slots[1], toks, tuple(range(len(toks)))), StepEntry(slots[2], others[1], ())]).cpu().numpy()
    for s in slots:
        eng.release(s)
    assert np.array_equal(out[1:], whole)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_unequal_batches_against_each_alone_then_decoded_together(name, dtype):
    from borrowed_compute_b200.engine import StepEntry

    eng, cfg, w = small(name, dtype)
    lengths, tail = [1, 37, 130, 66], 40
    seqs = [tokens_for(cfg, w, n + tail, seed=10 + n) for n in lengths]
    refs = [pl.forward(cfg, w, s) for s in seqs]
    slots = [eng.acquire() for _ in seqs]
    rows = [[] for _ in seqs]
    out = eng.step([StepEntry(sl, s[:n], tuple(range(n))) for sl, s, n in zip(slots, seqs, lengths)]).cpu().numpy()
    at = 0
    for i, n in enumerate(lengths):
        rows[i].append(out[at:at + n])
        at += n
    live = list(range(len(seqs)))
    for t in range(tail):
        if t == 25:                 # a shorter request ends earlier, its slot goes to a new one
            eng.release(slots[1])
            live.remove(1)
        out = eng.step([StepEntry(slots[i], [seqs[i][lengths[i] + t]], (0,)) for i in live]).cpu().numpy()
        for k, i in enumerate(live):
            rows[i].append(out[k:k + 1])
    for i in live:
        eng.release(slots[i])
    for i, r in enumerate(rows):
        got = np.concatenate(r)
        mostly_close(got, refs[i][: len(got)], dtype, f"sequence {i}")
    eng.cache.slots.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_slots_and_pages_used_again(dtype):
    """What a sequence left behind (pages, the token shift's state) does not reach the next one in its slot."""
    eng, cfg, w = small("A", dtype)
    a, b = tokens_for(cfg, w, 190, seed=20), tokens_for(cfg, w, 75, seed=21)
    ref_a, ref_b = pl.forward(cfg, w, a), pl.forward(cfg, w, b)
    for _ in range(3):
        mostly_close(run_cut(eng, a, [100]), ref_a, dtype, "the long one")
        mostly_close(run_cut(eng, b, [3, 70]), ref_b, dtype, "the short one in the same slot")
    eng.cache.slots.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_far_past_the_window(dtype):
    eng, cfg, w = small("B", dtype)
    toks = tokens_for(cfg, w, 420, seed=30)
    ref = pl.forward(cfg, w, toks)
    mostly_close(run_cut(eng, toks, [20]), ref, dtype)


@pytest.mark.parametrize("seed", range(10))
def test_drawn_configurations(seed):
    """Sizes, constants and the order of layers drawn at random, in float32: whole, in portions, and token by token."""
    rng = np.random.default_rng(1000 + seed)
    cfg = pl.draw_config(rng)
    w = pl.make_weights(cfg, seed)
    eng = engine_for(cfg, w, "float32", max_tokens=1024, max_slots=2, max_seq=512)
    toks = [int(t) for t in rng.integers(0, cfg["vocab"], 150)]
    ref = pl.forward(cfg, w, toks)
    close(run_whole(eng, toks), ref, "float32", f"whole, {json.dumps(cfg)}")
    close(run_cut(eng, toks, [2, 66, 30]), ref, "float32", f"portions, {json.dumps(cfg)}")


@pytest.mark.parametrize("seed", range(8))
def test_drawn_configurations_in_bfloat16(seed):
    rng = np.random.default_rng(2000 + seed)
    cfg = pl.draw_config(rng)
    w = pl.make_weights(cfg, seed)
    eng = engine_for(cfg, w, "bfloat16", max_tokens=1024, max_slots=2, max_seq=512)
    toks = tokens_for(cfg, w, 150, seed=seed)
    ref = pl.forward(cfg, w, toks)
    mostly_close(run_whole(eng, toks), ref, "bfloat16", f"whole, {json.dumps(cfg)}")
    mostly_close(run_cut(eng, toks, [2, 66, 30]), ref, "bfloat16", f"portions, {json.dumps(cfg)}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_sizes_that_are_multiples_of_nothing(dtype):
    """A width, heads, latents, feed-forwards and a vocabulary that no vector load and no tile divides."""
    cfg = pl.model(61, 50, [
        (pl.talking_mixer(3, 1, 10, 7, 2, 6, softcap=9.0), pl.moe(5, 2, 14, 6, 1.25)),
        (pl.latent_mixer(3, 6, 10, 10, 12, 2), pl.dense(14, 0.75)),
        (pl.talking_mixer(5, 5, 18, 50, 0, 18, softcap=0.0), None),
    ], eps=1e-4, embedding_scale=3.0, logit_scale=1.5)
    w = pl.make_weights(cfg, 77)
    eng = engine_for(cfg, w, dtype, max_tokens=1024, max_slots=2, max_seq=512)
    toks = tokens_for(cfg, w, 130, seed=9)
    ref = pl.forward(cfg, w, toks)
    mostly_close(run_whole(eng, toks), ref, dtype, "whole")
    mostly_close(run_cut(eng, toks, [3, 64, 2, 40]), ref, dtype, "portions")


# ------------------------------------------------------------------ the entry points

def folder_for(tmp_path, name, seed):
    from borrowed_compute_b200.weights.safetensors_io import write_safetensors

    cfg = pl.SMALL[name]
    w = pl.make_weights(cfg, seed)
    folder = str(tmp_path / f"logirax_{name}")
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), {n: torch.from_numpy(a).to(torch.bfloat16) for n, a in w.items()})
    return folder, cfg, w


def test_greedy_generation_through_the_library_and_the_command_line(tmp_path):
    from borrowed_compute_b200 import Local, Sampling

    folder, cfg, w = folder_for(tmp_path, "A", 41)
    prompts = [tokens_for(cfg, w, n, seed=50 + n) for n in (9, 30)]
    want = [pl.greedy(cfg, w, p, 12) for p in prompts]
    local = Local.load(folder, dtype="float32", max_tokens=1024, max_slots=4, max_seq=256)
    out, stats = local.generate(prompts, 12, Sampling(), stop_ids=())
    assert [list(g) for g in out] == want and stats.generated == 24
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "bc-infer"), "generate", folder, ";".join(",".join(map(str, p)) for p in prompts),
                          "--max-tokens", "12", "--dtype", "float32", "--stop-ids", ""], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [[int(t) for t in line.split(",")] for line in res.stdout.strip().splitlines()] == want
    # bfloat16 decodes through captured graphs: the tokens are the oracle's wherever its two best scores lie well apart
    out16, _ = Local.load(folder, dtype="bfloat16", max_tokens=1024, max_slots=4, max_seq=256).generate(prompts, 12, Sampling(), stop_ids=())
    for p, mine in zip(prompts, out16):
        toks = list(p)
        assert len(mine) == 12
        for t in mine:
            last = pl.forward(cfg, w, toks)[-1]
            best = np.sort(last)
            if best[-1] - best[-2] > 0.1 * (1.0 + np.abs(last).max()):
                assert t == int(last.argmax()), "a clear choice was missed"
            toks.append(int(t))


@pytest.mark.parametrize("dtype", DTYPES)
def test_replaying_steps_with_the_trace_tool(tmp_path, dtype):
    folder, cfg, w = folder_for(tmp_path, "B", 42)
    a, b = tokens_for(cfg, w, 80, seed=60), tokens_for(cfg, w, 33, seed=61)
    ref_a, ref_b = pl.forward(cfg, w, a), pl.forward(cfg, w, b)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": a[:70], "want": [0, 69]}, {"id": "y", "tokens": b[:30], "want": [29]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": a[70:71], "want": []}, {"id": "y", "tokens": b[30:31], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": a[71:72], "want": [0]}, {"id": "y", "tokens": b[31:32], "want": [0]}], "end": ["y"]},
             {"step": 3, "entries": [{"id": "x", "tokens": a[72:73], "want": [0]}], "end": ["x"]}]
    out = str(tmp_path / "scores")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out, "--max-tokens", "256"],
                         input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [line for line in res.stdout.splitlines() if line.startswith("done")] == [f"done {i}" for i in range(4)]
    read = lambda i: np.fromfile(os.path.join(out, f"{i}.f32"), dtype="<f4").reshape(-1, cfg["vocab"])      # noqa: E731
    assert not os.path.exists(os.path.join(out, "1.f32")) or read(1).shape[0] == 1
    mostly_close(read(0), np.stack([ref_a[0], ref_a[69], ref_b[29]]), dtype, "step 0")
    mostly_close(read(1), ref_b[30:31], dtype, "step 1")
    mostly_close(read(2), np.stack([ref_a[71], ref_b[31]]), dtype, "step 2")
    mostly_close(read(3), ref_a[72:73], dtype, "step 3")
