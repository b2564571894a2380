"""The Fudelorn decoder on the engine against the plain implementation (plain_fudelorn.py): each new mechanism alone
through its kernels, then whole models through the engine's step function, cache, scheduler and entry points: whole
prompts, token-by-token decoding, portions down to two tokens, unequal batches, slots and pages used again, keys at
the edges of windows and pages and far away, the first tokens, long decoding, and greedy generation.

The latent attention has three ways through the kernels (one warp a row and head; the split kernel over the cache as
it is; keys and values expanded for the prompt attention kernels).  Each is forced in turn on inputs and weights made so
that ONE position's key wins every softmax that sees it: a mask that is one position off then changes whole rows.

float32 engines are held to the float64 oracle tightly (1e-4 (1 + max|score|)), bfloat16 ones within 6e-2 (1 + max|score|)."""

from __future__ import annotations

import copy
import json
import math
import os

import numpy as np
import pytest

import plain_fudelorn as pf
from conftest import BF16_TOL, F32_TOL

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
DEV = "cuda:0"


def tol(dtype, ref):
    return (F32_TOL if dtype == "float32" else 2 * BF16_TOL) * (1.0 + float(np.abs(ref).max()))


def close(got, ref, dtype, what=""):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: {got.shape} against {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: not finite"
    worst = np.abs(got - ref).reshape(got.shape[0], -1).max(axis=-1)
    assert worst.max() <= tol(dtype, ref), f"{what}: row {int(worst.argmax())} differs by {worst.max():.4g} (allowed {tol(dtype, ref):.4g})"


def mostly_close(got, ref, dtype, what="", rounding=0.0):
    """For bfloat16 models whose sizes are drawn: a sublayer's result passes a norm before it joins the stream, so a row whose
    sublayer result is small (few experts' units above zero, say) has its rounding magnified, on every path through the kernels
    alike.  Nineteen rows in twenty are held to the tolerance; every row to three times that, or to twice ``rounding``, the
    farthest that the plain implementation's own scores move when it keeps in 16 bits what the design allows (rounding_alone)."""
    if dtype == "float32":
        return close(got, ref, dtype, what)
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape and np.isfinite(got).all(), f"{what}: shape or numbers"
    worst = np.abs(got - ref).reshape(got.shape[0], -1).max(axis=-1)
    top = max(3 * tol(dtype, ref), 2 * rounding)
    assert np.quantile(worst, 0.95) <= tol(dtype, ref) and worst.max() <= top, \
        f"{what}: row {int(worst.argmax())} differs by {worst.max():.4g} (allowed {top:.4g}), the 95th percentile by {np.quantile(worst, 0.95):.4g} (allowed {tol(dtype, ref):.4g})"


def rounding_alone(cfg, w, toks, ref):
    """The largest change of any score when the plain implementation rounds to bfloat16 wherever the design allows it, over
    four roundings that differ by a factor near one (which rows a rounding moves most is a matter of chance)."""
    return max(float(np.abs(pf.forward(cfg, w, toks, r=lambda a, f=f: pf.to_bf16(np.asarray(a) * f)) - ref).max())
               for f in (1.0, 1.0 + 2.0 ** -10, 1.0 - 2.0 ** -10, 1.0 + 2.0 ** -11))


def tokens_for(seed, n, vocab):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, n)]


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    return t if dtype is None else t.to(dtype)


def engine_for(cfg, weights, dtype, **kw):
    from borrowed_compute_b200.engine import Engine

    kw.setdefault("max_tokens", 2048)
    kw.setdefault("max_slots", 6)
    kw.setdefault("max_seq", 512)
    return Engine.from_tensors(cfg, {n: torch.from_numpy(np.ascontiguousarray(a)) for n, a in weights.items()}, dtype=dtype, **kw)


_made = {}


def small(name, dtype):
    key = (name, dtype)
    if key not in _made:
        cfg = pf.SMALL[name]
        w = pf.make_weights(cfg, seed=21 if name == "A" else 22)
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
def _the_part_chooses_again():
    from borrowed_compute_b200.parts import latent_attention

    yield
    latent_attention.force = None


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


def mixer_part(m, E, eps, own_kv=True):
    from borrowed_compute_b200.parts import MIXERS

    rot = int(m.get("rot_dim", 0))
    position = {"kind": "none"}
    if rot:
        s = m["rot"].get("scaling")
        position = {"kind": "rotary", "head_dim": rot, "theta": m["rot"]["base"], "pairing": "half", "max_positions": 512,
                    "scaling": None if not s else dict(s, type="yarn")}
    return MIXERS.get("latent_attention")(hidden_size=E, heads=m["heads"], head_dim=m["dim"], value_dim=m["vdim"], q_rank=m["q_rank"], kv_rank=m["kv_rank"],
                                          norm_eps=eps, rot_dim=rot, position=position, scale=m["scale"], window=m["mask"]["size"] if m.get("mask") else 0,
                                          own_kv=own_kv)


def load_part(part, w, dtype):
    from borrowed_compute_b200.parts import Runtime

    rt = Runtime(torch.device(DEV), dtype, max_positions=512)
    part.load({k: dev(w[k], torch.float32 if s.role == "vector" else dtype) for k, s in part.tensors().items()}, rt)
    return rt


def planted(rng, m, E, star, T):
    """Weights and inputs of one mixer in which position ``star``'s key wins every softmax that sees it: input channel 0 is zero
    but at ``star`` and alone feeds latent channel 0, which every head's key reads along a direction that every query has, fed by
    input channel 1 (one everywhere)."""
    H, D, DV, QR, R, rot = m["heads"], m["dim"], m["vdim"], m["q_rank"], m["kv_rank"], m.get("rot_dim", 0)
    mat = lambda r, c, s=1.0: rng.standard_normal((r, c)) * s / math.sqrt(c)                 # noqa: E731
    w = {"dq": mat(QR, E), "dq.norm": 1.0 + 0.2 * rng.uniform(-1, 1, QR), "uq": mat(H * (D + rot), QR), "dkv": mat(R + rot, E),
         "dkv.norm": 1.0 + 0.2 * rng.uniform(-1, 1, R), "uk": mat(H * D, R), "uv": mat(H * DV, R, 2.0), "g": mat(H, E, 2.0), "o": mat(E, H * DV)}
    w["dkv"][0, :], w["dkv"][:, 0], w["dkv"][0, 0] = 0.0, 0.0, 4.0
    w["dq"][0, :], w["dq"][0, 1] = 0.0, 3.0
    for h in range(H):
        v = rng.choice([-1.0, 1.0], D) * (3.0 / math.sqrt(D * m["scale"]))
        w["uq"][h * (D + rot):h * (D + rot) + D, 0] = v
        w["uk"][h * D:(h + 1) * D, 0] = v
    x = rng.standard_normal((T, E)) * 0.5
    x[:, 0], x[:, 1] = 0.0, 1.0
    x[star, 0] = 8.0
    return {k: pf.to_bf16(v) for k, v in w.items()}, pf.to_bf16(x)


def run_part(part, rt, x, portions, E, slots_before=0):
    """The mixer's output for one sequence's rows, fed in portions (then one row a step), from a cache of its own."""
    from borrowed_compute_b200 import StepEntry
    from borrowed_compute_b200.cache import PagedCache

    cache = PagedCache(rt, [part.cache_need()], [part.state_need()], [None], max_tokens=512, n_slots=2, max_seq=512)
    slot, at, got = cache.acquire(), 0, []
    for n in list(portions) + [1] * len(x):
        if at >= len(x):
            break
        rows = x[at:at + n]
        entry = StepEntry(slot, [0] * len(rows))
        cache.slots.reserve(slot, at + len(rows), rows=len(rows))
        cache.sync_tables()
        ctx = context([entry], [at])
        residual = torch.zeros((len(rows), E), dtype=torch.float32, device=DEV)
        part.forward(dev(rows, rt.dtype), residual, ctx, cache.memory(0))
        cache.slots.commit(slot, at + len(rows))
        got.append(residual.cpu().numpy())
        at += len(rows)
    cache.release(slot)
    return np.concatenate(got)


PATHS = [("float32", "rows"), ("bfloat16", "rows"), ("bfloat16", "split"), ("bfloat16", "expand")]


@pytest.mark.parametrize("dtype,path", PATHS)
@pytest.mark.parametrize("window,rot,star", [(0, 8, 5), (0, 0, 64), (1, 0, 63), (9, 0, 63), (64, 0, 63), (64, 8, 64), (70, 0, 63), (129, 16, 1)])
def test_latent_attention_with_one_key_that_matters_at_every_edge(dtype, path, window, rot, star):
    """Rows that see the planted key give its value, the row just past the window's edge does not: in a whole prompt, in portions
    of two and more rows whose borders fall beside the key, the edge and the pages' borders, and row by row."""
    from borrowed_compute_b200.parts import latent_attention

    E, T = 64, 210
    m = {"heads": 3, "dim": 16, "vdim": 24, "q_rank": 24, "kv_rank": 40, "scale": 0.25}
    if window:
        m["mask"] = {"size": window}
    if rot:
        m.update({"rot_dim": rot, "rot": {"base": 10000.0, "dims": rot, "scaling": {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}}})
    w, x = planted(np.random.default_rng(window * 7 + rot + star), m, E, star, T)
    ref, _ = pf.latent_attention(x, w, m, 1e-5)
    edge = star + window if window else T
    # the planted key decides: rows that see it differ from what they would be without it
    if window and edge + 1 < T:
        assert np.abs(ref[edge - 1] - ref[edge]).max() > 0.05 * np.abs(ref).max()
    part = mixer_part(m, E, 1e-5)
    rt = load_part(part, w, torch.float32 if dtype == "float32" else torch.bfloat16)
    latent_attention.force = path
    assert part.path(context([__import__("borrowed_compute_b200").StepEntry(0, [0] * 20)], [0]), rt.dtype) == path
    for portions in ([T], [star + 1], [star, 2, 2], [2, 61, 3, 62, 2, 9, 64]):
        close(run_part(part, rt, x, portions, E), ref, dtype, f"portions {portions}")


@pytest.mark.parametrize("dtype,path", PATHS)
@pytest.mark.parametrize("H,D,DV,QR,R,rot", [(1, 8, 8, 8, 8, 0), (17, 16, 8, 16, 24, 8), (2, 64, 128, 40, 136, 32), (5, 40, 80, 32, 64, 24)])
def test_latent_attention_in_other_sizes(dtype, path, H, D, DV, QR, R, rot):
    """One head, more heads than a block of the split kernel takes, values wider than keys, widths that are no power of two."""
    from borrowed_compute_b200.parts import latent_attention

    E, T = 48, 150
    m = {"heads": H, "dim": D, "vdim": DV, "q_rank": QR, "kv_rank": R, "scale": 0.3, "mask": {"size": 100}}
    if rot:
        m.update({"rot_dim": rot, "rot": {"base": 500.0, "dims": rot}})
        del m["mask"]
    w, x = planted(np.random.default_rng(H + D), m, E, 3, T)
    ref, _ = pf.latent_attention(x, w, m, 1e-6)
    part = mixer_part(m, E, 1e-6)
    rt = load_part(part, w, torch.float32 if dtype == "float32" else torch.bfloat16)
    latent_attention.force = path
    for portions in ([T], [70, 40, 2]):
        close(run_part(part, rt, x, portions, E), ref, dtype, f"portions {portions}")


def i32(a):
    return torch.tensor(list(a), dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("E,top,ff,K,shared,rows", [(5, 2, 24, 40, 16, 77), (3, 3, 8, 16, 0, 77), (9, 1, 72, 64, 24, 300), (1, 1, 16, 24, 8, 5), (12, 4, 40, 48, 0, 600)])
def test_experts_named_by_a_table_and_the_gated_shared_expert(E, top, ff, K, shared, rows):
    """Every row's experts come from its token's row of the table, each weighs 1 / top, the shared expert runs for all rows
    times the sigmoid of one number a row; rows of no sequence choose nothing and add nothing."""
    from borrowed_compute_b200.parts.base import Runtime, StepContext
    from borrowed_compute_b200.parts.moe import RoutedExperts

    rng, V = np.random.default_rng(E * 10 + top), 53
    w = {"table": np.stack([rng.permutation(E)[:top] for _ in range(V)]).astype(np.int32)}
    for e in range(E):
        w.update({f"e{e}.up": pf.to_bf16(rng.standard_normal((ff, K)) / math.sqrt(K)), f"e{e}.down": pf.to_bf16(rng.standard_normal((K, ff)) / math.sqrt(ff))})
    if shared:
        w.update({"shared.up": pf.to_bf16(rng.standard_normal((shared, K)) / 4), "shared.down": pf.to_bf16(rng.standard_normal((K, shared)) / 4),
                  "shared.sg": pf.to_bf16(rng.standard_normal((1, K)))})
    h = pf.to_bf16(rng.standard_normal((rows, K)))
    toks = rng.integers(0, V, rows)
    mlp = {"router": {"experts": E, "top": top}, "expert": {"ff": ff}}
    if shared:
        mlp["shared"] = {"ff": shared}
    ref = pf.table_experts(h, toks, w, mlp)
    for dtype, td in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
        part = RoutedExperts(K, E, top, ff, shared_size=shared, weight_on="output", router="table", expert="relu2", shared_gate=shared > 0, vocab_size=V)
        specs = part.tensors()
        part.load({n: dev(a) if n == "table" else dev(a, torch.float32 if specs[n].role == "vector" else td) for n, a in w.items()}, Runtime(torch.device(DEV), td))
        slot = np.zeros(rows + 3, dtype=np.int32)
        slot[rows:] = -1
        x = torch.cat([dev(h, td), torch.full((3, K), float("nan"), dtype=td, device=DEV)])
        residual = torch.ones((rows + 3, K), dtype=torch.float32, device=DEV)
        ctx = StepContext(rows=rows + 3, seqs=1, tokens=i32(list(toks) + [0, 0, 0]), row_pos=None, row_slot=i32(slot), seq_rows=None, seq_slot=None,
                          seq_start=None, max_new=rows, max_total=rows, decode=False)
        part.forward(x, residual, ctx)
        out = residual.cpu().numpy()
        close(out[:rows] - 1.0, ref, dtype, "experts")
        if not shared:
            assert (out[rows:] == 1.0).all(), "a row of no sequence added something"


@pytest.mark.parametrize("K,ff,rows", [(40, 24, 77), (64, 200, 3), (256, 1024, 300)])
def test_feed_forward_with_the_square_of_relu(K, ff, rows):
    from borrowed_compute_b200.parts.base import Runtime, StepContext
    from borrowed_compute_b200.parts.mlp import PlainMLP

    rng = np.random.default_rng(K)
    up, down = pf.to_bf16(rng.standard_normal((ff, K)) / math.sqrt(K)), pf.to_bf16(rng.standard_normal((K, ff)) / math.sqrt(ff))
    h = pf.to_bf16(rng.standard_normal((rows, K)))
    ref = pf.relu_squared_mlp(h, up, down)
    for dtype, td in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
        part = PlainMLP(K, ff, activation="relu2")
        part.load({"up": dev(up, td), "down": dev(down, td)}, Runtime(torch.device(DEV), td))
        residual = torch.ones((rows, K), dtype=torch.float32, device=DEV)
        ctx = StepContext(rows=rows, seqs=1, tokens=None, row_pos=None, row_slot=i32([0] * rows), seq_rows=None, seq_slot=None, seq_start=None, max_new=rows,
                          max_total=rows, decode=False)
        part.forward(dev(h, td), residual, ctx)
        close(residual.cpu().numpy() - 1.0, ref, dtype, "feed-forward")


def test_the_norm_after_a_sublayer_adds_into_the_stream():
    """x += N(y) in float, whatever the compute type: the stream keeps its 32 bits."""
    from borrowed_compute_b200 import ops

    rng = np.random.default_rng(3)
    for width, eps in ((96, 1e-5), (256, 1e-6), (1000, 1e-5)):
        y, x, w = rng.standard_normal((37, width)) * 3, rng.standard_normal((37, width)), 1.0 + 0.3 * rng.uniform(-1, 1, width)
        res = dev(x.astype(np.float32))
        ops.norm_add(dev(y.astype(np.float32)), dev(w.astype(np.float32)), res, eps)
        ref = x.astype(np.float32) + pf.rms_norm(y.astype(np.float32), w.astype(np.float32), eps)
        assert np.abs(res.cpu().numpy() - ref).max() <= 1e-5 * (1 + np.abs(ref).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_between_the_sublayers_one_kernel_norms_twice_and_clears(dtype):
    """x += N(y) in float, h = N(x) in the compute type for the feed-forward, y = 0: against the two norms one after the other;
    widths that four divides and others, a row that is all zeros."""
    from borrowed_compute_b200 import ops

    rng = np.random.default_rng(4)
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    for width, eps, eps2 in ((96, 1e-5, 1e-6), (250, 1e-6, 1e-5), (4096, 1e-5, 1e-5), (7, 1e-5, 1e-5)):
        y, x = rng.standard_normal((19, width)) * 3, rng.standard_normal((19, width))
        y[3] = 0.0
        w, w2 = 1.0 + 0.3 * rng.uniform(-1, 1, width), 1.0 + 0.3 * rng.uniform(-1, 1, width)
        yd, res = dev(y.astype(np.float32)), dev(x.astype(np.float32))
        h = torch.full((19, width), 7.0, dtype=td, device=DEV)
        ops.norm_add_norm(yd, dev(w.astype(np.float32)), res, eps, dev(w2.astype(np.float32)), h, eps2)
        ref = x.astype(np.float32) + pf.rms_norm(y.astype(np.float32), w.astype(np.float32), eps)
        assert np.abs(res.cpu().numpy() - ref).max() <= 1e-5 * (1 + np.abs(ref).max())
        close(h.float().cpu().numpy(), pf.rms_norm(ref, w2.astype(np.float32), eps2), dtype, f"width {width}")
        assert float(yd.abs().max()) == 0.0


def test_a_mixer_that_reads_another_layers_cache():
    """Two layers, the second without a down projection of its own: it reads what the first cached (the latent and the rotated
    key part as rotated there) with its own key and value matrices, queries and head count; prompts and single rows."""
    cfg = {"architecture": "Fudelorn", "vocab": 61, "width": 48, "norm": {"eps": 1e-5}, "layers": [
        {"type": "latent_attention", "mixer": pf._rotated(2, 16, 8, 24, 40, 8, 10000.0, {"factor": 8.0, "original": 16, "fast": 4.0, "slow": 1.0}), "mlp": None},
        {"type": "latent_attention", "mixer": pf._rotated(5, 8, 24, 16, 40, 8, 10000.0, {"factor": 8.0, "original": 16, "fast": 4.0, "slow": 1.0}, kv_from=0),
         "mlp": {"kind": "dense", "ff": 64}}]}
    w = pf.make_weights(cfg, 5)
    assert "l1.mix.dkv" not in w
    toks = tokens_for(2, 140, cfg["vocab"])
    ref = pf.forward(cfg, w, toks)
    for dtype in ("float32", "bfloat16"):
        eng = engine_for(cfg, w, dtype)
        assert len(eng.cache.groups) == 1 and [t.shape[0] for t in eng.cache.groups[0].planes] == [1, 1], "one layer's two planes serve both"
        close(run_whole(eng, toks), ref, dtype, "whole")
        close(run_cut(eng, toks, [100, 2, 20]), ref, dtype, "portions and single rows")


# ------------------------------------------------------------------ whole models through the engine

@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt(name, dtype):
    eng, cfg, w = small(name, dtype)
    toks = tokens_for(3, 150, cfg["vocab"])
    close(run_whole(eng, toks), pf.forward(cfg, w, toks), dtype)


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_token_by_token_and_portions(name, dtype):
    """Windows of 1, 5, 64 and 70 positions pass over decoded tokens and over the borders of 64-token pages; portions of two
    rows and of whole pages; bfloat16 portions go through the split kernel (short ones) and the expanded keys (long ones)."""
    eng, cfg, w = small(name, dtype)
    toks = tokens_for(5, 210, cfg["vocab"])
    ref = pf.forward(cfg, w, toks)
    close(run_cut(eng, toks, [60]), ref, dtype, "decoded from 60")
    close(run_cut(eng, toks, [1]), ref, dtype, "decoded from the first token")
    for cuts in ([2, 2, 61, 63, 2, 64, 16], [129, 2, 7, 70, 2], [64, 64, 64, 18], [9, 9, 100, 9]):
        close(run_cut(eng, toks, cuts), ref, dtype, f"portions {cuts}")


@pytest.mark.parametrize("dtype,name", [("float32", "A"), ("bfloat16", "A"), ("float32", "B"), ("bfloat16", "B")])
def test_unequal_batch_against_each_alone(dtype, name):
    from borrowed_compute_b200.engine import StepEntry

    eng, cfg, w = small(name, dtype)
    lens = [1, 77, 3, 130]
    seqs = [tokens_for(40 + i, n + 12, cfg["vocab"]) for i, n in enumerate(lens)]
    alone = [run_cut(eng, s, [n]) for s, n in zip(seqs, lens)]
    slots = [eng.acquire() for _ in seqs]
    got = [[rows] for rows in np.split(
        eng.step([StepEntry(s, q[:n], tuple(range(n))) for s, q, n in zip(slots, seqs, lens)]).cpu().numpy(), np.cumsum(lens)[:-1])]
    for t in range(12):
        live = [i for i in range(4) if t < 12 - 3 * (i == 2)]             # one sequence ends earlier
        out = eng.step([StepEntry(slots[i], [seqs[i][lens[i] + t]], (0,)) for i in live]).cpu().numpy()
        for j, i in enumerate(live):
            got[i].append(out[j:j + 1])
        if t == 8:
            eng.release(slots[2])
    for i in (0, 1, 3):
        eng.release(slots[i])
    for i in range(4):
        mine = np.concatenate(got[i])
        close(mine, pf.forward(cfg, w, seqs[i])[:len(mine)], dtype, f"sequence {i}")
        assert np.abs(mine - alone[i][:len(mine)]).max() <= (1e-5 if dtype == "float32" else 0.1), f"sequence {i} depends on the batch"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_slots_and_pages_used_again(dtype):
    from borrowed_compute_b200.engine import StepEntry

    cfg = pf.SMALL["A"]
    w = pf.make_weights(cfg, 21)
    eng = engine_for(cfg, w, dtype, max_tokens=448, max_slots=2, max_seq=320)
    first = None
    for turn in range(4):
        toks = tokens_for(60 + turn % 2, 200, cfg["vocab"])
        other = tokens_for(70 + turn, 100 + 20 * turn, cfg["vocab"])
        a, b = eng.acquire(), eng.acquire()
        eng.step([StepEntry(b, other, ())])
        got = eng.step([StepEntry(a, toks[:150], tuple(range(150)))]).cpu().numpy()
        eng.release(b)
        rest = [eng.step([StepEntry(a, [t], (0,))]).cpu().numpy() for t in toks[150:]]
        eng.release(a)
        got = np.concatenate([got] + rest)
        if turn < 2:
            close(got, pf.forward(cfg, w, toks), dtype, f"turn {turn}")
        if turn == 0:
            first = got
        if turn == 2:
            assert np.array_equal(got, first), "what a slot or a page held before shows"
    assert eng.cache.slots.live() == []


def test_a_page_that_held_numbers_that_are_none_changes_nothing():
    """A page comes back from another sequence with whatever that left; here every plane is filled with not-a-numbers between
    two runs of the same tokens, which then meet them past their last position and in pages they take anew."""
    eng, cfg, w = small("A", "bfloat16")
    toks = tokens_for(9, 100, cfg["vocab"])
    before = run_cut(eng, toks, [70, 3])
    for g in eng.cache.groups:
        for t in g.planes:
            t.fill_(float("nan"))
    after = run_cut(eng, toks, [70, 3])
    assert np.array_equal(before, after)


def test_long_decoding_and_the_first_tokens():
    for name, dtype in (("B", "float32"), ("A", "bfloat16")):
        eng, cfg, w = small(name, dtype)
        toks = tokens_for(8, 330, cfg["vocab"])
        ref = pf.forward(cfg, w, toks)
        close(run_cut(eng, toks, [3]), ref, dtype, "327 tokens decoded")
        for n in (1, 2, 3, 5):
            close(run_whole(eng, toks[:n]), ref[:n], dtype, f"the first {n}")


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 8])
def test_drawn_configurations(seed):
    """Sizes, layer orders, windows and constants drawn at random, among them values that make parts of the design equal or 1."""
    from borrowed_compute_b200.engine import StepEntry

    cfg = pf.drawn_config(np.random.default_rng(seed))
    w = pf.make_weights(cfg, seed)
    seqs = [tokens_for(seed * 10 + i, n, cfg["vocab"]) for i, n in enumerate([70, 5, 231])]
    refs = [pf.forward(cfg, w, q) for q in seqs]
    for dtype in ("float32", "bfloat16"):
        eng = engine_for(cfg, w, dtype, max_tokens=1024, max_slots=4, max_seq=256)
        slots = [eng.acquire() for _ in seqs]
        first = [30, 5, 229]
        out = eng.step([StepEntry(s, q[:n], tuple(range(n))) for s, q, n in zip(slots, seqs, first)]).cpu().numpy()
        got = [[a] for a in np.split(out, np.cumsum(first)[:-1])]
        got[0].append(eng.step([StepEntry(slots[0], seqs[0][30:68], tuple(range(38)))]).cpu().numpy())
        for t in range(2):
            out = eng.step([StepEntry(slots[0], [seqs[0][68 + t]], (0,)), StepEntry(slots[2], [seqs[2][229 + t]], (0,))]).cpu().numpy()
            got[0].append(out[:1])
            got[2].append(out[1:])
        for i in range(3):
            mostly_close(np.concatenate(got[i]), refs[i], dtype, f"{json.dumps(cfg)}: sequence {i} in {dtype}",
                         rounding=rounding_alone(cfg, w, seqs[i], refs[i]) if dtype == "bfloat16" else 0.0)


def test_sizes_that_are_multiples_of_nothing():
    """Widths, ranks, head sizes and a vocabulary that neither 8 nor 16 divides (two rotated dimensions, seven heads of four, one
    head): the products and the attention fall back to their plain kernels, and a window wider than the sequence hides nothing."""
    stretch = {"factor": 2.0, "original": 8, "fast": 2.0, "slow": 0.5}
    cfgs = [{"architecture": "Fudelorn", "vocab": 101, "width": 72, "norm": {"eps": 1e-5}, "layers": [
                {"type": "latent_attention", "mixer": pf._rotated(3, 12, 24, 12, 20, 2, 10000.0), "mlp": pf._moe(3, 2, 20, shared_ff=12)},
                {"type": "latent_attention_2", "mixer": pf._windowed(7, 4, 4, 20, 12, 3), "mlp": {"kind": "dense", "ff": 100}},
                {"type": "latent_attention", "mixer": pf._rotated(1, 20, 12, 4, 20, 2, 10000.0, kv_from=0), "mlp": pf._moe(2, 2, 36)}]},
            {"architecture": "Fudelorn", "vocab": 33, "width": 50, "norm": {"eps": 1e-6}, "layers": [
                {"type": "latent_attention_2", "mixer": pf._windowed(2, 6, 10, 6, 10, 1000), "mlp": None},
                {"type": "latent_attention", "mixer": pf._rotated(2, 10, 6, 14, 6, 6, 100.0, stretch), "mlp": {"kind": "dense", "ff": 30}}]}]
    for k, cfg in enumerate(cfgs):
        w = pf.make_weights(cfg, 50 + k)
        toks = tokens_for(5 + k, 150, cfg["vocab"])
        ref = pf.forward(cfg, w, toks)
        for dtype in ("float32", "bfloat16"):
            eng = engine_for(cfg, w, dtype, max_tokens=1024, max_slots=4, max_seq=256)
            mostly_close(run_cut(eng, toks, [70, 75]), ref, dtype, f"model {k} in {dtype}")


def write_folder(tmp_path, cfg, w):
    from borrowed_compute_b200.weights.safetensors_io import write_safetensors

    folder = str(tmp_path / "model")
    os.makedirs(folder)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      {n: torch.from_numpy(a) if a.dtype == np.int32 else torch.from_numpy(a).to(torch.bfloat16) for n, a in w.items()})
    return folder


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_trace_tool_replays_prompts_decoding_and_a_batch(tmp_path, dtype):
    """bin/trace_run on a folder of this design: whole prompts, single tokens after a prompt, and a batch of unequal requests that
    start together and end one after another, against the plain implementation."""
    import subprocess
    import sys

    from conftest import ROOT

    stretch = {"factor": 16.0, "original": 64, "fast": 16.0, "slow": 2.0}
    cfg = {"architecture": "Fudelorn", "vocab": 301, "width": 128, "norm": {"eps": 1e-6}, "layers": [
        {"type": "latent_attention", "mixer": pf._rotated(8, 32, 48, 64, 96, 32, 1e5, stretch), "mlp": pf._moe(8, 2, 32, shared_ff=64)},
        {"type": "latent_attention_2", "mixer": pf._windowed(2, 64, 64, 48, 64, 33), "mlp": {"kind": "dense", "ff": 192}},
        {"type": "latent_attention", "mixer": pf._rotated(3, 16, 16, 32, 96, 32, 1e5, stretch, kv_from=0), "mlp": None},
        {"type": "latent_attention_2", "mixer": pf._windowed(4, 16, 32, 32, 24, 100, scale=0.4), "mlp": pf._moe(6, 1, 40)},
    ]}
    w = pf.make_weights(cfg, 31)
    folder, out = write_folder(tmp_path, cfg, w), str(tmp_path / "out")
    a, b, c = (tokens_for(70 + i, n, cfg["vocab"]) for i, n in enumerate([150, 40, 9]))
    refs = {"a": pf.forward(cfg, w, a), "b": pf.forward(cfg, w, b), "c": pf.forward(cfg, w, c)}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:120], "want": [0, 64, 119]}], "end": []}]
    steps += [{"step": 1 + i, "entries": [{"id": "a", "tokens": [a[120 + i]], "want": [0]}], "end": ["a"] if i == 29 else []} for i in range(30)]
    steps.append({"step": 31, "entries": [{"id": "x", "tokens": a[:100], "want": [99]}, {"id": "y", "tokens": b[:30], "want": []},
                                          {"id": "z", "tokens": c[:5], "want": [4]}], "end": []})
    for i in range(10):
        live = [("x", a, 100), ("y", b, 30)] + ([("z", c, 5)] if i < 4 else [])
        steps.append({"step": 32 + i, "entries": [{"id": n, "tokens": [t[at + i]], "want": [0]} for n, t, at in live],
                      "end": (["z"] if i == 3 else []) + (["x", "y"] if i == 9 else [])})
    text = "".join(json.dumps(s) + "\n" for s in steps)
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out,
                          "--max-tokens", "512"], input=text, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [line for line in res.stdout.splitlines() if line.startswith("done")] == [f"done {s['step']}" for s in steps]
    V = cfg["vocab"]
    read = lambda n: np.fromfile(os.path.join(out, f"{n}.f32"), dtype="<f4").reshape(-1, V)      # noqa: E731
    got, want = [read(0)], [refs["a"][[0, 64, 119]]]
    for i in range(30):
        got.append(read(1 + i)), want.append(refs["a"][120 + i:121 + i])
    got.append(read(31)), want.append(np.stack([refs["a"][99], refs["c"][4]]))
    for i in range(10):
        got.append(read(32 + i)), want.append(np.stack([refs["a"][100 + i], refs["b"][30 + i]] + ([refs["c"][5 + i]] if i < 4 else [])))
    assert [g.shape for g in got] == [r.shape for r in want], "a step wrote other rows than were wanted"
    mostly_close(np.concatenate(got), np.concatenate(want), dtype, "the rows of all steps in their order")


def test_greedy_generation_through_the_entry_point(tmp_path):
    """A folder loaded by Local and by the command line; greedy tokens of a batch of unequal prompts against the plain loop."""
    import subprocess
    import sys

    from borrowed_compute_b200 import Local, Sampling
    from conftest import ROOT

    cfg = copy.deepcopy(pf.SMALL["A"])
    w = pf.make_weights(cfg, 21)
    folder = write_folder(tmp_path, cfg, w)
    prompts = [tokens_for(90 + i, n, cfg["vocab"]) for i, n in enumerate([3, 45, 1])]
    want = [pf.generate(cfg, w, p, 10) for p in prompts]
    model = Local.load(folder, dtype="float32", max_tokens=1024, max_slots=4, max_seq=128)
    out, stats = model.generate(prompts, 10, Sampling(), stop_ids=())
    assert out == want and stats.generated == 30
    assert model.engine.cache.slots.live() == []
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "bc-infer"), "generate", folder, ";".join(",".join(map(str, p)) for p in prompts),
                          "--max-tokens", "10", "--dtype", "float32", "--stop-ids", ""], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [[int(t) for t in line.split(",")] for line in res.stdout.strip().splitlines()] == want
    # bfloat16 decodes through captured graphs: the tokens are the oracle's wherever its two best scores lie apart
    model16 = Local.load(folder, dtype="bfloat16", max_tokens=1024, max_slots=4, max_seq=128)
    out16, _ = model16.generate(prompts, 10, Sampling(), stop_ids=())
    assert all(len(o) == 10 and all(0 <= t < cfg["vocab"] for t in o) for o in out16)
    for p, mine in zip(prompts, out16):
        toks = list(p)
        for t in mine:
            scores = np.sort(pf.forward(cfg, w, toks)[-1])
            if scores[-1] - scores[-2] > 0.25:
                assert t == int(np.argmax(pf.forward(cfg, w, toks)[-1])), "a clear choice was missed"
            toks.append(t)
