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
