"""A plain, slow NumPy restatement of the Fudelorn decoder, one function a mechanism, in float64.

It shares no code with the package: the tests hold the engine's kernels to it.  A model is a
config.json dictionary and a mapping from tensor names to arrays.  Notation: x is the residual
stream [T, E] of ONE sequence whose rows are positions 0 .. T-1; matrices are stored [out, in].

A layer:   x <- x + N1b(mixer(N1 x));  x <- x + N2b(ff(N2 x)),   N = RMS norm with a weight.

Latent attention.  From the layer's input h:
    cq = N(Wdq h) (weight dq.norm),  q = Wuq cq, head by head [dim plain | rot_dim rotated];
    Wdkv h = [z | r]:  c = N(z) (weight dkv.norm, kv_rank wide),  r = the one rotated key part all heads share;
    head n:  k_n = Wuk_n c,  v_n = Wuv_n c,  score = (q_plain . k_n + rot(q_rot) . rot(r)) * scale;
    softmax over the visible positions;  head output times sigmoid(Wg h)_n;  Wo on the heads side by side.
A layer with ``kv_from`` has no Wdkv and reads c and rot(r) of the named layer.  A ``mask.size`` w lets
position i see j with 0 <= i - j < w.  The second kind of mixer is the same without a rotated part.

Rotation of (u_i, u_{i + d/2}) by a = p f_i, with the frequencies stretched for long contexts
(``rot.scaling``) and cos and sin multiplied by a constant of that stretch.

Feed-forward: Wdown relu(Wup h)^2; or a table from token id to ``top`` experts of that form, each weighted
1 / top, plus a shared expert times sigmoid(wsg . h).
"""

from __future__ import annotations

import math

import numpy as np


def same(a):
    return a


def rms_norm(x, w, eps):
    x = np.asarray(x, dtype=np.float64)
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * np.asarray(w, dtype=np.float64)


def stretched_frequencies(dims, base, scaling):
    """(f [dims / 2], m): radians a position of every rotated pair, and the factor on cos and sin."""
    i = np.arange(dims // 2, dtype=np.float64)
    f = float(base) ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn(t):      # the (fractional) pair whose wave turns t times within the original length
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turn(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, f, m):
    """x [..., T, d] with pairs (i, i + d/2); positions [T]."""
    d = x.shape[-1]
    a = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    cos, sin = np.cos(a) * m, np.sin(a) * m
    u, v = x[..., : d // 2], x[..., d // 2:]
    return np.concatenate([u * cos - v * sin, v * cos + u * sin], axis=-1)


def visible(T, window):
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    ok = j <= i
    if window:
        ok &= (i - j) < window
    return ok


def softmax_rows(s, ok):
    s = np.where(ok, s, -np.inf)
    s = s - s.max(axis=-1, keepdims=True)
    p = np.exp(s)
    return p / p.sum(axis=-1, keepdims=True)


def latent_keys(h, w, m, eps, r=same):
    """What a layer caches: c [T, kv_rank] and the rotated shared key part [T, rot_dim] (or None)."""
    T = h.shape[0]
    R, rot = int(m["kv_rank"]), int(m.get("rot_dim", 0))
    z = r(h @ np.asarray(w["dkv"], dtype=np.float64).T)
    c = r(rms_norm(z[:, :R], w["dkv.norm"], eps))
    if rot == 0:
        return c, None
    f, mag = stretched_frequencies(int(m["rot"]["dims"]), float(m["rot"]["base"]), m["rot"].get("scaling"))
    return c, r(rotate(z[:, R:R + rot], np.arange(T), f, mag))


def latent_attention(h, w, m, eps, kept=None, r=same):
    """The mixer's output [T, E] for one sequence from position 0; ``kept`` = (c, rotated key part) of
    another layer for a mixer that has no down projection of its own.  Also returns what it keeps."""
    h = np.asarray(h, dtype=np.float64)
    T = h.shape[0]
    H, D, DV = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    R, rot = int(m["kv_rank"]), int(m.get("rot_dim", 0))
    window = int(m["mask"]["size"]) if m.get("mask") else 0
    W = {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}
    cq = r(rms_norm(r(h @ W["dq"].T), W["dq.norm"], eps))
    q = r(cq @ W["uq"].T).reshape(T, H, D + rot)
    c, kr = latent_keys(h, w, m, eps, r) if kept is None else kept
    k = r(c @ W["uk"].T).reshape(T, H, D)
    v = r(c @ W["uv"].T).reshape(T, H, DV)
    gate = 1.0 / (1.0 + np.exp(-(h @ W["g"].T)))           # [T, H]
    ok = visible(T, window)
    out = np.zeros((T, H, DV))
    if rot:
        f, mag = stretched_frequencies(int(m["rot"]["dims"]), float(m["rot"]["base"]), m["rot"].get("scaling"))
    for n in range(H):
        s = q[:, n, :D] @ k[:, n, :].T
        if rot:
            s = s + r(rotate(q[:, n, D:], np.arange(T), f, mag)) @ kr.T
        p = softmax_rows(s * float(m["scale"]), ok)
        out[:, n, :] = r(r(p @ v[:, n, :]) * gate[:, n:n + 1])
    return r(out.reshape(T, H * DV) @ W["o"].T), (c, kr)


def relu_squared_mlp(h, up, down, r=same):
    z = np.maximum(np.asarray(h, dtype=np.float64) @ np.asarray(up, dtype=np.float64).T, 0.0)
    return r(r(z * z) @ np.asarray(down, dtype=np.float64).T)


def table_experts(h, tokens, w, mlp, r=same):
    """w: the feed-forward's tensors by the names after 'mlp.'."""
    h = np.asarray(h, dtype=np.float64)
    top = int(mlp["router"]["top"])
    table = np.asarray(w["table"])
    out = np.zeros((h.shape[0], np.asarray(w["e0.down"]).shape[0]))
    for t, tok in enumerate(tokens):
        for e in table[int(tok)]:
            out[t] += relu_squared_mlp(h[t:t + 1], w[f"e{int(e)}.up"], w[f"e{int(e)}.down"], r)[0] / top
    if mlp.get("shared"):
        g = 1.0 / (1.0 + np.exp(-(h @ np.asarray(w["shared.sg"], dtype=np.float64).T)))      # [T, 1]
        out += relu_squared_mlp(h, w["shared.up"], w["shared.down"], r) * g
    return r(out)


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, tokens, taps=None, r=same):
    """Scores [T, vocab] of one sequence's tokens from position 0; ``taps`` (a list) receives the stream after every layer.
    ``r`` is applied wherever the design lets a value be kept in 16 bits (the inputs and results of matrix products and the
    activations between them; never the stream, a norm's sums, scores or softmax weights): with ``to_bf16`` the scores show how far
    rounding alone moves each row."""
    eps = float(config["norm"]["eps"])
    x = np.asarray(tensors["embed"], dtype=np.float64)[np.asarray(tokens)]
    kept = {}
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = r(rms_norm(x, tensors[p + "norm1"], eps))
        y, kept[i] = latent_attention(h, sub(tensors, p + "mix."), m, eps, kept.get(m.get("kv_from")) if "kv_from" in m else None, r)
        x = x + rms_norm(y, tensors[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = r(rms_norm(x, tensors[p + "norm2"], eps))
            if mlp["kind"] == "dense":
                y = relu_squared_mlp(h, tensors[p + "mlp.up"], tensors[p + "mlp.down"], r)
            else:
                y = table_experts(h, tokens, sub(tensors, p + "mlp."), mlp, r)
            x = x + rms_norm(y, tensors[p + "norm2b"], eps)
        if taps is not None:
            taps.append(x.copy())
    return r(rms_norm(x, tensors["final.norm"], eps)) @ np.asarray(tensors["head"], dtype=np.float64).T


# ------------------------------------------------------------------------------ small models for the tests

def _rot(dims, base, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling:
        out["scaling"] = scaling
    return out


def _windowed(heads, dim, vdim, q_rank, kv_rank, window, scale=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "mask": {"size": window}}
    m["scale"] = scale if scale is not None else 1.0 / math.sqrt(dim)
    return m


def _rotated(heads, dim, vdim, q_rank, kv_rank, rot_dim, base, scaling=None, kv_from=None, scale=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "rot_dim": rot_dim, "rot": _rot(rot_dim, base, scaling)}
    m["scale"] = scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _moe(experts, top, ff, shared_ff=0):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared_ff:
        out["shared"] = {"ff": shared_ff}
    return out


# A: windows of 5 and 70 positions (inside a page and across a page's border), a stretched rotation that the tests'
# positions pass, a layer that reads another's cache and has no feed-forward, three experts a token.
SMALL_A = {
    "architecture": "Fudelorn", "vocab": 160, "width": 96, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "latent_attention_2", "mixer": _windowed(3, 16, 24, 40, 48, 5), "mlp": {"kind": "dense", "ff": 176}},
        {"type": "latent_attention", "mixer": _rotated(2, 32, 16, 64, 72, 8, 10000.0, {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}),
         "mlp": _moe(5, 3, 40, shared_ff=56)},
        {"type": "latent_attention_2", "mixer": _windowed(5, 8, 8, 24, 32, 70, scale=0.5), "mlp": _moe(4, 2, 48)},
        {"type": "latent_attention", "mixer": _rotated(4, 24, 40, 32, 72, 8, 10000.0, {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}, kv_from=1),
         "mlp": None},
    ],
}
# B: one head, one expert a token, a window of one position (a row sees itself alone), a latent whose width is no
# multiple of eight, a rotation without a stretch, a window exactly a page long.
SMALL_B = {
    "architecture": "Fudelorn", "vocab": 97, "width": 64, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "latent_attention", "mixer": _rotated(1, 16, 16, 16, 36, 4, 500000.0, scale=0.3), "mlp": _moe(3, 1, 32, shared_ff=16)},
        {"type": "latent_attention_2", "mixer": _windowed(2, 12, 20, 8, 20, 1), "mlp": {"kind": "dense", "ff": 72}},
        {"type": "latent_attention_2", "mixer": _windowed(4, 16, 8, 32, 64, 64), "mlp": {"kind": "dense", "ff": 40}},
    ],
}
SMALL = {"A": SMALL_A, "B": SMALL_B}


def to_bf16(a):
    """Rounds float values to the nearest bfloat16 (ties to even), kept as float32."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32).reshape(np.shape(a))


def make_weights(config, seed, spread=1.0):
    """Seeded weights by tensor name, every value a bfloat16 (so that engines of both types hold the same numbers): matrices of
    spread ``spread`` / sqrt(inputs), norm weights around one, tables whose rows name different experts."""
    rng = np.random.default_rng(seed)
    E, V = int(config["width"]), int(config["vocab"])

    def mat(rows, cols, s=spread):
        return to_bf16(rng.standard_normal((rows, cols)) * s / math.sqrt(cols))

    def vec(n):
        return to_bf16(1.0 + 0.25 * rng.uniform(-1, 1, n))

    w = {"embed": to_bf16(rng.standard_normal((V, E))), "final.norm": vec(E), "head": mat(V, E)}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H, D, DV, R, rot = m["heads"], m["dim"], m["vdim"], m["kv_rank"], m.get("rot_dim", 0)
        w[p + "norm1"], w[p + "norm1b"] = vec(E), vec(E)
        w[p + "mix.dq"], w[p + "mix.dq.norm"] = mat(m["q_rank"], E, 2.0 * spread), vec(m["q_rank"])
        w[p + "mix.uq"] = mat(H * (D + rot), m["q_rank"], 2.0 * spread)
        if "kv_from" not in m:
            w[p + "mix.dkv"], w[p + "mix.dkv.norm"] = mat(R + rot, E, 2.0 * spread), vec(R)
        w[p + "mix.uk"], w[p + "mix.uv"] = mat(H * D, R, 2.0 * spread), mat(H * DV, R)
        w[p + "mix.g"], w[p + "mix.o"] = mat(H, E, 2.0 * spread), mat(E, H * DV)
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        w[p + "norm2"], w[p + "norm2b"] = vec(E), vec(E)
        if mlp["kind"] == "dense":
            w[p + "mlp.up"], w[p + "mlp.down"] = mat(mlp["ff"], E, 2.0 * spread), mat(E, mlp["ff"])
            continue
        n, top = mlp["router"]["experts"], mlp["router"]["top"]
        for e in range(n):
            w[p + f"mlp.e{e}.up"], w[p + f"mlp.e{e}.down"] = mat(mlp["expert"]["ff"], E, 2.0 * spread), mat(E, mlp["expert"]["ff"])
        w[p + "mlp.table"] = np.stack([rng.permutation(n)[:top] for _ in range(V)]).astype(np.int32)
        if mlp.get("shared"):
            f = mlp["shared"]["ff"]
            w[p + "mlp.shared.up"], w[p + "mlp.shared.down"], w[p + "mlp.shared.sg"] = mat(f, E, 2.0 * spread), mat(E, f), mat(1, E, 2.0 * spread)
    return w


def drawn_config(rng):
    """A configuration with sizes drawn at random: other widths, head counts, layer orders, windows and constants every time."""
    E = int(rng.choice([32, 48, 80, 128]))
    layers, owners = [], []
    for i in range(int(rng.integers(2, 5))):
        mlp = [None, {"kind": "dense", "ff": int(rng.choice([24, 56, 96]))},
               _moe(int(rng.integers(2, 7)), 1, int(rng.choice([16, 40])), shared_ff=int(rng.choice([0, 24])))][int(rng.integers(0, 3))]
        if mlp and mlp["kind"] == "moe":
            mlp["router"]["top"] = int(rng.integers(1, mlp["router"]["experts"] + 1))
        H, D, DV = int(rng.integers(1, 6)), int(rng.choice([8, 16, 24, 40])), int(rng.choice([8, 16, 48]))
        qr, R = int(rng.choice([8, 24, 48])), int(rng.choice([16, 36, 64, 136]))
        if rng.random() < 0.5:
            m = _windowed(H, D, DV, qr, R, int(rng.choice([1, 2, 7, 33, 64, 65, 200])), scale=float(rng.uniform(0.1, 0.5)))
            layers.append({"type": "latent_attention_2", "mixer": m, "mlp": mlp})
        else:
            scaling = None if rng.random() < 0.4 else {"factor": float(rng.choice([2.0, 8.0])), "original": int(rng.choice([16, 64])),
                                                      "fast": float(rng.choice([4.0, 32.0])), "slow": float(rng.choice([0.5, 1.0]))}
            rot, base = int(rng.choice([2, 4, 8, 16])), float(rng.choice([100.0, 10000.0, 500000.0]))
            kv_from = None
            if owners and rng.random() < 0.5:
                kv_from = int(rng.choice(owners))
                o = layers[kv_from]["mixer"]
                R, rot, base, scaling = o["kv_rank"], o["rot_dim"], o["rot"]["base"], o["rot"].get("scaling")
            m = _rotated(H, D, DV, qr, R, rot, base, scaling, kv_from=kv_from, scale=float(rng.uniform(0.1, 0.5)))
            layers.append({"type": "latent_attention", "mixer": m, "mlp": mlp})
            if kv_from is None:
                owners.append(i)
    return {"architecture": "Fudelorn", "vocab": int(rng.choice([50, 131, 300])), "width": E, "norm": {"eps": float(rng.choice([1e-5, 1e-6]))},
            "layers": layers}


def generate(config, tensors, prompt, n):
    """Greedy: the n tokens after ``prompt``, the lowest id winning a tie."""
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(forward(config, tensors, toks)[-1])))
    return toks[len(prompt):]
