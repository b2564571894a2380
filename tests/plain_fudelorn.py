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


def latent_keys(h, w, m, eps):
    """What a layer caches: c [T, kv_rank] and the rotated shared key part [T, rot_dim] (or None)."""
    T = h.shape[0]
    R, rot = int(m["kv_rank"]), int(m.get("rot_dim", 0))
    z = h @ np.asarray(w["dkv"], dtype=np.float64).T
    c = rms_norm(z[:, :R], w["dkv.norm"], eps)
    if rot == 0:
        return c, None
    f, mag = stretched_frequencies(int(m["rot"]["dims"]), float(m["rot"]["base"]), m["rot"].get("scaling"))
    return c, rotate(z[:, R:R + rot], np.arange(T), f, mag)


def latent_attention(h, w, m, eps, kept=None):
    """The mixer's output [T, E] for one sequence from position 0; ``kept`` = (c, rotated key part) of
    another layer for a mixer that has no down projection of its own.  Also returns what it keeps."""
    h = np.asarray(h, dtype=np.float64)
    T = h.shape[0]
    H, D, DV = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    R, rot = int(m["kv_rank"]), int(m.get("rot_dim", 0))
    window = int(m["mask"]["size"]) if m.get("mask") else 0
    W = {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}
    cq = rms_norm(h @ W["dq"].T, W["dq.norm"], eps)
    q = (cq @ W["uq"].T).reshape(T, H, D + rot)
    c, kr = latent_keys(h, w, m, eps) if kept is None else kept
    k = (c @ W["uk"].T).reshape(T, H, D)
    v = (c @ W["uv"].T).reshape(T, H, DV)
    gate = 1.0 / (1.0 + np.exp(-(h @ W["g"].T)))           # [T, H]
    ok = visible(T, window)
    out = np.zeros((T, H, DV))
    if rot:
        f, mag = stretched_frequencies(int(m["rot"]["dims"]), float(m["rot"]["base"]), m["rot"].get("scaling"))
    for n in range(H):
        s = q[:, n, :D] @ k[:, n, :].T
        if rot:
            s = s + rotate(q[:, n, D:], np.arange(T), f, mag) @ kr.T
        p = softmax_rows(s * float(m["scale"]), ok)
        out[:, n, :] = (p @ v[:, n, :]) * gate[:, n:n + 1]
    return out.reshape(T, H * DV) @ W["o"].T, (c, kr)


def relu_squared_mlp(h, up, down):
    z = np.maximum(np.asarray(h, dtype=np.float64) @ np.asarray(up, dtype=np.float64).T, 0.0)
    return (z * z) @ np.asarray(down, dtype=np.float64).T


def table_experts(h, tokens, w, mlp):
    """w: the feed-forward's tensors by the names after 'mlp.'."""
    h = np.asarray(h, dtype=np.float64)
    top = int(mlp["router"]["top"])
    table = np.asarray(w["table"])
    out = np.zeros((h.shape[0], np.asarray(w["e0.down"]).shape[0]))
    for t, tok in enumerate(tokens):
        for e in table[int(tok)]:
            out[t] += relu_squared_mlp(h[t:t + 1], w[f"e{int(e)}.up"], w[f"e{int(e)}.down"])[0] / top
    if mlp.get("shared"):
        g = 1.0 / (1.0 + np.exp(-(h @ np.asarray(w["shared.sg"], dtype=np.float64).T)))      # [T, 1]
        out += relu_squared_mlp(h, w["shared.up"], w["shared.down"]) * g
    return out


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, tokens, taps=None):
    """Scores [T, vocab] of one sequence's tokens from position 0; ``taps`` (a list) receives the stream after every layer."""
    eps = float(config["norm"]["eps"])
    x = np.asarray(tensors["embed"], dtype=np.float64)[np.asarray(tokens)]
    kept = {}
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = rms_norm(x, tensors[p + "norm1"], eps)
        y, kept[i] = latent_attention(h, sub(tensors, p + "mix."), m, eps, kept.get(m.get("kv_from")) if "kv_from" in m else None)
        x = x + rms_norm(y, tensors[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, tensors[p + "norm2"], eps)
            if mlp["kind"] == "dense":
                y = relu_squared_mlp(h, tensors[p + "mlp.up"], tensors[p + "mlp.down"])
            else:
                y = table_experts(h, tokens, sub(tensors, p + "mlp."), mlp)
            x = x + rms_norm(y, tensors[p + "norm2b"], eps)
        if taps is not None:
            taps.append(x.copy())
    return rms_norm(x, tensors["final.norm"], eps) @ np.asarray(tensors["head"], dtype=np.float64).T
