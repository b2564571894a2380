"""A plain, slow NumPy restatement of the Logirax decoder, one function a mechanism, in float64.

It shares no code with the package: the tests hold the engine's kernels to it.  A model is a
config.json dictionary and a mapping from tensor names to arrays.  Notation: x is the residual
stream [T, E] of ONE sequence whose rows are positions 0 .. T-1; matrices are stored [out, in].

A layer:   x <- x + N1b(mixer(shift(N1 x)));  x <- x + N2b(ff(N2 x)),   N(x) = x / rms(x) * (1 + w).
shift(h)_t = h_t + (h_{t-1} - h_t) * s, with h_{-1} = 0 and s one number a channel.

Mixer "attention" (H query heads on G key heads, head width d):
    q = Wq h + bq, k = Wk h + bk, and the values ARE the keys as projected: v = k.
    q, k <- rotate the first ``rot.dims`` dimensions (pairs (i, i + dims/2)), then each head divided by its rms.
    s_h(i, j) = cap * tanh(q_h(i) . k_g(j) * scale * temp_h / cap);   s'_h = sum_m T[h, m] s_m   (mixing across heads)
    i sees j <= i with i - j < size or j < keep_first;  softmax;  heads side by side times sigmoid(Wg h);  Wo . + bo.

Mixer "latent_attention":
    cq = Nw(Wdq h), q = Wuq cq (head n: [dim plain | rot_dim rotated]);  Wdkv h = [z | r]:  c = Nw(z), r shared by the heads;
    s_n(i, j) = (q_plain . Wuk_n c_j + rot(q_rot) . rot(r_j)) * scale, pairs (2i, 2i + 1);  causal;
    p = exp(s) / (sum_j exp(s) + exp(sink_n));  head n = (sum_j p Wuv_n c_j) * sigmoid(Wg h)_n;  Wo on the heads side by side.
    (Nw: RMS norm with a plain weight.)

Feed-forward, dense:  g = min(Wgate h, L), u = clip(Wup h, -L, L),  Wdown (g sigmoid(1.702 g) (u + 1)).
Feed-forward, experts:  s = sigmoid(Wr h); the ``top`` largest choose; weights s / (sum of the chosen + 1e-20) * router.scale;
    sum of weight * Wdown(silu(Wgate h) * Wup h) over the chosen, plus a shared expert of the same form for every row.

Output: N(x) with ``final.norm``, scores = embed N(x) * logit_scale; rows enter as embed[token] * embedding.scale.
"""

from __future__ import annotations

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def offset_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * (1 + w): the weight is stored around zero."""
    x = np.asarray(x, dtype=np.float64)
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * (1.0 + np.asarray(w, dtype=np.float64))


def weighted_norm(x, w, eps):
    x = np.asarray(x, dtype=np.float64)
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * np.asarray(w, dtype=np.float64)


def unit_rms(x, eps):
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def token_shift(h, s, before=None):
    """h [T, E]; ``before``: the row ahead of h[0] (None: the sequence starts here)."""
    prev = np.concatenate([np.zeros_like(h[:1]) if before is None else np.asarray(before, dtype=np.float64)[None, :], h[:-1]], axis=0)
    return h + (prev - h) * np.asarray(s, dtype=np.float64)[None, :]


def frequencies(dims, base):
    return float(base) ** (-2.0 * np.arange(dims // 2, dtype=np.float64) / dims)


def rotate_half(x, positions, dims, base):
    """x [..., T, d]: the first ``dims`` dimensions turn, pairs (i, i + dims/2)."""
    a = np.asarray(positions, dtype=np.float64)[:, None] * frequencies(dims, base)[None, :]
    cos, sin = np.cos(a), np.sin(a)
    u, v = x[..., : dims // 2], x[..., dims // 2: dims]
    return np.concatenate([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], axis=-1)


def rotate_adjacent(x, positions, dims, base):
    """x [..., T, d]: the first ``dims`` dimensions turn, pairs (2i, 2i + 1)."""
    a = np.asarray(positions, dtype=np.float64)[:, None] * frequencies(dims, base)[None, :]
    cos, sin = np.cos(a), np.sin(a)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = np.array(x, dtype=np.float64, copy=True)
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def window_with_first(T, size, keep_first):
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return (j <= i) & (((i - j) < size) | (j < keep_first))


def causal(T):
    return np.arange(T)[None, :] <= np.arange(T)[:, None]


def softmax_rows(s, ok, sink=None):
    """Rows of s [..., T, T] over the visible columns; ``sink`` [...] adds exp(sink) to the denominator."""
    s = np.where(ok, s, -np.inf)
    m = s.max(axis=-1, keepdims=True)
    if sink is not None:
        m = np.maximum(m, sink[..., None, None])
    p = np.exp(s - m)
    z = p.sum(axis=-1, keepdims=True)
    if sink is not None:
        z = z + np.exp(sink[..., None, None] - m)
    return p / z


def talking_attention(h, m, t, pre, eps):
    """The mixer "attention" on its (shifted) input h [T, E]."""
    T = h.shape[0]
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = (h @ t[pre + "q"].T + t[pre + "q.b"]).reshape(T, H, d).transpose(1, 0, 2)
    k = (h @ t[pre + "k"].T + t[pre + "k.b"]).reshape(T, G, d).transpose(1, 0, 2)
    v = k
    pos = np.arange(T)
    rot = m.get("rot")
    if rot:
        q, k = rotate_half(q, pos, int(rot["dims"]), rot["base"]), rotate_half(k, pos, int(rot["dims"]), rot["base"])
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    rep = H // G
    s = np.einsum("hid,hjd->hij", q, np.repeat(k, rep, axis=0)) * float(m["scale"]) * t[pre + "temp"][:, None, None]
    cap = float(m.get("softcap") or 0.0)
    if cap:
        s = cap * np.tanh(s / cap)
    s = np.einsum("hm,mij->hij", t[pre + "talk"], s)
    mask = m.get("mask")
    ok = window_with_first(T, int(mask["size"]), int(mask.get("keep_first", 0))) if mask else causal(T)
    p = softmax_rows(s, ok[None])
    o = np.einsum("hij,hjd->ihd", p, np.repeat(v, rep, axis=0)).reshape(T, H * d)
    o = o * sigmoid(h @ t[pre + "g"].T)
    return o @ t[pre + "o"].T + t[pre + "o.b"]


def latent_attention(h, m, t, pre, eps):
    """The mixer "latent_attention" on its (shifted) input h [T, E]."""
    T = h.shape[0]
    H, d, dv, R, rd = int(m["heads"]), int(m["dim"]), int(m["vdim"]), int(m["kv_rank"]), int(m["rot_dim"])
    cq = weighted_norm(h @ t[pre + "dq"].T, t[pre + "dq.norm"], eps)
    q = (cq @ t[pre + "uq"].T).reshape(T, H, d + rd).transpose(1, 0, 2)
    z = h @ t[pre + "dkv"].T
    c, r = weighted_norm(z[:, :R], t[pre + "dkv.norm"], eps), z[:, R:]
    pos = np.arange(T)
    base = m["rot"]["base"] if rd else 1.0
    kp = (c @ t[pre + "uk"].T).reshape(T, H, d).transpose(1, 0, 2)
    vv = (c @ t[pre + "uv"].T).reshape(T, H, dv).transpose(1, 0, 2)
    s = np.einsum("hid,hjd->hij", q[..., :d], kp)
    if rd:
        qr, kr = rotate_adjacent(q[..., d:], pos, rd, base), rotate_adjacent(r, pos, rd, base)
        s = s + np.einsum("hid,jd->hij", qr, kr)
    s = s * float(m["scale"])
    p = softmax_rows(s, causal(T)[None], sink=np.asarray(t[pre + "sink"], dtype=np.float64))
    o = np.einsum("hij,hjd->ihd", p, vv) * sigmoid(h @ t[pre + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ t[pre + "o"].T


def clipped_glu(h, f, t, pre):
    L = float(f["limit"])
    g = np.minimum(h @ t[pre + "gate"].T, L)
    u = np.clip(h @ t[pre + "up"].T, -L, L)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ t[pre + "down"].T


def silu_glu(h, t, pre):
    g = h @ t[pre + "gate"].T
    return (g * sigmoid(g) * (h @ t[pre + "up"].T)) @ t[pre + "down"].T


def choose(s, top):
    """The ``top`` largest of every row of s, the lower index first among equals."""
    return np.argsort(-s, axis=-1, kind="stable")[:, :top]


def experts(h, f, t, pre, chosen=None):
    """Returns (result, the chosen experts [T, top], the router's scores [T, experts])."""
    n, top, factor = int(f["router"]["experts"]), int(f["router"]["top"]), float(f["router"].get("scale", 1.0))
    s = sigmoid(h @ t[pre + "router"].T)
    pick = choose(s, top) if chosen is None else chosen
    w = np.take_along_axis(s, pick, axis=1)
    w = w / (w.sum(axis=1, keepdims=True) + 1e-20) * factor
    out = np.zeros_like(h)
    for e in range(n):
        rows, col = np.nonzero(pick == e)
        if rows.size:
            out[rows] += w[rows, col][:, None] * silu_glu(h[rows], t, f"{pre}e{e}.")
    if f.get("shared"):
        out = out + silu_glu(h, t, pre + "shared.")
    return out, pick, s


def feed_forward(h, f, t, pre):
    if f["kind"] == "dense":
        return clipped_glu(h, f, t, pre)
    return experts(h, f, t, pre)[0]


def layer(x, i, cfg, t, trace=None):
    L, eps, p = cfg["layers"][i], float(cfg["norm"]["eps"]), f"l{i}."
    h = token_shift(offset_norm(x, t[p + "norm1"], eps), t[p + "shift"])
    mix = talking_attention if L["type"] == "attention" else latent_attention
    y = mix(h, L["mixer"], t, p + "mix.", eps)
    if trace is not None:
        trace[f"mix{i}"] = y
    x = x + offset_norm(y, t[p + "norm1b"], eps)
    if L.get("mlp"):
        x = x + offset_norm(feed_forward(offset_norm(x, t[p + "norm2"], eps), L["mlp"], t, p + "mlp."), t[p + "norm2b"], eps)
    return x


def forward(cfg, t, tokens, streams=None):
    """Scores [T, vocab] of one sequence; ``streams`` (a list) receives the stream after every layer."""
    t = {k: np.asarray(v, dtype=np.float64) for k, v in t.items()}
    x = t["embed"][np.asarray(tokens)] * float(cfg.get("embedding", {}).get("scale", 1.0))
    for i in range(len(cfg["layers"])):
        x = layer(x, i, cfg, t)
        if streams is not None:
            streams.append(x.copy())
    return offset_norm(x, t["final.norm"], float(cfg["norm"]["eps"])) @ t["embed"].T * float(cfg.get("logit_scale", 1.0))


def greedy(cfg, t, prompt, n):
    """The prompt's continuation by the largest score, ``n`` tokens."""
    tokens = list(prompt)
    for _ in range(n):
        tokens.append(int(forward(cfg, t, tokens)[-1].argmax()))
    return tokens[len(prompt):]
