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

import math

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


# ------------------------------------------------------------------ models for the tests

def to_bf16(a):
    """Rounds to the nearest value that bfloat16 holds (ties to even), as float64."""
    f = np.ascontiguousarray(a, dtype=np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32).reshape(f.shape).astype(np.float64)


def talking_mixer(heads, kv_heads, dim, size, keep_first, rot_dims, softcap=15.0, scale=None, base=10000.0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale or 1.5 / math.sqrt(dim), "softcap": softcap,
         "mask": {"size": size, "keep_first": keep_first}}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
    return m


def latent_mixer(heads, dim, vdim, q_rank, kv_rank, rot_dim, scale=None, base=2000.0):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "rot_dim": rot_dim,
         "scale": scale or 1.0 / math.sqrt(dim + rot_dim)}
    if rot_dim:
        m["rot"] = {"base": base, "dims": rot_dim}
    return m


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff, shared, scale):
    f = {"kind": "moe", "router": {"experts": experts, "top": top, "scale": scale}, "expert": {"ff": ff}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def model(vocab, width, layers, eps=1e-5, embedding_scale=1.0, logit_scale=1.0):
    return {"architecture": "Logirax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embedding_scale},
            "logit_scale": logit_scale,
            "layers": [{"type": "attention" if "kv_heads" in m else "latent_attention", "mixer": m, "mlp": f} for m, f in layers]}


# Two small models that differ in every size and constant, in the order of their layers and in what they leave out.
SMALL = {
    "A": model(176, 64, [
        (talking_mixer(4, 2, 16, 24, 3, 8), moe(6, 2, 24, 16, 1.5)),
        (latent_mixer(3, 16, 24, 24, 40, 8), dense(48, 1.0)),
        (talking_mixer(4, 2, 16, 24, 3, 8), None),
        (latent_mixer(3, 16, 24, 24, 40, 8), moe(6, 2, 24, 16, 1.5)),
    ], eps=1e-5, embedding_scale=8.0, logit_scale=0.5),
    "B": model(97, 40, [
        (latent_mixer(2, 8, 8, 16, 16, 0), moe(3, 3, 8, 0, 1.0)),
        (talking_mixer(6, 6, 20, 70, 0, 20, softcap=0.0, base=300.0), dense(24, 0.5)),
        (talking_mixer(3, 1, 32, 9, 70, 0, softcap=4.0), moe(5, 1, 16, 8, 2.5)),
    ], eps=1e-6, embedding_scale=1.0, logit_scale=3.0),
}


def tensor_shapes(cfg):
    """name -> shape of every tensor a model of this configuration has."""
    E, out = cfg["width"], {"embed": (cfg["vocab"], cfg["width"]), "final.norm": (cfg["width"],)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out.update({p + "norm1": (E,), p + "norm1b": (E,), p + "shift": (E,)})
        if L["type"] == "attention":
            H, G, d = m["heads"], m["kv_heads"], m["dim"]
            out.update({p + "mix.q": (H * d, E), p + "mix.q.b": (H * d,), p + "mix.k": (G * d, E), p + "mix.k.b": (G * d,), p + "mix.talk": (H, H),
                        p + "mix.temp": (H,), p + "mix.g": (H * d, E), p + "mix.o": (E, H * d), p + "mix.o.b": (E,)})
        else:
            H, d, dv, QR, R, rd = m["heads"], m["dim"], m["vdim"], m["q_rank"], m["kv_rank"], m["rot_dim"]
            out.update({p + "mix.dq": (QR, E), p + "mix.dq.norm": (QR,), p + "mix.uq": (H * (d + rd), QR), p + "mix.dkv": (R + rd, E),
                        p + "mix.dkv.norm": (R,), p + "mix.uk": (H * d, R), p + "mix.uv": (H * dv, R), p + "mix.sink": (H,), p + "mix.g": (H, E),
                        p + "mix.o": (E, H * dv)})
        f = L.get("mlp")
        if f:
            out.update({p + "norm2": (E,), p + "norm2b": (E,)})
            if f["kind"] == "dense":
                out.update({p + "mlp.gate": (f["ff"], E), p + "mlp.up": (f["ff"], E), p + "mlp.down": (E, f["ff"])})
            else:
                ff = f["expert"]["ff"]
                for e in range(f["router"]["experts"]):
                    out.update({f"{p}mlp.e{e}.gate": (ff, E), f"{p}mlp.e{e}.up": (ff, E), f"{p}mlp.e{e}.down": (E, ff)})
                out[p + "mlp.router"] = (f["router"]["experts"], E)
                if f.get("shared"):
                    s = f["shared"]["ff"]
                    out.update({p + "mlp.shared.gate": (s, E), p + "mlp.shared.up": (s, E), p + "mlp.shared.down": (E, s)})
    return out


def make_weights(cfg, seed):
    """Random weights that bfloat16 holds exactly: matrices of spread 1 / sqrt(inputs) (gates and routers wider, so that they
    decide), norm weights and shifts around zero, heads' temperatures around one, a mix of heads near the identity, sinks that
    weigh about as much as a key."""
    rng = np.random.default_rng(seed)
    t = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if "norm" in name:
            a = 0.2 * rng.standard_normal(shape)
        elif last == "shift":
            a = rng.uniform(-0.2, 0.9, shape)
        elif last == "temp":
            a = rng.uniform(0.6, 1.6, shape)
        elif last == "talk":
            a = np.eye(shape[0]) + 0.4 * rng.standard_normal(shape) / math.sqrt(shape[0])
        elif last == "sink":
            a = rng.uniform(-1.0, 3.0, shape)
        elif last == "b":
            a = 0.3 * rng.standard_normal(shape)
        elif name == "embed":
            a = rng.standard_normal(shape)
        else:
            a = rng.standard_normal(shape) / math.sqrt(shape[-1]) * (3.0 if last in ("router", "g", "gate") else 1.0)
        t[name] = to_bf16(a)
    return t


def draw_config(rng):
    """A configuration whose sizes, constants and order of layers are drawn."""
    E = int(rng.choice([24, 40, 64, 72, 128]))
    layers = []
    for _ in range(int(rng.integers(2, 5))):
        if rng.random() < 0.5:
            G = int(rng.choice([1, 2, 3, 4, 8]))
            H = G * int(rng.choice([1, 2, 3, 4]))
            d = int(rng.choice([8, 12, 16, 32, 40, 64, 128]))
            rot = int(rng.choice([0, d // 2 // 2 * 2, d]))
            m = talking_mixer(H, G, d, int(rng.choice([1, 5, 33, 64, 100])), int(rng.choice([0, 1, 4, 66])), rot,
                              softcap=float(rng.choice([0.0, 5.0, 30.0])), base=float(rng.choice([100.0, 10000.0])))
        else:
            rd = int(rng.choice([0, 4, 8, 16]))
            m = latent_mixer(int(rng.choice([1, 2, 5, 18])), int(rng.choice([8, 16, 24, 48, 64])), int(rng.choice([8, 16, 40, 80])),
                             int(rng.choice([8, 12, 24, 96])), int(rng.choice([8, 16, 20, 48, 128])), rd, base=float(rng.choice([50.0, 50000.0])))
        kind = rng.random()
        if kind < 0.2:
            f = None
        elif kind < 0.5:
            f = dense(int(rng.choice([8, 20, 48])), float(rng.choice([0.5, 1.0, 7.0])))
        else:
            n = int(rng.choice([1, 3, 8]))
            f = moe(n, int(rng.integers(1, n + 1)), int(rng.choice([8, 12, 32])), int(rng.choice([0, 8, 24])), float(rng.choice([1.0, 2.5])))
        layers.append((m, f))
    return model(int(rng.choice([50, 131, 200])), E, layers, eps=float(rng.choice([1e-6, 1e-5, 1e-3])),
                 embedding_scale=float(rng.choice([1.0, 4.0, 12.0])), logit_scale=float(rng.choice([0.5, 1.0, 2.0])))


def router_margin(cfg, t, tokens):
    """The smallest gap between the last chosen and the first left-out router score over every row and layer of one sequence
    (infinite without routers): a sequence with a wide gap chooses the same experts under bfloat16 rounding."""
    t = {k: np.asarray(v, dtype=np.float64) for k, v in t.items()}
    x = t["embed"][np.asarray(tokens)] * float(cfg.get("embedding", {}).get("scale", 1.0))
    gap, eps = math.inf, float(cfg["norm"]["eps"])
    for i, L in enumerate(cfg["layers"]):
        f, p = L.get("mlp"), f"l{i}."
        h = token_shift(offset_norm(x, t[p + "norm1"], eps), t[p + "shift"])
        mix = talking_attention if L["type"] == "attention" else latent_attention
        x = x + offset_norm(mix(h, L["mixer"], t, p + "mix.", eps), t[p + "norm1b"], eps)
        if f:
            h2 = offset_norm(x, t[p + "norm2"], eps)
            if f["kind"] == "moe" and f["router"]["top"] < f["router"]["experts"]:
                s = np.sort(sigmoid(h2 @ t[p + "mlp.router"].T), axis=1)[:, ::-1]
                k = f["router"]["top"]
                gap = min(gap, float((s[:, k - 1] - s[:, k]).min()))
            x = x + offset_norm(feed_forward(h2, f, t, p + "mlp."), t[p + "norm2b"], eps)
    return gap
