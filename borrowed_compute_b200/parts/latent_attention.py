"""Latent attention: queries pass a normed low-rank bottleneck, and keys and values of every head are products of ONE
normed vector a position, the latent c (``kv_rank`` values), which is all the cache keeps, beside one rotated key part
(``rot_dim`` values) that the heads share if the mixer rotates at all.

    [zq | zc, zr | zg] = W h                fused down projection, float:  W = [dq; dkv; g]
    cq = N(zq),  c = N(zc),  r = rot(zr)     N: RMS norm with a plain weight; c and r go into the cache
    q  = Wuq cq                              head n: [dim plain values | rot_dim rotated values]
    score_n(i, j) = (q_n . Wuk_n c_j + rot(qr_n) . r_j) * scale,   softmax over the visible j
    out = Wo [ sigmoid(zg_n) * Wuv_n sum_j p_n(i, j) c_j ]_n

With few rows a sequence (decoding, short portions) the scores and the sum over positions run over the cache as it is: the
key products are moved to the query's side, a_n = Wuk_n^T q_n, and Wuv_n comes after the sum, so a position is read once
for all heads and never expanded.  With many rows a sequence (prompts) what the step sees of the cache is expanded once
into every head's keys and values, and the prompt attention kernels of the other mixers run over those.

Parameters: a sliding ``window`` (0: every earlier position), the score ``scale`` (default (dim + rot_dim)^-1/2), the
position encoding of the rotated part (a PartSpec-like mapping; {"kind": "none"} with ``rot_dim`` 0), ``own_kv``:
False for a mixer without a down projection to c and r, whose run reads another run's cache (RunSpec.memory_of) with
its own Wuk and Wuv, and ``sink``: every head's softmax has one more term e^sink_n in its denominator, a learned number a
head (tensor ``sink``) that has no key and no value, so that a row's weights add up to less than one.
Tensor names after the prefix: dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o, sink.

A position encoding that pairs neighbours, (2i, 2i + 1), needs no kernel of its own: a score is a sum over the rotated
dimensions, so the same permutation of them on the query's and on the key's side leaves it as it is.  The rows of Wuq and of
Wdkv that make the rotated parts are reordered once, when the weights are loaded, so that pair i sits at (i, i + rot_dim / 2),
and the kernels rotate those; the cache then keeps r in that order, which only this mixer reads.
"""

from __future__ import annotations

from typing import Any, Dict, Mapping, Optional

import torch

from .. import ops
from . import products
from .base import MIXERS, POSITION_ENCODINGS, CacheNeed, Mixer, RunMemory, Runtime, StepContext, TensorSpec


# Tests: "rows" (the one-warp-a-row kernel, the checked twin), "split" (the split kernel for few rows a sequence) or "expand"
# (keys and values expanded for the prompt attention kernels) wherever the sizes allow it; None: the part chooses.
force: Optional[str] = None
# A sequence that brings at most this many rows takes the split kernel row by row; more are worth expanding what they see.
SHORT_PORTION = 8


def seen_pages(ctx: StepContext, window: int, device: torch.device):
    """The pages of positions that this step's sequences see, as scratch pages in the order of the sequences: (pages, ints) with
    ints on the device [6, n]: the slot, first position and last live position of every scratch page; then a page table
    [seqs, widest] over scratch pages flattened, the sequences' scratch slots, and their starts counted from the first page
    each sees.  Planned once a step and window (the host knows the lengths of a prompt step)."""
    key = ("latent_pages", int(window))
    if key in ctx.extras:
        return ctx.extras[key]
    first, count, pg = [], [], []
    for s in range(ctx.seqs):
        slot, start = ctx.host_seq_slot[s], ctx.host_seq_start[s]
        new = ctx.host_seq_rows[s + 1] - ctx.host_seq_rows[s]
        if slot < 0 or new <= 0:
            first.append(0), count.append(0)
            continue
        lo = max(0, start - window + 1) if window > 0 else 0
        p0, p1 = lo // ops.PAGE, (start + new - 1) // ops.PAGE
        first.append(p0), count.append(p1 - p0 + 1)
        pg += [(slot, ops.PAGE * p, start + new - 1) for p in range(p0, p1 + 1)]
    pages, widest = len(pg), max(count + [1])
    table, at = [], 0
    for n in count:
        table += list(range(at, at + n)) + [-1] * (widest - n)
        at += n
    n = max(pages, ctx.seqs * widest, 1)
    rows = [[g[0] for g in pg], [g[1] for g in pg], [g[2] for g in pg], table,
            [s if count[s] else -1 for s in range(ctx.seqs)],
            [ctx.host_seq_start[s] - ops.PAGE * first[s] for s in range(ctx.seqs)]]
    ints = torch.tensor([r + [0] * (n - len(r)) for r in rows], dtype=torch.int32).to(device, non_blocking=True)
    ctx.extras[key] = (pages, widest, ints)
    return ctx.extras[key]


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    def __init__(self, hidden_size: int, heads: int, head_dim: int, value_dim: int, q_rank: int, kv_rank: int, norm_eps: float,
                 rot_dim: int = 0, position: Optional[Mapping[str, Any]] = None, scale: Optional[float] = None, window: int = 0,
                 own_kv: bool = True, sink: bool = False):
        super().__init__(hidden_size=hidden_size, heads=heads, head_dim=head_dim, value_dim=value_dim, q_rank=q_rank, kv_rank=kv_rank,
                         norm_eps=norm_eps, rot_dim=rot_dim, position=position, scale=scale, window=window, own_kv=own_kv, sink=sink)
        self.has_sink = bool(sink)
        self.hidden_size, self.heads, self.head_dim, self.value_dim = int(hidden_size), int(heads), int(head_dim), int(value_dim)
        self.q_rank, self.kv_rank, self.rot_dim, self.window = int(q_rank), int(kv_rank), int(rot_dim), int(window)
        self.norm_eps, self.own_kv = float(norm_eps), bool(own_kv)
        if min(self.heads, self.head_dim, self.value_dim, self.q_rank, self.kv_rank) <= 0 or self.rot_dim < 0 or self.window < 0:
            raise ValueError("latent attention wants positive sizes")
        if self.kv_rank > ops.LATENT_MAX_RANK or self.rot_dim > ops.LATENT_MAX_ROT:
            raise ValueError(f"a latent of {kv_rank} (at most {ops.LATENT_MAX_RANK}) or a rotated part of {rot_dim} (at most "
                             f"{ops.LATENT_MAX_ROT}) is refused by the latent attention kernels")
        self.scale = float(scale) if scale is not None else 1.0 / float(self.head_dim + self.rot_dim) ** 0.5
        pos = dict(position or {"kind": "none"})
        self.position = POSITION_ENCODINGS.get(pos.pop("kind"))(**pos)
        rotated = int(getattr(self.position, "head_dim", 0))
        if rotated != self.rot_dim:
            raise ValueError(f"the position encoding rotates {rotated} dimensions, the mixer's rotated part has {self.rot_dim}")
        self.adjacent = bool(self.rot_dim) and getattr(self.position, "pairing", "half") == "adjacent"

    def tensors(self) -> Dict[str, TensorSpec]:
        e, H = self.hidden_size, self.heads
        out = {"dq": TensorSpec((self.q_rank, e)), "dq.norm": TensorSpec((self.q_rank,), role="vector", init="ones"),
               "uq": TensorSpec((H * (self.head_dim + self.rot_dim), self.q_rank)),
               "uk": TensorSpec((H * self.head_dim, self.kv_rank)), "uv": TensorSpec((H * self.value_dim, self.kv_rank)),
               "g": TensorSpec((H, e)), "o": TensorSpec((e, H * self.value_dim))}
        if self.own_kv:
            out.update({"dkv": TensorSpec((self.kv_rank + self.rot_dim, e)), "dkv.norm": TensorSpec((self.kv_rank,), role="vector", init="ones")})
        if self.has_sink:
            out["sink"] = TensorSpec((H,), role="vector")
        return out

    def cache_need(self) -> Optional[CacheNeed]:
        planes = ((1, self.kv_rank),) + (((1, self.rot_dim),) if self.rot_dim else ())
        return CacheNeed(planes, self.window)

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        super().load(tensors, rt)
        if self.adjacent:
            # Neighbouring pairs (2i, 2i + 1) moved to (i, i + rot_dim / 2), on the query's side and on the key's alike.
            tensors = dict(tensors)
            D, ROT, H = self.head_dim, self.rot_dim, self.heads
            order = torch.cat([torch.arange(0, ROT, 2), torch.arange(1, ROT, 2)]).to(tensors["uq"].device)
            uq = tensors["uq"].reshape(H, D + ROT, self.q_rank)
            tensors["uq"] = torch.cat([uq[:, :D], uq[:, D:][:, order]], dim=1).reshape(H * (D + ROT), self.q_rank)
            if self.own_kv:
                tensors["dkv"] = torch.cat([tensors["dkv"][: self.kv_rank], tensors["dkv"][self.kv_rank:][order]], dim=0)
        self.sink = tensors["sink"].reshape(-1).contiguous() if self.has_sink else None
        down = [tensors["dq"]] + ([tensors["dkv"]] if self.own_kv else []) + [tensors["g"]]
        self.w_down = torch.cat(down, dim=0).contiguous()
        self.kv_at = self.q_rank if self.own_kv else -1
        self.gate_at = self.q_rank + (self.kv_rank + self.rot_dim if self.own_kv else 0)
        self.q_norm = tensors["dq.norm"].contiguous()
        self.kv_norm = tensors["dkv.norm"].contiguous() if self.own_kv else None
        self.w_uq, self.w_uk, self.w_uv, self.w_o = (tensors[n].contiguous() for n in ("uq", "uk", "uv", "o"))
        self.position.load({}, rt)
        # For prompts: one matrix [Wuk; Wuv] that expands gathered latents into every head's plain key part and values.
        self.widths = ops.latent_expand_widths(self.heads, self.head_dim + self.rot_dim, self.value_dim, self.kv_rank, self.rot_dim, rt.dtype)
        self.w_ukv = torch.cat([self.w_uk, self.w_uv], dim=0).contiguous() if self.widths is not None else None

    def path(self, ctx: StepContext, dtype: torch.dtype) -> str:
        split = ops.latent_decode_accepts(self.heads, self.kv_rank, self.rot_dim, dtype)
        expand = self.widths is not None and dtype == torch.bfloat16 and not ctx.decode and len(ctx.host_seq_rows) > ctx.seqs
        if force == "rows" or (force == "split" and split) or (force == "expand" and expand):
            return force
        if split and (ctx.decode or ctx.max_new <= SHORT_PORTION or not expand):
            return "split"
        return "expand" if expand else "rows"

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext, mem: RunMemory) -> None:
        rows, dev = x.shape[0], x.device
        H, D, DV, R, ROT = self.heads, self.head_dim, self.value_dim, self.kv_rank, self.rot_dim
        if mem.planes is None or len(mem.planes) != (2 if ROT else 1):
            raise RuntimeError("latent attention was given no cache of its shape: the run it reads keeps other planes")
        c_pages, r_pages = mem.planes[0], (mem.planes[1] if ROT else None)
        table = self.position.rotary()
        cos_sin = None if table is None else table.cos_sin
        proj = torch.empty((rows, self.w_down.shape[0]), dtype=torch.float32, device=dev)
        products.linear(x, self.w_down, proj, products.EPI_STORE_F32, "latent down product")
        cq = torch.empty((rows, self.q_rank), dtype=x.dtype, device=dev)
        gate = torch.empty((rows, H), dtype=torch.float32, device=dev)
        ops.latent_prepare(proj, self.q_rank, self.kv_at, R, ROT, self.gate_at, H, self.q_norm, self.kv_norm, cos_sin, ctx.row_pos, ctx.row_slot,
                           mem.page_table, c_pages, r_pages, cq, gate, self.norm_eps, write_cache=mem.writes and self.own_kv)
        q = torch.empty((rows, H * (D + ROT)), dtype=torch.float32, device=dev)
        products.linear(cq, self.w_uq, q, products.EPI_STORE_F32, "query up product")
        att = torch.empty((rows, H * DV), dtype=x.dtype, device=dev)
        path = self.path(ctx, x.dtype)
        if path == "expand":
            self.expanded(q, gate, att, ctx, c_pages, r_pages, mem.page_table, cos_sin)
        else:
            # The key products move to the query's side and the value products come after the sum over positions.
            a = torch.empty((rows, H, R + ROT), dtype=x.dtype, device=dev)
            ops.latent_query(q, self.w_uk, cos_sin, ctx.row_pos, a, H, D, ROT, R)
            found = torch.empty((rows, H, R), dtype=x.dtype, device=dev)
            if path == "split":
                ops.latent_decode(a, c_pages, r_pages, mem.page_table, ctx.row_pos, ctx.row_slot, found, H, R, ROT, self.window, self.scale,
                                  reach=ctx.max_total, sink=self.sink)
            else:
                ops.latent_rows(a, c_pages, r_pages, mem.page_table, ctx.row_pos, ctx.row_slot, found, H, R, ROT, self.window, self.scale,
                                sink=self.sink)
            ops.latent_values(found, self.w_uv, gate, att, H, R, DV)
        products.linear(att, self.w_o, residual, products.EPI_ADD_F32, "output product")

    def expanded(self, q: torch.Tensor, gate: torch.Tensor, att: torch.Tensor, ctx: StepContext, c_pages: torch.Tensor,
                 r_pages: Optional[torch.Tensor], page_table: torch.Tensor, cos_sin: Optional[torch.Tensor]) -> None:
        """Many rows a sequence: what the step sees of the cache is gathered, multiplied by [Wuk; Wuv] once, laid out as pages of
        every head's keys [Wuk_n c | r] and values, and the prompt attention kernels run over those pages."""
        rows, dev, dt = q.shape[0], q.device, att.dtype
        H, D, DV, R, ROT = self.heads, self.head_dim, self.value_dim, self.kv_rank, self.rot_dim
        KP, VP = self.widths
        pages, widest, ints = seen_pages(ctx, self.window, dev)
        qh = torch.empty((rows, H * KP), dtype=dt, device=dev)
        ops.latent_heads(q, cos_sin, ctx.row_pos, qh, H, D, ROT)
        found = torch.zeros((rows, H * VP), dtype=dt, device=dev)      # rows of no sequence are left as they are by the kernels
        if pages:
            S = pages * ops.PAGE
            seen_c = torch.empty((S, R), dtype=dt, device=dev)
            seen_r = torch.empty((S, ROT), dtype=dt, device=dev) if ROT else None
            ops.latent_gather(c_pages, r_pages, page_table, ints[0], ints[1], ints[2], seen_c, seen_r, pages)
            kv = torch.empty((S, H * (D + DV)), dtype=dt, device=dev)
            products.linear(seen_c, self.w_ukv, kv, products.EPI_STORE, "key and value up product")
            keys = torch.empty((pages, H, ops.PAGE, KP), dtype=dt, device=dev)
            values = torch.empty((pages, H, ops.PAGE, VP), dtype=dt, device=dev)
            ops.latent_spread(kv, seen_r, keys, values, H, D, DV, ROT)
            scratch_table = ints[3][: ctx.seqs * widest].view(ctx.seqs, widest)
            ops.attention_prefill(qh, H * KP, keys, values, scratch_table, ctx.seq_rows, ints[4], ints[5], found, ctx.seqs, ctx.max_new, H, H, KP,
                                  window=self.window, scale=self.scale, value_dim=VP, sink=self.sink)
        ops.latent_gate(found, gate, att, H, DV)
