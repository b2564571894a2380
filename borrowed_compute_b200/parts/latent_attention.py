"""Latent attention: queries pass a normed low-rank bottleneck, and keys and values of every head are products of ONE
normed vector a position, the latent c (``kv_rank`` values), which is all the cache keeps, beside one rotated key part
(``rot_dim`` values) that the heads share if the mixer rotates at all.

    [zq | zc, zr | zg] = W h                fused down projection, float:  W = [dq; dkv; g]
    cq = N(zq),  c = N(zc),  r = rot(zr)     N: RMS norm with a plain weight; c and r go into the cache
    q  = Wuq cq                              head n: [dim plain values | rot_dim rotated values]
    score_n(i, j) = (q_n . Wuk_n c_j + rot(qr_n) . r_j) * scale,   softmax over the visible j
    out = Wo [ sigmoid(zg_n) * Wuv_n sum_j p_n(i, j) c_j ]_n

The scores and the sum over positions run over the cache as it is (the key products are moved to the query's side,
a_n = Wuk_n^T q_n, and Wuv_n comes after the sum), so a position is read once for all heads and never expanded.

Parameters: a sliding ``window`` (0: every earlier position), the score ``scale`` (default (dim + rot_dim)^-1/2), the
position encoding of the rotated part (a PartSpec-like mapping; {"kind": "none"} with ``rot_dim`` 0), and ``own_kv``:
False for a mixer without a down projection to c and r, whose run reads another run's cache (RunSpec.memory_of) with
its own Wuk and Wuv.  Tensor names after the prefix: dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o.
"""

from __future__ import annotations

from typing import Any, Dict, Mapping, Optional

import torch

from .. import ops
from . import products
from .base import MIXERS, POSITION_ENCODINGS, CacheNeed, Mixer, RunMemory, Runtime, StepContext, TensorSpec


force_rows = False      # tests: the one-warp-a-row kernel (the checked twin) for bfloat16 too


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    def __init__(self, hidden_size: int, heads: int, head_dim: int, value_dim: int, q_rank: int, kv_rank: int, norm_eps: float,
                 rot_dim: int = 0, position: Optional[Mapping[str, Any]] = None, scale: Optional[float] = None, window: int = 0,
                 own_kv: bool = True):
        super().__init__(hidden_size=hidden_size, heads=heads, head_dim=head_dim, value_dim=value_dim, q_rank=q_rank, kv_rank=kv_rank,
                         norm_eps=norm_eps, rot_dim=rot_dim, position=position, scale=scale, window=window, own_kv=own_kv)
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
        if self.rot_dim and getattr(self.position, "pairing", "half") != "half":
            raise ValueError("latent attention rotates pairs (i, i + rot_dim / 2)")

    def tensors(self) -> Dict[str, TensorSpec]:
        e, H = self.hidden_size, self.heads
        out = {"dq": TensorSpec((self.q_rank, e)), "dq.norm": TensorSpec((self.q_rank,), role="vector", init="ones"),
               "uq": TensorSpec((H * (self.head_dim + self.rot_dim), self.q_rank)),
               "uk": TensorSpec((H * self.head_dim, self.kv_rank)), "uv": TensorSpec((H * self.value_dim, self.kv_rank)),
               "g": TensorSpec((H, e)), "o": TensorSpec((e, H * self.value_dim))}
        if self.own_kv:
            out.update({"dkv": TensorSpec((self.kv_rank + self.rot_dim, e)), "dkv.norm": TensorSpec((self.kv_rank,), role="vector", init="ones")})
        return out

    def cache_need(self) -> Optional[CacheNeed]:
        planes = ((1, self.kv_rank),) + (((1, self.rot_dim),) if self.rot_dim else ())
        return CacheNeed(planes, self.window)

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        super().load(tensors, rt)
        down = [tensors["dq"]] + ([tensors["dkv"]] if self.own_kv else []) + [tensors["g"]]
        self.w_down = torch.cat(down, dim=0).contiguous()
        self.kv_at = self.q_rank if self.own_kv else -1
        self.gate_at = self.q_rank + (self.kv_rank + self.rot_dim if self.own_kv else 0)
        self.q_norm = tensors["dq.norm"].contiguous()
        self.kv_norm = tensors["dkv.norm"].contiguous() if self.own_kv else None
        self.w_uq, self.w_uk, self.w_uv, self.w_o = (tensors[n].contiguous() for n in ("uq", "uk", "uv", "o"))
        self.position.load({}, rt)

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
        a = torch.empty((rows, H, R + ROT), dtype=x.dtype, device=dev)
        ops.latent_query(q, self.w_uk, cos_sin, ctx.row_pos, a, H, D, ROT, R)
        found = torch.empty((rows, H, R), dtype=x.dtype, device=dev)
        self.attend(a, found, ctx, c_pages, r_pages, mem.page_table)
        att = torch.empty((rows, H * DV), dtype=x.dtype, device=dev)
        ops.latent_values(found, self.w_uv, gate, att, H, R, DV)
        products.linear(att, self.w_o, residual, products.EPI_ADD_F32, "output product")

    def attend(self, a: torch.Tensor, out: torch.Tensor, ctx: StepContext, c_pages: torch.Tensor, r_pages: Optional[torch.Tensor],
               page_table: torch.Tensor) -> None:
        H, R, ROT = self.heads, self.kv_rank, self.rot_dim
        if not force_rows and hasattr(ops, "latent_tiles") and ops.latent_tiles_accepts(H, R, ROT, a.dtype):
            ops.latent_tiles(a, c_pages, r_pages, page_table, ctx.seq_rows, ctx.seq_slot, ctx.seq_start, out, ctx.seqs, ctx.max_new, H, R, ROT,
                             self.window, self.scale)
            return
        ops.latent_rows(a, c_pages, r_pages, page_table, ctx.row_pos, ctx.row_slot, out, H, R, ROT, self.window, self.scale)
