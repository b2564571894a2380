"""Grouped-query attention whose heads talk to one another before the softmax, whose values are its keys, and whose window
keeps a sequence's first positions.

    [zq | zk | zg] = W h                      fused projection, float:  W = [q; k; g]
    q = zq + bq,  k = zk + bk,  v = k          the values are the keys as projected: there is no value projection
    q, k <- rot(q), rot(k)                     the first ``rotary_dims`` dimensions of every head, pairs (i, i + rotary_dims / 2)
    q, k <- q / rms(q), k / rms(k)             every head by itself, over its ``head_dim`` values, without a weight
    raw_m(i, j) = q_m(i) . k_g(j) * scale * temp_m,  bounded: cap * tanh(raw / cap)  (``softcap`` 0: not bounded)
    s_h(i, j)   = sum_m talk[h, m] raw_m(i, j)                       every head's score mixes all heads' raw scores
    i sees j <= i with i - j < window or j < keep_first              (``window`` 0: every j <= i)
    out = Wo [ sigmoid(zg) * softmax_j(s_h) v_g ]_h + bo              the gate has one number a value

The cache keeps two planes a position, the rotated unit keys and the keys as projected, and never lets go of the pages of the
first ``keep_first`` positions.  Scores, the bound, the mix and the softmax are float on every path; q and both planes take the
activation type.  Tensor names after the prefix: q, q.b, k, k.b, g, o, o.b, temp [heads], talk [heads, heads].
"""

from __future__ import annotations

from typing import Any, Dict, Mapping, Optional

import torch

from .. import ops
from . import products
from .base import MIXERS, POSITION_ENCODINGS, CacheNeed, Mixer, RunMemory, Runtime, StepContext, TensorSpec


# Tests: "rows" (one block a row: the checked twin) or "tiles" (tensor-core tiles, bfloat16) wherever the sizes allow it;
# None: the part chooses.
force: Optional[str] = None


@MIXERS.register("talking_attention")
class TalkingAttention(Mixer):
    def __init__(self, hidden_size: int, heads: int, kv_heads: int, head_dim: int, norm_eps: float, position: Optional[Mapping[str, Any]] = None,
                 scale: Optional[float] = None, softcap: float = 0.0, window: int = 0, keep_first: int = 0, bias: bool = True):
        super().__init__(hidden_size=hidden_size, heads=heads, kv_heads=kv_heads, head_dim=head_dim, norm_eps=norm_eps, position=position,
                         scale=scale, softcap=softcap, window=window, keep_first=keep_first, bias=bias)
        self.hidden_size, self.heads, self.kv_heads, self.head_dim = int(hidden_size), int(heads), int(kv_heads), int(head_dim)
        self.norm_eps, self.softcap, self.window, self.keep_first, self.bias = float(norm_eps), float(softcap), int(window), int(keep_first), bool(bias)
        if self.heads <= 0 or self.kv_heads <= 0 or self.heads % self.kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} kv heads")
        if self.heads > ops.TALK_MAX_HEADS or not 0 < self.head_dim <= ops.TALK_MAX_DIM:
            raise ValueError(f"{heads} heads (at most {ops.TALK_MAX_HEADS}) of {head_dim} (at most {ops.TALK_MAX_DIM}) are refused by the "
                             "kernels of attention whose heads talk")
        if self.window < 0 or self.keep_first < 0 or self.softcap < 0.0:
            raise ValueError("a window, the positions it keeps and the bound on scores are not negative")
        self.scale = float(scale) if scale is not None else 1.0 / float(self.head_dim) ** 0.5
        pos = dict(position or {"kind": "none"})
        self.position = POSITION_ENCODINGS.get(pos.pop("kind"))(**pos)
        self.rotary_dims = int(getattr(self.position, "head_dim", 0))
        if self.rotary_dims > self.head_dim:
            raise ValueError(f"{self.rotary_dims} rotated dimensions do not fit a head of {self.head_dim}")
        if self.rotary_dims and getattr(self.position, "pairing", "half") != "half":
            raise ValueError("attention whose heads talk rotates pairs (i, i + rotary_dims / 2)")

    def tensors(self) -> Dict[str, TensorSpec]:
        q, kv, e, H = self.heads * self.head_dim, self.kv_heads * self.head_dim, self.hidden_size, self.heads
        out = {"q": TensorSpec((q, e)), "k": TensorSpec((kv, e)), "g": TensorSpec((q, e)), "o": TensorSpec((e, q)),
               "temp": TensorSpec((H,), role="vector", init="ones"), "talk": TensorSpec((H, H), role="vector", init="identity")}
        if self.bias:
            out.update({"q.b": TensorSpec((q,), role="vector", init="zeros"), "k.b": TensorSpec((kv,), role="vector", init="zeros"),
                        "o.b": TensorSpec((e,), role="vector", init="zeros")})
        return out

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed.keys_values(self.kv_heads, self.head_dim, self.window, keep_first=self.keep_first if self.window else 0)

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        super().load(tensors, rt)
        self.w_qkg = torch.cat([tensors["q"], tensors["k"], tensors["g"]], dim=0).contiguous()
        self.gate_at = (self.heads + self.kv_heads) * self.head_dim
        self.w_o = tensors["o"].contiguous()
        self.b_qk = torch.cat([tensors["q.b"].reshape(-1), tensors["k.b"].reshape(-1)]).contiguous() if self.bias else None
        self.b_o = tensors["o.b"].reshape(-1).contiguous() if self.bias else None
        self.temp, self.talk = tensors["temp"].reshape(-1).contiguous(), tensors["talk"].contiguous()
        self.position.load({}, rt)

    def path(self, ctx: StepContext, dtype: torch.dtype) -> str:
        tiles = ops.talk_tiles_accepts(self.heads, self.kv_heads, self.head_dim, dtype)
        if force == "rows" or (force == "tiles" and tiles):
            return force
        return "tiles" if tiles else "rows"

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext, mem: RunMemory) -> None:
        rows, dev = x.shape[0], x.device
        H, G, D = self.heads, self.kv_heads, self.head_dim
        if mem.planes is None or len(mem.planes) != 2:
            raise RuntimeError("attention whose heads talk was given no cache of its shape")
        proj = torch.empty((rows, self.w_qkg.shape[0]), dtype=torch.float32, device=dev)
        products.linear(x, self.w_qkg, proj, products.EPI_STORE_F32, "qkv product")
        table = self.position.rotary()
        q = torch.empty((rows, H * D), dtype=x.dtype, device=dev)
        gate = torch.empty((rows, H * D), dtype=torch.float32, device=dev)
        ops.talk_prepare(proj, self.gate_at, self.b_qk, None if table is None else table.cos_sin, ctx.row_pos, ctx.row_slot, mem.page_table, q,
                         mem.k_pages, mem.v_pages, gate, H, G, D, self.rotary_dims if table is not None else 0, self.norm_eps,
                         write_cache=mem.writes)
        att = torch.empty((rows, H * D), dtype=x.dtype, device=dev)
        if self.path(ctx, x.dtype) == "tiles":
            # Few rows a sequence (single rows above all) leave few blocks: the positions are then shared out over several.
            splits = ops.talk_tiles_splits(ctx.seqs, H, ctx.max_total, self.window, self.keep_first) if ctx.max_new <= 16 else 1
            ops.talk_tiles(q, mem.k_pages, mem.v_pages, mem.page_table, ctx.seq_rows, ctx.seq_slot, ctx.seq_start, gate, self.temp, self.talk, att,
                           ctx.seqs, ctx.max_new, H, G, D, self.window, self.keep_first, self.scale, self.softcap, splits=splits,
                           row_slot=ctx.row_slot)
        else:
            ops.talk_rows(q, mem.k_pages, mem.v_pages, mem.page_table, ctx.row_pos, ctx.row_slot, gate, self.temp, self.talk, att, H, G, D,
                          self.window, self.keep_first, self.scale, self.softcap)
        if self.b_o is not None:
            ops.add_bias(residual, self.b_o)
        products.linear(att, self.w_o, residual, products.EPI_ADD_F32, "output product")
