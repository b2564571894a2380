"""A feed-forward of many small gated experts of which every row uses a few, plus (optionally) a shared expert
that every row uses.

Router scores are sigmoid(W_router h) (or a softmax over the experts) in float; the ``top`` largest choose a row's
experts and are its weights, as they are or divided by their sum (``renormalize``), times ``weight_factor``.  The weight multiplies the
expert's input (``weight_on="input"``: the sum over the chosen experts of expert(w h)) or its output.  An expert is
down( silu(gate x) * (up x) ).

Variations a configuration may ask for: ``router="table"``: no router at all, a table [vocabulary, top] of expert numbers
(the entries of a row differ) names every token id's experts, each with weight 1 / top; ``expert="relu2"``: experts without a
gate, down( relu(up x)^2 ), the shared expert too; ``shared_gate``: the shared expert's result is multiplied by
sigmoid(w . h), one number a row (tensor ``shared.sg`` [1, width]).

Rows are sorted by expert on the device (nothing of a step's routing reaches the host, so a captured step replays),
the experts' two products run over the sorted rows, and a last kernel adds every row's results in the order of its
choices: no two blocks add into one place, so a row's result does not depend on the batch.
"""

from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from .. import ops
from .base import FEED_FORWARDS, FeedForward, Runtime, StepContext, TensorSpec
from . import products
from .mlp import PlainMLP, SwiGLU


force_simt = False      # tests: the CUDA-core products (the checked twin) for bfloat16 too


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    def __init__(self, hidden_size: int, experts: int, top: int, intermediate_size: int, shared_size: int = 0, score: str = "sigmoid",
                 renormalize: bool = False, weight_on: str = "input", router: str = "learned", expert: str = "swiglu", shared_gate: bool = False,
                 vocab_size: int = 0, weight_factor: float = 1.0):
        super().__init__(hidden_size=hidden_size, experts=experts, top=top, intermediate_size=intermediate_size, shared_size=shared_size,
                         score=score, renormalize=renormalize, weight_on=weight_on, router=router, expert=expert, shared_gate=shared_gate,
                         vocab_size=vocab_size, weight_factor=weight_factor)
        self.weight_factor = float(weight_factor)
        self.hidden_size, self.experts, self.top = int(hidden_size), int(experts), int(top)
        self.intermediate_size, self.shared_size = int(intermediate_size), int(shared_size)
        if not 0 < self.top <= self.experts or self.top > 16:
            raise ValueError(f"{top} of {experts} experts a row is outside what the router takes (1 to 16, at most all)")
        if score not in ("sigmoid", "softmax") or weight_on not in ("input", "output"):
            raise ValueError(f"score {score!r} must be 'sigmoid' or 'softmax', weight_on {weight_on!r} 'input' or 'output'")
        if router not in ("learned", "table") or expert not in ("swiglu", "relu2"):
            raise ValueError(f"router {router!r} must be 'learned' or 'table', expert {expert!r} 'swiglu' or 'relu2'")
        self.softmax, self.renormalize, self.on_input = score == "softmax", bool(renormalize), weight_on == "input"
        self.by_table, self.gated, self.shared_gate, self.vocab_size = router == "table", expert == "swiglu", bool(shared_gate), int(vocab_size)
        if self.by_table and self.weight_factor != 1.0:
            raise ValueError("experts named by a table weigh 1 / top each and take no factor")
        if self.by_table and (self.vocab_size <= 0 or self.on_input):
            raise ValueError("experts named by a table want the vocabulary's size and their weights on the output")
        if not self.gated and self.on_input:
            raise ValueError("experts without a gate take their weight on the output")
        if self.shared_gate and self.shared_size <= 0:
            raise ValueError("a gate on the shared expert needs a shared expert")
        self.shared = None
        if self.shared_size > 0:
            self.shared = SwiGLU(hidden_size, shared_size, gate="shared.gate", up="shared.up", down="shared.down") if self.gated else \
                PlainMLP(hidden_size, shared_size, activation=expert, up="shared.up", down="shared.down")

    def tensors(self) -> Dict[str, TensorSpec]:
        e, f = self.hidden_size, self.intermediate_size
        out = {"table": TensorSpec((self.vocab_size, self.top), role="index", init=f"distinct:{self.experts}")} if self.by_table else \
            {"router": TensorSpec((self.experts, e), role="vector")}
        for i in range(self.experts):
            if self.gated:
                out[f"e{i}.gate"] = TensorSpec((f, e))
            out.update({f"e{i}.up": TensorSpec((f, e)), f"e{i}.down": TensorSpec((e, f))})
        if self.shared is not None:
            out.update(self.shared.tensors())
        if self.shared_gate:
            out["shared.sg"] = TensorSpec((1, e))
        return out

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        super().load(tensors, rt)
        self.router = None if self.by_table else tensors["router"].contiguous()
        self.table = tensors["table"].contiguous() if self.by_table else None
        # [experts, 2 ff, width]: an expert's gate rows, then its up rows (without a gate: [experts, ff, width]); [experts, width, ff].
        self.w_gate_up = torch.stack([torch.cat([tensors[f"e{i}.gate"], tensors[f"e{i}.up"]], dim=0) if self.gated else tensors[f"e{i}.up"]
                                      for i in range(self.experts)]).contiguous()
        self.w_down = torch.stack([tensors[f"e{i}.down"] for i in range(self.experts)]).contiguous()
        if self.shared is not None:
            self.shared.load({n: tensors[n] for n in self.shared.tensors()}, rt)
        self.w_shared_gate = tensors["shared.sg"].reshape(-1).contiguous() if self.shared_gate else None

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext) -> None:
        rows, E, top, dev = x.shape[0], self.experts, self.top, x.device
        pairs = rows * top
        i32 = dict(dtype=torch.int32, device=dev)
        choice = torch.empty((rows, top), **i32)
        weight = torch.empty((rows, top), dtype=torch.float32, device=dev)
        if self.by_table:
            ops.moe_table_route(self.table, ctx.tokens, ctx.row_slot, choice, weight, E)
        else:
            logits = torch.empty((rows, E), dtype=torch.float32, device=dev)
            ops.moe_route(x, self.router, ctx.row_slot, logits, choice, weight, softmax=self.softmax, renorm=self.renormalize,
                          factor=self.weight_factor)
        # bfloat16 whose widths the tensor cores take: the rows are gathered in sorted order (times their weights: the weight
        # multiplies the expert's input) and both products run on tcgen05 tiles; else on the CUDA cores, gathering as they go.
        tensor_cores = not force_simt and self.intermediate_size % 8 == 0 and ops.gemm_tc_grouped_accepts(x, self.w_gate_up)
        tile_rows = ops.moe_simt_tile_rows()
        if tensor_cores:
            tile_rows = next((t for t in ops.GROUPED_TILE_ROWS if pairs <= t * E), ops.GROUPED_TILE_ROWS[-1])      # by the rows an expert gets on average
        max_tiles = ops.moe_max_tiles(pairs, E, tile_rows)
        ints = torch.empty(E + (E + 1) + (1 + 3 * max_tiles) + 2 * pairs, **i32)
        counts, offsets, table, perm, place = torch.split(ints, [E, E + 1, 1 + 3 * max_tiles, pairs, pairs])
        ops.moe_plan(choice, E, counts, offsets, table, perm, place, tile_rows)
        act = torch.empty((pairs, self.intermediate_size), dtype=x.dtype, device=dev)
        y = torch.empty((pairs, self.hidden_size), dtype=torch.float32, device=dev)
        if tensor_cores or not self.gated:
            xs = torch.empty((pairs, self.hidden_size), dtype=x.dtype, device=dev)
            ops.moe_gather(x, perm, offsets, weight, xs, E, top, weight_on_input=self.on_input)
        if not self.gated:
            # Experts without a gate: the activation works on the up product's float sums and rounds once, in the product's
            # epilogue on the tensor cores.
            if tensor_cores:
                ops.gemm_tc_grouped(xs, self.w_gate_up, act, table, False, tile_rows, max_tiles, relu2=True)
            else:
                z = torch.empty((pairs, self.intermediate_size), dtype=torch.float32, device=dev)
                ops.moe_product(False, xs, self.w_gate_up, table, perm, weight, z, top)
                ops.relu2(z, act)
        elif tensor_cores:
            ops.gemm_tc_grouped(xs, self.w_gate_up, act, table, True, tile_rows, max_tiles)
        else:
            ops.moe_product(True, x, self.w_gate_up, table, perm, weight, act, top, weight_on_input=self.on_input)
        if tensor_cores:
            ops.gemm_tc_grouped(act, self.w_down, y, table, False, tile_rows, max_tiles)
        else:
            ops.moe_product(False, act, self.w_down, table, perm, weight, y, top)
        ops.moe_combine(y, choice, place, weight, residual, weight_on_output=not self.on_input)
        if self.shared is not None and self.shared_gate:
            ys = torch.zeros((rows, self.hidden_size), dtype=torch.float32, device=dev)
            self.shared.forward(x, ys, ctx)
            ops.gated_add(x, self.w_shared_gate, ys, residual)
        elif self.shared is not None:
            self.shared.forward(x, residual, ctx)
