"""The dense gated feed-forward: down( silu(x gate^T) * (x up^T) ), added into the residual
stream (crates/bc-infer/src/model.rs:341-345).  Gate and up are one product whose epilogue
applies the gate."""

from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from . import products
from .base import FEED_FORWARDS, FeedForward, Runtime, StepContext, TensorSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """``gate``, ``up`` and ``down`` are the names the three matrices carry after the part's prefix."""

    def __init__(self, hidden_size: int, intermediate_size: int, gate: str = "gate_proj.weight", up: str = "up_proj.weight",
                 down: str = "down_proj.weight"):
        super().__init__(hidden_size=hidden_size, intermediate_size=intermediate_size, gate=gate, up=up, down=down)
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.names = (str(gate), str(up), str(down))

    def tensors(self) -> Dict[str, TensorSpec]:
        e, f = self.hidden_size, self.intermediate_size
        gate, up, down = self.names
        return {gate: TensorSpec((f, e)), up: TensorSpec((f, e)), down: TensorSpec((e, f))}

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        super().load(tensors, rt)
        gate, up, down = self.names
        # Gate rows stacked on up rows: the product's epilogue pairs row j with row F + j.
        self.w_gate_up = torch.cat([tensors[gate], tensors[up]], dim=0).contiguous()
        self.w_down = tensors[down].contiguous()

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext) -> None:
        h = torch.empty((x.shape[0], self.intermediate_size), dtype=x.dtype, device=x.device)
        products.linear(x, self.w_gate_up, h, products.EPI_SWIGLU, "gate/up product")
        products.linear(h, self.w_down, residual, products.EPI_ADD_F32, "down product")


@FEED_FORWARDS.register("plain_mlp")
class PlainMLP(FeedForward):
    """down( act(up x) ) without a gate; ``activation``: "relu2", the square of relu, applied to the up product's float sums in its
    epilogue and rounded once.  ``up`` and ``down`` are the names the matrices carry after the part's prefix."""

    ACTIVATIONS = ("relu2",)

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "relu2", up: str = "up", down: str = "down"):
        super().__init__(hidden_size=hidden_size, intermediate_size=intermediate_size, activation=activation, up=up, down=down)
        if activation not in self.ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is not known (known: {list(self.ACTIVATIONS)})")
        self.hidden_size, self.intermediate_size, self.activation = int(hidden_size), int(intermediate_size), activation
        self.names = (str(up), str(down))

    def tensors(self) -> Dict[str, TensorSpec]:
        e, f = self.hidden_size, self.intermediate_size
        return {self.names[0]: TensorSpec((f, e)), self.names[1]: TensorSpec((e, f))}

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        super().load(tensors, rt)
        self.w_up, self.w_down = tensors[self.names[0]].contiguous(), tensors[self.names[1]].contiguous()

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext) -> None:
        act = torch.empty((x.shape[0], self.intermediate_size), dtype=x.dtype, device=x.device)
        products.linear(x, self.w_up, act, products.EPI_RELU2, "up product")
        products.linear(act, self.w_down, residual, products.EPI_ADD_F32, "down product")


@FEED_FORWARDS.register("clipped_glu")
class ClippedGLU(FeedForward):
    """down( g sigmoid(alpha g) (u + 1) ) with g = min(gate x, limit) and u = clamp(up x, -limit, limit): a gated feed-forward
    whose gate saturates from above, whose up branch is bounded on both sides and carries a one.  Gate and up are one product
    with float sums; the activation works on those and rounds once: in the product's epilogue on the tensor cores, in a kernel
    of its own after the CUDA-core product (the 32-bit path, and the checked twin: ``fused = False``)."""

    fused = True

    def __init__(self, hidden_size: int, intermediate_size: int, limit: float, alpha: float = 1.702, gate: str = "gate", up: str = "up",
                 down: str = "down"):
        super().__init__(hidden_size=hidden_size, intermediate_size=intermediate_size, limit=limit, alpha=alpha, gate=gate, up=up, down=down)
        self.hidden_size, self.intermediate_size, self.limit, self.alpha = int(hidden_size), int(intermediate_size), float(limit), float(alpha)
        if self.limit <= 0.0:
            raise ValueError(f"the bound of a clipped gate must be positive, got {limit}")
        self.names = (str(gate), str(up), str(down))

    def tensors(self) -> Dict[str, TensorSpec]:
        e, f = self.hidden_size, self.intermediate_size
        gate, up, down = self.names
        return {gate: TensorSpec((f, e)), up: TensorSpec((f, e)), down: TensorSpec((e, f))}

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        super().load(tensors, rt)
        gate, up, down = self.names
        self.w_gate_up = torch.cat([tensors[gate], tensors[up]], dim=0).contiguous()      # gate rows, then up rows
        self.w_down = tensors[down].contiguous()

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext) -> None:
        rows, F = x.shape[0], self.intermediate_size
        act = torch.empty((rows, F), dtype=x.dtype, device=x.device)
        if self.fused and products.takes_tensor_cores(x, self.w_gate_up):
            products.linear(x, self.w_gate_up, act, products.EPI_SWIGLU, "gate/up product", glu=(self.limit, self.alpha))
        else:
            z = torch.empty((rows, 2 * F), dtype=torch.float32, device=x.device)
            products.linear(x, self.w_gate_up, z, products.EPI_STORE_F32, "gate/up product")
            ops.glu_clipped(z, act, self.limit, self.alpha)
        products.linear(act, self.w_down, residual, products.EPI_ADD_F32, "down product")
