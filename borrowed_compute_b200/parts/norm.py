"""RMSNorm: x / sqrt(mean(x^2) + eps) * w, statistics in float32
(crates/bc-infer/src/model.rs:381-389).  A folder may store the weight around zero: ``offset`` is what is added to
the stored values to give w (1 for such folders), once, in float32, when the weights are loaded."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from .base import NORMS, Norm, Runtime, TensorSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """``tensor`` is the name the weight carries after the part's prefix ("weight" in
    published Llama folders; other formats name the norm itself)."""

    def __init__(self, size: int, eps: float, tensor: str = "weight", offset: float = 0.0):
        super().__init__(size=size, eps=eps, tensor=tensor, offset=offset)
        self.size, self.eps, self.tensor, self.offset = int(size), float(eps), str(tensor), float(offset)

    def tensors(self) -> Dict[str, TensorSpec]:
        return {self.tensor: TensorSpec((self.size,), role="vector", init="ones" if self.offset == 0.0 else "normal")}

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        super().load(tensors, rt)
        self.weight = tensors[self.tensor] if self.offset == 0.0 else (tensors[self.tensor] + self.offset).contiguous()

    def forward(self, residual: torch.Tensor, out: torch.Tensor, gather: Optional[torch.Tensor] = None) -> None:
        ops.rmsnorm(residual, self.weight, out, self.eps, gather)
