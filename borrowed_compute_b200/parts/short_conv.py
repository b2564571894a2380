"""A short causal convolution over time, channel by channel, added to its own input:

    out_t = h_t + sum_{j < taps} w[:, j] * h_(t - taps + 1 + j)        (zeros before position 0)

The last ``taps - 1`` inputs of every sequence are per-sequence state, so that a prompt cut
into portions, or continued token by token, convolves over the same inputs as a whole one.

Token shift is the case of two taps with one number a channel: every channel moves part of the way towards its value at
the position before,

    out_t = h_t + (h_(t - 1) - h_t) * s = h_t + s * h_(t - 1) + (-s) * h_t        (h before position 0 is zero),

so it is that convolution with the taps (s, -s), and the one row of state is the input at the last position.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from .base import CONVOLUTIONS, Runtime, ShortConvolution, StateNeed, StepContext, TensorSpec


@CONVOLUTIONS.register("causal_conv_residual")
class CausalConvResidual(ShortConvolution):
    def __init__(self, width: int, taps: int, tensor: str = "weight"):
        super().__init__(width=width, taps=taps, tensor=tensor)
        if int(taps) < 1:
            raise ValueError(f"a convolution needs at least one tap, got {taps}")
        self.width, self.taps, self.tensor = int(width), int(taps), str(tensor)

    def tensors(self) -> Dict[str, TensorSpec]:
        return {self.tensor: TensorSpec((self.width, self.taps), role="vector")}

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        super().load(tensors, rt)
        self.weight_t = tensors[self.tensor].t().contiguous()      # [taps, width]: neighbouring channels are neighbours in memory

    def state_need(self) -> Optional[StateNeed]:
        # One row more than needed when taps is 1, so that the tensor is never empty.
        return StateNeed((max(self.taps - 1, 1), self.width), None)     # the activation type

    def forward(self, h: torch.Tensor, out: torch.Tensor, ctx: StepContext, state: Optional[torch.Tensor], writes: bool = True) -> None:
        if state is None:
            raise RuntimeError("the convolution was given no state: the cache does not serve this block")
        tail = state if self.taps > 1 else state[:, :0]
        ops.short_conv(h, self.weight_t, tail, ctx.seq_rows, ctx.seq_slot, out, ctx.seqs, ctx.max_new, write_tail=writes)


@CONVOLUTIONS.register("token_shift")
class TokenShift(CausalConvResidual):
    """``tensor`` holds s, one number a channel."""

    def __init__(self, width: int, tensor: str = "shift"):
        super().__init__(width=width, taps=2, tensor=tensor)
        self.params = {"width": int(width), "tensor": str(tensor)}

    def tensors(self) -> Dict[str, TensorSpec]:
        return {self.tensor: TensorSpec((self.width,), role="vector")}

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        ShortConvolution.load(self, tensors, rt)
        s = tensors[self.tensor].reshape(-1)
        self.weight_t = torch.stack([s, -s]).contiguous()      # [2, width]: the tap on the position before, the tap on the row itself
