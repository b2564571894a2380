"""Block arrangements.

The pre-norm residual block: x += mixer(norm1(x)); x += feed_forward(norm2(x))
(crates/bc-infer/src/model.rs:323-345).

The parallel block: x += mixer(conv(norm1(x))) + feed_forward(norm2(x)), both branches reading
the same x, the mixer's input first passing a short causal convolution over time whose last
inputs are per-sequence state.  The feed-forward (and its norm) may be left out; a feed-forward
without a norm of its own reads what the mixer reads, x += mixer(h) + feed_forward(h) with
h = norm1(x).

The sandwich block: a norm before and after each sublayer, x += norm1b(mixer(conv(norm1(x)))); x += norm2b(ff(norm2(x))).
The second half may be left out, and so may the short convolution (or token shift) of the mixer's input."""

from __future__ import annotations

import torch

from typing import Dict, Mapping

from .. import ops
from .norm import RMSNorm
from .short_conv import CausalConvResidual
from .base import BLOCKS, CONVOLUTIONS, FEED_FORWARDS, MIXERS, NORMS, Block, RunMemory, Runtime, StateNeed, StepContext


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    ROLES = {"norm1": NORMS, "mixer": MIXERS, "norm2": NORMS, "feed_forward": FEED_FORWARDS}

    def forward(self, residual: torch.Tensor, ctx: StepContext, mem: RunMemory, rt: Runtime) -> None:
        h = torch.empty((residual.shape[0], self.hidden_size), dtype=rt.dtype, device=residual.device)
        self.norm1.forward(residual, h)
        self.mixer.forward(h, residual, ctx, mem)
        self.norm2.forward(residual, h)
        self.feed_forward.forward(h, residual, ctx)


@BLOCKS.register("parallel")
class ParallelBlock(Block):
    ROLES = {"norm1": NORMS, "conv": CONVOLUTIONS, "mixer": MIXERS, "norm2": NORMS, "feed_forward": FEED_FORWARDS}
    OPTIONAL = ("conv", "norm2", "feed_forward")

    def __init__(self, parts, hidden_size: int):
        super().__init__(parts, hidden_size)
        if self.norm2 is not None and self.feed_forward is None:
            raise ValueError("a parallel block has no second norm without a feed-forward")
        if self.norm2 is None and self.feed_forward is not None and self.conv is not None:
            raise ValueError("a feed-forward that shares the mixer's norm cannot follow a convolution of the mixer's input")

    def _one_statistic(self) -> bool:
        """Whether both norms are plain RMS norms with the same eps, so that they share the row's statistic."""
        return type(self.norm1) is RMSNorm and (self.norm2 is None or (type(self.norm2) is RMSNorm and self.norm2.eps == self.norm1.eps))

    def state_needs(self) -> Dict[str, StateNeed]:
        needs = super().state_needs()
        need = None if self.conv is None else self.conv.state_need()
        if need is not None:
            needs["conv"] = need
        return needs

    def forward(self, residual: torch.Tensor, ctx: StepContext, mem: RunMemory, rt: Runtime) -> None:
        rows = residual.shape[0]
        # Both branches read the stream as it is now, so both norms run before either adds to it.
        h = torch.empty((rows, self.hidden_size), dtype=rt.dtype, device=residual.device)
        h2 = torch.empty_like(h) if self.norm2 is not None else None
        if self._one_statistic():
            # Two RMS norms of the same rows are one kernel; in a step of single rows the convolution rides in it too.
            conv = self.conv if self.conv is not None and ctx.decode and isinstance(self.conv, CausalConvResidual) else None
            tail = None if conv is None else mem.states.get("conv")
            if conv is not None and tail is None:
                raise RuntimeError("the convolution was given no state: the cache does not serve this block")
            ops.norm_pair(residual, self.norm1.weight, None if h2 is None else self.norm2.weight, h, h2, self.norm1.eps,
                          None if conv is None else conv.weight_t, None if conv is None else (tail if conv.taps > 1 else tail[:, :0]),
                          ctx.row_slot, write_tail=mem.writes)
            done = conv is not None
        else:
            self.norm1.forward(residual, h)
            if h2 is not None:
                self.norm2.forward(residual, h2)
            done = False
        if self.conv is not None and not done:
            hc = torch.empty_like(h)
            self.conv.forward(h, hc, ctx, mem.states.get("conv"), mem.writes)
            h = hc
        self.mixer.forward(h, residual, ctx, mem)
        if self.feed_forward is not None:
            self.feed_forward.forward(h if h2 is None else h2, residual, ctx)


@BLOCKS.register("sandwich")
class SandwichBlock(Block):
    """Every sublayer's result passes a norm of its own before it joins the stream, so no product can add into the stream
    itself: the sublayer adds into a cleared float buffer, and one kernel norms that and adds it."""

    ROLES = {"norm1": NORMS, "conv": CONVOLUTIONS, "mixer": MIXERS, "norm1b": NORMS, "norm2": NORMS, "feed_forward": FEED_FORWARDS, "norm2b": NORMS}
    OPTIONAL = ("conv", "norm2", "feed_forward", "norm2b")

    def __init__(self, parts, hidden_size: int):
        super().__init__(parts, hidden_size)
        if len({self.norm2 is None, self.feed_forward is None, self.norm2b is None}) != 1:
            raise ValueError("a sandwich block has a feed-forward with both of its norms, or none of the three")
        for role in ("norm1b", "norm2b"):
            if getattr(self, role) is not None and type(getattr(self, role)) is not RMSNorm:
                raise ValueError(f"the norm after a sublayer ('{role}') must be a plain RMS norm")

    def state_needs(self) -> Dict[str, StateNeed]:
        needs = super().state_needs()
        need = None if self.conv is None else self.conv.state_need()
        if need is not None:
            needs["conv"] = need
        return needs

    def forward(self, residual: torch.Tensor, ctx: StepContext, mem: RunMemory, rt: Runtime) -> None:
        rows = residual.shape[0]
        h = torch.empty((rows, self.hidden_size), dtype=rt.dtype, device=residual.device)
        y = torch.zeros((rows, self.hidden_size), dtype=torch.float32, device=residual.device)
        if self.conv is not None and ctx.decode and type(self.norm1) is RMSNorm and isinstance(self.conv, CausalConvResidual):
            # Single rows: the convolution over the mixer's input rides in the norm's kernel.
            tail = mem.states.get("conv")
            if tail is None:
                raise RuntimeError("the convolution was given no state: the cache does not serve this block")
            ops.norm_pair(residual, self.norm1.weight, None, h, None, self.norm1.eps, self.conv.weight_t,
                          tail if self.conv.taps > 1 else tail[:, :0], ctx.row_slot, write_tail=mem.writes)
        else:
            if self.conv is not None and type(self.norm1) is RMSNorm:
                ops.norm_pair(residual, self.norm1.weight, None, h, None, self.norm1.eps)      # the same sums as in a step of single rows
            else:
                self.norm1.forward(residual, h)
            if self.conv is not None:
                hc = torch.empty_like(h)
                self.conv.forward(h, hc, ctx, mem.states.get("conv"), mem.writes)
                h = hc
        self.mixer.forward(h, y, ctx, mem)
        if self.feed_forward is None:
            ops.norm_add(y, self.norm1b.weight, residual, self.norm1b.eps)
        else:
            # Between the sublayers one kernel: the mixer's result normed into the stream, the stream normed for the
            # feed-forward, and the buffer cleared for its result.
            if type(self.norm2) is RMSNorm:
                ops.norm_add_norm(y, self.norm1b.weight, residual, self.norm1b.eps, self.norm2.weight, h, self.norm2.eps)
            else:
                ops.norm_add(y, self.norm1b.weight, residual, self.norm1b.eps)
                y.zero_()
                self.norm2.forward(residual, h)
            self.feed_forward.forward(h, y, ctx)
            ops.norm_add(y, self.norm2b.weight, residual, self.norm2b.eps)
