"""Dense SwiGLU feed-forward: down( silu(gate(h)) * up(h) ).

The reference's FfnForward (src/forward.cc:313-322) with SiLU as x / (1 + exp(-x))
(src/ops.cc:135-151).  The gate and up matrices are fused at bind time into one
[2I, D] matrix so that one product feeds the activation kernel; when I is a multiple of
8 their rows are interleaved in blocks of 8 (gate rows 0-7, up rows 0-7, gate rows
8-15, ...), which puts a gate value and its up value into the same thread of a
tensor-core accumulator tile.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import kernels as K
from .base import BuildContext, FeedForward, PreNormed, WeightSpec, register_part
from .linear import Linear

INTERLEAVE = 8


def fuse_gate_up(gate: torch.Tensor, up: torch.Tensor):
    """Return (fused [2I, D], block) with block = INTERLEAVE, or 0 for plain halves."""
    inter, width = gate.shape
    if gate.dtype != up.dtype:
        gate, up = gate.float(), up.float()
    if inter % INTERLEAVE:
        return torch.cat([gate, up], dim=0).contiguous(), 0
    fused = torch.stack([gate.view(inter // INTERLEAVE, INTERLEAVE, width),
                         up.view(inter // INTERLEAVE, INTERLEAVE, width)], dim=1)
    return fused.reshape(2 * inter, width).contiguous(), INTERLEAVE


class SwiGLUFeedForward(FeedForward):
    """params: intermediate, names {"gate","up","down"} (tensor name stems)."""

    capturable = True
    takes_prenormed = True  # the gate/up product may read rows whose norm it finishes itself
    adds_residual = True    # the down product may add to the residual stream and prepare the next norm

    def __init__(self, params, ctx: BuildContext):
        super().__init__(params, ctx)
        self.inter = int(params["intermediate"])
        self.names = dict(params["names"])
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None
        self.block = 0

    def weight_specs(self) -> List[WeightSpec]:
        D = self.ctx.hidden_size
        return [WeightSpec(self.names["gate"] + ".weight", (self.inter, D)),
                WeightSpec(self.names["up"] + ".weight", (self.inter, D)),
                WeightSpec(self.names["down"] + ".weight", (D, self.inter))]

    def bind(self, store) -> None:
        fused, self.block = fuse_gate_up(store.take(self.names["gate"] + ".weight"),
                                         store.take(self.names["up"] + ".weight"))
        self.gate_up = Linear(fused, self.names["gate"] + "+up")
        self.down = Linear(store.take(self.names["down"] + ".weight"), self.names["down"])

    def parameter_bytes(self) -> int:
        return self.gate_up.parameter_bytes() + self.down.parameter_bytes()

    def forward(self, step, h, into=None):
        values, row_norm = (h.values, K.RowNorm(h.sumsq, h.partials, h.eps)) if isinstance(h, PreNormed) else (h, None)
        rows = values.shape[0]
        w = self.gate_up.weight
        fused = (rows <= step.small_rows and self.block == INTERLEAVE and w.dtype == torch.bfloat16
                 and values.dtype == torch.bfloat16
                 and bool(K.small_linear_kind(rows, 2 * self.inter, w.shape[1], K.EPI_SWIGLU)))
        if fused:
            # few rows: one weight-streaming kernel whose epilogue applies the activation
            act = step.ws.buffer("act", (rows, self.inter), torch.bfloat16)
            K.small_linear(values, w, None, act, K.EPI_SWIGLU, row_norm)
        elif (row_norm is not None and w.dtype == torch.bfloat16 and self.inter % 8 == 0
              and not K.small_linear_kind(rows, 2 * self.inter, w.shape[1], K.EPI_BF16)):
            # the library product cannot finish the norm in front of it: it runs on the rows as they are and
            # the activation kernel multiplies gate and up by the rows' factors
            gu = self.gate_up.forward(step, values, "gu")
            act = step.ws.buffer("act", (rows, self.inter), torch.bfloat16)
            K.swiglu(gu, act, self.block, row_norm, w.shape[1])
        else:
            gu = self.gate_up.forward(step, h, "gu")
            act = step.ws.buffer("act", (rows, self.inter), gu.dtype)
            K.swiglu(gu, act, self.block)
        return self.down.forward(step, act, "down", into=into)


register_part("feed_forward", "swiglu", SwiGLUFeedForward)
