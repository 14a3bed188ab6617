"""RMSNorm, fused with the residual add that precedes it.

y_i = x_i * w_i / sqrt(mean_j(x_j^2) + eps): eps inside the root, the weight multiplies
(no 1 + w), no bias - src/ops.cc:95-110.  The residual stream x is float32; the add of
the previous part's output and the norm are one kernel.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import kernels as K
from .base import BuildContext, Norm, PreNormed, WeightSpec, register_part


class RMSNorm(Norm):
    """params: width, eps, name (tensor name of the weight)."""

    capturable = True

    def __init__(self, params, ctx: BuildContext):
        super().__init__(params, ctx)
        self.width = int(params["width"])
        self.eps = float(params["eps"])
        self.name = params["name"]
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name, (self.width,), kind="vector", init="norm")]

    def bind(self, store) -> None:
        self.weight = store.take(self.name)

    def parameter_bytes(self) -> int:
        return self.width * 4

    def prenorm_weight(self):
        return self.weight, self.eps

    def forward(self, step, x, delta, rows=None, out_name: str = "h"):
        if isinstance(delta, PreNormed):
            if delta.norm is not self or rows is not None:
                raise RuntimeError(f"{self.name}: given rows that were prepared for another norm")
            return delta  # x is up to date; the product that reads the rows applies the factor
        n = x.shape[0] if rows is None else rows.shape[0]
        out = step.ws.buffer(out_name, (n, self.width), self.ctx.act_dtype)
        K.add_rmsnorm(x, delta, self.weight, out, self.eps, rows)
        return out


register_part("norm", "rms_norm", RMSNorm)
