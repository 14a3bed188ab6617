"""`Linear`: y[T, N] = x[T, K] . W[N, K]^T, the one contraction every part uses.

W is row-major [out, in] as in the reference (src/cuda_matmul.cc:181-186, one
`cublasSgemm` per call there).  The product runs in the dtype of the weight:
  * bfloat16 weight, bfloat16 x: tensor-core product with float32 accumulation;
  * float32 weight: a true float32 product (TF32 must be off; it is refused otherwise);
    bfloat16 activations are widened first and the result narrowed afterwards.
Large products go to the library GEMM (as the reference's do); small batches of rows go
to this package's own weight-streaming kernel when it is available for the shape.  That kernel can
also finish the norm in front of the product (input `PreNormed`) and start the one behind it
(`into`, a `ResidualTarget`), so that neither norm is a kernel of its own.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import kernels as K
from .base import PreNormed, ResidualTarget


class Linear:
    def __init__(self, weight: torch.Tensor, name: str = "linear"):
        if weight.dim() != 2:
            raise ValueError(f"{name}: weight must be [out, in], got {tuple(weight.shape)}")
        if weight.dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"{name}: weight dtype {weight.dtype} not supported")
        self.weight = weight.contiguous()
        self.name = name
        self.out_features, self.in_features = weight.shape

    def parameter_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, step, x, out_name: str, out_dtype: Optional[torch.dtype] = None,
                into: Optional[ResidualTarget] = None):
        """x [T, K] in the activation dtype -> [T, N] in `out_dtype` (default: x's dtype).

        x may be a `PreNormed` (bfloat16 only: nothing else makes one).  With `into`, the product may add
        its result to the residual stream and return a `PreNormed` for the norm named there; it does so for
        the few rows of a decode step, and returns the plain result otherwise."""
        row_norm = None
        if isinstance(x, PreNormed):
            row_norm = K.RowNorm(x.sumsq, x.partials, x.eps)
            x = x.values
        rows = x.shape[0]
        if x.shape[1] != self.in_features:
            raise ValueError(f"{self.name}: input width {x.shape[1]} != {self.in_features}")
        out_dtype = out_dtype or x.dtype
        w = self.weight
        ws = step.ws
        if w.dtype == torch.float32:
            if torch.backends.cuda.matmul.allow_tf32:
                raise RuntimeError(f"{self.name}: TF32 is enabled; the float32 path needs true 32-bit products")
            if row_norm is not None:
                # a matrix stored in 32-bit inside a bfloat16 run, behind a product that folded the norm away:
                # finish the norm here, then widen like any other bfloat16 input
                normed = ws.buffer(out_name + ".x", (rows, self.in_features), torch.bfloat16)
                K.apply_row_norm(x, row_norm, normed)
                x = normed
            if x.dtype != torch.float32:
                wide = ws.buffer(out_name + ".x32", (rows, self.in_features), torch.float32)
                K.cast(x, wide)
                x = wide
            if out_dtype == torch.float32:
                out = ws.buffer(out_name, (rows, self.out_features), torch.float32)
                torch.mm(x, w.t(), out=out)
                return out
            wide_out = ws.buffer(out_name + ".y32", (rows, self.out_features), torch.float32)
            torch.mm(x, w.t(), out=wide_out)
            out = ws.buffer(out_name, (rows, self.out_features), out_dtype)
            K.cast(wide_out, out)
            return out
        # bfloat16 weight
        if x.dtype != torch.bfloat16:
            raise RuntimeError(f"{self.name}: bfloat16 weight with {x.dtype} activations; "
                               "a float32 run widens its matrices when it loads them")
        if into is not None and rows <= step.small_rows and out_dtype == torch.bfloat16:
            made = self._into_residual(ws, x, row_norm, out_name, into)
            if made is not None:
                return made
        out = ws.buffer(out_name, (rows, self.out_features), out_dtype)
        if rows <= step.small_rows and K.small_linear(x, w, None, out,
                                                       K.EPI_F32 if out_dtype == torch.float32 else K.EPI_BF16,
                                                       row_norm):
            return out
        if row_norm is not None:  # no kernel of this package takes the shape: finish the norm first
            normed = ws.buffer(out_name + ".x", (rows, self.in_features), torch.bfloat16)
            K.apply_row_norm(x, row_norm, normed)
            x = normed
        if out_dtype == torch.bfloat16:
            torch.mm(x, w.t(), out=out)
        else:  # bfloat16 operands, float32 result (the logits)
            _mm_bf16_to_f32(x, w, out)
        return out


    def _into_residual(self, ws, x, row_norm, out_name: str, into: ResidualTarget) -> Optional[PreNormed]:
        prenorm = into.norm.prenorm_weight()
        rows, width = x.shape[0], self.out_features
        if prenorm is None or into.x.shape != (rows, width) or not K.fused_norm_rows(rows):
            return None
        weight, eps = prenorm
        partials = -(-width // K.NORM_TILE)
        values = ws.buffer(out_name + ".pre", (rows, width), torch.bfloat16)
        sumsq = ws.buffer(out_name + ".sumsq", (rows, partials), torch.float32)
        if not K.small_linear(x, self.weight, None, values, K.EPI_RESID, row_norm, K.ResidualOut(into.x, weight, sumsq)):
            return None
        return PreNormed(values, sumsq, partials, eps, into.norm)


_MM_OUT_DTYPE_WITH_OUT = None


def _mm_bf16_to_f32(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    global _MM_OUT_DTYPE_WITH_OUT
    if _MM_OUT_DTYPE_WITH_OUT is None:
        try:
            torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
            _MM_OUT_DTYPE_WITH_OUT = True
            return
        except (TypeError, RuntimeError):
            _MM_OUT_DTYPE_WITH_OUT = False
    if _MM_OUT_DTYPE_WITH_OUT:
        torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
    else:
        out.copy_(torch.mm(x, w.t(), out_dtype=torch.float32))
