"""Python face of the kernel library: typed wrappers that check tensors on the host
and launch on the current CUDA stream.

Every function here needs the compiled library and CUDA tensors; there is no other
implementation behind them.  Argument faults raise `KernelError` before any launch.
"""
from __future__ import annotations

import ctypes
from typing import Dict, NamedTuple, Optional

import torch

from ..cache.paged import PAGE  # cache positions per page; the library's MLL_PAGE is checked against it on load
from .build import KernelBuildError, load_library

ABI_VERSION = 27
MAX_TOP_K = 1024


class KernelError(RuntimeError):
    pass


class DeviceKernelError(KernelError):
    """A kernel gave up on the device (a bounded wait ran out, or its shared memory was misplaced): what the
    step computed is not to be used."""


_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        handle = load_library()
        handle.mll_last_error.restype = ctypes.c_char_p
        handle.mll_attn_decode_scratch_floats.restype = ctypes.c_longlong
        if handle.mll_abi_version() != ABI_VERSION:
            raise KernelBuildError(
                f"kernel library reports ABI {handle.mll_abi_version()}, the package expects {ABI_VERSION}; "
                "remove csrc/_build and rebuild")
        if handle.mll_page() != PAGE:
            raise KernelBuildError(f"kernel library built for pages of {handle.mll_page()} positions, the cache uses {PAGE}")
        _lib = handle
    return _lib


def multiprocessor_count() -> int:
    """Multiprocessors of the current CUDA device (the library asks the driver once per device)."""
    return int(lib().mll_multiprocessor_count())


launches = 0  # kernels of this library launched so far (counted per successful call)
calls: Dict[str, int] = {}  # the same, per kind of launch (the name each wrapper gives its kernel)


def _check(code: int, what: str, kernels: int = 1) -> None:
    global launches
    launches += kernels
    calls[what] = calls.get(what, 0) + 1
    if code != 0:
        message = lib().mll_last_error().decode("utf-8", "replace")
        raise KernelError(f"{what}: {message} (code {code})")


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, name: str, dtype=None, ndim=None) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name}: expected a CUDA tensor (the kernels have no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name}: tensor must be contiguous, strides {tuple(t.stride())}")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name}: expected {ndim} dimensions, got shape {tuple(t.shape)}")


def dtype_code(dtype: torch.dtype) -> int:
    if dtype not in _DTYPE_CODE:
        raise KernelError(f"dtype {dtype} not supported by the kernels (float32, bfloat16)")
    return _DTYPE_CODE[dtype]


# --------------------------------------------------------------------------- #
def embedding(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, :] = float32(table[tokens[t], :]); tokens int32 [T], out float32 [T, D]."""
    _need(tokens, "embedding tokens", torch.int32, 1)
    _need(table, "embedding table", None, 2)
    _need(out, "embedding out", torch.float32, 2)
    n, width = tokens.shape[0], table.shape[1]
    if out.shape[0] < n or out.shape[1] != width:
        raise KernelError(f"embedding: out {tuple(out.shape)} does not fit [{n}, {width}]")
    _check(lib().mll_embedding(_ptr(tokens), _ptr(table), dtype_code(table.dtype), _ptr(out),
                               ctypes.c_int(n), ctypes.c_int(width), _stream()), "embedding")


def cast(src: torch.Tensor, dst: torch.Tensor) -> None:
    _need(src, "cast src")
    _need(dst, "cast dst")
    if src.numel() != dst.numel():
        raise KernelError("cast: sizes differ")
    _check(lib().mll_cast(_ptr(src), dtype_code(src.dtype), _ptr(dst), dtype_code(dst.dtype),
                          ctypes.c_longlong(src.numel()), _stream()), "cast")


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> None:
    """x[t, :] += bias (float32 bias, in place)."""
    _need(x, "add_bias x", None, 2)
    _need(bias, "add_bias bias", torch.float32, 1)
    if bias.shape[0] != x.shape[1]:
        raise KernelError("add_bias: bias length differs from the row width")
    _check(lib().mll_add_bias(_ptr(x), _ptr(bias), dtype_code(x.dtype), ctypes.c_int(x.shape[0]),
                              ctypes.c_int(x.shape[1]), _stream()), "add_bias")


def scatter_rows(table: torch.Tensor, staged: torch.Tensor, n_rows: int) -> None:
    """table[staged[r, 0], :] = staged[r, 1:] for r < n_rows: block-table rows that changed on the host.
    table int32 [rows, width]; staged int32, n_rows * (1 + width) values."""
    _need(table, "scatter_rows table", torch.int32, 2)
    _need(staged, "scatter_rows staged", torch.int32)
    if staged.numel() < n_rows * (1 + table.shape[1]):
        raise KernelError("scatter_rows: staged rows shorter than the count says")
    _check(lib().mll_scatter_rows(_ptr(table), _ptr(staged), ctypes.c_int(n_rows), ctypes.c_int(table.shape[1]),
                                  ctypes.c_int(table.shape[0]), _stream()), "scatter_rows")


def gather_int32(dst: torch.Tensor, src: torch.Tensor, index: torch.Tensor, n: int) -> None:
    """dst[i] = src[index[i]] for i < n (int32; an index outside src gives 0): the tokens that a step sampled,
    brought into the order of the next step's rows on the device."""
    for name, t in (("dst", dst), ("src", src), ("index", index)):
        _need(t, f"gather_int32 {name}", torch.int32, 1)
    if dst.shape[0] < n or index.shape[0] < n:
        raise KernelError("gather_int32: dst or index shorter than the count says")
    _check(lib().mll_gather_int32(_ptr(dst), _ptr(src), _ptr(index), ctypes.c_int(n), ctypes.c_int(src.shape[0]),
                                  _stream()), "gather_int32")


EPI_BF16, EPI_F32, EPI_SWIGLU, EPI_RESID = 0, 1, 2, 3
NORM_TILE = 16  # columns per partial sum of squares that the residual epilogue writes


class RowNorm(NamedTuple):
    """Rows that still lack their RMS norm's factor: `sumsq` float32 [rows, stride] holds `partials`
    partial sums of squares per row; the factor is 1 / sqrt(sum / width + eps)."""
    sumsq: torch.Tensor
    partials: int
    eps: float


class ResidualOut(NamedTuple):
    """Where the residual epilogue writes: `resid` float32 [rows, N] (+= result), `next_weight` float32 [N]
    (out = resid * next_weight in bfloat16), `sumsq` float32 [rows, stride >= ceil(N / NORM_TILE)]."""
    resid: torch.Tensor
    next_weight: torch.Tensor
    sumsq: torch.Tensor


def _row_norm_args(row_norm: Optional["RowNorm"], rows: int, what: str):
    if row_norm is None:
        return ctypes.c_void_p(None), ctypes.c_int(0), ctypes.c_int(0), ctypes.c_float(0.0)
    _need(row_norm.sumsq, what + " partial sums", torch.float32, 2)
    if row_norm.sumsq.shape[0] < rows or row_norm.sumsq.shape[1] < row_norm.partials:
        raise KernelError(f"{what}: partial sums {tuple(row_norm.sumsq.shape)} for {rows} rows of {row_norm.partials}")
    return (_ptr(row_norm.sumsq), ctypes.c_int(row_norm.partials), ctypes.c_int(row_norm.sumsq.shape[1]),
            ctypes.c_float(row_norm.eps))


def linear_small_supported(rows: int, out_features: int, in_features: int, epilogue: int = EPI_BF16) -> bool:
    return bool(lib().mll_linear_small_supported(rows, out_features, in_features, epilogue))


def linear_small(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                 epilogue: int = EPI_BF16, ranks: int = 0, row_norm: Optional[RowNorm] = None,
                 residual: Optional[ResidualOut] = None) -> None:
    """out = x . w^T for at most 64 rows of bfloat16 x [M, K] and bfloat16 w [N, K], read once.

    epilogue EPI_BF16 / EPI_F32: out [M, N] in that dtype (+ float32 bias [N]);
    EPI_SWIGLU: w holds gate and up rows interleaved in blocks of 8, out [M, N / 2] = silu(gate) * up;
    EPI_RESID (at most 16 rows, with `residual`): the result is added to the residual stream, out [M, N]
    is the new stream times the next norm's weight (not yet its factor), with partial sums of squares.
    `row_norm`: x is such an output; the result is multiplied by the rows' factors."""
    _need(x, "linear_small x", torch.bfloat16, 2)
    _need(w, "linear_small w", torch.bfloat16, 2)
    rows, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise KernelError(f"linear_small: x width {k} differs from w width {w.shape[1]}")
    want = (rows, n // 2) if epilogue == EPI_SWIGLU else (rows, n)
    _need(out, "linear_small out", torch.float32 if epilogue == EPI_F32 else torch.bfloat16, 2)
    if tuple(out.shape) != want:
        raise KernelError(f"linear_small: out {tuple(out.shape)}, expected {want}")
    if bias is not None:
        _need(bias, "linear_small bias", torch.float32, 1)
        if bias.shape[0] != n:
            raise KernelError("linear_small: bias length differs from the output width")
    if (epilogue == EPI_RESID) != (residual is not None):
        raise KernelError("linear_small: the residual epilogue and its outputs go together")
    resid = next_w = out_sumsq = None
    out_stride = 0
    if residual is not None:
        resid, next_w, out_sumsq = residual
        _need(resid, "linear_small resid", torch.float32, 2)
        _need(next_w, "linear_small next weight", torch.float32, 1)
        _need(out_sumsq, "linear_small sums of squares", torch.float32, 2)
        if tuple(resid.shape) != (rows, n) or next_w.shape[0] != n or out_sumsq.shape[0] < rows:
            raise KernelError(f"linear_small: resid {tuple(resid.shape)}, next weight {tuple(next_w.shape)}, sums "
                              f"{tuple(out_sumsq.shape)} do not fit out {(rows, n)}")
        out_stride = out_sumsq.shape[1]
    _check(lib().mll_linear_small_fused(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), ctypes.c_int(rows), ctypes.c_int(n),
                                        ctypes.c_int(k), ctypes.c_int(epilogue), ctypes.c_int(ranks),
                                        *_row_norm_args(row_norm, rows, "linear_small"), _ptr(resid), _ptr(next_w),
                                        _ptr(out_sumsq), ctypes.c_int(out_stride), _stream()), "linear_small")


def linear_tma_supported(rows: int, out_features: int, in_features: int, epilogue: int = EPI_BF16) -> bool:
    return bool(lib().mll_linear_tma_supported(rows, out_features, in_features, epilogue))


def linear_tma(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
               epilogue: int = EPI_BF16, ranks: int = 0, row_norm: Optional[RowNorm] = None) -> None:
    """As `linear_small`, with the weights streamed through a TMA + mbarrier pipeline.  Takes
    any N, any K that is a multiple of 8, at most 64 rows."""
    _need(x, "linear_tma x", torch.bfloat16, 2)
    _need(w, "linear_tma w", torch.bfloat16, 2)
    rows, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise KernelError(f"linear_tma: x width {k} differs from w width {w.shape[1]}")
    want = (rows, n // 2) if epilogue == EPI_SWIGLU else (rows, n)
    _need(out, "linear_tma out", torch.float32 if epilogue == EPI_F32 else torch.bfloat16, 2)
    if tuple(out.shape) != want:
        raise KernelError(f"linear_tma: out {tuple(out.shape)}, expected {want}")
    if bias is not None:
        _need(bias, "linear_tma bias", torch.float32, 1)
        if bias.shape[0] != n:
            raise KernelError("linear_tma: bias length differs from the output width")
    _check(lib().mll_linear_tma_fused(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), ctypes.c_int(rows), ctypes.c_int(n),
                                      ctypes.c_int(k), ctypes.c_int(epilogue), ctypes.c_int(ranks),
                                      *_row_norm_args(row_norm, rows, "linear_tma"), _stream()), "linear_tma")


def linear_tc5_supported(rows: int, out_features: int, in_features: int, epilogue: int = EPI_BF16) -> bool:
    return bool(lib().mll_linear_tc5_supported(rows, out_features, in_features, epilogue))


def linear_tc5(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
               epilogue: int = EPI_BF16, ranks: int = 0, row_norm: Optional[RowNorm] = None,
               residual: Optional[ResidualOut] = None) -> None:
    """As `linear_small` (the residual epilogue included, here for up to 64 rows), with the product on the
    fifth-generation tensor cores: tcgen05.mma reads the TMA-filled stages from shared memory and
    accumulates in tensor memory.  Takes any N, any K that is a multiple of 8, at most 64 rows."""
    _need(x, "linear_tc5 x", torch.bfloat16, 2)
    _need(w, "linear_tc5 w", torch.bfloat16, 2)
    rows, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise KernelError(f"linear_tc5: x width {k} differs from w width {w.shape[1]}")
    want = (rows, n // 2) if epilogue == EPI_SWIGLU else (rows, n)
    _need(out, "linear_tc5 out", torch.float32 if epilogue == EPI_F32 else torch.bfloat16, 2)
    if tuple(out.shape) != want:
        raise KernelError(f"linear_tc5: out {tuple(out.shape)}, expected {want}")
    if bias is not None:
        _need(bias, "linear_tc5 bias", torch.float32, 1)
        if bias.shape[0] != n:
            raise KernelError("linear_tc5: bias length differs from the output width")
    if (epilogue == EPI_RESID) != (residual is not None):
        raise KernelError("linear_tc5: the residual epilogue and its outputs go together")
    resid = next_w = out_sumsq = None
    out_stride = 0
    if residual is not None:
        resid, next_w, out_sumsq = residual
        _need(resid, "linear_tc5 resid", torch.float32, 2)
        _need(next_w, "linear_tc5 next weight", torch.float32, 1)
        _need(out_sumsq, "linear_tc5 sums of squares", torch.float32, 2)
        if tuple(resid.shape) != (rows, n) or next_w.shape[0] != n or out_sumsq.shape[0] < rows:
            raise KernelError(f"linear_tc5: resid {tuple(resid.shape)}, next weight {tuple(next_w.shape)}, sums "
                              f"{tuple(out_sumsq.shape)} do not fit out {(rows, n)}")
        out_stride = out_sumsq.shape[1]
    _check(lib().mll_linear_tc5_fused(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), ctypes.c_int(rows), ctypes.c_int(n),
                                      ctypes.c_int(k), ctypes.c_int(epilogue), ctypes.c_int(ranks),
                                      *_row_norm_args(row_norm, rows, "linear_tc5"), _ptr(resid), _ptr(next_w),
                                      _ptr(out_sumsq), ctypes.c_int(out_stride), _stream()), "linear_tc5")


DEVICE_ERROR_BITS = ("the TMA linear kernel", "the tcgen05 linear kernel", "the tcgen05 prefill attention kernel",
                     "the TMA decode attention kernel")


def take_device_error() -> int:
    """Non-zero when a kernel gave up since the flags were last read (then cleared): bit i stands for
    DEVICE_ERROR_BITS[i]; synchronises.  The sampling kernels read and clear the same flags on the
    device and hand them to `DeviceSampler.collect` in their status word."""
    return int(lib().mll_take_device_error())


def raise_device_error(mask: int) -> None:
    """Set the flags of `mask` from the host, as a kernel that gave up would (for tests of the host side)."""
    _check(lib().mll_raise_device_error(ctypes.c_int(mask)), "raise_device_error", kernels=0)


def device_error_message(mask: int) -> str:
    names = [name for i, name in enumerate(DEVICE_ERROR_BITS) if mask & (1 << i)] or [f"mask {mask}"]
    return ("a bounded wait ran out (or a block's shared memory was misplaced) in " + ", ".join(names)
            + "; the step's results are not valid")


TMA_MAX_ROWS = 8      # rows up to which tall matrices go to the direct kernel, or the TMA + mma.sync kernel (one batch tile of 8 rows)
TC5_TALL_MAX_ROWS = 16  # rows up to which tall matrices go to the tcgen05 kernel (beyond: the library, which shares the
                        # batch tile between the blocks of a cluster)
DIRECT_MAX_ROWS = 16  # rows up to which the other matrices go to the direct kernel
TALL = 16384          # output features from which a matrix counts as tall


def small_linear_kind(rows: int, out_features: int, in_features: int, epilogue: int = EPI_BF16) -> str:
    """Which of this library's weight-streaming kernels takes the problem: "tc5", "tma", "direct" or "".

    Measured on B200 (CUDA-graph timing) on the shapes of the 8B, 7B and 1B Llama models.  Tall matrices
    (gate/up, lm_head) up to 8 rows: the direct kernel, as it stands since it got its register targets and eight
    warps a block (us at 8 rows, direct / TMA + mma.sync / tcgen05: 8B gate/up + SwiGLU 38.7 / 41.5 / 42.6, lm_head
    154.7 / 159.5 / 161.5; 7B 31.1 / 32.3 / 33.0 and 42.5 / 46.3 / 46.2; 1B 13.3 / 15.2 / 16.1 and 78.3 / 80.4 /
    83.0; the TMA kernel stays for widths the direct kernel does not take); from 9 to 16 rows the tcgen05 kernel
    (8B gate/up 43.0 against 45.3 direct and 54.5 TMA with their second batch tile).  The other projections: the
    direct kernel up to 16 rows (it chooses its variant by rows and tiles).  From 17 rows on the library GEMM: the tcgen05 kernel takes up to 64 rows (32 or 64 batch
    columns per MMA), but inside a CUDA graph the library's kernels are ahead on every shape tried
    (64 rows, us, library / tcgen05: 8B q/k/v 11.8 / 16.2, o 9.9 / 13.1, down 24.9 / 26.5, gate/up 42.8 /
    46.9; 1B q/k/v 5.9 / 9.6, o 5.7 / 9.1, down 13.2 / 14.5, gate/up 13.2 / 19.1), and in a batch-64 step
    the three small products took 60.6 us a layer on it against 46.6 + two norm kernels on the library."""
    if SMALL_LINEAR == "none":
        return ""
    if SMALL_LINEAR != "auto":  # a forced kind (tests, experiments)
        supported = {"tc5": linear_tc5_supported, "tma": linear_tma_supported, "direct": linear_small_supported}
        return SMALL_LINEAR if rows <= 64 and supported[SMALL_LINEAR](rows, out_features, in_features, epilogue) else ""
    if out_features >= TALL:
        if rows <= TMA_MAX_ROWS:  # one batch tile of 8 rows in either kernel
            if linear_small_supported(rows, out_features, in_features, epilogue):
                return "direct"
            if linear_tma_supported(rows, out_features, in_features, epilogue):
                return "tma"
        if rows <= TC5_TALL_MAX_ROWS and linear_tc5_supported(rows, out_features, in_features, epilogue):
            return "tc5"
    if rows <= DIRECT_MAX_ROWS:
        if linear_small_supported(rows, out_features, in_features, epilogue):
            return "direct"
        if linear_tma_supported(rows, out_features, in_features, epilogue):
            return "tma"
    return ""


def small_linear(x, w, bias, out, epilogue: int = EPI_BF16, row_norm: Optional[RowNorm] = None,
                 residual: Optional[ResidualOut] = None) -> bool:
    """Run the product on the kernel that `small_linear_kind` names; False when there is none (then
    nothing ran).  The residual epilogue exists in the direct kernel and in the tcgen05 kernel."""
    kind = small_linear_kind(x.shape[0], w.shape[0], w.shape[1], EPI_BF16 if epilogue == EPI_RESID else epilogue)
    if epilogue == EPI_RESID and kind not in ("direct", "tc5"):
        return False
    if kind == "tc5":
        linear_tc5(x, w, bias, out, epilogue, 0, row_norm, residual)
    elif kind == "tma":
        linear_tma(x, w, bias, out, epilogue, 1 if x.shape[0] > 8 else 0, row_norm)
    elif kind == "direct":
        linear_small(x, w, bias, out, epilogue, 0, row_norm, residual)
    return bool(kind)


def fused_norm_rows(rows: int) -> bool:
    """Whether products over `rows` rows may fold the norms around them in (the residual epilogue
    exists in the kernels that take decode steps' row counts)."""
    return FUSE_NORM and 1 <= rows <= (64 if SMALL_LINEAR == "tc5" else DIRECT_MAX_ROWS)


FUSE_NORM = True  # off: every norm is a kernel of its own


SMALL_LINEAR = "auto"  # "auto", a forced kind ("tc5", "tma", "direct"), or "none" (library GEMM only)


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, block: int, row_norm: Optional[RowNorm] = None,
           width: int = 0) -> None:
    """out[t, i] = silu(gate) * up; gate_up [T, 2I] holds halves (block 0) or blocks of `block`.
    `row_norm` (bfloat16, I a multiple of 8): gate_up was computed from rows of `width` columns that lacked their
    norm's factor; gate and up are multiplied by it first."""
    _need(gate_up, "swiglu gate_up", None, 2)
    _need(out, "swiglu out", gate_up.dtype, 2)
    tokens, inter = out.shape
    if gate_up.shape[0] != tokens or gate_up.shape[1] != 2 * inter:
        raise KernelError(f"swiglu: gate_up {tuple(gate_up.shape)} does not match out {tuple(out.shape)}")
    if row_norm is not None:
        if gate_up.dtype != torch.bfloat16 or inter % 8 or block not in (0, 8) or width <= 0:
            raise KernelError("swiglu: rows without their norm's factor need bfloat16, I % 8 == 0 and the rows' width")
        sumsq, partials, stride, eps = _row_norm_args(row_norm, tokens, "swiglu")
        _check(lib().mll_swiglu_rows(_ptr(gate_up), _ptr(out), ctypes.c_int(tokens), ctypes.c_int(inter),
                                     ctypes.c_int(block), sumsq, partials, stride, eps, ctypes.c_int(width), _stream()),
               "swiglu_rows")
        return
    _check(lib().mll_swiglu(_ptr(gate_up), _ptr(out), dtype_code(out.dtype), ctypes.c_int(tokens),
                            ctypes.c_int(inter), ctypes.c_int(block), _stream()), "swiglu")


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, out: torch.Tensor,
                eps: float, rows: Optional[torch.Tensor] = None) -> None:
    """x += delta (float32 residual, in place); out = rmsnorm(x) * weight.

    With `rows` (int32 [n]) only those rows of x are normalised into out [n, D] and x is
    left unchanged."""
    _need(x, "rmsnorm x", torch.float32, 2)
    _need(weight, "rmsnorm weight", torch.float32, 1)
    _need(out, "rmsnorm out", None, 2)
    width = x.shape[1]
    if weight.shape[0] != width or out.shape[1] != width:
        raise KernelError(f"rmsnorm: widths differ: x {width}, weight {weight.shape[0]}, out {out.shape[1]}")
    if delta is not None:
        _need(delta, "rmsnorm delta", out.dtype, 2)
        if delta.shape != x.shape:
            raise KernelError(f"rmsnorm: delta {tuple(delta.shape)} differs from x {tuple(x.shape)}")
    if rows is not None:
        _need(rows, "rmsnorm rows", torch.int32, 1)
        n_rows = rows.shape[0]
    else:
        n_rows = x.shape[0]
    if out.shape[0] != n_rows:
        raise KernelError(f"rmsnorm: out has {out.shape[0]} rows, expected {n_rows}")
    _check(lib().mll_add_rmsnorm(_ptr(x), _ptr(delta), _ptr(weight), _ptr(out), _ptr(rows),
                                 dtype_code(out.dtype), ctypes.c_int(n_rows), ctypes.c_int(width),
                                 ctypes.c_float(eps), _stream()), "rmsnorm")


def apply_row_norm(values: torch.Tensor, row_norm: RowNorm, out: torch.Tensor) -> None:
    """out = values * the rows' norm factors (bfloat16 [T, D]): finishes a norm that the product behind it
    cannot finish itself."""
    _need(values, "apply_row_norm values", torch.bfloat16, 2)
    _need(out, "apply_row_norm out", torch.bfloat16, 2)
    if out.shape != values.shape:
        raise KernelError(f"apply_row_norm: out {tuple(out.shape)} differs from values {tuple(values.shape)}")
    sumsq, partials, stride, eps = _row_norm_args(row_norm, values.shape[0], "apply_row_norm")
    _check(lib().mll_apply_row_norm(_ptr(values), sumsq, partials, stride, eps, _ptr(out),
                                    ctypes.c_int(values.shape[0]), ctypes.c_int(values.shape[1]), _stream()),
           "apply_row_norm")


def rope_cache_write(qkv, bias, cos, sin, tok_pos, tok_seq, seq_slot, block_table, q_out, k_cache, v_cache,
                     n_heads: int, n_kv_heads: int, head_dim: int, interleaved: bool,
                     write_kv: bool = True) -> None:
    """Rotate q and k of qkv [T, (Hq + 2 Hk) d], write q to q_out [T, Hq d] and k, v into the
    paged cache [n_pages, Hk, PAGE, d] at each token's slot and position."""
    _need(qkv, "rope qkv", None, 2)
    _need(q_out, "rope q_out", qkv.dtype, 2)
    n = qkv.shape[0]
    for name, t in (("tok_pos", tok_pos), ("tok_seq", tok_seq), ("seq_slot", seq_slot)):
        _need(t, f"rope {name}", torch.int32, 1)
    _need(block_table, "rope block_table", torch.int32, 2)
    if tok_pos.shape[0] < n or tok_seq.shape[0] < n:
        raise KernelError("rope: token metadata shorter than the token count")
    if q_out.shape[0] < n or q_out.shape[1] != n_heads * head_dim:
        raise KernelError(f"rope: q_out {tuple(q_out.shape)} does not fit [{n}, {n_heads * head_dim}]")
    if cos is not None:
        _need(cos, "rope cos", torch.float32, 2)
        _need(sin, "rope sin", torch.float32, 2)
        if cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
            raise KernelError(f"rope: table {tuple(cos.shape)} does not match head_dim {head_dim}")
    if bias is not None:
        _need(bias, "rope bias", torch.float32, 1)
        if bias.shape[0] != qkv.shape[1]:
            raise KernelError("rope: bias length differs from the qkv width")
    if write_kv:
        _need(k_cache, "rope k_cache", qkv.dtype, 4)
        _need(v_cache, "rope v_cache", qkv.dtype, 4)
        want = (n_kv_heads, PAGE, head_dim)
        if tuple(k_cache.shape[1:]) != want or k_cache.shape != v_cache.shape:
            raise KernelError(f"rope: cache shape {tuple(k_cache.shape)} is not [pages, {want}]")
    _check(lib().mll_rope_cache(_ptr(qkv), _ptr(bias), _ptr(cos), _ptr(sin), _ptr(tok_pos), _ptr(tok_seq),
                                _ptr(seq_slot), _ptr(block_table), _ptr(q_out), _ptr(k_cache), _ptr(v_cache),
                                dtype_code(qkv.dtype), ctypes.c_int(n), ctypes.c_int(qkv.shape[1]),
                                ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads), ctypes.c_int(head_dim),
                                ctypes.c_int(block_table.shape[1]), ctypes.c_int(int(interleaved)),
                                ctypes.c_int(int(write_kv)), _stream()), "rope_cache_write")


def _check_attention(q, k_cache, v_cache, out, n_heads, n_kv_heads, head_dim):
    _need(q, "attention q", None, 2)
    _need(out, "attention out", q.dtype, 2)
    _need(k_cache, "attention k_cache", q.dtype, 4)
    _need(v_cache, "attention v_cache", q.dtype, 4)
    if head_dim % 16 != 0 or not 16 <= head_dim <= 256:
        raise KernelError(f"attention: head_dim {head_dim} is not a multiple of 16 in [16, 256]")
    if n_heads % n_kv_heads != 0:
        raise KernelError(f"attention: {n_heads} heads are not a multiple of {n_kv_heads} kv heads")
    if q.shape[1] != n_heads * head_dim or out.shape[1] != n_heads * head_dim:
        raise KernelError("attention: q/out width differs from heads * head_dim")
    if tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, head_dim) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention: cache shape {tuple(k_cache.shape)} is not "
                          f"[pages, {n_kv_heads}, {PAGE}, {head_dim}]")


def attention_decode_scratch_floats(n_seqs: int, n_heads: int, head_dim: int, n_splits: int) -> int:
    return int(lib().mll_attn_decode_scratch_floats(n_seqs, n_heads, head_dim, n_splits))


USE_TENSOR_CORE_DECODE = True  # tests switch these off to reach the general kernels at every size
USE_TENSOR_CORE_PREFILL = True
USE_TCGEN05_PREFILL = True      # off: the mma.sync kernel takes the tensor-core prefill


def attention_decode(q, k_cache, v_cache, seq_slot, seq_ctx, block_table, scratch, out, n_seqs: int,
                     n_heads: int, n_kv_heads: int, head_dim: int, n_splits: int, window: int,
                     scale: float, counters: Optional[torch.Tensor] = None, order: Optional[torch.Tensor] = None,
                     work: Optional[torch.Tensor] = None) -> None:
    """One query token per sequence (q row i belongs to sequence i) over the paged cache.
    bfloat16 runs on tensor cores (head sizes 16 .. 256 in steps of 16), float32 on the general kernel.
    `order`: optional int32 permutation of the sequences, longest context first; the TMA-fed kernel starts its
    blocks in that order so that short sequences fill the end of the launch (the others ignore it)."""
    _check_attention(q, k_cache, v_cache, out, n_heads, n_kv_heads, head_dim)
    _need(seq_slot, "attention seq_slot", torch.int32, 1)
    _need(seq_ctx, "attention seq_ctx", torch.int32, 1)
    _need(block_table, "attention block_table", torch.int32, 2)
    if q.shape[0] < n_seqs or out.shape[0] < n_seqs or seq_slot.shape[0] < n_seqs or seq_ctx.shape[0] < n_seqs:
        raise KernelError("attention decode: an input has fewer rows than sequences")
    if n_splits > 1:
        _need(scratch, "attention scratch", torch.float32)
        if scratch.numel() < attention_decode_scratch_floats(n_seqs, n_heads, head_dim, n_splits):
            raise KernelError("attention decode: scratch too small for the split count")
    code = dtype_code(q.dtype)
    if counters is not None:
        _need(counters, "attention counters", torch.int32, 1)
        group = n_heads // n_kv_heads
        if counters.shape[0] < n_seqs * n_kv_heads * ((group + 15) // 16):
            raise KernelError("attention decode: counters shorter than sequences x kv heads x head chunks")
    if q.dtype == torch.bfloat16 and _tma_decode(q, None, None, None, False, False, k_cache, v_cache, seq_slot, seq_ctx,
                                                block_table, scratch, out, n_seqs, n_heads, n_kv_heads, head_dim,
                                                n_splits, window, scale, counters, _order(order, n_seqs), work):
        return
    if work is not None:
        raise KernelError("attention decode: a work list was given, but the kernel that takes one does not run here")
    if USE_TENSOR_CORE_DECODE and lib().mll_attn_decode_mma_supported(code, head_dim):
        _check(lib().mll_attn_decode_mma(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(seq_slot), _ptr(seq_ctx),
                                         _ptr(block_table), _ptr(scratch), _ptr(out), ctypes.c_int(n_seqs),
                                         ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads), ctypes.c_int(head_dim),
                                         ctypes.c_int(block_table.shape[1]), ctypes.c_int(n_splits),
                                         ctypes.c_int(window), ctypes.c_float(scale),
                                         _ptr(counters if n_splits > 1 else None), _stream()),
               "attention_decode (tensor cores)")
        if n_splits > 1 and counters is None:
            _check(lib().mll_attn_combine(_ptr(scratch), _ptr(out), code, ctypes.c_int(n_seqs), ctypes.c_int(n_heads),
                                          ctypes.c_int(head_dim), ctypes.c_int(n_splits), _stream()),
                   "attention_combine")
        return
    _check(lib().mll_attn_decode(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(seq_slot), _ptr(seq_ctx),
                                 _ptr(block_table), _ptr(scratch), _ptr(out), code,
                                 ctypes.c_int(n_seqs), ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads),
                                 ctypes.c_int(head_dim), ctypes.c_int(block_table.shape[1]),
                                 ctypes.c_int(n_splits), ctypes.c_int(window), ctypes.c_float(scale),
                                 _stream()), "attention_decode", kernels=2 if n_splits > 1 else 1)


USE_FUSED_DECODE = True  # off: rotary encoding and cache write stay a kernel of their own in decode steps
USE_TMA_DECODE = True    # off: the cp.async / mma.sync decode kernel also takes head sizes 64 and 128
USE_CLUSTER_MERGE = True  # off: the TMA decode kernel merges its context splits through global memory and counters


def _order(order, n_seqs: int):
    if order is not None:
        _need(order, "attention order", torch.int32, 1)
        if order.shape[0] < n_seqs:
            raise KernelError("attention decode: the order is shorter than the batch")
    return order


WORK_LIST_MAX_SPLITS = 32  # splits a sequence of a work list can have (the stride of the partial results)


def decode_work_entry(sequence: int, split: int, n_splits: int) -> int:
    """One place of a decode work list: block `split` of the `n_splits` that `sequence` is cut into."""
    return sequence | (split << 16) | (n_splits << 24)


def _work(work, n_seqs: int, n_splits: int):
    if work is not None:
        _need(work, "attention work list", torch.int32, 1)
        if work.shape[0] < n_seqs or work.shape[0] > 65535 or n_seqs > 65535:
            raise KernelError(f"attention decode: a work list of {work.shape[0]} places for {n_seqs} sequences")
        if n_splits > 127:
            raise KernelError("attention decode: a work list takes at most 127 splits a sequence")
    return work


def _tma_decode(q, qkv, cos, sin, interleaved, write_kv, k_cache, v_cache, seq_slot, seq_ctx, block_table, scratch, out,
                n_seqs, n_heads, n_kv_heads, head_dim, n_splits, window, scale, counters, order=None, work=None) -> bool:
    """Runs the TMA-fed decode kernel when it takes the problem (bfloat16, head_dim 64/128, arrival
    counters whenever the context is split); returns whether it did."""
    if not (USE_TMA_DECODE and USE_TENSOR_CORE_DECODE and lib().mll_attn_decode_tma_supported(dtype_code(out.dtype), head_dim)):
        return False
    if n_splits > 1 and counters is None:
        return False
    work = _work(work, n_seqs, n_splits)
    _check(lib().mll_attn_decode_tma(_ptr(q), _ptr(qkv), ctypes.c_int(qkv.shape[1] if qkv is not None else 0),
                                     _ptr(cos), _ptr(sin), ctypes.c_int(int(interleaved)), ctypes.c_int(int(write_kv)),
                                     _ptr(k_cache), _ptr(v_cache), ctypes.c_longlong(k_cache.shape[0]), _ptr(seq_slot),
                                     _ptr(seq_ctx), _ptr(block_table), _ptr(scratch), _ptr(out), ctypes.c_int(n_seqs),
                                     ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads), ctypes.c_int(head_dim),
                                     ctypes.c_int(block_table.shape[1]), ctypes.c_int(n_splits), ctypes.c_int(window),
                                     ctypes.c_float(scale), _ptr(counters if n_splits > 1 else None),
                                     ctypes.c_int(int(USE_CLUSTER_MERGE)), _ptr(order), _ptr(work),
                                     ctypes.c_int(work.shape[0] if work is not None else 0), _stream()),
           "attention_decode (TMA, work list)" if work is not None
           else "attention_decode (TMA, cluster merge)" if USE_CLUSTER_MERGE and 2 <= n_splits <= 16
           else "attention_decode (TMA)")
    return True


_cluster_capacity = {}


def attention_decode_cluster_capacity(dtype: torch.dtype, head_dim: int, fused: bool):
    """capacity[s], s = 0 .. 16: how many clusters of s blocks of the TMA decode kernel the device holds at once
    (0: no such cluster), or None when that kernel or its cluster merge is not what runs for this dtype and
    head size.  A launch with more clusters than that runs in two waves; measured on B200 at 8 kv heads of
    128, contexts of 128 .. 2,048: 3 sequences with 12 splits (24 clusters, 21 fit) 14.2 us, with 10 splits
    8.8 us; 4 sequences 9 / 8 splits 14.4 / 9.1 us; 5 sequences 7 / 6 splits 15.1 / 9.9 us."""
    if not (USE_TMA_DECODE and USE_TENSOR_CORE_DECODE and USE_CLUSTER_MERGE and dtype == torch.bfloat16
            and lib().mll_attn_decode_tma_supported(dtype_code(dtype), head_dim)):
        return None
    key = (head_dim, bool(fused))
    if key not in _cluster_capacity:
        _cluster_capacity[key] = (0, 0) + tuple(
            int(lib().mll_attn_decode_tma_resident_clusters(ctypes.c_int(head_dim), ctypes.c_int(int(fused)), ctypes.c_int(s)))
            for s in range(2, 17))
    return _cluster_capacity[key]


def attention_decode_fused_supported(dtype: torch.dtype, head_dim: int) -> bool:
    """Whether a decode step's rotary encoding, cache write and attention can be one launch."""
    return bool(USE_FUSED_DECODE and USE_TENSOR_CORE_DECODE
                and lib().mll_attn_decode_mma_supported(dtype_code(dtype), head_dim))


def attention_decode_fused(qkv, cos, sin, interleaved: bool, write_kv: bool, k_cache, v_cache, seq_slot, seq_ctx,
                           block_table, scratch, out, n_seqs: int, n_heads: int, n_kv_heads: int, head_dim: int,
                           n_splits: int, window: int, scale: float, counters: Optional[torch.Tensor] = None,
                           order: Optional[torch.Tensor] = None, work: Optional[torch.Tensor] = None) -> None:
    """Decode step: row i of qkv [B, (Hq + 2 Hk) d] is sequence i's new token at position seq_ctx[i] - 1.
    Rotates q and k (tables as for rope_cache_write, or None), writes k and v into the paged cache and
    attends over it, in one launch (bfloat16, head sizes 16 .. 256 in steps of 16).
    `work`: int32 list of `decode_work_entry` places (-1: unused) that gives every sequence its own number of
    splits, long ones more than short ones; n_splits is then the most any has (the TMA-fed kernel only)."""
    _need(qkv, "attention qkv", torch.bfloat16, 2)
    _need(out, "attention out", torch.bfloat16, 2)
    _need(k_cache, "attention k_cache", torch.bfloat16, 4)
    _need(v_cache, "attention v_cache", torch.bfloat16, 4)
    if tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, head_dim) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention: cache shape {tuple(k_cache.shape)} is not [pages, {n_kv_heads}, {PAGE}, {head_dim}]")
    if out.shape[1] != n_heads * head_dim or qkv.shape[1] < (n_heads + (2 * n_kv_heads if write_kv else 0)) * head_dim:
        raise KernelError("attention decode (fused): qkv/out width differs from the heads")
    for name, t in (("seq_slot", seq_slot), ("seq_ctx", seq_ctx)):
        _need(t, f"attention {name}", torch.int32, 1)
    _need(block_table, "attention block_table", torch.int32, 2)
    if min(qkv.shape[0], out.shape[0], seq_slot.shape[0], seq_ctx.shape[0]) < n_seqs:
        raise KernelError("attention decode (fused): an input has fewer rows than sequences")
    if cos is not None:
        _need(cos, "rope cos", torch.float32, 2)
        _need(sin, "rope sin", torch.float32, 2)
        if cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
            raise KernelError(f"rope: table {tuple(cos.shape)} does not match head_dim {head_dim}")
    if n_splits > 1:
        _need(scratch, "attention scratch", torch.float32)
        if scratch.numel() < attention_decode_scratch_floats(n_seqs, n_heads, head_dim, n_splits):
            raise KernelError("attention decode: scratch too small for the split count")
        if counters is None:
            raise KernelError("attention decode (fused): splits need arrival counters")
        _need(counters, "attention counters", torch.int32, 1)
        if counters.shape[0] < n_seqs * n_kv_heads * ((n_heads // n_kv_heads + 15) // 16):
            raise KernelError("attention decode: counters shorter than sequences x kv heads x head chunks")
    if _tma_decode(None, qkv, cos, sin, interleaved, write_kv, k_cache, v_cache, seq_slot, seq_ctx, block_table, scratch,
                   out, n_seqs, n_heads, n_kv_heads, head_dim, n_splits, window, scale, counters, _order(order, n_seqs), work):
        return
    if work is not None:
        raise KernelError("attention decode: a work list was given, but the kernel that takes one does not run here")
    _check(lib().mll_attn_decode_mma_fused(_ptr(qkv), ctypes.c_int(qkv.shape[1]), _ptr(cos), _ptr(sin),
                                           ctypes.c_int(int(interleaved)), ctypes.c_int(int(write_kv)), _ptr(k_cache),
                                           _ptr(v_cache), _ptr(seq_slot), _ptr(seq_ctx), _ptr(block_table),
                                           _ptr(scratch), _ptr(out), ctypes.c_int(n_seqs), ctypes.c_int(n_heads),
                                           ctypes.c_int(n_kv_heads), ctypes.c_int(head_dim),
                                           ctypes.c_int(block_table.shape[1]), ctypes.c_int(n_splits),
                                           ctypes.c_int(window), ctypes.c_float(scale),
                                           _ptr(counters if n_splits > 1 else None), _stream()),
           "attention_decode (fused)")


PREFILL_TILE = 64  # query rows per entry of the work list that `attention_prefill` takes


def attention_prefill(q, k_cache, v_cache, seq_slot, seq_ctx, seq_qstart, seq_qlen, tile_seq, tile_row0,
                      block_table, out, n_tiles: int, n_heads: int, n_kv_heads: int, head_dim: int,
                      window: int, scale: float, wide_tiles=None) -> None:
    """Tiles of up to 64 query tokens of sequences with unequal lengths over the paged cache.
    `wide_tiles`: (sequence, first row) int32 lists of the same rows in tiles of 128, which the tcgen05 kernel
    works on; without them it walks the 64-row list and every other block finds nothing to do."""
    _check_attention(q, k_cache, v_cache, out, n_heads, n_kv_heads, head_dim)
    for name, t in (("seq_slot", seq_slot), ("seq_ctx", seq_ctx), ("seq_qstart", seq_qstart),
                    ("seq_qlen", seq_qlen), ("tile_seq", tile_seq), ("tile_row0", tile_row0)):
        _need(t, f"attention {name}", torch.int32, 1)
    _need(block_table, "attention block_table", torch.int32, 2)
    if tile_seq.shape[0] < n_tiles or tile_row0.shape[0] < n_tiles:
        raise KernelError("attention prefill: tile lists shorter than the tile count")
    if (USE_TENSOR_CORE_PREFILL and USE_TCGEN05_PREFILL
            and lib().mll_attn_prefill_tc5_supported(dtype_code(q.dtype), head_dim)):
        if wide_tiles is not None:
            tile_seq, tile_row0 = wide_tiles
            _need(tile_seq, "attention wide tile_seq", torch.int32, 1)
            _need(tile_row0, "attention wide tile_row0", torch.int32, 1)
            n_tiles = tile_seq.shape[0]
            if tile_row0.shape[0] != n_tiles:
                raise KernelError("attention prefill: the wide tile lists differ in length")
        _check(lib().mll_attn_prefill_tc5(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(seq_slot), _ptr(seq_ctx),
                                          _ptr(seq_qstart), _ptr(seq_qlen), _ptr(tile_seq), _ptr(tile_row0),
                                          _ptr(block_table), _ptr(out), ctypes.c_int(q.shape[0]),
                                          ctypes.c_longlong(k_cache.shape[0]), ctypes.c_int(n_tiles),
                                          ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads), ctypes.c_int(head_dim),
                                          ctypes.c_int(block_table.shape[1]), ctypes.c_int(window),
                                          ctypes.c_float(scale), _stream()), "attention_prefill (tcgen05)")
        return
    if USE_TENSOR_CORE_PREFILL and lib().mll_attn_prefill_mma_supported(dtype_code(q.dtype), head_dim):
        _check(lib().mll_attn_prefill_mma(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(seq_slot), _ptr(seq_ctx),
                                          _ptr(seq_qstart), _ptr(seq_qlen), _ptr(tile_seq), _ptr(tile_row0),
                                          _ptr(block_table), _ptr(out), ctypes.c_int(n_tiles), ctypes.c_int(n_heads),
                                          ctypes.c_int(n_kv_heads), ctypes.c_int(head_dim),
                                          ctypes.c_int(block_table.shape[1]), ctypes.c_int(window),
                                          ctypes.c_float(scale), _stream()), "attention_prefill (tensor cores)")
        return
    _check(lib().mll_attn_prefill(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(seq_slot), _ptr(seq_ctx),
                                  _ptr(seq_qstart), _ptr(seq_qlen), _ptr(tile_seq), _ptr(tile_row0),
                                  _ptr(block_table), _ptr(out), dtype_code(q.dtype), ctypes.c_int(n_tiles),
                                  ctypes.c_int(n_heads), ctypes.c_int(n_kv_heads), ctypes.c_int(head_dim),
                                  ctypes.c_int(block_table.shape[1]), ctypes.c_int(window),
                                  ctypes.c_float(scale), _stream()), "attention_prefill")


def argmax(logits: torch.Tensor, tokens: torch.Tensor, status: torch.Tensor) -> None:
    """tokens[r] = first index of the maximum of logits[r]; status[r] = 1 if a logit is not finite."""
    _need(logits, "argmax logits", torch.float32, 2)
    _need(tokens, "argmax tokens", torch.int32, 1)
    _need(status, "argmax status", torch.int32, 1)
    n = logits.shape[0]
    if tokens.shape[0] < n or status.shape[0] < n:
        raise KernelError("argmax: outputs shorter than the row count")
    _check(lib().mll_argmax(_ptr(logits), ctypes.c_int(n), ctypes.c_int(logits.shape[1]), _ptr(tokens),
                            _ptr(status), _stream()), "argmax")


def sample(logits: torch.Tensor, temperature: float, top_k: int, seed: int, request: torch.Tensor,
           step: torch.Tensor, tokens: torch.Tensor, status: torch.Tensor) -> None:
    """Temperature (top_k == 0) or top-k sampling with u = f(seed, request[r], step[r])."""
    _need(logits, "sample logits", torch.float32, 2)
    for name, t in (("request", request), ("step", step), ("tokens", tokens), ("status", status)):
        _need(t, f"sample {name}", torch.int32, 1)
        if t.shape[0] < logits.shape[0]:
            raise KernelError(f"sample: {name} shorter than the row count")
    _check(lib().mll_sample(_ptr(logits), ctypes.c_int(logits.shape[0]), ctypes.c_int(logits.shape[1]),
                            ctypes.c_float(temperature), ctypes.c_int(top_k),
                            ctypes.c_ulonglong(seed & 0xFFFFFFFFFFFFFFFF), _ptr(request), _ptr(step),
                            _ptr(tokens), _ptr(status), _stream()), "sample")
