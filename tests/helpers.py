"""Shared test helpers: tolerances and the comparison rule.

float32: the reference's golden rule (scripts/compare_logits.py:14-16,189-217): absolute
error <= 1e-4 and relative error <= 1e-4 wherever |reference| >= 1e-3, no NaN/Inf, and
the same top-1 token unless the reference's two best logits are closer than the
absolute tolerance.
bfloat16: the plain implementation rounds activations to bfloat16 where the engine
stores them, so what is left is accumulation order and rounding flips of single values
(2^-8 relative each).  Bound chosen before the first run and not to be widened: maximum
error <= 2% and mean error <= 0.4% of the largest |reference logit| of the comparison.
"""
import numpy as np

import plain_llama as pl

F32_ABS = 1e-4
F32_REL = 1e-4
REL_FLOOR = 1e-3
BF16_MAX_FRACTION = 2e-2
BF16_MEAN_FRACTION = 4e-3


def plain_logits(folder, tokens, dtype):
    cfg, weights = pl.read_model_folder(folder)
    if dtype == "bfloat16":  # weights are used as stored; only activations are rounded
        return pl.forward_sequence(cfg, weights, tokens, act_round=pl.round_bf16)
    return pl.forward_sequence(cfg, weights, tokens)


def assert_close(got, ref, dtype, what=""):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    err = np.abs(got - ref)
    worst = np.unravel_index(np.argmax(err), err.shape)
    if dtype == "float32":
        assert err.max() <= F32_ABS, f"{what}: abs err {err.max():.3e} at {worst} (ref {ref[worst]:.6f})"
        big = np.abs(ref) >= REL_FLOOR
        if big.any():
            rel = (err[big] / np.abs(ref[big])).max()
            assert rel <= F32_REL, f"{what}: rel err {rel:.3e}"
        tol = F32_ABS
    else:
        scale = np.abs(ref).max()
        assert err.max() <= BF16_MAX_FRACTION * scale, \
            f"{what}: max err {err.max():.3e} at {worst} exceeds {BF16_MAX_FRACTION} * {scale:.3f}"
        assert err.mean() <= BF16_MEAN_FRACTION * scale, \
            f"{what}: mean err {err.mean():.3e} exceeds {BF16_MEAN_FRACTION} * {scale:.3f}"
        tol = BF16_MAX_FRACTION * scale
    if ref.ndim == 2:  # top-1 agrees unless the reference's best two are within the tolerance
        for row in range(ref.shape[0]):
            best = int(np.argmax(ref[row]))
            if int(np.argmax(got[row])) != best:
                second = np.partition(ref[row], -2)[-2]
                assert ref[row, best] - second <= 2 * tol, f"{what}: top-1 differs at row {row}"
