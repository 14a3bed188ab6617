"""Shared test helpers: tolerances and the comparison rule.

float32: absolute error <= 1e-4 on every logit (the reference's golden bound,
scripts/compare_logits.py:14-16), no NaN/Inf, the same top-1 token unless the
reference's two best logits are closer than the tolerance, and error <= 1e-4 relative to
the largest |logit| of the comparison.  The reference also bounds the element-wise
relative error where |reference| >= 1e-3; that holds there because both of its sides sum
in float32 in nearly the same order.  Against a float64 oracle it is ill-conditioned: a
logit is a sum of terms ~100 times larger than a 1e-3 result, so an error of 3e-7 (one
float32 rounding of a term) already reads as 3e-4 "relative".  The norm-wise bound used
here is the stricter of the two whenever the largest |logit| is below 1.
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
        scale = np.abs(ref).max()
        assert err.max() <= F32_REL * max(scale, REL_FLOOR), \
            f"{what}: err {err.max():.3e} exceeds {F32_REL} of the largest logit {scale:.4f}"
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
