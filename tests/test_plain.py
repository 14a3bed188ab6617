"""The plain implementation itself (no GPU): against the reference project's own outputs
(tests/golden, made by tests/golden/make_golden.py from scripts/reference_forward.py and from
the C++ CPU engine), and against properties of each part."""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

import plain_llama as pl
import tiny_configs as tc

GOLDEN = Path(__file__).parent / "golden"


@pytest.fixture(scope="module")
def tiny_a(tmp_path_factory):
    folder = tc.write_folder("A", "float32", tmp_path_factory.mktemp("goldenA"))
    meta = json.loads((GOLDEN / "tinyA_reference.json").read_text())
    digest = hashlib.sha256((Path(folder) / "model.safetensors").read_bytes()).hexdigest()
    if digest != meta["model_sha256"]:
        pytest.fail("the seeded tiny-A weights differ from those the golden files were made with; "
                    "rerun tests/golden/make_golden.py")
    cfg, weights = pl.read_model_folder(folder)
    return cfg, weights, meta


def test_matches_the_references_numpy_oracle(tiny_a):
    cfg, weights, meta = tiny_a
    golden = np.load(GOLDEN / "tinyA_reference_numpy_logits.npy")
    ours = pl.forward_sequence(cfg, weights, meta["numpy_tokens"])
    assert ours.shape == golden.shape == (24, 131)
    # the reference accumulates in float32; the bound is its own golden tolerance
    np.testing.assert_allclose(ours, golden, atol=1e-4, rtol=0)
    assert (ours.argmax(axis=1) == golden.argmax(axis=1)).all()
    assert np.abs(ours - golden).max() < 2e-6


def test_matches_the_references_cpp_engine(tiny_a):
    cfg, weights, meta = tiny_a
    golden = np.load(GOLDEN / "tinyA_reference_cpp_logits.npy")
    prompt, generated = meta["cpp_prompt_tokens"], meta["cpp_generated"]
    assert prompt == [128] + [ord(c) for c in "hello"]
    # the dump holds one step per fed token: the prompt, then every generated token but the last
    fed = prompt + generated[:-1]
    assert golden.shape == (len(fed), 131)
    ours = pl.forward_sequence(cfg, weights, fed)
    np.testing.assert_allclose(ours, golden, atol=1e-4, rtol=0)
    # greedy generation: every generated token is the plain argmax of the step before it
    for i, token in enumerate(generated):
        assert pl.greedy(ours[len(prompt) - 1 + i]) == token


def test_tiny_b_without_rope_scaling_matches_the_references_cpp_engine(tmp_path):
    # what the reference can run of tiny B: multi-query attention (6 heads on 1), half-split rotary pairs, eps
    # 1e-6, theta 500000, a tied head, three layers - everything but the llama3 rope scaling, which it does
    # not have.  Its C++ forward ran these four sequences one token per forward (tests/golden/reference_driver.cc).
    folder = tc.write_folder("B", "float32", tmp_path)
    meta = json.loads((GOLDEN / "tinyB_noscale_reference.json").read_text())
    digest = hashlib.sha256((Path(folder) / "model.safetensors").read_bytes()).hexdigest()
    assert digest == meta["model_sha256"], "the seeded tiny-B weights changed: rerun tests/golden/make_golden.py"
    cfg, weights = pl.read_model_folder(folder)
    assert cfg["rope_scaling"] is not None and cfg["tie_word_embeddings"] and cfg["num_key_value_heads"] == 1
    cfg = dict(cfg, rope_scaling=None)
    golden = np.load(GOLDEN / "tinyB_noscale_reference_cpp_logits.npy")
    assert [len(s) for s in meta["sequences"]] == [29, 13, 52, 18] and golden.shape == (112, 257)
    ours = np.concatenate([pl.forward_sequence(cfg, weights, tokens) for tokens in meta["sequences"]])
    np.testing.assert_allclose(ours, golden, atol=1e-4, rtol=0)
    assert (ours.argmax(axis=1) == golden.argmax(axis=1)).all()
    # the scaling does matter for these sequences: with it the logits move by far more than the tolerance
    scaled = pl.forward_sequence(dict(cfg, rope_scaling=tc.TINY["B"]["rope_scaling"]), weights, meta["sequences"][2])
    assert np.abs(scaled - golden[42:94]).max() > 1e-3


def test_rms_norm_and_swiglu_values():
    x = np.array([[3.0, -4.0]])
    np.testing.assert_allclose(pl.rms_norm(x, np.array([1.0, 2.0]), 0.0), [[3 / np.sqrt(12.5), -8 / np.sqrt(12.5)]])
    # eps sits inside the root (src/ops.cc:104-106)
    np.testing.assert_allclose(pl.rms_norm(np.zeros((1, 4)), np.ones(4), 1e-5), np.zeros((1, 4)))
    big = pl.rms_norm(np.array([[1e-3, 0.0]]), np.ones(2), 1e-2)
    np.testing.assert_allclose(big[0, 0], 1e-3 / np.sqrt(0.5e-6 + 1e-2))
    np.testing.assert_allclose(pl.swiglu(np.array([0.0, 1.0, -20.0]), np.array([5.0, 2.0, 1.0])),
                               [0.0, 2.0 / (1 + np.exp(-1.0)), -20.0 / (1 + np.exp(20.0))])


@pytest.mark.parametrize("interleaved", [True, False])
def test_rope_is_a_rotation_that_composes(interleaved):
    rng = np.random.RandomState(0)
    x = rng.randn(3, 2, 16)
    inv = pl.rope_inverse_frequencies(16, 37.0)
    assert inv[0] == 1.0 and np.isclose(inv[-1], 37.0 ** (-14 / 16))
    at0 = pl.apply_rope(x, [0, 0, 0], inv, interleaved)
    np.testing.assert_allclose(at0, x)                                   # position 0 changes nothing
    y = pl.apply_rope(x, [5, 7, 63], inv, interleaved)
    np.testing.assert_allclose(np.linalg.norm(y, axis=-1), np.linalg.norm(x, axis=-1))
    twice = pl.apply_rope(pl.apply_rope(x, [2, 2, 2], inv, interleaved), [3, 5, 61], inv, interleaved)
    np.testing.assert_allclose(twice, y, atol=1e-12)                     # angles add (test/ops_test.cc:749-835)
    # the score of a rotated pair depends on the distance only
    q, k = rng.randn(1, 1, 16), rng.randn(1, 1, 16)
    a = (pl.apply_rope(q, [9], inv, interleaved) * pl.apply_rope(k, [4], inv, interleaved)).sum()
    b = (pl.apply_rope(q, [25], inv, interleaved) * pl.apply_rope(k, [20], inv, interleaved)).sum()
    np.testing.assert_allclose(a, b)
    if interleaved:
        np.testing.assert_allclose(y[0, 0, 0], x[0, 0, 0] * np.cos(5.0) - x[0, 0, 1] * np.sin(5.0))
    else:
        np.testing.assert_allclose(y[0, 0, 0], x[0, 0, 0] * np.cos(5.0) - x[0, 0, 8] * np.sin(5.0))


def test_llama3_scaling_regimes():
    scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 8192}
    plain = pl.rope_inverse_frequencies(128, 500000.0)
    scaled = pl.rope_inverse_frequencies(128, 500000.0, scaling)
    wavelength = 2 * np.pi / plain
    high, low = wavelength < 8192 / 4, wavelength > 8192 / 1
    assert high.any() and low.any() and (~high & ~low).any()
    np.testing.assert_array_equal(scaled[high], plain[high])
    np.testing.assert_allclose(scaled[low], plain[low] / 8)
    mid = ~high & ~low
    assert ((scaled[mid] < plain[mid]) & (scaled[mid] > plain[mid] / 8)).all()
    assert (np.diff(scaled) < 0).all()                                   # still monotone in the pair index


def test_attention_is_causal_grouped_and_windowed():
    rng = np.random.RandomState(1)
    q, k, v = rng.randn(6, 4, 8), rng.randn(6, 2, 8), rng.randn(6, 2, 8)
    out = pl.causal_attention(q, k, v)
    np.testing.assert_allclose(out[0, :, :], v[0, [0, 0, 1, 1], :])      # the first token sees itself only
    changed = pl.causal_attention(q, np.concatenate([k[:5], k[5:] + 9]), np.concatenate([v[:5], v[5:] - 3]))
    np.testing.assert_allclose(changed[:5], out[:5])                     # later keys do not reach earlier queries
    np.testing.assert_allclose(pl.causal_attention(q, k, v, window=1), v[:, [0, 0, 1, 1], :])
    np.testing.assert_allclose(pl.causal_attention(q, k, v, window=6), out)
    one = pl.causal_attention(q[4:5], k, v, q_positions=[4])
    np.testing.assert_allclose(one[0], out[4])
    # stable for huge scores (the reference's softmax test, tests/test_cuda_ops.cc:24-26)
    big = pl.causal_attention(np.full((2, 1, 8), 100.0), np.full((2, 1, 8), 100.0), v[:2, :1])
    assert np.isfinite(big).all()


def test_sampling_rules():
    logits = np.array([1.0, 3.0, 3.0, -2.0], dtype=np.float32)
    assert pl.greedy(logits) == 1                                        # first of equal maxima
    assert pl.sample(logits, 0.0, 0, 0.9) == 1 and pl.sample(logits, 1.0, 1, 0.9) == 1
    w = np.exp(logits - 3.0)
    cdf = np.cumsum(w) / w.sum()
    for u, want in ((0.0, 0), (float(cdf[0]) + 1e-3, 1), (float(cdf[1]) + 1e-3, 2), (0.9999, 3 if cdf[2] < 0.9999 else 2)):
        assert pl.sample(logits, 1.0, 0, u) == want
    # top-k walks the k largest in descending order, equal logits by lower id
    assert pl.sample(logits, 1.0, 2, 0.1) == 1 and pl.sample(logits, 1.0, 2, 0.9) == 2
    us = [float(pl.uniform_from_counter(7, r, s)) for r in range(20) for s in range(20)]
    assert all(0.0 <= u < 1.0 for u in us) and len(set(us)) > 390 and 0.4 < np.mean(us) < 0.6
    assert pl.uniform_from_counter(7, 3, 5) == pl.uniform_from_counter(7, 3, 5) != pl.uniform_from_counter(8, 3, 5)


def test_bf16_rounding():
    assert pl.round_bf16(np.float32(1.0)) == 1.0
    assert pl.round_bf16(np.float32(1.0 + 2 ** -8)) == 1.0               # tie goes to the even mantissa
    assert pl.round_bf16(np.float32(1.0 + 3 * 2 ** -8)) == 1.0 + 2 ** -6
    assert pl.round_bf16(np.float32(1.0 + 2 ** -7)) == 1.0 + 2 ** -7
    x = np.random.RandomState(2).randn(1000).astype(np.float32)
    assert np.abs(pl.round_bf16(x) - x).max() <= np.abs(x).max() * 2 ** -8
