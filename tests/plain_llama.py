"""Plain, slow Llama decoder used as the oracle of the tests.

Whole sequences, no cache, one function per part, NumPy only.  Nothing here is
imported by the product and nothing of the product is imported here: the model
folder reader, the rotary tables, the sampler and its random numbers are all
restated so that a fault in the product cannot hide in shared code.

All arithmetic is float64 on the stored (float32 or bfloat16) weight values.
`act_round` optionally rounds activations where a bfloat16 engine stores them
(norm outputs, projection outputs, rotated q/k, attention output, SwiGLU
output), so that the bfloat16 comparison measures accumulation order and not the
storage format.

Formulas follow the reference engine (paths are inside the reference project):
  src/forward.cc:385-414   block: pre-norm attention + residual, pre-norm FFN + residual
  src/forward.cc:415-424   final norm and lm_head
  scripts/reference_forward.py:166-275  the reference's own NumPy oracle
The llama3 `rope_scaling` rule has no counterpart in the reference (it has no
rope scaling); it follows the published Llama-3.1 frequency rule.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np


# --------------------------------------------------------------------------- #
# model folder                                                                #
# --------------------------------------------------------------------------- #
def _bf16_bits_to_f32(raw: np.ndarray) -> np.ndarray:
    return (raw.astype(np.uint32) << 16).view(np.float32)


def read_model_folder(path):
    """Read `config.json` and `model.safetensors` of a folder.

    Returns (config dict, {tensor name: float32 array}).  bfloat16 tensors are
    widened exactly.  The container layout (8-byte little-endian header length,
    JSON header with dtype/shape/data_offsets, raw bytes) is the public
    safetensors format.
    """
    path = Path(path)
    config = json.loads((path / "config.json").read_text())
    blob = (path / "model.safetensors").read_bytes()
    (header_len,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + header_len].decode("utf-8"))
    base = 8 + header_len
    tensors = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        begin, end = info["data_offsets"]
        raw = blob[base + begin:base + end]
        shape = tuple(info["shape"])
        if info["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype="<f4").reshape(shape).copy()
        elif info["dtype"] == "BF16":
            arr = _bf16_bits_to_f32(np.frombuffer(raw, dtype="<u2")).reshape(shape).copy()
        elif info["dtype"] == "F16":
            arr = np.frombuffer(raw, dtype="<f2").astype(np.float32).reshape(shape)
        else:
            raise ValueError(f"plain reader: dtype {info['dtype']} of {name} not handled")
        tensors[name] = arr
    return config, tensors


def round_bf16(x):
    """Round float values to the nearest bfloat16 (ties to even), return float64."""
    f = np.asarray(x, dtype=np.float32)
    bits = f.view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    return rounded.astype(np.uint32).view(np.float32).astype(np.float64).reshape(f.shape)


def _identity(x):
    return x


# --------------------------------------------------------------------------- #
# parts                                                                       #
# --------------------------------------------------------------------------- #
def embedding(table, tokens):
    """x[t, :] = E[token_t, :] (src/forward.cc:198-205)."""
    tokens = np.asarray(tokens, dtype=np.int64)
    if tokens.min() < 0 or tokens.max() >= table.shape[0]:
        raise ValueError("token outside the vocabulary")  # src/forward.cc:437-439
    return table[tokens].astype(np.float64)


def rms_norm(x, weight, eps):
    """y_i = x_i * w_i / sqrt(mean_j(x_j^2) + eps), eps inside the root
    (src/ops.cc:95-110; scripts/reference_forward.py:166-172)."""
    x = x.astype(np.float64)
    denom = np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + float(eps))
    return x * weight.astype(np.float64) / denom


def linear(x, weight, bias=None):
    """y[o] = sum_k W[o, k] x[k], W row-major [out, in]
    (matumal/matuml_ops.cc:155-161); the bias is added only where the tensor
    exists (src/forward.cc:159-161, 328-335)."""
    y = np.asarray(x, dtype=np.float64) @ np.asarray(weight, dtype=np.float64).T
    if bias is not None:
        y = y + bias.astype(np.float64)
    return y


def rope_inverse_frequencies(head_dim, theta, scaling=None):
    """f_i = theta^(-2i/d) for pair i in [0, d/2) (src/ops.cc:200-203).

    With `scaling` of type llama3 (factor, low_freq_factor, high_freq_factor,
    original_max_position_embeddings = L0) each frequency is changed by its
    wavelength lam = 2*pi/f: kept when lam < L0/high, divided by factor when
    lam > L0/low, and blended linearly in between with
    s = (L0/lam - low) / (high - low): f' = (1-s) f/factor + s f.
    """
    half = head_dim // 2
    freqs = np.array([float(theta) ** (-2.0 * i / head_dim) for i in range(half)],
                     dtype=np.float64)
    if scaling is None:
        return freqs
    kind = scaling.get("rope_type", scaling.get("type"))
    if kind in (None, "default"):
        return freqs
    if kind != "llama3":
        raise ValueError(f"plain rope: scaling type {kind!r} not handled")
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    original = float(scaling["original_max_position_embeddings"])
    out = np.empty_like(freqs)
    for i, f in enumerate(freqs):
        wavelength = 2.0 * math.pi / f
        if wavelength < original / high:
            out[i] = f
        elif wavelength > original / low:
            out[i] = f / factor
        else:
            s = (original / wavelength - low) / (high - low)
            out[i] = (1.0 - s) * f / factor + s * f
    return out


def apply_rope(x, positions, inv_freq, interleaved):
    """Rotate pairs of x [T, H, d] by angle pos * f_i.

    interleaved=True pairs (2i, 2i+1): the reference's "Normal" type;
    interleaved=False pairs (i, i + d/2): its "NeoX" type (src/ops.cc:206-221).
    (a, b) <- (a cos - b sin, a sin + b cos).
    """
    x = x.astype(np.float64)
    T, H, d = x.shape
    half = d // 2
    angle = np.asarray(positions, dtype=np.float64)[:, None] * inv_freq[None, :]  # [T, half]
    cos = np.cos(angle)[:, None, :]
    sin = np.sin(angle)[:, None, :]
    out = np.empty_like(x)
    if interleaved:
        a, b = x[..., 0::2], x[..., 1::2]
        out[..., 0::2] = a * cos - b * sin
        out[..., 1::2] = a * sin + b * cos
    else:
        a, b = x[..., :half], x[..., half:]
        out[..., :half] = a * cos - b * sin
        out[..., half:] = a * sin + b * cos
    return out


def causal_attention(q, k, v, window=None, q_positions=None):
    """q [T, Hq, d], k/v [S, Hk, d] -> [T, Hq, d]; query t sits at position
    q_positions[t] (default t, with S == T) and reads keys 0..its position.

    Head h reads kv head h // (Hq/Hk); score_t = (q . k_t) / sqrt(d) for
    t <= position (the scale multiplies after the dot); softmax with the
    maximum subtracted; out = sum_t p_t v_t (src/forward.cc:265-298).
    `window` keeps only the last `window` keys (not used by the reference).
    """
    T, Hq, d = q.shape
    Hk = k.shape[1]
    group = Hq // Hk
    scale = 1.0 / math.sqrt(d)
    out = np.zeros((T, Hq, d), dtype=np.float64)
    for t in range(T):
        pos = t if q_positions is None else int(q_positions[t])
        first = 0 if not window else max(0, pos - window + 1)
        for h in range(Hq):
            g = h // group
            keys = k[first:pos + 1, g].astype(np.float64)
            values = v[first:pos + 1, g].astype(np.float64)
            scores = (keys @ q[t, h].astype(np.float64)) * scale
            e = np.exp(scores - scores.max())
            p = e / e.sum()
            out[t, h] = p @ values
    return out


def swiglu(gate, up):
    """f = gate * 1/(1 + exp(-gate)) * up (src/ops.cc:135-151)."""
    gate = gate.astype(np.float64)
    return gate * (1.0 / (1.0 + np.exp(-gate))) * up.astype(np.float64)


def feed_forward(h, w_gate, w_up, w_down, act_round=_identity):
    """Wdown . (silu(Wgate h) * (Wup h)) (src/forward.cc:313-322)."""
    g = act_round(linear(h, w_gate))
    u = act_round(linear(h, w_up))
    return act_round(linear(act_round(swiglu(g, u)), w_down))


def attention_block(h, positions, weights, prefix, cfg, inv_freq, act_round=_identity):
    """q/k/v projections, head split, RoPE on q and k, causal GQA attention,
    output projection (src/forward.cc:393-407)."""
    Hq = cfg["num_attention_heads"]
    Hk = cfg.get("num_key_value_heads", Hq)
    d = cfg.get("head_dim") or cfg["hidden_size"] // Hq
    T = h.shape[0]
    name = prefix + "self_attn."
    def project(which):
        # a bfloat16 engine stores the product, then adds the bias in float32
        y = act_round(linear(h, weights[name + which + "_proj.weight"]))
        bias = weights.get(name + which + "_proj.bias")
        return y if bias is None else y + bias.astype(np.float64)

    q, k, v = project("q"), project("k"), act_round(project("v"))
    q = q.reshape(T, Hq, d)
    k = k.reshape(T, Hk, d)
    v = v.reshape(T, Hk, d)
    interleaved = bool(cfg.get("rope_interleaved", False))
    q = act_round(apply_rope(q, positions, inv_freq, interleaved))
    k = act_round(apply_rope(k, positions, inv_freq, interleaved))
    a = act_round(causal_attention(q, k, v, cfg.get("sliding_window")))
    out = act_round(linear(a.reshape(T, Hq * d), weights[name + "o_proj.weight"]))
    bias = weights.get(name + "o_proj.bias")
    return out if bias is None else act_round(out + bias.astype(np.float64))


def forward_sequence(cfg, weights, tokens, act_round=_identity, return_hidden=False):
    """Logits [T, vocab] of one whole sequence that starts at position 0."""
    Hq = cfg["num_attention_heads"]
    d = cfg.get("head_dim") or cfg["hidden_size"] // Hq
    eps = cfg.get("rms_norm_eps", 1e-5)
    inv_freq = rope_inverse_frequencies(d, cfg.get("rope_theta", 10000.0), cfg.get("rope_scaling"))
    positions = np.arange(len(tokens))
    x = embedding(weights["model.embed_tokens.weight"], tokens)
    for layer in range(cfg["num_hidden_layers"]):
        prefix = f"model.layers.{layer}."
        h = act_round(rms_norm(x, weights[prefix + "input_layernorm.weight"], eps))
        x = x + attention_block(h, positions, weights, prefix, cfg, inv_freq, act_round)
        h = act_round(rms_norm(x, weights[prefix + "post_attention_layernorm.weight"], eps))
        x = x + feed_forward(h, weights[prefix + "mlp.gate_proj.weight"],
                             weights[prefix + "mlp.up_proj.weight"],
                             weights[prefix + "mlp.down_proj.weight"], act_round)
    if return_hidden:
        return x
    h = act_round(rms_norm(x, weights["model.norm.weight"], eps))
    head = weights["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) \
        else weights["lm_head.weight"]
    return linear(h, head)


# --------------------------------------------------------------------------- #
# sampling                                                                    #
# --------------------------------------------------------------------------- #
_MASK64 = (1 << 64) - 1


def _mix64(z):
    """splitmix64 finaliser on Python integers."""
    z = (z + 0x9E3779B97F4A7C15) & _MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
    return z ^ (z >> 31)


def uniform_from_counter(seed, request, step):
    """The sampler's uniform number in [0, 1) for (seed, request, step): three
    chained splitmix64 rounds, top 24 bits as a float32 fraction."""
    z = _mix64(seed & _MASK64)
    z = _mix64(z ^ (request & _MASK64))
    z = _mix64(z ^ (step & _MASK64))
    return np.float32((z >> 40) / float(1 << 24))


def greedy(logits):
    """First index of the maximum (src/sampler.cc:31-41)."""
    return int(np.argmax(np.asarray(logits)))


def sample(logits, temperature, top_k, u):
    """Temperature / top-k sampling by inverse CDF (src/sampler.cc:42-79, 110-147).

    temperature < 1e-6 or top_k == 1 is greedy.  Without top-k the candidates
    are walked in id order; with top-k they are the k largest logits in
    descending order (equal logits: lower id first).  w_i = exp((l_i - max)/T),
    the first candidate whose cumulative w/sum reaches u is returned, else the last.
    All in float32.
    """
    logits = np.asarray(logits, dtype=np.float32)
    if temperature < 1e-6 or top_k == 1:
        return greedy(logits)
    ids = np.arange(len(logits))
    if top_k and top_k > 0:
        k = min(int(top_k), len(logits))
        order = np.lexsort((ids, -logits.astype(np.float64)))
        ids = order[:k]
    cand = logits[ids]
    w = np.exp((cand - cand.max()) / np.float32(temperature)).astype(np.float32)
    total = np.float32(0)
    for value in w:
        total = np.float32(total + value)
    threshold = np.float32(u) * total
    cumulative = np.float32(0)
    for i, value in enumerate(w):
        cumulative = np.float32(cumulative + value)
        if threshold <= cumulative:
            return int(ids[i])
    return int(ids[-1])
