"""The engine at the layer widths of a real model, against the plain implementation.

The tiny configurations never reach the schedule that a model of real size runs: every product
of a small decode step on the weight-streaming kernels with the norms folded in (the direct kernel
up to 8 rows, the tall matrices - gate/up with the fused activation, the head - on the tcgen05
kernel from 9 to 16 rows, and the TMA kernel where it is forced), 32/8 heads of 128
in the tcgen05 prefill attention and the cluster-merged decode attention, decode steps of
more than 16 rows on the library product.  Here the layers have the widths of Llama-3.1-8B
(hidden 4096, 32 query / 8 key-value heads of 128, intermediate 14336, llama3 rope scaling
8 / 1 / 4 / 8192, untied head) with **2 layers instead of 32 and a vocabulary of 16,640
instead of 128,256** (fewer layers and a shorter head are no smaller layers; the head keeps
more than 16,384 rows so that it still counts as a tall matrix).

One folder of bfloat16 weights serves both runs: the bfloat16 run takes it as it is, the
float32 run widens the same values and multiplies in true 32-bit (every tensor is then
float32 on the device).  The comparison is the reference's per-step one
(scripts/compare_logits.py:189-239; test/forward_test.cc:118-181 for batches against single
sequences), with the bounds of `helpers.py`.
"""
import numpy as np
import pytest
import torch

import cpp_minilamma_b200 as ml
import plain_llama as pl
from cpp_minilamma_b200 import EngineBackend, SamplingParams, StepEntry
from cpp_minilamma_b200.csrc import kernels as K
from cpp_minilamma_b200.engine.generate import generate
from helpers import assert_close

pytestmark = pytest.mark.gpu

LAYERS, VOCAB = 2, 16640      # of 32 layers and 128,256 tokens: see the header
REAL = dict(architectures=["LlamaForCausalLM"], vocab_size=VOCAB, hidden_size=4096, intermediate_size=14336,
            num_hidden_layers=LAYERS, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
            max_position_embeddings=1024, rope_theta=500000.0,
            rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                          "original_max_position_embeddings": 8192},
            rope_interleaved=False, rms_norm_eps=1e-5, tie_word_embeddings=False, torch_dtype="bfloat16",
            eos_token_id=None)
DTYPES = ["float32", "bfloat16"]


class Oracle:
    """The plain implementation on the folder's weights, widened to float64 once."""

    def __init__(self, folder):
        self.cfg, weights = pl.read_model_folder(folder)
        self.weights = {name: w.astype(np.float64) for name, w in weights.items()}
        self._seen = {}

    def logits(self, tokens, dtype):
        key = (tuple(tokens), dtype)
        if key not in self._seen:
            act_round = pl.round_bf16 if dtype == "bfloat16" else (lambda x: x)
            self._seen[key] = pl.forward_sequence(self.cfg, self.weights, list(tokens), act_round=act_round)
        return self._seen[key]


@pytest.fixture(scope="module")
def real(tmp_path_factory):
    folder = str(tmp_path_factory.mktemp("real_widths"))
    ml.write_random_model(ml.config_from_dict(REAL), folder, seed=21, matrix_std=0.02, norm_std=0.1)
    return folder, Oracle(folder)


def tokens_of(length, seed):
    rng = np.random.RandomState(seed)
    return [int(t) for t in rng.randint(0, VOCAB, size=length)]


def load(folder, dtype, **kw):
    kw.setdefault("max_tokens", 64 * 160)
    return ml.load(folder, dtype=dtype, **kw)


def test_the_float32_run_holds_no_reduced_precision_tensor(real):
    folder, _ = real
    llm = load(folder, "float32")
    layer = llm.model.layers[0]
    for weight in (layer.mixer.qkv.weight, layer.mixer.o.weight, layer.feed_forward.gate_up.weight,
                   layer.feed_forward.down.weight, llm.model.embedding.table, llm.model.lm_head.linear.weight):
        assert weight.dtype == torch.float32
    assert not torch.backends.cuda.matmul.allow_tf32


@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_requests(real, dtype):
    folder, oracle = real
    llm = load(folder, dtype)
    K.calls.clear()
    for i, length in enumerate((1, 65, 200, 333)):
        tokens = tokens_of(length, 100 + i)
        slot, = llm.engine.acquire(1)
        got = llm.engine.step([StepEntry(slot, tokens, list(range(length)))]).cpu().numpy()
        llm.engine.release(slot)
        assert_close(got, oracle.logits(tokens, dtype), dtype, f"real widths whole len {length}")
    if dtype == "bfloat16":
        assert K.calls.get("attention_prefill (tcgen05)", 0) >= 3 * LAYERS, K.calls
    llm.engine.cache.check()
    assert K.take_device_error() == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_last_32_one_by_one(real, dtype):
    folder, oracle = real
    llm = load(folder, dtype)
    K.calls.clear()
    for i, length in enumerate((40, 200)):
        tokens = tokens_of(length, 200 + i)
        head = length - 32
        slot, = llm.engine.acquire(1)
        rows = [llm.engine.step([StepEntry(slot, tokens[:head], list(range(head)))]).cpu().numpy()]
        for t in range(head, length):
            rows.append(llm.engine.step([StepEntry(slot, [tokens[t]], [0])]).cpu().numpy())
        llm.engine.release(slot)
        assert_close(np.concatenate(rows), oracle.logits(tokens, dtype), dtype, f"real widths last-32 len {length}")
    if dtype == "bfloat16":
        # one row: every product, the tall gate/up and head too, streams through the direct kernel, and the
        # 200-token context is split over a cluster
        assert K.calls.get("linear_small", 0) >= 64 * (4 * LAYERS + 1), K.calls
        assert K.calls.get("attention_decode (TMA, cluster merge)", 0) >= 32 * LAYERS, K.calls
    assert K.take_device_error() == 0


# Requests of the batched test: 48 of unequal prompt lengths on 40 slots, so that a second batch uses slots
# again.  The numbers of decoded tokens are chosen so that the first batch's decode steps have
# 40, 17, 16, 9, 8 and 1 rows as its requests end one after the other.
PROMPTS = [1, 2, 3, 5, 7, 9, 12, 17, 23, 30, 33, 40, 47, 63, 64, 65, 70, 90, 127, 128, 129, 150, 190, 200,
           4, 6, 8, 10, 11, 13, 14, 15, 16, 18, 19, 20, 21, 22, 24, 25,
           26, 66, 1, 130, 31, 2, 80, 35]
DECODED = [2] * 23 + [4] + [6] * 7 + [8] + [10] * 7 + [12] + [3, 5, 5, 7, 7, 7, 9, 9]


def batched_requests():
    order = np.random.RandomState(7).permutation(40)  # which request ends when does not follow its length
    decoded = [0] * 48
    for place, request in enumerate(order):
        decoded[request] = DECODED[place]
    decoded[40:] = DECODED[40:]
    return [tokens_of(p + d, 300 + i) for i, (p, d) in enumerate(zip(PROMPTS, decoded))], decoded


def replay_in_batches(llm, requests, prompt_lens, batch_size):
    """Prompts in one step, then one token each until a request's tokens are used up; a request that is
    through gives its slot back at once.  Returns per-request logits at every position and the row
    counts of the decode steps."""
    results = [None] * len(requests)
    decode_rows = []
    for begin in range(0, len(requests), batch_size):
        group = list(range(begin, min(begin + batch_size, len(requests))))
        slots = dict(zip(group, llm.engine.acquire(len(group))))
        fed = {r: prompt_lens[r] for r in group}
        pieces = {r: [] for r in group}
        out = llm.engine.step([StepEntry(slots[r], requests[r][:fed[r]], list(range(fed[r]))) for r in group]).cpu().numpy()
        at = 0
        for r in group:
            pieces[r].append(out[at:at + fed[r]])
            at += fed[r]
        live = group
        while True:
            for r in [r for r in live if fed[r] == len(requests[r])]:
                llm.engine.release(slots[r])
            live = [r for r in live if fed[r] < len(requests[r])]
            if not live:
                break
            decode_rows.append(len(live))
            out = llm.engine.step([StepEntry(slots[r], [requests[r][fed[r]]], [0]) for r in live]).cpu().numpy()
            for j, r in enumerate(live):
                pieces[r].append(out[j:j + 1])
                fed[r] += 1
        for r in group:
            results[r] = np.concatenate(pieces[r])
        llm.engine.cache.check()
    return results, decode_rows


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batches_with_decode_steps_of_1_to_40_rows(real, dtype):
    folder, oracle = real
    requests, _ = batched_requests()
    llm = load(folder, dtype, max_seqs=40)
    K.calls.clear()
    got, decode_rows = replay_in_batches(llm, requests, PROMPTS, batch_size=40)
    assert {40, 17, 16, 9, 8, 1} <= set(decode_rows), decode_rows
    for i, tokens in enumerate(requests):
        assert_close(got[i], oracle.logits(tokens, dtype), dtype, f"real widths batched request {i}")
    assert llm.engine.cache.n_free_slots == llm.engine.cache.n_slots
    if dtype == "bfloat16":
        for kind in ("linear_tc5", "linear_small", "attention_prefill (tcgen05)"):
            assert K.calls.get(kind, 0) > 0, (kind, K.calls)
    assert K.take_device_error() == 0


def test_unequal_batches_with_every_product_on_the_tcgen05_kernel(real, monkeypatch):
    """The engine sends decode steps of more than 16 rows to the library product (it is ahead there).  Forced
    onto the tcgen05 kernel, the same steps run its 32- and 64-column variants, the residual epilogue at
    17 and 40 rows and the norms folded in at every row count - inside a model, against the same oracle."""
    folder, oracle = real
    requests, _ = batched_requests()
    monkeypatch.setattr(K, "SMALL_LINEAR", "tc5")
    llm = load(folder, "bfloat16", max_seqs=40)
    K.calls.clear()
    norm_calls = []
    real_norm = K.add_rmsnorm
    monkeypatch.setattr(K, "add_rmsnorm", lambda *a, **kw: (norm_calls.append(a[3].shape[0]), real_norm(*a, **kw))[1])
    got, decode_rows = replay_in_batches(llm, requests[:40], PROMPTS[:40], batch_size=40)
    assert {40, 17, 16, 9, 8, 1} <= set(decode_rows), decode_rows
    for i, tokens in enumerate(requests[:40]):
        assert_close(got[i], oracle.logits(tokens, "bfloat16"), "bfloat16", f"real widths, tcgen05 forced, request {i}")
    # decode steps (every norm call of 40 or fewer rows): only the first layer's input norm and the final norm are kernels
    decode_norms = [rows for rows in norm_calls if rows <= 40]
    assert len(decode_norms) == 2 * len(decode_rows), (len(decode_norms), len(decode_rows))
    assert K.calls.get("linear_tc5", 0) >= len(decode_rows) * (4 * LAYERS + 1)
    assert K.take_device_error() == 0


def test_unequal_batches_with_the_small_steps_on_the_tma_kernel(real, monkeypatch):
    """The engine prefers the direct kernel up to 8 rows; the TMA + mma.sync kernel is what takes a width the direct
    kernel does not.  Forced onto it, the decode steps of up to 64 rows run its one to eight batch tiles with the
    norm folded in and the fused activation - inside a model, against the same oracle."""
    folder, oracle = real
    requests, _ = batched_requests()
    monkeypatch.setattr(K, "SMALL_LINEAR", "tma")
    llm = load(folder, "bfloat16", max_seqs=40)
    K.calls.clear()
    got, decode_rows = replay_in_batches(llm, requests[:40], PROMPTS[:40], batch_size=40)
    assert {40, 17, 16, 9, 8, 1} <= set(decode_rows), decode_rows
    for i, tokens in enumerate(requests[:40]):
        assert_close(got[i], oracle.logits(tokens, "bfloat16"), "bfloat16", f"real widths, TMA kernel forced, request {i}")
    assert K.calls.get("linear_tma", 0) >= len(decode_rows) * 2 * LAYERS, K.calls
    assert K.take_device_error() == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_generation_under_graphs_with_run_ahead(real, dtype):
    """The same requests through the generation loop: decode steps replay captured graphs one step ahead
    of the host while the batch shrinks from 40 rows to 1.  Same tokens as eager step-by-step launches,
    and every token of some requests is the plain implementation's argmax (ties aside)."""
    folder, oracle = real
    requests, decoded = batched_requests()
    prompts = [r[:p] for r, p in zip(requests, PROMPTS)]
    budgets = [d + 1 for d in decoded]  # n tokens cost n - 1 decode steps
    llm = load(folder, dtype, max_seqs=40)
    eager = generate(EngineBackend(llm.engine, SamplingParams(), use_graphs=False), prompts, budgets)
    tokens = None
    for _ in range(2):  # the second round replays every graph that the first one captured
        backend = EngineBackend(llm.engine, SamplingParams())
        K.calls.clear()
        tokens = [c.tokens for c in generate(backend, prompts, budgets)]
        assert tokens == [c.tokens for c in eager]
    assert backend.graphs.replays > 0
    for r in (0, 13, 23, 39, 43):
        ref = oracle.logits(list(prompts[r]) + tokens[r], dtype)  # causal: row t depends on tokens 0..t only
        for i, token in enumerate(tokens[r]):
            row = ref[len(prompts[r]) - 1 + i]
            best = int(np.argmax(row))
            if token != best:
                assert row[best] - row[token] <= (2e-4 if dtype == "float32" else 0.04 * np.abs(row).max()), \
                    f"request {r}: token {i} is {token}, plain argmax {best}"
    llm.engine.cache.check()
    assert K.take_device_error() == 0


def test_decode_splits_keep_every_cluster_resident(real):
    """Up to 16 context splits the decode attention's blocks of one (sequence, kv head) form a cluster, and a
    launch with more clusters than the device holds at once runs in two waves (measured: 14 us against 9 at
    3 to 6 sequences).  The split count chosen for every batch size keeps the clusters in one wave, never
    exceeds the pages of the longest context and falls back to one block per (sequence, kv head) only when
    two splits no longer fit."""
    folder, _ = real
    llm = load(folder, "bfloat16")
    attention = llm.model.layers[0].mixer
    capacity = K.attention_decode_cluster_capacity(torch.bfloat16, 128, True)
    assert capacity is not None and capacity[2] >= capacity[8] >= capacity[16] >= 1
    kv_heads = REAL["num_key_value_heads"]
    for context in (64, 200, 1024, 131072):
        pages = -(-context // 64)
        for batch in range(1, 41):
            splits = attention.decode_splits(batch, context)
            assert 1 <= splits <= pages
            if 2 <= splits <= 16:
                assert batch * kv_heads <= capacity[splits], (batch, context, splits)
            if splits == 1 and pages >= 2:
                assert batch * kv_heads > capacity[2], (batch, context)
            if context >= 1024 and splits < 16 and batch * kv_heads <= capacity[16]:
                raise AssertionError(f"batch {batch}, context {context}: {splits} splits although 16 fit")
