"""The engine against the plain implementation, under every way of cutting the work:
each request alone and whole; with the last 32 tokens one by one; in batches of unequal
lengths whose shorter requests end earlier, one batch after another so that slots are
used again; long decoding; the first tokens of a sequence.  In float32 and bfloat16."""
import os

import numpy as np
import pytest
import torch

import cpp_minilamma_b200 as ml
import tiny_configs as tc
from cpp_minilamma_b200 import StepEntry
from helpers import assert_close, plain_logits

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
CASES = [(name, dtype) for name in "ABCD" for dtype in DTYPES]


def load(model_folders, name, dtype, storage=None, **kw):
    storage = storage or dtype  # by default a bfloat16 run reads a bfloat16 folder, a float32 run a float32 one
    folder = model_folders(name, storage)
    kw.setdefault("max_tokens", 4096)
    return folder, ml.load(folder, dtype=dtype, **kw)


def request_lengths(name):
    top = tc.TINY[name]["max_position_embeddings"]
    return [n for n in (1, 2, 5, 33, 64, 65, 100, 200) if n <= top]


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_requests(model_folders, name, dtype):
    folder, llm = load(model_folders, name, dtype)
    for i, length in enumerate(request_lengths(name)):
        tokens = tc.random_tokens(name, length, 100 + i)
        slot, = llm.engine.acquire(1)
        got = llm.engine.step([StepEntry(slot, tokens, list(range(length)))]).cpu().numpy()
        llm.engine.release(slot)
        assert_close(got, plain_logits(folder, tokens, dtype), dtype, f"{name} whole len {length}")
    llm.engine.cache.check()


@pytest.mark.parametrize("name,dtype", CASES)
def test_last_32_one_by_one(model_folders, name, dtype):
    folder, llm = load(model_folders, name, dtype)
    for i, length in enumerate(request_lengths(name)):
        tokens = tc.random_tokens(name, length, 200 + i)
        ref = plain_logits(folder, tokens, dtype)
        head = max(length - 32, 0)
        slot, = llm.engine.acquire(1)
        rows = []
        if head:
            rows.append(llm.engine.step([StepEntry(slot, tokens[:head], list(range(head)))]).cpu().numpy())
        for t in range(head, length):
            rows.append(llm.engine.step([StepEntry(slot, [tokens[t]], [0])]).cpu().numpy())
        llm.engine.release(slot)
        assert_close(np.concatenate(rows), ref, dtype, f"{name} last-32 len {length}")


def _batched_replay(llm, requests, prompt_lens, batch_size):
    """Run requests in consecutive batches: prompts in one step, then one token each until
    each request's tokens are used up.  Returns per-request logits at every position."""
    results = [None] * len(requests)
    for begin in range(0, len(requests), batch_size):
        group = list(range(begin, min(begin + batch_size, len(requests))))
        slots = dict(zip(group, llm.engine.acquire(len(group))))
        fed = {r: prompt_lens[r] for r in group}
        pieces = {r: [] for r in group}
        out = llm.engine.step([StepEntry(slots[r], requests[r][:fed[r]], list(range(fed[r]))) for r in group])
        at = 0
        for r in group:
            pieces[r].append(out[at:at + fed[r]].cpu().numpy())
            at += fed[r]
        live = [r for r in group if fed[r] < len(requests[r])]
        for r in group:
            if r not in live:
                llm.engine.release(slots[r])
        while live:
            out = llm.engine.step([StepEntry(slots[r], [requests[r][fed[r]]], [0]) for r in live])
            for j, r in enumerate(live):
                pieces[r].append(out[j:j + 1].cpu().numpy())
                fed[r] += 1
            for r in [r for r in live if fed[r] == len(requests[r])]:
                llm.engine.release(slots[r])
            live = [r for r in live if fed[r] < len(requests[r])]
        for r in group:
            results[r] = np.concatenate(pieces[r])
        llm.engine.cache.check()
    return results


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_batches_reuse_slots(model_folders, name, dtype):
    # the BASELINE workloads (A: prompts 5/9/2 + 8 steps; B: 17/1/40/6 + 12 steps) and more,
    # on a cache with fewer slots than requests
    workloads = {"A": ([5, 9, 2, 1, 30, 7, 3], 8), "B": ([17, 1, 40, 6, 64, 65, 2, 100], 12),
                 "C": ([3, 130, 64, 1, 257, 20], 20), "D": ([70, 1, 128, 5, 200, 64, 129], 40)}
    prompt_lens, steps = workloads[name]
    extra = [steps + 3 * (i % 3) for i in range(len(prompt_lens))]  # unequal ends
    top = tc.TINY[name]["max_position_embeddings"]
    requests = [tc.random_tokens(name, min(p + e, top), 300 + i) for i, (p, e) in enumerate(zip(prompt_lens, extra))]
    prompt_lens = [min(p, len(r)) for p, r in zip(prompt_lens, requests)]
    folder, llm = load(model_folders, name, dtype, max_seqs=4)
    got = _batched_replay(llm, requests, prompt_lens, batch_size=4 if name != "A" else 3)
    for i, tokens in enumerate(requests):
        assert_close(got[i], plain_logits(folder, tokens, dtype), dtype, f"{name} batched request {i}")
    assert llm.engine.cache.n_free_slots == llm.engine.cache.n_slots


@pytest.mark.parametrize("name", ["C", "D"])
@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(model_folders, name, dtype):
    # 3 prompt tokens, then single-token steps up to 600: crosses many pages
    tokens = tc.random_tokens(name, min(603, tc.TINY[name]["max_position_embeddings"]), 400)
    folder, llm = load(model_folders, name, dtype)
    slot, = llm.engine.acquire(1)
    rows = [llm.engine.step([StepEntry(slot, tokens[:3], [0, 1, 2])]).cpu().numpy()]
    for t in range(3, len(tokens)):
        rows.append(llm.engine.step([StepEntry(slot, [tokens[t]], [0])]).cpu().numpy())
    llm.engine.release(slot)
    assert_close(np.concatenate(rows), plain_logits(folder, tokens, dtype), dtype, "long decoding")


@pytest.mark.parametrize("name,dtype", CASES)
def test_first_tokens(model_folders, name, dtype):
    # a sequence's first positions, fed one by one from an empty slot
    tokens = tc.random_tokens(name, 6, 500)
    folder, llm = load(model_folders, name, dtype)
    slot, = llm.engine.acquire(1)
    rows = [llm.engine.step([StepEntry(slot, [t], [0])]).cpu().numpy() for t in tokens]
    llm.engine.release(slot)
    assert_close(np.concatenate(rows), plain_logits(folder, tokens, dtype), dtype, f"{name} first tokens")


@pytest.mark.parametrize("dtype", DTYPES)
def test_chunked_step_equals_whole(model_folders, dtype):
    # a step longer than max_step_tokens is cut into chunks inside the engine
    name = "C"
    tokens = tc.random_tokens(name, 300, 600)
    folder, llm = load(model_folders, name, dtype, max_step_tokens=128)
    slots = llm.engine.acquire(2)
    other = tc.random_tokens(name, 70, 601)
    out = llm.engine.step([StepEntry(slots[0], tokens, list(range(300))),
                           StepEntry(slots[1], other, [69, 0])]).cpu().numpy()
    assert_close(out[:300], plain_logits(folder, tokens, dtype), dtype, "chunked long")
    ref_other = plain_logits(folder, other, dtype)
    assert_close(out[300:], ref_other[[69, 0]], dtype, "chunked short, want out of order")


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("D", "bfloat16"), ("D", "float32"), ("C", "bfloat16")])
@pytest.mark.parametrize("length", [65, 66, 129])
def test_chunk_edges_portions_of_one_and_two_tokens(model_folders, name, dtype, length):
    # with chunks of 64 tokens a prompt of 65, 66 or 129 leaves a last portion of 1 or 2 tokens whose first
    # position is the first row of a new page: alone it is a step of single tokens (the decode kernels, in D
    # bfloat16 with rope and cache write fused into the attention), next to a longer neighbour a one-row tile
    top = tc.TINY[name]["max_position_embeddings"]
    if length > top:
        pytest.skip("longer than the model's positions")
    tokens = tc.random_tokens(name, length, 610 + length)
    ref = plain_logits(folder := model_folders(name, dtype), tokens, dtype)
    llm = ml.load(folder, dtype=dtype, max_tokens=4096, max_step_tokens=64)
    slot, = llm.engine.acquire(1)
    alone = llm.engine.step([StepEntry(slot, tokens, list(range(length)))]).cpu().numpy()
    llm.engine.release(slot)
    assert_close(alone, ref, dtype, f"{name} chunks of 64, {length} tokens alone")
    other = tc.random_tokens(name, min(100, top), 611)
    a, b = llm.engine.acquire(2)
    out = llm.engine.step([StepEntry(a, other, [len(other) - 1]), StepEntry(b, tokens, list(range(length)))]).cpu().numpy()
    assert_close(out[1:], ref, dtype, f"{name} chunks of 64, {length} tokens behind a neighbour")
    assert_close(out[:1], plain_logits(folder, other, dtype)[-1:], dtype, "the neighbour")
    llm.engine.cache.check()


@pytest.mark.parametrize("name,dtype", CASES)
def test_greedy_generation_through_entry_point(model_folders, name, dtype):
    folder, llm = load(model_folders, name, dtype)
    prompts = [tc.random_tokens(name, n, 700 + n) for n in (5, 9, 2)]
    outs = llm.generate(prompts, max_new_tokens=8, ignore_eos=True)
    for prompt, out in zip(prompts, outs):
        assert len(out) == 8
        seq = list(prompt)
        for token in out:  # each generated token is the argmax of the plain logits, ties aside
            ref = plain_logits(folder, seq, dtype)[-1]
            best = int(np.argmax(ref))
            if token != best:
                margin = ref[best] - ref[token]
                assert margin <= (2e-4 if dtype == "float32" else 0.04 * np.abs(ref).max()), \
                    f"{name} {dtype}: generated {token}, plain argmax {best}, margin {margin}"
            seq.append(token)


@pytest.mark.parametrize("dtype,storage", [("bfloat16", "float32"), ("float32", "bfloat16")])
def test_run_dtype_differs_from_storage(model_folders, dtype, storage):
    # tensors stored in 32-bit stay 32-bit in a bfloat16 run (their products run in float32);
    # a float32 run widens bfloat16 tensors
    name = "A"
    folder, llm = load(model_folders, name, dtype, storage=storage)
    want = torch.float32 if (storage == "float32" or dtype == "float32") else torch.bfloat16
    assert llm.model.layers[0].mixer.qkv.weight.dtype == want
    assert llm.model.embedding.table.dtype == want
    tokens = tc.random_tokens(name, 40, 800)
    slot, = llm.engine.acquire(1)
    got = [llm.engine.step([StepEntry(slot, tokens[:30], list(range(30)))]).cpu().numpy()]
    for t in range(30, 40):
        got.append(llm.engine.step([StepEntry(slot, [tokens[t]], [0])]).cpu().numpy())
    assert_close(np.concatenate(got), plain_logits(folder, tokens, dtype), dtype, f"run {dtype} on {storage}")


def test_bfloat16_run_with_some_matrices_stored_in_32_bit(model_folders, tmp_path):
    # a matrix stored in 32-bit stays 32-bit in a bfloat16 run.  When only some are (here layer 1's q_proj and
    # gate_proj), a decode step's bfloat16 o/down product folds the following norm away and the float32
    # product behind it has to finish that norm itself
    import shutil
    import plain_llama as pl
    from cpp_minilamma_b200.weights.safetensors_io import write_safetensors
    name = "B"
    folder = str(tmp_path / "mixed")
    shutil.copytree(model_folders(name, "bfloat16"), folder)
    _, weights = pl.read_model_folder(folder)
    wide = {"model.layers.1.self_attn.q_proj.weight", "model.layers.1.mlp.gate_proj.weight"}
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      {n: torch.tensor(w).to(torch.float32 if n in wide else torch.bfloat16) for n, w in weights.items()},
                      {"format": "pt"})
    llm = ml.load(folder, dtype="bfloat16", max_tokens=4096)
    assert llm.model.layers[1].mixer.qkv.weight.dtype == torch.float32
    assert llm.model.layers[1].feed_forward.gate_up.weight.dtype == torch.float32
    assert llm.model.layers[0].mixer.qkv.weight.dtype == torch.bfloat16
    lengths = [40, 70, 9]
    requests = [tc.random_tokens(name, n, 850 + i) for i, n in enumerate(lengths)]
    slots = llm.engine.acquire(len(requests))
    heads = [n - 8 for n in lengths]
    first = llm.engine.step([StepEntry(s, t[:h], list(range(h))) for s, t, h in zip(slots, requests, heads)]).cpu().numpy()
    rows = [[] for _ in requests]
    for k in range(8):
        got = llm.engine.step([StepEntry(s, [t[h + k]], [0]) for s, t, h in zip(slots, requests, heads)]).cpu().numpy()
        for i in range(len(requests)):
            rows[i].append(got[i])
    at = 0
    for i, (tokens, h) in enumerate(zip(requests, heads)):
        ref = plain_logits(folder, tokens, "bfloat16")
        assert_close(np.concatenate([first[at:at + h], np.stack(rows[i])]), ref, "bfloat16", f"mixed storage request {i}")
        at += h


@pytest.mark.parametrize("dtype", DTYPES)
def test_folder_stored_in_float16(model_folders, dtype):
    # a float16 folder (Llama-2's storage) loads in either run: widened exactly for float32, rounded once to
    # bfloat16 for bfloat16.  The plain implementation gets the same weights, rounded the same way.
    import plain_llama as pl
    name = "B"
    folder = model_folders(name, "float16")
    cfg, weights = pl.read_model_folder(folder)
    assert cfg["torch_dtype"] == "float16"
    llm = ml.load(folder, dtype=dtype, max_tokens=2048)
    assert llm.model.layers[0].mixer.qkv.weight.dtype == (torch.float32 if dtype == "float32" else torch.bfloat16)
    if dtype == "bfloat16":  # matrices are rounded; vectors (norm weights) are kept as float32
        weights = {n: (pl.round_bf16(w).astype(np.float32) if w.ndim == 2 else w) for n, w in weights.items()}
    tokens = tc.random_tokens(name, 50, 860)
    slot, = llm.engine.acquire(1)
    got = [llm.engine.step([StepEntry(slot, tokens[:40], list(range(40)))]).cpu().numpy()]
    for t in range(40, 50):
        got.append(llm.engine.step([StepEntry(slot, [tokens[t]], [0])]).cpu().numpy())
    act_round = pl.round_bf16 if dtype == "bfloat16" else (lambda x: x)
    assert_close(np.concatenate(got), pl.forward_sequence(cfg, weights, tokens, act_round=act_round), dtype, f"float16 folder, {dtype} run")


def test_cli_generate_matches_the_api(model_folders, capsys):
    from cpp_minilamma_b200.cli import main
    folder, llm = load(model_folders, "B", "float32")
    prompts = [[5, 17, 3], [9, 9], [200]]
    expect = llm.generate(prompts, max_new_tokens=5, ignore_eos=True)
    argv = ["generate", folder, "--dtype", "float32", "-n", "5", "--ignore-eos"]
    for p in prompts:
        argv += ["-p", " ".join(map(str, p))]
    assert main(argv) == 0
    lines = capsys.readouterr().out.splitlines()
    assert [[int(t) for t in line.split()] for line in lines[:3]] == expect
    assert lines[-1].startswith("trace summary: trace_id=") and lines[-1].endswith("status=ok")
    # sampling with a seed is reproducible and differs between seeds
    a = llm.generate(prompts, max_new_tokens=12, temperature=1.0, top_k=50, seed=7, ignore_eos=True)
    b = llm.generate(prompts, max_new_tokens=12, temperature=1.0, top_k=50, seed=7, ignore_eos=True)
    c = llm.generate(prompts, max_new_tokens=12, temperature=1.0, top_k=50, seed=8, ignore_eos=True)
    assert a == b and a != c
    # a request's samples do not depend on its neighbours in the batch
    alone = llm.generate(prompts[:1], max_new_tokens=12, temperature=1.0, top_k=50, seed=7, ignore_eos=True)
    assert alone[0] == a[0]
    # stop tokens end a sequence and are not emitted
    stops = llm.generate(prompts, max_new_tokens=5, stop_ids=[expect[0][2]])
    assert stops[0] == expect[0][:2]
    assert main(["generate", folder, "-p", "1 2 3", "-n", "400", "--dtype", "float32"]) == 2   # over the context


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16"), ("C", "bfloat16"), ("D", "bfloat16")])
def test_graph_replay_equals_eager_steps(model_folders, name, dtype):
    # the same generation with captured decode graphs and with eager launches; budgets differ so
    # the batch shrinks and other graph sizes come into play; a second round reuses the graphs
    from cpp_minilamma_b200 import EngineBackend, SamplingParams
    from cpp_minilamma_b200.engine.generate import generate
    folder, llm = load(model_folders, name, dtype)
    prompts = [tc.random_tokens(name, n, 950 + n) for n in (5, 30, 2, 9)]
    budgets = [20, 7, 12, 20]
    for params in (SamplingParams(), SamplingParams(temperature=0.9, top_k=20, seed=3)):
        eager = generate(EngineBackend(llm.engine, params, use_graphs=False), prompts, budgets)
        for _ in range(2):
            backend = EngineBackend(llm.engine, params, use_graphs=True)
            replayed = generate(backend, prompts, budgets)
            assert [c.tokens for c in replayed] == [c.tokens for c in eager]
        assert backend.graphs.replays > 0
    llm.engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_context_chunked_prefill_then_decode(tmp_path, dtype):
    """5,000 prompt tokens (80 pages) in chunks of 2,048 that continue from the cache, then
    single-token steps whose attention is split 16 ways over the context; head size 128.  Random
    weights spread attention evenly, which would hide a wrong page or a lost split, so one early
    position gets a key that every later query prefers (one token id that stands at position 70 only)."""
    import plain_llama as pl
    raw = dict(vocab_size=160, hidden_size=128, intermediate_size=200, num_hidden_layers=2, num_attention_heads=2,
               num_key_value_heads=1, head_dim=128, max_position_embeddings=8192, rope_theta=1.0e6,
               rope_interleaved=False, rms_norm_eps=1e-5, tie_word_embeddings=False, architectures=["LlamaForCausalLM"],
               torch_dtype=dtype)
    cfg = ml.config_from_dict(raw)
    folder = str(tmp_path / "long")
    ml.write_random_model(cfg, folder, seed=11, matrix_std=0.05, norm_std=0.1)
    rng = np.random.RandomState(5)
    marked = 159
    tokens = [int(t) for t in rng.randint(0, marked, size=5040)]   # the marked id appears once
    tokens[70] = marked
    # Plant the key (the file is rewritten; the engine and the plain implementation read it afterwards).
    # RMSNorm removes an embedding's length, so the mark is a direction: every token gets a
    # common component on hidden dim 0, the marked token one on dim 1; layer 0's query rows for
    # head dim 63 read dim 0, its key row for dim 63 reads dim 1.  Dim 63 pairs with 127 at the
    # lowest rotary frequency (1e6 ** (-63/64) per position): the product survives 5,000 positions.
    from cpp_minilamma_b200.weights.safetensors_io import write_safetensors
    _, weights = pl.read_model_folder(folder)
    storage = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    tensors = {name: torch.tensor(np.asarray(w, dtype=np.float32)) for name, w in weights.items()}
    tensors["model.embed_tokens.weight"][:, 0] += 3.0
    tensors["model.embed_tokens.weight"][marked, 1] += 8.0
    for head in range(2):
        tensors["model.layers.0.self_attn.q_proj.weight"][head * 128 + 63, 0] += 4.0
    tensors["model.layers.0.self_attn.k_proj.weight"][63, 1] += 4.0
    write_safetensors(os.path.join(folder, "model.safetensors"), {n: t.to(storage) for n, t in tensors.items()},
                      {"format": "pt"})
    ref = plain_logits(folder, tokens, dtype)
    llm = ml.load(folder, dtype=dtype, max_tokens=64 * 90, max_seqs=2, max_step_tokens=2048)
    slot, = llm.engine.acquire(1)
    want = [0, 69, 70, 71, 2047, 2048, 4095, 4096, 4999]
    rows = [llm.engine.step([StepEntry(slot, tokens[:5000], want)]).cpu().numpy()]
    for t in range(5000, 5040):
        rows.append(llm.engine.step([StepEntry(slot, [tokens[t]], [0])]).cpu().numpy())
    llm.engine.release(slot)
    assert_close(np.concatenate(rows), ref[want + list(range(5000, 5040))], dtype, "long context")
    # the planted key does carry weight: without position 70 the last logits differ visibly
    cut = plain_logits(folder, tokens[:70] + tokens[71:], dtype)
    assert np.abs(cut[-1] - ref[-1]).max() > 0.02 * np.abs(ref[-1]).max()


@pytest.mark.parametrize("name,dtype,sampling", [("A", "float32", {}), ("D", "bfloat16", {}),
                                                   ("B", "bfloat16", dict(temperature=0.9, top_k=20, seed=5))])
def test_generation_one_step_ahead_equals_step_by_step(model_folders, name, dtype, sampling):
    """The generation loop keeps the device one step ahead of the host (the next step takes its input
    tokens on the device).  The same requests through a backend without that ability give the same
    tokens, with stop tokens that end sequences in the middle of a batch."""
    from cpp_minilamma_b200 import EngineBackend, SamplingParams
    from cpp_minilamma_b200.engine.generate import generate

    class StepByStep:
        """The engine backend without `submit`: the loop falls back to one synchronous call a step."""
        def __init__(self, inner):
            self.inner = inner
            self.n_slots, self.n_pages, self.max_positions = inner.n_slots, inner.n_pages, inner.max_positions
        def acquire(self, count): return self.inner.acquire(count)
        def release(self, slot): self.inner.release(slot)
        def step_and_sample(self, entries, requests, steps): return self.inner.step_and_sample(entries, requests, steps)

    folder, llm = load(model_folders, name, dtype, max_seqs=4)
    prompts = [tc.random_tokens(name, n, 800 + n) for n in (5, 9, 2, 17, 3, 30)]
    params = SamplingParams(sampling.get("temperature", 0.0), sampling.get("top_k", 0), sampling.get("seed", 1))
    free_run = generate(StepByStep(EngineBackend(llm.engine, params)), prompts, 24, set())
    # stop tokens taken from the free run, so that sequences really end early at different steps
    stops = {free_run[0].tokens[3], free_run[3].tokens[10]}
    plain = generate(StepByStep(EngineBackend(llm.engine, params)), prompts, [24, 24, 1, 24, 2, 24], stops)
    ahead_backend = EngineBackend(llm.engine, params)
    ahead = generate(ahead_backend, prompts, [24, 24, 1, 24, 2, 24], stops)
    assert [(c.tokens, c.finish_reason) for c in ahead] == [(c.tokens, c.finish_reason) for c in plain]
    assert any(c.finish_reason == "stop" for c in ahead) and any(c.finish_reason == "length" for c in ahead)
    assert llm.engine.cache.n_free_slots == llm.engine.cache.n_slots
    llm.engine.cache.check()


@pytest.mark.parametrize("name,dtype", [("D", "bfloat16"), ("C", "float32")])
def test_long_generation_crosses_pages_under_graphs_and_run_ahead(model_folders, name, dtype):
    """80 new tokens from prompts of 60 and 3 tokens: the sequences cross page boundaries (64, 128)
    while decode steps replay a captured graph one step ahead of the host.  Same tokens as the
    step-by-step loop, and each token is the plain implementation's argmax (ties aside)."""
    from cpp_minilamma_b200 import EngineBackend, SamplingParams
    from cpp_minilamma_b200.engine.generate import generate

    class StepByStep:
        def __init__(self, inner):
            self.inner = inner
            self.n_slots, self.n_pages, self.max_positions = inner.n_slots, inner.n_pages, inner.max_positions
        def acquire(self, count): return self.inner.acquire(count)
        def release(self, slot): self.inner.release(slot)
        def step_and_sample(self, entries, requests, steps): return self.inner.step_and_sample(entries, requests, steps)

    folder, llm = load(model_folders, name, dtype, max_seqs=2)
    prompts = [tc.random_tokens(name, 60, 901), tc.random_tokens(name, 3, 902)]
    ahead = generate(EngineBackend(llm.engine, SamplingParams()), prompts, 80, set())
    plain = generate(StepByStep(EngineBackend(llm.engine, SamplingParams(), use_graphs=False)), prompts, 80, set())
    assert [c.tokens for c in ahead] == [c.tokens for c in plain]
    for prompt, completion in zip(prompts, ahead):
        ref = plain_logits(folder, list(prompt) + completion.tokens, dtype)
        for i, token in enumerate(completion.tokens):
            row = ref[len(prompt) - 1 + i]
            best = int(np.argmax(row))
            if token != best:
                assert row[best] - row[token] <= (2e-4 if dtype == "float32" else 0.04 * np.abs(row).max()), \
                    f"{name} {dtype}: token {i} is {token}, plain argmax {best}"
    llm.engine.cache.check()


@pytest.mark.parametrize("name,dtype", [("D", "bfloat16"), ("B", "bfloat16"), ("C", "float32")])
def test_graphs_of_a_small_batch_survive_a_larger_batch_in_between(model_folders, name, dtype):
    """A batch of 2, then a batch of 5, then the batch of 2 again on one engine whose prompt steps are cut
    into portions of 64 tokens.  No portion of the larger batch's prompts holds more sequences than the
    smaller batch had, so the first buffers to grow are those of the larger batch's first decode step, and
    the smaller batch's captured step was recorded with them; it must not be replayed with the old
    addresses.  Same tokens as an engine without graphs, and no captured step is older than the workspace."""
    from cpp_minilamma_b200 import EngineBackend, SamplingParams
    from cpp_minilamma_b200.engine.generate import generate
    folder, llm = load(model_folders, name, dtype, max_seqs=5, max_step_tokens=64)
    _, plain_llm = load(model_folders, name, dtype, max_seqs=5, max_step_tokens=64)
    two = [tc.random_tokens(name, n, 950 + n) for n in (70, 67)]
    five = [tc.random_tokens(name, n, 960 + n) for n in (66, 70, 65, 72, 68)]
    graphs = llm.engine.shared_decode_graphs()
    generations = []
    for round_, prompts in enumerate((two, five, two, five, two)):
        got = generate(EngineBackend(llm.engine, SamplingParams()), prompts, 12, set())
        ref = generate(EngineBackend(plain_llm.engine, SamplingParams(), use_graphs=False), prompts, 12, set())
        assert [c.tokens for c in got] == [c.tokens for c in ref], f"{name} {dtype}: batch {round_} of {len(prompts)}"
        for cap in graphs._captured.values():
            assert cap.graph is None or cap.generation == llm.engine.ws.generation
        generations.append(llm.engine.ws.generation)
    assert generations[1] > generations[0], "the larger batch grew no buffer: the test does not reach its case"
    assert graphs.replays > 0
    llm.engine.cache.check()


@pytest.mark.parametrize("name,dtype,sampling", [("D", "bfloat16", {}), ("B", "bfloat16", {}),
                                                   ("C", "float32", dict(temperature=0.8, top_k=30, seed=4))])
def test_batches_above_16_run_at_rounded_up_sizes_with_padding_rows(model_folders, name, dtype, sampling):
    """40 requests that end two steps apart: the decode steps of 17 to 40 live sequences replay the graphs of
    batch 24, 32 and 40, their spare rows filled with the cache's padding slot.  A product of 25 rows and one of
    32 need not round alike in bfloat16, so the greedy bfloat16 runs are held to the plain implementation
    (every token its argmax, near-ties aside); the float32 run, sampled, gives the tokens of an engine without
    graphs, which runs every step at its own size.  No slot or page is lost."""
    from cpp_minilamma_b200 import EngineBackend, SamplingParams
    from cpp_minilamma_b200.engine.generate import generate
    folder, llm = load(model_folders, name, dtype, max_seqs=40, max_tokens=40 * 192)
    prompts = [tc.random_tokens(name, 1 + (7 * i) % 50, 1200 + i) for i in range(40)]
    budgets = [3 + 2 * i for i in range(40)]
    params = SamplingParams(sampling.get("temperature", 0.0), sampling.get("top_k", 0), sampling.get("seed", 1))
    if sampling:
        _, plain_llm = load(model_folders, name, dtype, max_seqs=40, max_tokens=40 * 192)
        ref = generate(EngineBackend(plain_llm.engine, params, use_graphs=False), prompts, budgets, set())
    for _ in range(2):  # the second time no buffer grows any more, so every captured step is still there at the end
        got = generate(EngineBackend(llm.engine, params), prompts, budgets, set())
        if sampling:
            assert [c.tokens for c in got] == [c.tokens for c in ref]
    if not sampling:
        for prompt, completion, budget in zip(prompts, got, budgets):
            assert len(completion.tokens) == budget
            rows = plain_logits(folder, list(prompt) + completion.tokens, dtype)
            for i, token in enumerate(completion.tokens):
                row = rows[len(prompt) - 1 + i]
                best = int(np.argmax(row))
                assert token == best or row[best] - row[token] <= 0.04 * np.abs(row).max(), \
                    f"{name}: token {i} of a request with {len(prompt)} prompt tokens is {token}, plain argmax {best}"
    sizes = sorted({key[0] for key, cap in llm.engine.shared_decode_graphs()._captured.items() if cap.graph is not None})
    assert [b for b in sizes if b > 16] == [24, 32, 40], sizes
    assert llm.engine.cache.n_free_slots == llm.engine.cache.n_slots
    llm.engine.cache.check()


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("room,prompts,extra", [
    ((0, 0, 4, 2, 2, 1, 1, 1, 1), [300, 5, 70, 2, 129], [70, 40, 70, 12, 55]),  # no split of every sequence fits
    ((0, 0, 10, 5, 2, 1, 1, 1, 1), [5, 430, 70], [40, 70, 70]),                 # two splits each fit, one is far longer
])
def test_decode_batch_with_one_long_sequence_cut_by_the_work_list(model_folders, monkeypatch, graphs, room, prompts, extra):
    """A batch too large for a split of every sequence, or one whose longest sequence is far longer than the
    rest, runs its decode attention from a list of (sequence, split) pairs in which only the long sequences
    are cut.  The device is made to look small (room for a few clusters of two) and the shortest piece one
    page, so that the tiny model reaches that path: one request of 300 or 430 tokens beside short ones, decoded for
    70 steps (the long one crosses a page, the short ones end earlier, so that the batch shrinks and the kind of
    step changes), eagerly and under graph replay, against the plain implementation."""
    from cpp_minilamma_b200.csrc import kernels as K
    from cpp_minilamma_b200.parts.attention import Attention
    real = K.attention_decode_cluster_capacity
    monkeypatch.setattr(K, "attention_decode_cluster_capacity",
                        lambda *a: None if real(*a) is None else tuple(room) + (0,) * 8)
    monkeypatch.setattr(Attention, "work_list_min_pages", 1)
    name, dtype = "D", "bfloat16"
    folder, llm = load(model_folders, name, dtype, max_seqs=5)
    requests = [tc.random_tokens(name, p + e, 970 + i) for i, (p, e) in enumerate(zip(prompts, extra))]
    K.calls.clear()
    if graphs:
        from cpp_minilamma_b200 import EngineBackend, SamplingParams
        from cpp_minilamma_b200.engine.generate import generate
        got = generate(EngineBackend(llm.engine, SamplingParams()), [r[:p] for r, p in zip(requests, prompts)], extra, set())
        for prompt_len, request, completion in zip(prompts, requests, got):
            ref = plain_logits(folder, request[:prompt_len] + completion.tokens, dtype)
            for i, token in enumerate(completion.tokens):
                row = ref[prompt_len - 1 + i]
                best = int(np.argmax(row))
                assert token == best or row[best] - row[token] <= 0.04 * np.abs(row).max(), f"token {i}: {token} vs {best}"
    else:
        got = _batched_replay(llm, requests, prompts, batch_size=5)
        for i, tokens in enumerate(requests):
            assert_close(got[i], plain_logits(folder, tokens, dtype), dtype, f"request {i}")
    assert K.calls.get("attention_decode (TMA, work list)", 0) > 0, K.calls
    if len(prompts) == 3:  # once the long request is alone or the lengths are alike, the clusters are back
        assert K.calls.get("attention_decode (TMA, cluster merge)", 0) > 0 or not graphs, K.calls
    assert K.take_device_error() == 0
    llm.engine.cache.check()


@pytest.mark.parametrize("name", ["B", "D"])
def test_decode_with_norms_folded_into_products_and_apart(model_folders, name, monkeypatch):
    # decode steps of few rows fold every norm but the first and the last into the products around it;
    # with that switched off each norm is a kernel of its own.  Both against the plain implementation.
    from cpp_minilamma_b200.csrc import kernels as K
    folder, llm = load(model_folders, name, "bfloat16")
    layers = tc.TINY[name]["num_hidden_layers"]
    lengths = [40, 70, 9]
    requests = [tc.random_tokens(name, n, 900 + i) for i, n in enumerate(lengths)]
    refs = [plain_logits(folder, tokens, "bfloat16") for tokens in requests]
    norm_calls = []
    real = K.add_rmsnorm
    monkeypatch.setattr(K, "add_rmsnorm", lambda *a, **kw: (norm_calls.append(1), real(*a, **kw))[1])
    for folded in (True, False):
        monkeypatch.setattr(K, "FUSE_NORM", folded)
        slots = llm.engine.acquire(len(requests))
        heads = [n - 8 for n in lengths]
        llm.engine.step([StepEntry(s, t[:h], []) for s, t, h in zip(slots, requests, heads)])
        rows = [[] for _ in requests]
        for k in range(8):
            del norm_calls[:]
            got = llm.engine.step([StepEntry(s, [t[h + k]], [0]) for s, t, h in zip(slots, requests, heads)]).cpu().numpy()
            # B: every width is a multiple of 32; D: the direct kernel does not take the down product (K = 328),
            # so that each layer's input norm stays a kernel
            expected = {"B": 2, "D": 2 + layers - 1}[name] if folded else 2 * layers + 1
            assert len(norm_calls) == expected, (folded, len(norm_calls))
            for i in range(len(requests)):
                rows[i].append(got[i])
        for s in slots:
            llm.engine.release(s)
        for i, (n, h) in enumerate(zip(lengths, heads)):
            assert_close(np.stack(rows[i]), refs[i][h:], "bfloat16", f"{name} folded={folded} request {i}")
