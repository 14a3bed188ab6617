"""Configurations drawn at random (fixed seeds) through the engine against the plain implementation:
head sizes in steps of 16 up to 256, any number of heads and groups, widths, intermediate sizes and
vocabularies that are no multiple of anything, one to three layers, both pairings, scaled and unscaled
rotation, tied and untied heads, biases.  Every case runs one batch of unequal prompts in one step, then
one token each with the shorter requests ending earlier, in float32 and in bfloat16, and its first
request once more alone and whole.  A head size outside the steps of 16 is refused with a clear error
before anything is built."""
import numpy as np
import pytest

import cpp_minilamma_b200 as ml
from cpp_minilamma_b200 import StepEntry
from helpers import assert_close, plain_logits

HEAD_SIZES = [16, 32, 48, 64, 80, 96, 112, 128, 144, 160, 176, 192, 208, 224, 240, 256]
SEEDS = list(range(16))


def draw(seed):
    """A configuration, prompt lengths and requests from one seed; head size HEAD_SIZES[seed % 16], so that
    the seeds 0..15 cover every head size once."""
    rng = np.random.RandomState(1000 + seed)
    head_dim = HEAD_SIZES[seed % len(HEAD_SIZES)]
    groups = int(rng.choice([1, 2, 3, 4, 5, 8]))
    kv_heads = int(rng.choice([1, 2, 3, 4]))
    while kv_heads > 1 and kv_heads * groups * head_dim > 1024:
        kv_heads -= 1
    heads = kv_heads * groups
    hidden = int(rng.choice([heads * head_dim, 8 * int(rng.randint(4, 60)), 2 * int(rng.randint(9, 200)),
                             int(rng.randint(17, 300))]))
    scaling = None
    if rng.rand() < 0.35:
        scaling = {"rope_type": "llama3", "factor": float(rng.choice([2.0, 8.0, 32.0])), "low_freq_factor": 1.0,
                   "high_freq_factor": float(rng.choice([2.0, 4.0])),
                   "original_max_position_embeddings": int(rng.choice([16, 64, 128]))}
    raw = dict(architectures=["LlamaForCausalLM"],
               vocab_size=int(rng.choice([int(rng.randint(50, 3000)), 8 * int(rng.randint(8, 300)), 1024])),
               hidden_size=hidden,
               intermediate_size=int(rng.choice([8 * int(rng.randint(4, 120)), int(rng.randint(9, 700)),
                                                 16 * int(rng.randint(2, 50))])),
               num_hidden_layers=int(rng.randint(1, 4)), num_attention_heads=heads, num_key_value_heads=kv_heads,
               head_dim=head_dim, max_position_embeddings=int(rng.choice([300, 512, 1000])),
               rope_theta=float(rng.choice([100.0, 10000.0, 500000.0])), rope_scaling=scaling,
               rope_interleaved=bool(rng.rand() < 0.5), rms_norm_eps=float(rng.choice([1e-6, 1e-5, 3e-4])),
               tie_word_embeddings=bool(rng.rand() < 0.5), attention_bias=bool(rng.rand() < 0.3), eos_token_id=None)
    n_requests = int(rng.choice([1, 2, 3, 5, 8, 9, 13, 17]))
    prompts = [int(rng.choice([1, 2, 7, 31, 63, 64, 65, 100, 129, 200, 260])) for _ in range(n_requests)]
    requests = [[int(t) for t in rng.randint(0, raw["vocab_size"], size=p + int(rng.randint(1, 20)))] for p in prompts]
    return raw, prompts, requests


def replay(llm, requests, prompts):
    """The requests as one batch: prompts in one step, then one token each; a request's slot goes back when
    its tokens are used up.  Logits at every position of every request."""
    slots = llm.engine.acquire(len(requests))
    fed = list(prompts)
    pieces = [[] for _ in requests]
    out = llm.engine.step([StepEntry(slots[r], tokens[:fed[r]], list(range(fed[r]))) for r, tokens in enumerate(requests)])
    at = 0
    for r in range(len(requests)):
        pieces[r].append(out[at:at + fed[r]].cpu().numpy())
        at += fed[r]
    live = list(range(len(requests)))
    while live:
        for r in [r for r in live if fed[r] == len(requests[r])]:
            llm.engine.release(slots[r])
        live = [r for r in live if fed[r] < len(requests[r])]
        if not live:
            break
        out = llm.engine.step([StepEntry(slots[r], [requests[r][fed[r]]], [0]) for r in live])
        for j, r in enumerate(live):
            pieces[r].append(out[j:j + 1].cpu().numpy())
            fed[r] += 1
    llm.engine.cache.check()
    assert llm.engine.cache.n_free_slots == llm.engine.cache.n_slots
    return [np.concatenate(p) for p in pieces]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", SEEDS)
def test_random_configuration(tmp_path, seed, dtype):
    raw, prompts, requests = draw(seed)
    raw["torch_dtype"] = dtype
    folder = str(tmp_path / "model")
    ml.write_random_model(ml.config_from_dict(raw), folder, seed, matrix_std=0.02, norm_std=0.1)
    llm = ml.load(folder, dtype=dtype, max_tokens=8192, max_seqs=max(len(requests), 2))
    got = replay(llm, requests, prompts)
    what = (f"seed {seed}: head size {raw['head_dim']}, heads {raw['num_attention_heads']}/{raw['num_key_value_heads']}, "
            f"width {raw['hidden_size']}, prompts {prompts}")
    for r, tokens in enumerate(requests):
        assert_close(got[r], plain_logits(folder, tokens, dtype), dtype, f"{what}, request {r}")
    alone = replay(llm, requests[:1], [len(requests[0])])[0]
    assert_close(alone, plain_logits(folder, requests[0], dtype), dtype, f"{what}, first request whole")


@pytest.mark.parametrize("head_dim", [8, 40, 72, 272])
def test_head_sizes_outside_the_steps_of_16_are_refused(tmp_path, head_dim):
    raw, _, _ = draw(0)
    raw.update(head_dim=head_dim, num_attention_heads=2, num_key_value_heads=1, torch_dtype="bfloat16")
    with pytest.raises(ValueError, match="head_dim .* must be a multiple of 16"):
        ml.write_random_model(ml.config_from_dict(raw), str(tmp_path / "model"), 0)
