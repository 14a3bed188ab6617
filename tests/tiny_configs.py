"""Tiny Llama configurations for the tests.  They differ in every size and option: head
counts and groups (GQA, MQA, MHA), head sizes, widths that are no power of two, layer
counts, vocabulary, eps, rope base, rope scaling, pairing, tied head, biases.  "D" has the head
size and widths at which the bfloat16 engine runs its tensor-core and TMA kernels."""
import numpy as np

import cpp_minilamma_b200 as ml

TINY = {
    # 2 layers, GQA 4/2, head 16, interleaved pairs, untied
    "A": dict(vocab_size=131, hidden_size=64, intermediate_size=176, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, max_position_embeddings=64,
              rope_theta=10000.0, rope_scaling=None, rope_interleaved=True, rms_norm_eps=1e-5,
              tie_word_embeddings=False, eos_token_id=130),
    # 3 layers, MQA 6/1, head 32, llama3 scaling, tied
    "B": dict(vocab_size=257, hidden_size=192, intermediate_size=512, num_hidden_layers=3,
              num_attention_heads=6, num_key_value_heads=1, head_dim=32, max_position_embeddings=256,
              rope_theta=500000.0,
              rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                            "high_freq_factor": 4.0, "original_max_position_embeddings": 32},
              rope_interleaved=False, rms_norm_eps=1e-6, tie_word_embeddings=True, eos_token_id=[255, 256]),
    # 1 layer, MHA 3/3, head 48 (hidden != heads * head), odd intermediate (no interleave), biases, long context
    "C": dict(vocab_size=1000, hidden_size=100, intermediate_size=250, num_hidden_layers=1,
              num_attention_heads=3, num_key_value_heads=3, head_dim=48, max_position_embeddings=1024,
              rope_theta=1000.0, rope_scaling=None, rope_interleaved=False, rms_norm_eps=3e-4,
              tie_word_embeddings=False, attention_bias=True, eos_token_id=None),
    # 2 layers, GQA 4/2, head 64: the head size that the tensor-core attention kernels take; widths that
    # the TMA-fed linear kernels take (multiples of 8), interleaved pairs, tied
    "D": dict(vocab_size=300, hidden_size=256, intermediate_size=328, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=64, max_position_embeddings=512,
              rope_theta=20000.0, rope_scaling=None, rope_interleaved=True, rms_norm_eps=2e-5,
              tie_word_embeddings=True, eos_token_id=7),
}
SEEDS = {"A": 0, "B": 1, "C": 2, "D": 3}


def config(name, storage="float32"):
    raw = dict(TINY[name])
    raw["architectures"] = ["LlamaForCausalLM"]
    raw["torch_dtype"] = storage
    return ml.config_from_dict(raw)


def write_folder(name, storage, folder):
    ml.write_random_model(config(name, storage), folder, SEEDS[name], matrix_std=0.02, norm_std=0.1)
    return str(folder)


def random_tokens(name, length, seed):
    rng = np.random.RandomState(seed)
    return [int(t) for t in rng.randint(0, TINY[name]["vocab_size"], size=length)]
