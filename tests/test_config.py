"""Configuration and registry (no GPU)."""
import json

import pytest

import cpp_minilamma_b200 as ml
import tiny_configs as tc
from cpp_minilamma_b200.config import ConfigError, known_architectures
from cpp_minilamma_b200.models.llama import build_llama_spec


def raw(name="A", **over):
    r = dict(tc.TINY[name], architectures=["LlamaForCausalLM"])
    r.update(over)
    return r


def test_reads_every_key_and_round_trips(tmp_path):
    for name in "ABC":
        cfg = ml.config_from_dict(raw(name))
        for key, value in tc.TINY[name].items():
            if key == "eos_token_id":
                expect = [] if value is None else ([value] if isinstance(value, int) else value)
                assert cfg.eos_token_ids == expect
            elif key == "rope_scaling":
                assert (cfg.rope_scaling.to_dict() if cfg.rope_scaling else None) == value
            else:
                assert getattr(cfg, key) == value, key
        ml.config.save_config(cfg, tmp_path / name)
        assert ml.load_config(tmp_path / name) == cfg


def test_defaults():
    r = raw("A")
    for key in ("num_key_value_heads", "head_dim", "rope_theta", "rms_norm_eps", "tie_word_embeddings",
                "rope_scaling", "rope_interleaved", "eos_token_id"):
        r.pop(key)
    cfg = ml.config_from_dict(r)
    assert cfg.num_key_value_heads == cfg.num_attention_heads == 4
    assert cfg.head_dim == 16 and cfg.rope_theta == 10000.0 and cfg.rms_norm_eps == 1e-5
    assert cfg.tie_word_embeddings is False and cfg.rope_scaling is None and cfg.eos_token_ids == []


@pytest.mark.parametrize("change,match", [
    (dict(architectures=["NoSuchModel"]), "unknown architecture.*LlamaForCausalLM"),
    (dict(architectures=[]), "exactly one"),
    (dict(vocab_size=None), "missing required key 'vocab_size'"),
    (dict(hidden_size="64"), "must be an integer"),
    (dict(num_hidden_layers=0), ">= 1"),
    (dict(num_key_value_heads=3), "multiple of"),
    (dict(head_dim=15), "even"),
    (dict(rope_theta=0.0), "rope_theta"),
    (dict(rms_norm_eps=float("nan")), "finite"),
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(mlp_bias=True), "mlp_bias"),
    (dict(rope_scaling={"rope_type": "yarn", "factor": 2.0}), "rope_scaling type"),
    (dict(rope_scaling={"rope_type": "llama3", "factor": 8.0}), "low_freq_factor"),
    (dict(eos_token_id=5000), "outside the vocabulary"),
    (dict(torch_dtype="float8"), "torch_dtype"),
    (dict(tie_word_embeddings="yes"), "true or false"),
])
def test_rejects(change, match):
    with pytest.raises(ConfigError, match=match):
        ml.config_from_dict(raw("A", **change))


def test_load_config_errors(tmp_path):
    with pytest.raises(ConfigError, match="no config.json"):
        ml.load_config(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        ml.load_config(tmp_path)


def test_registry_and_spec_are_data():
    assert "LlamaForCausalLM" in known_architectures()
    cfg = ml.config_from_dict(raw("B"))
    spec = build_llama_spec(cfg)
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    assert spec.lm_head.params["tied_to"] == "model.embed_tokens.weight"
    attn = spec.layers[1].mixer
    assert attn.kind == "attention" and attn.params["n_kv_heads"] == 1 and attn.params["head_dim"] == 32
    assert attn.params["position"].params["scaling"]["factor"] == 8.0
    assert spec.layers[2].norms["input"].params["eps"] == 1e-6
    assert spec.stop_token_ids == [255, 256]


def test_no_size_in_code():
    # the builder takes every size from the configuration: a config unlike any test model builds
    cfg = ml.config_from_dict(raw("A", hidden_size=48, num_attention_heads=3, num_key_value_heads=1,
                                  head_dim=16, intermediate_size=40, vocab_size=77, num_hidden_layers=5,
                                  eos_token_id=None))
    model = ml.build_model(cfg, "float32", "cpu", max_positions=8)
    shapes = {s.name: s.shape for s in model.weight_specs()}
    assert shapes["model.layers.4.self_attn.k_proj.weight"] == (16, 48)
    assert shapes["model.layers.0.mlp.down_proj.weight"] == (48, 40)
    assert shapes["lm_head.weight"] == (77, 48)
    assert model.parameter_count() == sum(__import__("math").prod(s) for s in shapes.values())


def test_float16_storage_is_a_known_dtype():
    # the dtype a folder is stored in; a run converts to its own (float32 or bfloat16) when it loads
    cfg = ml.config_from_dict(raw("A", torch_dtype="float16"))
    assert cfg.torch_dtype == "float16" and cfg.to_dict()["torch_dtype"] == "float16"
