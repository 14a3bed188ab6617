"""Weights by tensor name: the container, the error that lists every fault, placement
dtypes, random folders (no GPU)."""
import json
import struct

import numpy as np
import pytest
import torch

import cpp_minilamma_b200 as ml
import plain_llama as pl
import tiny_configs as tc
from cpp_minilamma_b200.parts.base import WeightSpec
from cpp_minilamma_b200.weights import (ModelFiles, WeightError, WeightFileError, check_tensors, load_tensors,
                                        placement_dtype, write_safetensors)


def specs_of(name):
    return ml.build_model(tc.config(name), "float32", "cpu", max_positions=4).weight_specs()


def test_random_folder_round_trip(tmp_path):
    for storage in ("float32", "bfloat16"):
        folder = tc.write_folder("B", storage, tmp_path / storage)
        specs = specs_of("B")
        tensors = load_tensors(folder, specs, torch.float32, "cpu")
        assert set(tensors) == {s.name for s in specs}
        assert "lm_head.weight" not in tensors  # tied
        _, plain = pl.read_model_folder(folder)  # the independent reader sees the same values
        for name, t in tensors.items():
            np.testing.assert_array_equal(t.float().numpy(), plain[name])
        again = tc.write_folder("B", storage, tmp_path / (storage + "2"))
        assert open(folder + "/model.safetensors", "rb").read() == open(again + "/model.safetensors", "rb").read()


def test_random_weights_statistics(tmp_path):
    folder = tc.write_folder("B", "float32", tmp_path)
    _, w = pl.read_model_folder(folder)
    m = w["model.layers.1.mlp.gate_proj.weight"]
    assert abs(m.std() - 0.02) < 0.002 and abs(m.mean()) < 0.001
    n = w["model.layers.0.input_layernorm.weight"]
    assert abs(n.mean() - 1.0) < 0.05 and 0.05 < n.std() < 0.15
    assert not np.array_equal(w["model.layers.0.self_attn.q_proj.weight"], w["model.layers.1.self_attn.q_proj.weight"])


def test_placement():
    mat, vec = WeightSpec("m", (2, 2)), WeightSpec("v", (2,), kind="vector")
    assert placement_dtype(mat, torch.bfloat16, torch.bfloat16) == torch.bfloat16
    assert placement_dtype(mat, torch.bfloat16, torch.float32) == torch.float32
    assert placement_dtype(mat, torch.float32, torch.bfloat16) == torch.float32   # stored in 32-bit: stays so
    assert placement_dtype(vec, torch.bfloat16, torch.bfloat16) == torch.float32
    assert placement_dtype(WeightSpec("t", (2,), kind="int_table"), torch.int64, torch.bfloat16) == torch.int32


def test_one_error_lists_everything(tmp_path):
    folder = tc.write_folder("A", "float32", tmp_path)
    _, w = pl.read_model_folder(folder)
    tensors = {k: torch.from_numpy(v) for k, v in w.items()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["extra.weight"] = torch.zeros(1)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64)
    tensors["lm_head.weight"] = torch.zeros(131, 64, dtype=torch.int32)
    write_safetensors(tmp_path / "model.safetensors", tensors)
    with pytest.raises(WeightError) as err:
        load_tensors(folder, specs_of("A"), torch.float32, "cpu")
    e = err.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["extra.weight", "model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert len(e.wrong) == 2 and "k_proj" in e.wrong[0] and "(16, 64)" in e.wrong[0] and "(32, 64)" in e.wrong[0]
    text = str(e)
    for piece in ("missing (2)", "unexpected (2)", "wrong shape or dtype (2)", "up_proj", "extra.weight"):
        assert piece in text


def test_untied_model_needs_lm_head_and_tied_rejects_it(tmp_path):
    folder = tc.write_folder("B", "float32", tmp_path)  # tied
    _, w = pl.read_model_folder(folder)
    tensors = {k: torch.from_numpy(v) for k, v in w.items()}
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(tmp_path / "model.safetensors", tensors)
    with pytest.raises(WeightError, match="unexpected.*lm_head.weight"):
        load_tensors(folder, specs_of("B"), torch.float32, "cpu")


def _damaged(tmp_path, mutate):
    folder = tc.write_folder("A", "float32", tmp_path)
    path = tmp_path / "model.safetensors"
    blob = bytearray(path.read_bytes())
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(bytes(blob[8:8 + n]))
    data = bytes(blob[8 + n:])
    header, data = mutate(header, data)
    enc = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(enc)) + enc + data)
    return folder


def test_container_faults(tmp_path):
    def truncated(h, d):
        return h, d[:-10]

    def trailing(h, d):
        return h, d + b"1234"

    def overlap(h, d):
        names = sorted((v["data_offsets"][0], k) for k, v in h.items() if k != "__metadata__")
        first, second = names[0][1], names[1][1]
        size = h[second]["data_offsets"][1] - h[second]["data_offsets"][0]
        h[second]["data_offsets"] = [h[first]["data_offsets"][0] + 4, h[first]["data_offsets"][0] + 4 + size]
        return h, d

    def bad_size(h, d):
        h["model.norm.weight"]["shape"] = [63]
        return h, d

    def bad_dtype(h, d):
        h["model.norm.weight"]["dtype"] = "F8_E4M3"
        return h, d

    for i, (mutate, match) in enumerate([(truncated, "beyond the end"), (trailing, "trailing bytes"),
                                         (overlap, "overlap"), (bad_size, "spans"), (bad_dtype, "unsupported dtype")]):
        folder = _damaged(tmp_path / str(i), mutate)
        with pytest.raises(WeightFileError, match=match):
            ModelFiles(folder)
    (tmp_path / "short").mkdir()
    (tmp_path / "short" / "model.safetensors").write_bytes(b"\x01\x02")
    with pytest.raises(WeightFileError, match="8-byte"):
        ModelFiles(tmp_path / "short")
    (tmp_path / "none").mkdir()
    with pytest.raises(WeightFileError, match="neither"):
        ModelFiles(tmp_path / "none")


def test_sharded_folder(tmp_path):
    folder = tc.write_folder("A", "bfloat16", tmp_path)
    _, w = pl.read_model_folder(folder)
    whole = load_tensors(folder, specs_of("A"), torch.bfloat16, "cpu")
    names = sorted(whole)
    half = len(names) // 2
    write_safetensors(tmp_path / "model-00001-of-00002.safetensors", {n: whole[n] for n in names[:half]})
    write_safetensors(tmp_path / "model-00002-of-00002.safetensors", {n: whole[n] for n in names[half:]})
    index = {"weight_map": {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
                            for i, n in enumerate(names)}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    (tmp_path / "model.safetensors").unlink()
    sharded = load_tensors(folder, specs_of("A"), torch.bfloat16, "cpu")
    for n in names:
        assert torch.equal(sharded[n], whole[n])
    assert whole["model.norm.weight"].dtype == torch.float32          # vectors are held in float32
    assert whole["model.embed_tokens.weight"].dtype == torch.bfloat16  # matrices stay bfloat16


def test_check_tensors_accepts_exact_match():
    specs = specs_of("C")
    check_tensors({s.name: (torch.bfloat16, s.shape) for s in specs}, specs)
    assert any(s.name.endswith("q_proj.bias") for s in specs) and any(s.name.endswith("o_proj.bias") for s in specs)
