#!/usr/bin/env python3
"""Makes the golden logits under tests/golden/ from the reference project's own code.

    python tests/golden/make_golden.py --reference /path/to/cpp-minilamma [--cpp-binary build/mini-llama]
                                       [--cpp-library build/libyan_minillama.a]

Steps: write the tiny-A model (this repo's seeded random weights, float32) in the
reference's model.json / model.bin format (src/load.cc:386-406 names, row-major [out, in]);
run the reference's NumPy oracle (scripts/reference_forward.py: load_model, forward_token) on
a fixed random token sequence; optionally run its C++ CPU engine
(`mini-llama --config --model --dump-logits`, app/main.cc:137-269) on the prompt "hello",
which feeds BOS (128) + the ASCII bytes and then generates greedily.  With
`--cpp-library` (the reference's static library, CPU build) it also compiles `reference_driver.cc` against it
and runs the reference's C++ forward on tiny B without rope scaling: multi-query attention, half-split rotary
pairs (its "NeoX" type), eps 1e-6, theta 500000, the tied head written out as a second tensor, on the
BASELINE workload's four sequences (prompts 17/1/40/6 + 12 tokens each).  The llama3 rope scaling itself has no
counterpart in the reference, so that rule stays anchored on its published formula alone.  The outputs are
small and are committed; tests/test_plain.py compares the plain implementation with them.
Needs the reference checkout, so it runs where that is mounted, not in the test suite.
"""
import argparse
import hashlib
import json
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE.parent))

NAME_MAP = {"model.embed_tokens.weight": "token_embedding", "model.norm.weight": "final_norm",
            "lm_head.weight": "lm_head"}
LAYER_MAP = {"input_layernorm.weight": "attention_norm", "self_attn.q_proj.weight": "wq",
             "self_attn.k_proj.weight": "wk", "self_attn.v_proj.weight": "wv", "self_attn.o_proj.weight": "wo",
             "post_attention_layernorm.weight": "ffn_norm", "mlp.gate_proj.weight": "w_gate",
             "mlp.up_proj.weight": "w_up", "mlp.down_proj.weight": "w_down"}


def reference_name(name):
    if name in NAME_MAP:
        return NAME_MAP[name]
    _, _, layer, rest = name.split(".", 3)
    return f"layers.{layer}.{LAYER_MAP[rest]}"


def export_reference_format(cfg, weights, folder):
    """model.json + model.bin as model/tinymodel/export_model.py:94-129 lays them out."""
    if "lm_head.weight" not in weights:  # a tied head: the reference wants the tensor written out
        weights = dict(weights, **{"lm_head.weight": weights["model.embed_tokens.weight"]})
    order = ["model.embed_tokens.weight"]
    for layer in range(cfg["num_hidden_layers"]):
        order += [f"model.layers.{layer}.{k}" for k in LAYER_MAP]
    order += ["model.norm.weight", "lm_head.weight"]
    entries, blob, offset = [], bytearray(), 0
    for name in order:
        data = np.ascontiguousarray(weights[name], dtype="<f4")
        entries.append({"name": reference_name(name), "shape": list(data.shape), "dtype": "float32",
                        "offset": offset, "byte_size": data.nbytes})
        blob += data.tobytes()
        offset += data.nbytes
    manifest = {"config": {"vocab_size": cfg["vocab_size"], "dim": cfg["hidden_size"],
                           "hidden_dim": cfg["intermediate_size"], "layers": cfg["num_hidden_layers"],
                           "n_heads": cfg["num_attention_heads"], "n_kv_heads": cfg["num_key_value_heads"],
                           "head_dim": cfg["head_dim"], "max_seq_len": cfg["max_position_embeddings"],
                           "rope_theta": cfg["rope_theta"], "rms_norm_eps": cfg["rms_norm_eps"]},
                "tokenizer": {"type": "ASCII", "bos_id": 128, "eos_id": 129, "unk_id": 130},
                "tensors": entries}
    (folder / "model.json").write_text(json.dumps(manifest, indent=2))
    (folder / "model.bin").write_bytes(bytes(blob))


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True)
    parser.add_argument("--cpp-binary", default=None)
    parser.add_argument("--cpp-library", default=None)
    args = parser.parse_args()
    import plain_llama as pl
    import tiny_configs as tc

    with tempfile.TemporaryDirectory() as tmp:
        tmp = Path(tmp)
        folder = Path(tc.write_folder("A", "float32", tmp / "ours"))
        digest = hashlib.sha256((folder / "model.safetensors").read_bytes()).hexdigest()
        cfg, weights = pl.read_model_folder(folder)
        ref_dir = tmp / "ref"
        ref_dir.mkdir()
        export_reference_format(cfg, weights, ref_dir)

        sys.path.insert(0, str(Path(args.reference) / "scripts"))
        import reference_forward as rf
        model = rf.load_model(ref_dir / "model.json", ref_dir / "model.bin")
        tokens = tc.random_tokens("A", 24, 4242)
        model.reset_cache()
        logits = np.stack([rf.forward_token(model, pos, tok) for pos, tok in enumerate(tokens)])
        np.save(HERE / "tinyA_reference_numpy_logits.npy", logits.astype(np.float32))
        meta = {"model_sha256": digest, "config": "tiny_configs.TINY['A'], float32, seed 0",
                "numpy_tokens": tokens, "source": "scripts/reference_forward.py forward_token"}

        if args.cpp_binary:
            out = tmp / "dump"
            subprocess.run([args.cpp_binary, "--config", str(ref_dir / "model.json"), "--model",
                            str(ref_dir / "model.bin"), "--dump-logits", str(out), "--prompt", "hello",
                            "--n-predict", "9"], check=True, capture_output=True)
            run = json.loads((out / "cpp_run.json").read_text())
            steps = [np.fromfile(out / f"logits_step{i}.bin", dtype="<f4") for i in range(run["step_count"])]
            generated = [int(t) for t in (out / "generation_tokens.txt").read_text().split()]
            np.save(HERE / "tinyA_reference_cpp_logits.npy", np.stack(steps).astype(np.float32))
            meta.update({"cpp_prompt_tokens": run["prompt_tokens"], "cpp_generated": generated,
                         "cpp_source": "mini-llama --dump-logits (CPU build, app/main.cc:137-269)"})
        (HERE / "tinyA_reference.json").write_text(json.dumps(meta, indent=1) + "\n")

        if args.cpp_library:
            # tiny B as far as the reference can run it: everything but the rope scaling
            folder_b = Path(tc.write_folder("B", "float32", tmp / "ours_b"))
            digest_b = hashlib.sha256((folder_b / "model.safetensors").read_bytes()).hexdigest()
            cfg_b, weights_b = pl.read_model_folder(folder_b)
            ref_b = tmp / "ref_b"
            ref_b.mkdir()
            export_reference_format(cfg_b, weights_b, ref_b)
            driver = tmp / "reference_driver"
            subprocess.run(["g++", "-std=c++17", "-O2", "-I", args.reference, str(HERE / "reference_driver.cc"),
                            args.cpp_library, "-lpthread", "-o", str(driver)], check=True)
            lengths = [17 + 12, 1 + 12, 40 + 12, 6 + 12]
            sequences = [tc.random_tokens("B", n, 5150 + i) for i, n in enumerate(lengths)]
            rows = []
            for i, tokens in enumerate(sequences):
                out = tmp / f"b{i}.f32"
                subprocess.run([str(driver), str(ref_b / "model.json"), str(ref_b / "model.bin"), "neox", str(out)]
                               + [str(t) for t in tokens], check=True)
                rows.append(np.fromfile(out, dtype="<f4").reshape(len(tokens), cfg_b["vocab_size"]))
            np.save(HERE / "tinyB_noscale_reference_cpp_logits.npy", np.concatenate(rows).astype(np.float32))
            (HERE / "tinyB_noscale_reference.json").write_text(json.dumps({
                "model_sha256": digest_b, "config": "tiny_configs.TINY['B'] with rope_scaling = None, float32, seed 1",
                "sequences": sequences, "source": "reference_driver.cc: ParseModel, rope_type = kNeoX, ForwardBatch one "
                "token per forward (src/forward.cc:473-488), CPU build"}, indent=1) + "\n")
        print("wrote golden files:", sorted(p.name for p in HERE.iterdir()))


if __name__ == "__main__":
    main()
