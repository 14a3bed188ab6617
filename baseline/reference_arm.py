"""`bench.py --impl reference`: the unmodified reference engine on the bench's model shape.

The reference (a CMake C++ project; pip has nothing to install: it ships neither setup.py nor
pyproject.toml) is built as it is with its own CUDA backend switched on:

    cmake -S baseline/_ref/src -B baseline/_ref/build -G Ninja -DCMAKE_BUILD_TYPE=Release \
          -DBUILD_TESTING=OFF -DMINI_LLAMA_CUDA=ON -DCMAKE_CUDA_ARCHITECTURES=100
    cmake --build baseline/_ref/build --target mini-llama

(`baseline/_ref/src` is a copy of the reference tree; CMakeLists.txt:10,51-58 of the reference).
This module writes a model of the bench's shape in the reference's own format (model.json +
model.bin, float32: its CUDA backend has no other dtype; src/load.cc:510-566), a vocabulary file for
its JsonVocab tokenizer (src/jsonvocab.cc), and runs its stock strict bench

    mini-llama bench <folder> --backend cuda --prompt <text> -n <K + 1> --warmup 0

(src/bench_strict.cc:255-282), whose report gives prefill ms, decode ms and tokens/s (decode) with
the timers around the forwards only.  None of this repository's engine, kernels or model code is on
that path; torch is used to draw the random weights and write the files.

The reference runs one sequence, one token per forward: a batch of 8 is, for it, 8 sequences one
after the other, so its decode rate at "batch 8" is its single-sequence rate.  Measured on a B200: one
forward of the 32-layer float32 model takes 172 ms (prompt and decode forwards alike: 2,813 ms for 16
prompt tokens, 858 ms for 5 decoded ones), writing the 32 GB model takes 26 s and the engine's start-up
(read + upload) 31 s.  The bench's own workload - 8 prompts of 128 to 2,047 tokens, 1,088 on average -
would be 8,700 prompt forwards, 25 minutes, before the first timed decode step.  So one sequence is run
with the workload's shortest prompt (128 tokens) and no warm-up run of the engine's own (a warm-up
run would repeat the prompt; the 128 prompt forwards precede the timed decode forwards).  A forward's
time grows with the context, so the short prompt flatters the reference, not this library.  The JSON
line says all of this in `config`.
If the run cannot be had (no build, no room for the files, the time limit), one line
{"impl": "reference", "unavailable": why} is printed and the exit code is 0.
"""
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
BINARY = os.path.join(REF, "build", "mini-llama")

LAYER_TENSORS = [("attention_norm", "norm"), ("wq", "q"), ("wk", "kv"), ("wv", "kv"), ("wo", "o"),
                 ("ffn_norm", "norm"), ("w_gate", "up"), ("w_up", "up"), ("w_down", "down")]


def unavailable(why):
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def ensure_binary():
    """The reference's `mini-llama` with its CUDA backend; built here if the tree is there and the binary is not."""
    if os.path.isfile(BINARY):
        return None
    src = os.path.join(REF, "src")
    if not os.path.isfile(os.path.join(src, "CMakeLists.txt")):
        return "the reference tree is not under baseline/_ref/src (it is not part of this repository)"
    cmake = shutil.which("cmake")
    if cmake is None:
        return "cmake not found: the reference cannot be built"
    build = os.path.join(REF, "build")
    steps = [[cmake, "-S", src, "-B", build, "-G", "Ninja", "-DCMAKE_BUILD_TYPE=Release", "-DBUILD_TESTING=OFF",
              "-DMINI_LLAMA_CUDA=ON", "-DCMAKE_CUDA_ARCHITECTURES=100", "-DCMAKE_CUDA_COMPILER=/usr/local/cuda/bin/nvcc"],
             [cmake, "--build", build, "--target", "mini-llama", "-j", "8"]]
    for cmd in steps:
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode != 0:
            return "building the reference failed: " + (done.stderr or done.stdout).strip().splitlines()[-1][:200]
    return None if os.path.isfile(BINARY) else "the reference build left no mini-llama binary"


def token_text(token_id):
    return "t%05x" % token_id  # six characters each, none a prefix of another: the greedy matcher finds them back


def write_vocabulary(path, vocab):
    """Entries {"id", "context"} for every id (src/jsonvocab.cc:140-200); the last three ids are the special
    tokens that the tokenizer insists on."""
    specials = {vocab - 3: "<BOS>", vocab - 2: "<EOS>", vocab - 1: "<UNK>"}
    with open(path, "w") as fh:
        fh.write("[")
        for i in range(vocab):
            fh.write(("," if i else "") + json.dumps({"id": i, "context": specials.get(i, token_text(i))}))
        fh.write("]")
    return vocab - 3, vocab - 2, vocab - 1


def write_model(folder, shape, layers, max_seq_len, seed=0):
    """model.json + model.bin (headerless little-endian float32, row-major [out, in], tensors back to back;
    names as src/load.cc:386-406).  Weights N(0, 0.02), norms 1.0, drawn on the GPU and streamed to the file."""
    import torch
    cfg = shape["config"]
    d, hq, hk, hd, inter, vocab = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                                   cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"])
    shapes = {"norm": (d,), "q": (hq * hd, d), "kv": (hk * hd, d), "o": (d, hq * hd), "up": (inter, d), "down": (d, inter)}
    tensors = [("token_embedding", (vocab, d))]
    for layer in range(layers):
        tensors += [(f"layers.{layer}.{name}", shapes[kind]) for name, kind in LAYER_TENSORS]
    tensors += [("final_norm", (d,)), ("lm_head", (vocab, d))]
    entries, offset = [], 0
    device = "cuda:0" if torch.cuda.is_available() else "cpu"
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    with open(os.path.join(folder, "model.bin"), "wb") as fh:
        for name, dims in tensors:
            if len(dims) == 1:
                data = torch.ones(dims, dtype=torch.float32)
            else:
                data = (torch.randn(dims, generator=gen, dtype=torch.float32, device=device) * 0.02).cpu()
            data.numpy().tofile(fh)
            size = data.numel() * 4
            entries.append({"name": name, "shape": list(dims), "dtype": "float32", "offset": offset, "byte_size": size})
            offset += size
    bos, eos, unk = write_vocabulary(os.path.join(folder, "vocab.json"), vocab)
    manifest = {"config": {"vocab_size": vocab, "dim": d, "hidden_dim": inter, "layers": layers, "n_heads": hq,
                           "n_kv_heads": hk, "head_dim": hd, "max_seq_len": max_seq_len,
                           "rope_theta": cfg["rope_theta"], "rms_norm_eps": cfg["rms_norm_eps"]},
                "tokenizer": {"type": "JsonVocab", "pathname": "vocab.json", "bos_id": bos, "eos_id": eos, "unk_id": unk},
                "tensors": entries}
    with open(os.path.join(folder, "model.json"), "w") as fh:
        json.dump(manifest, fh, indent=2)
    return offset


def parse_report(text):
    """The strict bench's "key: value" lines (src/bench_strict.cc:200-252)."""
    fields = {}
    for line in text.splitlines():
        key, sep, value = line.partition(":")
        if sep:
            fields[key.strip()] = value.strip()
    return fields


def run_reference(shape, layers, prompt_tokens, new_tokens, warmup_runs, limit_s, seed=0, keep=None, backend="cuda"):
    """Write the model, run the stock bench once, return (report fields, timings) or raise RuntimeError."""
    import numpy as np
    cfg = shape["config"]
    need = 4 * (2 * cfg["vocab_size"] * cfg["hidden_size"] + layers * (
        cfg["hidden_size"] * (2 * cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"]
        + 3 * cfg["hidden_size"] * cfg["intermediate_size"]))
    base = keep
    if base is None:
        # memory-backed storage when it has room for the file beside the engine's own host copy of the weights
        shm = "/dev/shm"
        roomy = os.path.isdir(shm) and shutil.disk_usage(shm).free > 3 * need + (8 << 30)
        base = tempfile.mkdtemp(prefix="mll_reference_", dir=shm if roomy else None)
    try:
        free = shutil.disk_usage(base).free
        if free < need + (1 << 30):
            raise RuntimeError(f"{need / 1e9:.1f} GB of float32 weights do not fit into {base} ({free / 1e9:.1f} GB free)")
        began = time.time()
        write_model(base, shape, layers, max_seq_len=prompt_tokens + new_tokens + 8, seed=seed)
        wrote_s = time.time() - began
        rng = np.random.RandomState(seed + 1)
        # the tokenizer puts <BOS> in front: prompt_tokens - 1 ordinary tokens follow
        ids = rng.randint(0, cfg["vocab_size"] - 3, size=prompt_tokens - 1)
        text = "".join(token_text(int(t)) for t in ids)
        cmd = [BINARY, "bench", base, "--backend", backend, "--prompt", text, "-n", str(new_tokens),
               "--warmup", str(warmup_runs), "--seed", "1"]
        began = time.time()
        try:
            done = subprocess.run(cmd, capture_output=True, text=True, timeout=limit_s)
        except subprocess.TimeoutExpired:
            raise RuntimeError(f"the reference's bench did not finish {warmup_runs + 1} runs of {prompt_tokens} prompt "
                               f"forwards + {new_tokens - 1} decode forwards within {limit_s:.0f} s "
                               f"({need / 1e9:.1f} GB float32 model, written in {wrote_s:.0f} s)")
        ran_s = time.time() - began
        if done.returncode != 0:
            raise RuntimeError("the reference's bench failed: " + (done.stderr.strip().splitlines() or ["no message"])[-1][:300])
        fields = parse_report(done.stdout)
        return fields, {"write_s": round(wrote_s, 1), "run_s": round(ran_s, 1), "model_gb": round(need / 1e9, 2)}
    finally:
        if keep is None:
            shutil.rmtree(base, ignore_errors=True)


def main(args):
    sys.path.insert(0, os.path.dirname(HERE))
    import bench
    if args.gpus != 1:
        return unavailable("the reference runs on one GPU")
    problem = ensure_binary()
    if problem:
        return unavailable(problem)
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device")
    except ImportError:
        return unavailable("torch is needed to draw the random weights")
    shape = bench.SHAPES["llama31_8b"]
    layers = args.layers or shape["config"]["num_hidden_layers"]
    steps = max(args.steps, 1)
    prompt_tokens = bench.PROMPT_RANGE[0]  # the shortest prompt of the workload: see the header
    limit = float(os.environ.get("MLL_REFERENCE_LIMIT_S", "420"))
    try:
        fields, timings = run_reference(shape, layers, prompt_tokens, steps + 1, warmup_runs=0, limit_s=limit)
        decode_ms = float(fields["decode ms"])
        prefill_ms = float(fields["prefill ms"])
        n_prompt = int(fields["prompt tokens"])
    except (RuntimeError, KeyError, ValueError, OSError) as error:
        return unavailable(str(error)[:400])
    per_token_ms = decode_ms / steps
    batch = bench.BATCH
    cfg = shape["config"]
    line = {
        "metric": "decode tok/s at batch 8 (Llama-3.1-8B shape, random weights)", "impl": "reference",
        "value": round(1000.0 / per_token_ms, 2), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": args.warmup,
        "ms_per_step": round(batch * per_token_ms, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32 (the reference's CUDA backend has no other)", "data": "synthetic token ids, random-init weights",
        "config": {"model": "Llama-3.1-8B shape", "layers": layers, "layers_full": cfg["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "global_batch": batch, "seq_len": bench.CONTEXT, "prompt_tokens": n_prompt,
                   "sequences": "one sequence with the shortest prompt of uniform[128,2048): the engine runs a batch one "
                                "sequence after the other (a step of 8 tokens is 8 of its forwards) and a prompt one "
                                "forward per token, 172 ms each at this size",
                   "warmup_runs": "none of its own; the prompt's forwards precede the timed ones", "parallelism": "1 gpu",
                   "command": "mini-llama bench <folder> --backend cuda"},
        "e2e": {"value": round(1000.0 / per_token_ms, 2), "unit": "tokens/s",
                "h2d_bytes_per_step": 0, "d2h_bytes_per_step": batch * 4 * cfg["vocab_size"],
                "note": "its timers already include the logits' copy to the host after every forward; its own counters: "
                        f"host->device copies {fields.get('host->device copies')}, device->host copies "
                        f"{fields.get('device->host copies')}"},
        "gpu_launches": int(fields.get("cuda linear calls", "0") or 0),
        "prefill": {"value": round(n_prompt * 1000.0 / prefill_ms, 1), "tokens": n_prompt, "ms": round(prefill_ms, 1)},
        "timings": timings,
    }
    print(json.dumps(line))
    return 0
