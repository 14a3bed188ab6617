#!/usr/bin/env python3
"""Decode and prefill throughput of the Llama-3.1-8B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints one JSON line.  A step is one decode step of a batch of 8 sequences with unequal
prompts (uniform in [128, 2048)) on a cache sized for 4096 tokens each; `value` is decoded
tokens per second measured with CUDA events around K steps after W warm-up steps (the loop of
K steps is repeated and the median repeat reported).  Before anything is timed the bfloat16
engine's tokens are compared with a float32 run at the same layer widths (`checked`).  The
same line carries: `e2e` (the same metric through one `LLM.generate` call, token ids in host lists
in and out, the last K of its W + K decode steps on the host clock), `prefill` (one 2,048-token prompt), `roofline` (bytes a decode step must
read / its time, against the measured HBM copy bandwidth), `points` (decode at batch 1
and 64, with their fractions of the HBM peak) and `workloads` (the Llama-2-7B shape at batch
16 and the Llama-3.2-1B shape at batch 64, each with its own bytes and fraction).  Weights are
random (N(0, 0.02)), token ids synthetic; every decode step reads gigabytes of weights and
cache, far more than the 126 MB L2, so no L2 flush is needed between iterations.  The metric definitions follow the reference's strict bench (timers around
forwards only, warm-ups first, fresh cache: src/bench_strict.cc:146-176).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
BATCH = 8
CONTEXT = 4096
PROMPT_RANGE = (128, 2048)
PREFILL_TOKENS = 2048


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peaks = dict(FALLBACK_PEAKS)
    if os.path.isfile(path):
        try:
            raw = json.load(open(path))
            flat = {}

            def walk(node):
                if isinstance(node, dict):
                    for k, v in node.items():
                        if isinstance(v, (int, float)):
                            flat.setdefault(k, float(v))
                        else:
                            walk(v)
            walk(raw)
            if "hbm_gbs" in flat:
                peaks["hbm_gbs"] = flat["hbm_gbs"]
                peaks["source"] = "measured"
            if "bf16_tflops" in flat:
                peaks["bf16_tflops"] = flat["bf16_tflops"]
            if "bf16_tflops_sustained" in flat:
                peaks["bf16_tflops_sustained"] = flat["bf16_tflops_sustained"]
        except (OSError, ValueError):
            pass
    return peaks


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.samples = []      # (time of arrival, fields)
        self.proc = None
        self.index = index
        self.window = [None, None]

    def wait_for_first_line(self, limit=3.0):
        deadline = time.monotonic() + limit
        while self.proc is not None and not self.samples and time.monotonic() < deadline:
            time.sleep(0.01)

    def begin(self):
        """The timed region starts now: earlier samples are dropped."""
        self.window[0] = time.monotonic()

    def end(self):
        self.window[1] = time.monotonic()

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append((time.monotonic(), parts))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        clocks, reasons, top = [], set(), None
        lo, hi = self.window
        for at, (sm, mx, hw, hwt, swt, cap) in self.samples:
            # a line arrives up to one period after its reading
            if (lo is not None and at < lo + 0.05) or (hi is not None and at > hi + 0.05):
                continue
            try:
                clocks.append(int(float(sm)))
                top = int(float(mx))
            except ValueError:
                continue
            for name, flag in (("hw_slowdown", hw), ("hw_thermal_slowdown", hwt), ("sw_thermal_slowdown", swt),
                               ("sw_power_cap", cap)):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None, "sm_max_mhz": top,
                "reasons": sorted(reasons), "samples": len(clocks)}


SHAPES = {
    # BASELINE's configurations 3, 4 and 5: sizes as config.json keys, then the workload
    "llama31_8b": dict(
        config={"vocab_size": 128256, "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 32,
                "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
                "max_position_embeddings": 131072, "rope_theta": 500000.0,
                "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                 "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
                "rms_norm_eps": 1e-5, "tie_word_embeddings": False},
        batch=8, context=4096, prompts=(128, 2048)),
    "llama2_7b": dict(
        config={"vocab_size": 32000, "hidden_size": 4096, "intermediate_size": 11008, "num_hidden_layers": 32,
                "num_attention_heads": 32, "num_key_value_heads": 32, "head_dim": 128,
                "max_position_embeddings": 4096, "rope_theta": 10000.0, "rope_scaling": None,
                "rms_norm_eps": 1e-5, "tie_word_embeddings": False},
        batch=16, context=4096, prompts=(256, 1025), decode_steps=256),
    "llama32_1b": dict(
        config={"vocab_size": 128256, "hidden_size": 2048, "intermediate_size": 8192, "num_hidden_layers": 16,
                "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
                "max_position_embeddings": 131072, "rope_theta": 500000.0,
                "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                                 "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
                "rms_norm_eps": 1e-5, "tie_word_embeddings": True},
        batch=64, context=8192, prompts=(64, 4097), decode_steps=128),
}


def shape_config(name, layers=None):
    import cpp_minilamma_b200 as ml
    raw = dict(SHAPES[name]["config"], architectures=["LlamaForCausalLM"], torch_dtype="bfloat16")
    if layers:
        raw["num_hidden_layers"] = layers
    return ml.config_from_dict(raw)


def llama31_8b(layers=None):
    return shape_config("llama31_8b", layers)


def prompts_for(batch, vocab, seed, prompt_range=PROMPT_RANGE):
    import numpy as np
    rng = np.random.RandomState(seed)
    lens = rng.randint(prompt_range[0], prompt_range[1], size=batch)
    return [[int(t) for t in rng.randint(0, vocab, size=n)] for n in lens]


def release_model(llm):
    """Give a model's memory back before the next one is built."""
    import gc
    import torch
    llm.engine.__dict__.clear()
    llm.__dict__.clear()
    gc.collect()
    torch.cuda.empty_cache()


def time_decode(llm, batch, steps, warmup, seed, sampler=None, prompt_range=PROMPT_RANGE, repeats=1, context=CONTEXT):
    """Prefill `batch` unequal prompts, then time `steps` decode steps (greedy sampling on
    the device included) with CUDA events, `repeats` times over on the same growing sequences.
    Returns (median ms per step, live context tokens at the middle of the timed steps, launches
    of this library's kernels per step, the times of all repeats, ms of the prompt step)."""
    import torch
    from cpp_minilamma_b200 import EngineBackend, SamplingParams, StepEntry
    from cpp_minilamma_b200.csrc import kernels as K
    engine = llm.engine
    backend = EngineBackend(engine, SamplingParams())
    prompts = prompts_for(batch, llm.config.vocab_size, seed, prompt_range)
    longest = max(len(p) for p in prompts)
    repeats = max(1, min(repeats, (context - longest - warmup - 2) // steps))
    slots = engine.acquire(batch)
    try:
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        begin.record()
        tokens = backend.step_and_sample([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)],
                                         list(range(batch)), [0] * batch)
        end.record()
        torch.cuda.synchronize()
        prompt_ms = begin.elapsed_time(end)
        for i in range(warmup):
            tokens = backend.step_and_sample([StepEntry(s, [t], [0]) for s, t in zip(slots, tokens)],
                                             list(range(batch)), [i + 1] * batch)
        torch.cuda.synchronize()
        if sampler:
            sampler.wait_for_first_line()
            sampler.begin()
        launches_before = K.launches
        times = []
        done = warmup
        for _ in range(repeats):
            # as the generation loop runs it: step i + 1, fed on the device with the tokens of step i, is
            # enqueued before the host collects step i
            begin.record()
            ticket = backend.submit([StepEntry(s, [t], [0]) for s, t in zip(slots, tokens)], list(range(batch)),
                                    [done + 1] * batch)
            for i in range(steps):
                ahead = backend.submit_ahead(slots, list(range(batch)), [done + i + 2] * batch) if i + 1 < steps else None
                tokens = backend.collect(ticket)
                ticket = ahead
            end.record()
            torch.cuda.synchronize()
            times.append(begin.elapsed_time(end) / steps)
            done += steps
        if sampler:
            sampler.end()
        ordered = sorted(times)
        ms = ordered[len(ordered) // 2]
        live = sum(len(p) for p in prompts) + batch * (warmup + (repeats * steps) // 2)
        return ms, live, (K.launches - launches_before) / (steps * repeats), times, prompt_ms
    finally:
        for s in slots:
            engine.release(s)


def decode_bytes(llm, live_tokens):
    """Bytes a decode step has to read: every weight it uses once, and the cache of the live tokens."""
    return llm.model.step_weight_bytes() + llm.engine.cache.kv_bytes_per_token() * live_tokens


def check_against_float32(peaks_note=None):
    """Before anything is timed: the bfloat16 engine at the benchmark's layer widths and vocabulary (2 of the
    32 layers) generates greedily for a batch of 8 unequal prompts through `LLM.generate` (captured graphs,
    the device one step ahead), and a float32 run of the same weights scores those sequences.  Every
    generated token must be the float32 run's best token, or within 4 % of its largest |logit| of it
    (bfloat16 rounding moves near ties)."""
    import numpy as np
    import torch
    import cpp_minilamma_b200 as ml
    from cpp_minilamma_b200 import StepEntry
    cfg = shape_config("llama31_8b", layers=2)
    new_tokens = 6
    prompts = prompts_for(BATCH, cfg.vocab_size, seed=5, prompt_range=(128, 700))
    fast = ml.random_model(cfg, seed=0, dtype="bfloat16", max_tokens=BATCH * 1024, max_positions=1024, max_seqs=BATCH)
    generated = fast.generate(prompts, max_new_tokens=new_tokens, ignore_eos=True)
    release_model(fast)
    exact = ml.random_model(cfg, seed=0, dtype="float32", stored_as="bfloat16", max_tokens=2048, max_positions=1024,
                            max_seqs=2)
    worst = 0.0
    for prompt, tokens in zip(prompts, generated):
        assert len(tokens) == new_tokens
        slot, = exact.engine.acquire(1)
        whole = list(prompt) + tokens[:-1]
        want = list(range(len(prompt) - 1, len(whole)))
        logits = exact.engine.step([StepEntry(slot, whole, want)]).cpu().numpy()
        exact.engine.release(slot)
        for row, token in zip(logits, tokens):
            margin = float(row.max() - row[token]) / float(np.abs(row).max())
            worst = max(worst, margin)
            if margin > 0.04:
                raise AssertionError(f"bench check: the bfloat16 engine generated token {token}, which the float32 "
                                     f"run puts {margin:.3f} of its largest logit below its best token")
    release_model(exact)
    return {"checked": True, "check": f"8 prompts x {new_tokens} greedy tokens of the bfloat16 engine (2 layers, full widths "
                                       f"and vocabulary) against a float32 run of the same weights; worst margin {worst:.4f}"}


def time_workload(name, peaks, warmup, layers=None):
    """One of the further workloads: its batch of unequal prompts in one step, then all its decode steps,
    timed as the reference's strict bench times them (timers around the steps only, device sampling
    included; src/bench_strict.cc:146-176,200-209)."""
    import cpp_minilamma_b200 as ml
    spec = SHAPES[name]
    cfg = shape_config(name, layers)
    batch, steps, context = spec["batch"], spec["decode_steps"], spec["context"]
    budget = batch * (spec["prompts"][1] + warmup + steps + 64)
    llm = ml.random_model(cfg, seed=0, dtype="bfloat16", max_tokens=budget, max_positions=context, max_seqs=batch,
                          max_step_tokens=8192)
    ms, live, _, _, prompt_ms = time_decode(llm, batch, steps, warmup, seed=21, prompt_range=spec["prompts"],
                                            context=context)
    prompt_tokens = live - batch * (warmup + steps // 2)
    achieved = decode_bytes(llm, live) / (ms * 1e-3) / 1e9
    out = {"decode_tok_s": round(batch * 1000.0 / ms, 1), "ms_per_step": round(ms, 4), "batch": batch,
           "decode_steps": steps, "layers": cfg.num_hidden_layers, "layers_full": spec["config"]["num_hidden_layers"],
           "live_tokens": live, "gb_per_step": round(decode_bytes(llm, live) / 1e9, 3),
           "hbm_gbs": round(achieved, 1), "frac": round(achieved / peaks["hbm_gbs"], 4),
           "prefill_tok_s": round(prompt_tokens * 1000.0 / prompt_ms, 1), "prefill_tokens": prompt_tokens}
    release_model(llm)
    return out


def time_e2e(llm, batch, steps, warmup, seed):
    """Decoded tokens per second through LLM.generate, host token lists in, host lists out: one call that
    generates warmup + steps + 1 tokens per prompt; the host clock is read as each step's tokens arrive, and the
    last `steps` decode steps count (the `warmup` steps before them are the warm-up, as for the device-timed
    figure).  Also returned: the rate of the first `steps` decode steps, which follow the prompt step into the
    power cap and run slower."""
    prompts = prompts_for(batch, llm.config.vocab_size, seed)
    stats = {}
    llm.generate(prompts, max_new_tokens=warmup + steps + 1, ignore_eos=True, stats=stats)
    stamps = stats["step_stamps"]  # [0]: the prompt step's tokens, [k]: decode step k's
    if len(stamps) < warmup + steps + 1:
        raise RuntimeError(f"the generation made {len(stamps) - 1} decode steps, {warmup + steps} were asked for")
    timed = stamps[warmup + steps] - stamps[warmup]
    first = stamps[steps] - stamps[0]
    return batch * steps / timed, batch * steps / first


def time_prefill(llm, tokens, reps, warmup, seed, pause=0.0):
    """Mean time of one prompt step of `tokens` tokens (CUDA events around the engine's step call,
    host planning included).  `pause` seconds of idling before each timed step make it an isolated
    step, as a request meets it; without pauses the steps run back to back under the power cap."""
    import numpy as np
    import torch
    from cpp_minilamma_b200 import StepEntry
    rng = np.random.RandomState(seed)
    prompt = [int(t) for t in rng.randint(0, llm.config.vocab_size, size=tokens)]
    times = []
    for i in range(warmup + reps):
        slot, = llm.engine.acquire(1)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        if pause and i >= warmup:
            time.sleep(pause)
        begin.record()
        llm.engine.step_borrowed([StepEntry(slot, prompt, [tokens - 1])])
        end.record()
        torch.cuda.synchronize()
        llm.engine.release(slot)
        if i >= warmup:
            times.append(begin.elapsed_time(end))
    return sum(times) / len(times)


def prefill_flops(cfg, tokens):
    d, hq, hk = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    per_layer = 2 * tokens * cfg.hidden_size * ((hq + 2 * hk) * d + hq * d) \
        + 2 * tokens * cfg.hidden_size * cfg.intermediate_size * 3 \
        + 2 * hq * tokens * tokens * d  # causal: half of 4 T^2 d per head
    return cfg.num_hidden_layers * per_layer + 2 * cfg.hidden_size * cfg.vocab_size  # head on one row


def profile_region(args):
    """One eager step inside cudaProfilerStart/Stop, after warm-up steps of the same kind."""
    import numpy as np
    import torch
    import cpp_minilamma_b200 as ml
    from cpp_minilamma_b200 import StepEntry
    cfg = shape_config(args.shape, args.layers or 4)
    context = max(SHAPES[args.shape]["context"], args.context + 64)  # room for a longer --context than the workload's
    llm = ml.random_model(cfg, seed=0, dtype="bfloat16", max_tokens=(args.batch + 1) * context, max_positions=context,
                          max_seqs=args.batch + 2, max_step_tokens=8192)
    rng = np.random.RandomState(0)
    engine = llm.engine
    draw = lambda n: [int(t) for t in rng.randint(0, cfg.vocab_size, size=n)]
    if args.profile == "decode":
        slots = engine.acquire(args.batch)
        engine.step_borrowed([StepEntry(s, draw(args.context), [args.context - 1]) for s in slots])
        for _ in range(2):
            engine.step_borrowed([StepEntry(s, [5], [0]) for s in slots])
        step = lambda: engine.step_borrowed([StepEntry(s, [7], [0]) for s in slots])
    else:
        prompt = draw(PREFILL_TOKENS)
        slot, = engine.acquire(1)
        engine.step_borrowed([StepEntry(slot, prompt, [PREFILL_TOKENS - 1])])
        engine.release(slot)
        slot, = engine.acquire(1)
        step = lambda: engine.step_borrowed([StepEntry(slot, prompt, [PREFILL_TOKENS - 1])])
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    step()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print(f"profiled one {args.profile} step: {args.shape}, {cfg.num_hidden_layers} layers, batch {args.batch}")
    return 0


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (named in config)")
    parser.add_argument("--skip-points", action="store_true", help="leave out batch 1 and 64 and the further workloads")
    parser.add_argument("--skip-check", action="store_true", help="leave out the comparison with a float32 run")
    parser.add_argument("--profile", choices=["decode", "prefill"], default=None,
                        help="run one step of that kind between cudaProfilerStart/Stop (for ncu "
                             "--profile-from-start off) on a small case and exit; use with --layers")
    parser.add_argument("--shape", choices=sorted(SHAPES), default="llama31_8b", help="model shape of the --profile step")
    parser.add_argument("--batch", type=int, default=BATCH, help="batch of the --profile decode step")
    parser.add_argument("--context", type=int, default=1024, help="prompt length of the --profile decode step")
    args = parser.parse_args()

    if args.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import reference_arm
        return reference_arm.main(args)
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not supported by this single-GPU library")
        return 2

    import torch
    import cpp_minilamma_b200 as ml
    if args.profile:
        return profile_region(args)
    sampler = ClockSampler()
    sampler.start()  # nvidia-smi needs a moment before its first line: it runs through the set-up
    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)
    peaks = load_peaks()
    checked = {"checked": False, "check": "skipped"} if args.skip_check else check_against_float32()
    cfg = llama31_8b(args.layers)
    budget = 64 * (PROMPT_RANGE[1] + warmup + steps + 64)  # room for the batch-64 point
    llm = ml.random_model(cfg, seed=0, dtype="bfloat16", max_tokens=max(budget, BATCH * CONTEXT),
                          max_positions=CONTEXT, max_seqs=64, max_step_tokens=4096)
    # The prefill is one short step.  "ms" is the mean of isolated steps (half a second apart), the
    # condition of the burst GEMM figure it is held against; "ms_hot" is the same step back to back
    # after the decode loops, under the power cap, held against the sustained figure.
    prefill_ms = time_prefill(llm, PREFILL_TOKENS, reps=5, warmup=3, seed=3, pause=0.5)
    # the timed loop of exactly `steps` steps is repeated (at least 5 times and for at least 0.6 s, as far as the
    # context allows) and the median repeat is reported
    first_ms, _, _, _, _ = time_decode(llm, BATCH, steps, warmup, seed=1)
    repeats = max(5, min(60, int(600.0 / (first_ms * steps)) + 1))
    ms, live_tokens, launches, all_ms, _ = time_decode(llm, BATCH, steps, warmup, seed=1, sampler=sampler, repeats=repeats)
    clocks = sampler.summary()
    sampler.stop()
    value = BATCH * 1000.0 / ms
    achieved = decode_bytes(llm, live_tokens) / (ms * 1e-3) / 1e9

    e2e_value, e2e_after_prompt = time_e2e(llm, BATCH, steps, warmup, seed=2)
    # what a replayed decode step copies to the device: the captured step's index arrays and the parts' own lists
    # (counted from the buffer the engine copies; block-table rows ride along when a page is crossed)
    captured = [cap for key, cap in llm.engine.shared_decode_graphs()._captured.items() if key[0] == BATCH and cap.graph is not None]
    meta_ints = captured[0].updates_at if captured else 11 * BATCH
    d2h_ints = 2 * llm.engine.shared_sampler().rows  # the sampler's token ids and status words

    prefill_hot_ms = time_prefill(llm, PREFILL_TOKENS, reps=5, warmup=1, seed=3)
    flops = prefill_flops(cfg, PREFILL_TOKENS)
    points, workloads = {}, {}
    if not args.skip_points:
        for b in (1, 64):
            p_ms, p_live, _, _, _ = time_decode(llm, b, max(steps // 2, 8), warmup, seed=10 + b, repeats=5)
            points[f"decode_b{b}"] = round(b * 1000.0 / p_ms, 1)
            points[f"decode_b{b}_hbm_frac"] = round(decode_bytes(llm, p_live) / (p_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)
    release_model(llm)
    if not args.skip_points:
        for name in ("llama2_7b", "llama32_1b"):
            workloads[name] = time_workload(name, peaks, warmup, layers=None)

    line = {
        "metric": "decode tok/s at batch 8 (Llama-3.1-8B shape, random bf16 weights)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic token ids, random-init weights", "impl": "ours",
        "config": {"model": "Llama-3.1-8B shape", "layers": cfg.num_hidden_layers, "layers_full": 32,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": BATCH, "seq_len": CONTEXT, "prompt_lens": "uniform[128,2048)",
                   "parallelism": "1 gpu", "l2": "inputs larger than L2 (15 GB of weights per step)",
                   "peaks": peaks["source"], "repeats": len(all_ms), "reported": "median repeat of `steps` steps"},
        "clocks": clocks,
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": 4 * meta_ints,
                "d2h_bytes_per_step": 4 * d2h_ints, "warmup_steps": warmup,
                "first_steps_after_prompt": round(e2e_after_prompt, 1)},
        "gpu_launches": int(round(launches * steps)),
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / prefill_ms, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4),
                    "ms_hot": round(prefill_hot_ms, 3),
                    "frac_hot": round(flops / (prefill_hot_ms * 1e-3) / (peaks["bf16_tflops_sustained"] * 1e12), 4),
                    "timing": "ms: 5 isolated steps 0.5 s apart; ms_hot: 5 steps back to back after the decode loops"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
        "workloads": workloads,
        "repeat_ms": [round(t, 4) for t in all_ms],
    }
    line.update(checked)
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
