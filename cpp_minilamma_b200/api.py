"""The Python entry point: load a model folder (or make random weights) and generate.

    import cpp_minilamma_b200 as ml
    llm = ml.load("/path/to/model", dtype="bfloat16", max_tokens=8192)
    outputs = llm.generate([[1, 5, 9], [1, 7]], max_new_tokens=16)          # lists of token ids
    outputs = llm.generate(prompts, max_new_tokens=16, temperature=0.8, top_k=40, seed=1)

The reference has no Python API (its scripts spawn the `mini-llama` binary); option names
follow its CLI and sampler: `n_predict` is accepted as an alias of `max_new_tokens`
(app/backend_cli.cc:96), `temperature`, `top_k`, `seed` are the fields of its
`SamplerParmas` (include/sampler.h:7-15).
"""
from __future__ import annotations

from pathlib import Path
from typing import List, Optional, Sequence

import torch

from . import models  # noqa: F401  (registers architectures)
from .config.base import ModelConfig, load_config, lookup_architecture
from .engine.generate import Backend, Completion, generate
from .engine.model import Model
from .engine.step import Engine, StepEntry
from .sampling.sampler import DeviceSampler, SamplingParams
from .weights.loader import load_tensors
from .weights.random_init import random_tensors

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    if dtype not in _DTYPES:
        raise ValueError(f"dtype {dtype!r} not supported (bfloat16 or float32)")
    return _DTYPES[dtype]


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError("cpp_minilamma_b200 runs on a CUDA device only (there is no CPU path); "
                           f"asked for {device}, cuda available: {torch.cuda.is_available()}")
    return device


class EngineBackend(Backend):
    """Connects the generation loop to an engine and a device sampler.  Steps in which
    every sequence brings one token run through captured CUDA graphs."""

    def __init__(self, engine: Engine, params: SamplingParams, use_graphs: bool = True):
        self.engine = engine
        self.params = params
        self.n_slots = engine.cache.n_slots
        self.n_pages = engine.cache.n_pages
        self.max_positions = engine.model.max_positions
        self.sampler = engine.shared_sampler()
        self.graphs = engine.shared_decode_graphs() if use_graphs and engine.model.capturable() else None
        self.steps = 0

    def acquire(self, count):
        return self.engine.acquire(count)

    def release(self, slot):
        self.engine.release(slot)

    def step_and_sample(self, entries, requests, steps):
        return self.collect(self.submit(entries, requests, steps))

    def submit(self, entries, requests, steps):
        """Enqueue a step and its sampling; `collect` brings the token ids to the host."""
        self.steps += 1
        self._rows = {e.slot: i for i, e in enumerate(entries)}  # where each slot's sampled token will lie
        if self.graphs is not None and all(len(e.tokens) == 1 for e in entries):
            return self.graphs.submit([e.slot for e in entries], [e.tokens[0] for e in entries], self.params,
                                      requests, steps)
        if self.params.is_greedy:
            return self.sampler.sample_ticket(self.engine.step_borrowed(entries), self.params, requests, steps)
        # the sampler's random-number counters cross to the device with the step's index arrays
        logits = self.engine.step_borrowed(entries, extras={"rng_request": requests, "rng_step": steps})
        return self.sampler.sample_ticket(logits, self.params, requests, steps,
                                          on_device=(self.engine.extras["rng_request"], self.engine.extras["rng_step"]))

    def submit_ahead(self, slots, requests, steps):
        """Enqueue one more token for `slots`, all of which the previous `submit` or `submit_ahead` must
        have had (it may have had more: sequences that end with it): that step's sampled tokens are taken
        on the device, before the host has collected them.  Returns None when this backend cannot run
        ahead (no captured decode)."""
        if self.graphs is None:
            return None
        rows = getattr(self, "_rows", {})
        if any(s not in rows for s in slots):
            raise ValueError("submit_ahead: a slot that the step before did not have")
        source_rows = [rows[s] for s in slots]
        self.steps += 1
        self._rows = {s: i for i, s in enumerate(slots)}
        return self.graphs.submit(list(slots), None, self.params, requests, steps, source_rows=source_rows)

    def collect(self, ticket):
        from .csrc.kernels import DeviceKernelError
        try:
            return self.sampler.collect(ticket)
        except DeviceKernelError:
            self.engine.after_device_error()
            raise


class LLM:
    def __init__(self, config: ModelConfig, model: Model, max_tokens: int, max_seqs: Optional[int] = None,
                 max_step_tokens: int = 8192):
        self.config = config
        self.model = model
        self.engine = Engine(model, max_tokens, max_seqs, max_step_tokens)

    @property
    def stop_token_ids(self) -> List[int]:
        return list(self.model.spec.stop_token_ids)

    def generate_detailed(self, prompts: Sequence[Sequence[int]], max_new_tokens=None, temperature: float = 0.0,
                          top_k: int = 0, seed: int = 1, stop_ids: Optional[Sequence[int]] = None,
                          ignore_eos: bool = False, max_batch: Optional[int] = None, clip: bool = False,
                          n_predict=None, stats: Optional[dict] = None) -> List[Completion]:
        if max_new_tokens is None:
            max_new_tokens = 4 if n_predict is None else n_predict  # the reference CLI's default of 4
        params = SamplingParams(float(temperature), int(top_k), int(seed))
        params.validate(self.model.spec.vocab_size)
        stops = set(self.stop_token_ids) | set(stop_ids or ())
        backend = EngineBackend(self.engine, params)
        return generate(backend, prompts, max_new_tokens, stops, ignore_eos, max_batch, clip, stats)

    def generate(self, prompts: Sequence[Sequence[int]], **options) -> List[List[int]]:
        """Token ids generated for each prompt (stop tokens are not included)."""
        return [c.tokens for c in self.generate_detailed(prompts, **options)]

    def step(self, entries: Sequence[StepEntry]):
        return self.engine.step(entries)


def build_model(config: ModelConfig, dtype, device, max_positions: Optional[int] = None) -> Model:
    _, builder = lookup_architecture(config.architecture)
    return Model(builder(config), parse_dtype(dtype), device, max_positions)


def load(folder, dtype="bfloat16", device="cuda:0", max_tokens: int = 16384, max_seqs: Optional[int] = None,
         max_positions: Optional[int] = None, max_step_tokens: int = 8192) -> LLM:
    """Load `config.json` + safetensors from `folder`; the model class is chosen by
    `architectures` in config.json."""
    device = require_cuda(device)
    config = load_config(folder)
    model = build_model(config, dtype, device, max_positions)
    model.bind(load_tensors(Path(folder), model.weight_specs(), parse_dtype(dtype), device))
    return LLM(config, model, max_tokens, max_seqs, max_step_tokens)


def random_model(config: ModelConfig, seed: int = 0, dtype="bfloat16", device="cuda:0", max_tokens: int = 16384,
                 max_seqs: Optional[int] = None, max_positions: Optional[int] = None, matrix_std: float = 0.02,
                 norm_std: float = 0.0, max_step_tokens: int = 8192, stored_as=None) -> LLM:
    """A model with seeded random weights drawn on the device (no files).  `stored_as`: the dtype a folder
    would store the matrices in; they are rounded to it before they take the run's dtype, so that a
    float32 run with stored_as="bfloat16" holds the very values of a bfloat16 run of the same seed."""
    device = require_cuda(device)
    run_dtype = parse_dtype(dtype)
    stored = parse_dtype(stored_as) if stored_as is not None else run_dtype
    model = build_model(config, run_dtype, device, max_positions)
    tensors = {}
    specs = model.weight_specs()
    for index, spec in enumerate(specs):  # one at a time: the float32 draft of a tensor is freed before the next
        drawn = random_tensors([spec], seed * 4099 + index, torch.float32, device, matrix_std, norm_std)[spec.name]
        tensors[spec.name] = drawn.to(torch.float32) if spec.kind == "vector" else drawn.to(stored).to(run_dtype)
    model.bind(tensors)
    return LLM(config, model, max_tokens, max_seqs, max_step_tokens)
