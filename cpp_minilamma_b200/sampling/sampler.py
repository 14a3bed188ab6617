"""Sampling parameters and the device sampler.

`SamplingParams` mirrors the reference's `SamplerParmas` (include/sampler.h:7-15):
temperature 0 means greedy, top_k 0 means off, top_k 1 means greedy; values are checked
as in src/sampler.cc:20-29.  Unlike the reference, whose seed 0 draws from
std::random_device (src/sampler.cc:84-91), every seed is reproducible here: the uniform
number of a draw depends only on (seed, request index, index of the generated token).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Sequence

import torch

GREEDY_TEMPERATURE = 1e-6  # below this the reference falls back to greedy (src/sampler.cc:7,140)
MAX_TOP_K = 1024


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    seed: int = 1

    def validate(self, vocab_size: int) -> None:
        if not math.isfinite(self.temperature) or self.temperature < 0:
            raise ValueError(f"temperature must be finite and >= 0, got {self.temperature}")
        if self.top_k < 0:
            raise ValueError(f"top_k must be >= 0, got {self.top_k}")
        if not self.is_greedy and min(self.top_k, vocab_size) > MAX_TOP_K:
            raise ValueError(f"top_k {self.top_k} exceeds the device sampler's maximum of {MAX_TOP_K}")
        if self.seed < 0:
            raise ValueError(f"seed must be >= 0, got {self.seed}")

    @property
    def is_greedy(self) -> bool:
        return self.temperature < GREEDY_TEMPERATURE or self.top_k == 1


class DeviceSampler:
    """Samples one token per logits row on the device; only token ids and a status word
    per row cross to the host."""

    def __init__(self, device, max_rows: int = 64):
        self.device = device
        self._alloc(max_rows)

    def _alloc(self, rows: int) -> None:
        self.rows = rows
        self.out = torch.zeros(2 * rows, dtype=torch.int32, device=self.device)   # tokens | status
        self.counters = torch.zeros(2 * rows, dtype=torch.int32, device=self.device)  # request | step
        # two pinned copies and their events: the tokens of one step can be on their way to the
        # host while the next step, which overwrites `out`, is already enqueued
        self.hosts = [torch.zeros(2 * rows, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self.events = [torch.cuda.Event(), torch.cuda.Event()]
        self._turn = 0

    def launch(self, logits: torch.Tensor, params: SamplingParams, request: torch.Tensor, step: torch.Tensor) -> None:
        """Enqueue the sampling kernel for logits float32 [n, vocab]; `request` and `step`
        are int32 device tensors with the random-number counters of each row."""
        from ..csrc import kernels as K
        n = logits.shape[0]
        if n > self.rows:
            raise ValueError(f"sampler sized for {self.rows} rows, got {n}")
        tokens, status = self.out[:n], self.out[self.rows:self.rows + n]
        if params.is_greedy:
            K.argmax(logits, tokens, status)
        else:
            K.sample(logits, params.temperature, min(params.top_k, logits.shape[1]), params.seed, request, step,
                     tokens, status)

    def ticket(self, n: int):
        """Enqueue the copy of the n token ids just sampled to the host; `collect` waits for it.
        At most two tickets may be outstanding."""
        turn = self._turn
        self._turn ^= 1
        self.hosts[turn].copy_(self.out, non_blocking=True)
        self.events[turn].record()
        return (turn, n, self.rows)

    def collect(self, ticket) -> List[int]:
        """The token ids of a ticket (waits for that step, not for later ones)."""
        turn, n, rows = ticket
        self.events[turn].synchronize()
        host = self.hosts[turn]
        status = host[rows:rows + n]
        # row 0's word also carries, in bits 8 and up, the error flags of kernels that gave up during the step
        gave_up = int(status[0]) >> 8
        if gave_up:
            from ..csrc.kernels import DeviceKernelError, device_error_message
            raise DeviceKernelError(device_error_message(gave_up))
        if int((status & 0xFF).max()) != 0:
            raise FloatingPointError("logits are not finite")  # src/sampler.cc:10-19
        return host[:n].tolist()

    def fetch(self, n: int) -> List[int]:
        """Bring the n sampled token ids to the host (waits for the step)."""
        return self.collect(self.ticket(n))

    def sample(self, logits: torch.Tensor, params: SamplingParams, requests: Sequence[int],
               steps: Sequence[int]) -> List[int]:
        """logits float32 [n, vocab] -> n token ids on the host (this call synchronises)."""
        return self.collect(self.sample_ticket(logits, params, requests, steps))

    def sample_ticket(self, logits: torch.Tensor, params: SamplingParams, requests: Sequence[int],
                      steps: Sequence[int], on_device=None):
        """As `sample`, but returns a ticket for `collect` instead of waiting.  `on_device`: the same
        counters as int32 device tensors (request, step), when the caller has brought them over already."""
        n = logits.shape[0]
        if n > self.rows:
            self._alloc(max(n, 2 * self.rows))
        if on_device is not None and not params.is_greedy:
            self.launch(logits, params, on_device[0], on_device[1])
            return self.ticket(n)
        if not params.is_greedy:
            self.counters[:n].copy_(torch.tensor(list(requests), dtype=torch.int32))
            self.counters[self.rows:self.rows + n].copy_(torch.tensor(list(steps), dtype=torch.int32))
        self.launch(logits, params, self.counters[:n], self.counters[self.rows:self.rows + n])
        return self.ticket(n)
