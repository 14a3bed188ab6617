"""Decode steps as CUDA graphs.

A decode step launches a few hundred small kernels; launched one by one from Python the
host, not the GPU, sets the pace.  `DecodeGraphs` captures the whole step - every layer,
the final norm, the head and the sampling kernel - once per (batch size, sampling
parameters) and replays it.  What changes from step to step (token ids, positions, slots,
context lengths, random-number counters) lives in one small int32 buffer at a fixed
address that is refreshed with a single host-to-device copy before each replay; block
tables are updated by the cache outside the graph.  The first step of a new batch size
runs eagerly (it also sizes the workspace); the second one is captured.

The reference launches every kernel separately, allocates its output and synchronises
several times per layer (src/forward.cc:337-383, src/cuda_attention.cu:21-24).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..sampling.sampler import DeviceSampler, SamplingParams
from .step import Engine, StepState

_FIELDS = 10  # tokens, tok_pos, tok_seq, seq_slot, seq_ctx, seq_qstart, seq_qlen, want, rng request, rng step


class _Captured:
    def __init__(self, engine: Engine, batch: int):
        self.batch = batch
        self.host = torch.zeros(_FIELDS * batch, dtype=torch.int32, pin_memory=True)
        self.dev = torch.zeros(_FIELDS * batch, dtype=torch.int32, device=engine.device)
        self.copied = torch.cuda.Event()
        self.graph = None
        self.failures = 0  # captures that did not go through (the step then ran eagerly)
        self.launches = 0
        h = self.host.numpy().reshape(_FIELDS, batch)
        h[2] = np.arange(batch)   # sequence of each token
        h[5] = np.arange(batch)   # first query row of each sequence
        h[6] = 1                  # one query token per sequence
        h[7] = np.arange(batch)   # the logits of every row are wanted
        self.fields = h
        d = self.dev.view(_FIELDS, batch)
        self.state = StepState(
            ws=engine.ws, n_tokens=batch, n_seqs=batch, tokens=d[0], tok_pos=d[1], tok_seq=d[2], seq_slot=d[3],
            seq_ctx=d[4], seq_qstart=d[5], seq_qlen=d[6], tile_seq=d[5][:0], tile_row0=d[5][:0], n_tiles=0,
            want_rows=d[7], all_decode=True, max_ctx=engine.model.max_positions, small_rows=engine.small_rows)
        self.rng_request, self.rng_step = d[8], d[9]


class DecodeGraphs:
    def __init__(self, engine: Engine, sampler: DeviceSampler):
        self.engine = engine
        self.sampler = sampler
        self._captured: Dict[Tuple, _Captured] = {}
        self._generation = engine.ws.generation
        self.replays = 0

    def _splits(self, batch: int) -> int:
        """One split count for all attention layers of a captured step: chosen from the batch
        size alone, since the graph must serve every context length."""
        best = 1
        for layer in self.engine.model.layers:
            chooser = getattr(layer.mixer, "decode_splits", None)
            if chooser is not None:
                best = max(best, chooser(batch, self.engine.model.max_positions))
        return best

    def step(self, slots: Sequence[int], tokens: Sequence[int], params: SamplingParams,
             requests: Sequence[int], steps: Sequence[int]) -> List[int]:
        """One token for each slot, brought to the host (waits for the step)."""
        return self.sampler.collect(self.submit(slots, tokens, params, requests, steps))

    def submit(self, slots: Sequence[int], tokens: Optional[Sequence[int]], params: SamplingParams,
               requests: Sequence[int], steps: Sequence[int]):
        """Enqueue one token for each slot: reserve, refresh the index buffer, run (eagerly the
        first time, then from the graph), sample; returns the sampler's ticket for the token ids.

        `tokens` None: the inputs are the tokens that the previous step sampled for the same
        slots in the same order; they are taken on the device, so the host can enqueue this
        step before it has seen them."""
        from ..csrc import kernels as K
        engine = self.engine
        batch = len(slots)
        vocab = engine.vocab_size
        for t in tokens or ():
            if not 0 <= t < vocab:
                raise ValueError(f"token {t} outside the vocabulary [0, {vocab})")
        starts = [engine.cache.seq_len[s] for s in slots]
        engine.cache.reserve([(s, 1) for s in slots])
        engine.cache.flush()
        if self._generation != engine.ws.generation:  # a workspace buffer moved: old graphs point at freed memory
            self._captured.clear()
            self._generation = engine.ws.generation
        key = (batch, params.is_greedy, params.temperature, params.top_k, params.seed)
        cap = self._captured.get(key)
        fresh = cap is None
        if fresh:
            cap = self._captured[key] = _Captured(engine, batch)
            cap.state.decode_splits = self._splits(batch)
        else:
            cap.copied.synchronize()  # the previous replay's copy has read the pinned buffer
        f = cap.fields
        f[0], f[1], f[3] = (tokens if tokens is not None else 0), starts, slots
        f[4] = np.asarray(starts, dtype=np.int32) + 1
        f[8], f[9] = requests, steps
        cap.dev.copy_(cap.host, non_blocking=True)
        cap.copied.record()
        if tokens is None:
            cap.state.tokens.copy_(self.sampler.out[:batch])  # device to device, after the index buffer's copy
        if cap.graph is None and not fresh and cap.failures < 3:
            before = K.launches
            graph = torch.cuda.CUDAGraph()
            try:
                # relaxed: a driver call made elsewhere in the process while this stream captures
                # (a tensor or an older graph being released, a lazily loaded module) must not
                # invalidate the capture
                with torch.cuda.graph(graph, capture_error_mode="relaxed"):
                    self._body(cap, params)
            except Exception:
                # the capture ran nothing: do this step eagerly and try again on a later one
                cap.failures += 1
                K.launches = before
                torch.cuda.synchronize()
                self._body(cap, params)
                return self.sampler.ticket(batch)
            cap.launches = K.launches - before
            K.launches = before
            if self._generation != engine.ws.generation:
                # the capture itself grew the workspace: its addresses are stale, run eagerly and try again later
                self._generation = engine.ws.generation
                self._captured.pop(key, None)
                self._body(cap, params)
                return self.sampler.ticket(batch)
            cap.graph = graph
        if cap.graph is not None:
            cap.graph.replay()
            K.launches += cap.launches
            self.replays += 1
        else:
            self._body(cap, params)
            if self._generation != engine.ws.generation:
                self._generation = engine.ws.generation
        return self.sampler.ticket(batch)

    def _body(self, cap: _Captured, params: SamplingParams) -> None:
        logits = self.engine.model.forward(cap.state, self.engine.cache, cap.state.tokens, cap.state.want_rows)
        self.sampler.launch(logits, params, cap.rng_request, cap.rng_step)
