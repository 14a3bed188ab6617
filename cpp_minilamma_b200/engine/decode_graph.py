"""Decode steps as CUDA graphs.

A decode step launches a few hundred small kernels; launched one by one from Python the
host, not the GPU, sets the pace.  `DecodeGraphs` captures the whole step - every layer,
the final norm, the head and the sampling kernel - once per (batch size, sampling
parameters, kind of step that a part may name) and replays it; above 16 sequences the batch
size is rounded up and the spare rows run in the cache's padding slot.  What changes from step to step (token ids, positions, slots,
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

from ..parts.base import StepShape
from ..sampling.sampler import DeviceSampler, SamplingParams
from .step import Engine, StepState

_FIELDS = 11  # tokens, tok_pos, tok_seq, seq_slot, seq_ctx, seq_qstart, seq_qlen, want, rng request, rng step, source row


def decode_bucket(batch: int) -> int:
    """The batch size a decode step of `batch` sequences is captured and replayed at.  Up to 16 its own (the
    kernels differ from row to row there); beyond, the next multiple of 8 (to 64), 16 (to 128) or 32, the spare
    rows filled with the cache's padding slot.  A batch whose sequences end one after the other then replays a
    handful of graphs instead of capturing one for every size on its way down: 64 requests that end three steps
    apart took 3.3 ms a step the first time and 1.95 ms later, against 1.33 ms for a batch that stays whole."""
    if batch <= 16:
        return batch
    unit = 8 if batch <= 64 else 16 if batch <= 128 else 32
    return -(-batch // unit) * unit


class _Captured:
    """The fixed-address buffers of one captured step: the ten index arrays of `batch` integers each, then
    the index arrays that parts prepare for decode steps (sizes fixed by the batch size), then room for the
    block-table rows that changed.  One copy from pinned memory refreshes the part that is in use."""

    def __init__(self, engine: Engine, batch: int, shape: StepShape):
        self.batch = batch
        # parts' own index arrays: laid out once from what they prepare for this first step
        self.meta_layout = []  # (key, part, name, offset, count)
        at = _FIELDS * batch
        for key, part in engine.providers.items():
            for name, values in part.prepare_step(shape).items():
                count = len(values)
                self.meta_layout.append((key, part, name, at, count))
                at += count
        self.updates_at = at
        size = at + engine.cache.table_update_capacity(batch)
        self.host = torch.zeros(size, dtype=torch.int32, pin_memory=True)
        self.dev = torch.zeros(size, dtype=torch.int32, device=engine.device)
        self.copied = torch.cuda.Event()
        self.graph = None
        self.generation = -1  # the workspace's generation when the graph was captured
        self.failures = 0  # captures that did not go through (the step then ran eagerly)
        self.launches = 0
        h = self.host.numpy()[:_FIELDS * batch].reshape(_FIELDS, batch)
        h[2] = np.arange(batch)   # sequence of each token
        h[5] = np.arange(batch)   # first query row of each sequence
        h[6] = 1                  # one query token per sequence
        h[7] = np.arange(batch)   # the logits of every row are wanted
        self.fields = h
        d = self.dev[:_FIELDS * batch].view(_FIELDS, batch)
        self.state = StepState(
            ws=engine.ws, n_tokens=batch, n_seqs=batch, tokens=d[0], tok_pos=d[1], tok_seq=d[2], seq_slot=d[3],
            seq_ctx=d[4], seq_qstart=d[5], seq_qlen=d[6], want_rows=d[7], all_decode=True,
            max_ctx=engine.model.max_positions, small_rows=engine.small_rows, shape=shape)
        for key, _, name, offset, count in self.meta_layout:
            self.state.meta.setdefault(key, {})[name] = self.dev[offset:offset + count]
        for part in engine.model.all_parts():
            fixed = part.capture_parameters(batch, engine.model.max_positions)
            if fixed:
                self.state.fixed[part] = fixed
        self.rng_request, self.rng_step = d[8], d[9]
        self.source_rows = d[10]  # for a step fed on the device: the row of the previous step that sampled each input

    def refresh_meta(self, shape: StepShape) -> None:
        """The parts' index arrays for this step, into their fixed places."""
        h = self.host.numpy()
        prepared = {}
        for key, part, name, offset, count in self.meta_layout:
            if key not in prepared:
                prepared[key] = part.prepare_step(shape)
            values = prepared[key].get(name, ())
            if len(values) != count:
                raise RuntimeError(f"{type(part).__name__}: index array {name!r} has {len(values)} entries in this "
                                   f"decode step and had {count} in the first one; decode steps are replayed from a "
                                   "graph and need index arrays whose sizes follow from the batch size alone")
            h[offset:offset + count] = values


class DecodeGraphs:
    def __init__(self, engine: Engine, sampler: DeviceSampler):
        self.engine = engine
        self.sampler = sampler
        self._captured: Dict[Tuple, _Captured] = {}
        self._generation = engine.ws.generation
        self.replays = 0

    def drop(self) -> None:
        """Forget every captured graph (they are captured again on later steps)."""
        self._captured.clear()

    def step(self, slots: Sequence[int], tokens: Sequence[int], params: SamplingParams,
             requests: Sequence[int], steps: Sequence[int]) -> List[int]:
        """One token for each slot, brought to the host (waits for the step)."""
        return self.sampler.collect(self.submit(slots, tokens, params, requests, steps))

    def submit(self, slots: Sequence[int], tokens: Optional[Sequence[int]], params: SamplingParams,
               requests: Sequence[int], steps: Sequence[int], source_rows: Optional[Sequence[int]] = None):
        """Enqueue one token for each slot: reserve, refresh the index buffer, run (eagerly the
        first time, then from the graph), sample; returns the sampler's ticket for the token ids.

        `tokens` None: the inputs are the tokens that the previous step sampled; slot i takes the one of
        that step's row `source_rows[i]` (default: row i).  They are taken on the device, so the host can
        enqueue this step before it has seen them."""
        from ..csrc import kernels as K
        engine = self.engine
        n_live = len(slots)
        vocab = engine.vocab_size
        for t in tokens or ():
            if not 0 <= t < vocab:
                raise ValueError(f"token {t} outside the vocabulary [0, {vocab})")
        if tokens is None:
            if source_rows is None:
                source_rows = list(range(n_live))
            if len(source_rows) != n_live or any(not 0 <= r < self.sampler.rows for r in source_rows):
                raise ValueError("a step fed on the device needs, for each slot, the row of the previous step that sampled its token")
            source_rows = list(source_rows)
        starts = [engine.cache.seq_len[s] for s in slots]
        engine.cache.reserve([(s, 1) for s in slots])
        updates = engine.cache.take_table_updates()
        self._forget_stale_graphs()  # a prompt step or another engine call may have moved a workspace buffer
        # the step runs at a rounded-up batch size; its spare rows are one-token sequences in the padding slot
        batch = decode_bucket(n_live)
        if batch > self.sampler.rows:
            batch = n_live
        spare = batch - n_live
        slots = list(slots) + [engine.cache.pad_slot] * spare
        starts = starts + [0] * spare
        requests = list(requests) + [0] * spare
        steps = list(steps) + [0] * spare
        if tokens is not None:
            tokens = list(tokens) + [0] * spare
        shape = StepShape(list(slots), starts, [1] * batch)
        # parts that launch differently for different kinds of steps (a batch with one very long sequence, say)
        # have a captured step for each kind
        variants = tuple(part.step_variant(shape) for part in engine.providers.values())
        key = (batch, params.is_greedy, params.temperature, params.top_k, params.seed, variants)
        cap = self._captured.get(key)
        fresh = cap is None
        if fresh:
            cap = self._captured[key] = _Captured(engine, batch, shape)
        else:
            cap.copied.synchronize()  # the previous replay's copy has read the pinned buffer
        cap.state.shape = shape
        f = cap.fields
        f[0], f[1], f[3] = (tokens if tokens is not None else 0), starts, slots
        f[4] = np.asarray(starts, dtype=np.int32) + 1
        f[8], f[9] = requests, steps
        if source_rows is not None:
            f[10] = source_rows + [0] * spare
        if cap.meta_layout:
            cap.refresh_meta(shape)
        used = cap.updates_at
        staged = []
        h = cap.host.numpy()
        for group, rows in updates:  # block-table rows that changed: behind the index arrays, in the same copy
            if used + rows.size > h.shape[0]:
                # more rows than this batch can have changed itself (left over from a step that never ran):
                # bring them over one by one
                for row in rows:
                    group.table_dev[int(row[0])].copy_(torch.from_numpy(row[1:].copy()))
                continue
            h[used:used + rows.size] = rows.reshape(-1)
            staged.append((group, cap.dev[used:used + rows.size], rows.shape[0]))
            used += rows.size
        cap.dev[:used].copy_(cap.host[:used], non_blocking=True)
        cap.copied.record()
        for group, region, n_rows in staged:
            K.scatter_rows(group.table_dev, region, n_rows)
        if tokens is None:  # on the device, after the index buffer's copy: the previous step's tokens in this step's order
            K.gather_int32(cap.state.tokens, self.sampler.out[:self.sampler.rows], cap.source_rows, batch)
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
                return self.sampler.ticket(n_live)
            cap.launches = K.launches - before
            K.launches = before
            if self._forget_stale_graphs():
                # the capture itself grew the workspace: its addresses are stale (and so are those of every
                # other batch size's graph), run eagerly and try again later
                self._body(cap, params)
                self._forget_stale_graphs()
                return self.sampler.ticket(n_live)
            cap.graph = graph
            cap.generation = engine.ws.generation
        if cap.graph is not None:
            if cap.generation != engine.ws.generation:
                raise RuntimeError("decode graphs: a captured step outlived the workspace buffers it was captured with")
            cap.graph.replay()
            K.launches += cap.launches
            self.replays += 1
        else:
            self._body(cap, params)
            # an eager step of a new batch size may have grown buffers that the graphs of other batch sizes
            # were captured with; this one has no graph yet and keeps its index buffers
            self._forget_stale_graphs(keep=key)
        return self.sampler.ticket(n_live)

    def _forget_stale_graphs(self, keep=None) -> bool:
        """Drop every captured step if a workspace buffer has moved since the last look (a graph replays the
        addresses it was captured with, and the old buffer is freed); True if one had.  `keep`: a key whose
        entry has no graph yet and stays."""
        if self._generation == self.engine.ws.generation:
            return False
        self._generation = self.engine.ws.generation
        kept = self._captured.get(keep) if keep is not None else None
        self._captured.clear()
        if kept is not None and kept.graph is None:
            self._captured[keep] = kept
        return True

    def _body(self, cap: _Captured, params: SamplingParams) -> None:
        logits = self.engine.model.forward(cap.state, self.engine.cache, cap.state.tokens, cap.state.want_rows)
        self.sampler.launch(logits, params, cap.rng_request, cap.rng_step)
