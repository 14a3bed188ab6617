"""The step function: a batch of sequences, the tokens each brings, logits where wanted.

`Engine.step(entries)` runs only the tokens it is given, as one batch, from the cache
that earlier steps left: each entry names a slot, its next tokens (a whole prompt or one
decoded token - lengths may differ) and the places among those tokens whose logits are
wanted.  A sequence's tokens start at its cached length.  The reference's counterpart is
`ForwardBatch(model, context, batch)` for one sequence, which loops single-token
forwards and keeps only the last logits (src/forward.cc:473-488); its checks before any
work (token range, position range: :434-450) are made here on the host for the whole
batch, so that no kernel is launched on a bad argument.

All per-step index arrays (token ids, positions, sequence of each token, slots, context
lengths, attention tiles, wanted rows) are packed into one int32 buffer that crosses to
the device in one copy.  Activations live in a workspace that is reused from layer to
layer and from step to step.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.paged import PAGE, CacheError, SequenceCache
from .model import Model

ATTN_TILE = 64  # query rows per prefill attention tile


class StepError(ValueError):
    """A step that cannot run: unknown slot, token outside the vocabulary, bad `want`."""


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


class Workspace:
    """Named device buffers that persist between steps.  A request larger than the
    buffer's capacity reallocates it and bumps `generation` (captured graphs that used
    the old address must be dropped)."""

    def __init__(self, device):
        self.device = device
        self._flat: Dict[str, torch.Tensor] = {}
        self.generation = 0

    def buffer(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        count = 1
        for dim in shape:
            count *= dim
        flat = self._flat.get(name)
        if flat is None or flat.dtype != dtype or flat.numel() < count:
            flat = torch.empty(max(count, 1), dtype=dtype, device=self.device)
            self._flat[name] = flat
            self.generation += 1
        return flat[:count].view(shape)

    def zeros(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        """As `buffer`, but zero-filled when it is (re)allocated - for counters that the
        kernels using them leave at zero."""
        count = 1
        for dim in shape:
            count *= dim
        flat = self._flat.get(name)
        if flat is None or flat.dtype != dtype or flat.numel() < count:
            self._flat[name] = torch.zeros(max(count, 64), dtype=dtype, device=self.device)
            self.generation += 1
        return self._flat[name][:count].view(shape)

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._flat.values())


@dataclass
class StepState:
    """Everything the parts see of a step (device tensors are int32 views of one buffer)."""

    ws: Workspace
    n_tokens: int
    n_seqs: int
    tokens: torch.Tensor
    tok_pos: torch.Tensor
    tok_seq: torch.Tensor
    seq_slot: torch.Tensor
    seq_ctx: torch.Tensor
    seq_qstart: torch.Tensor
    seq_qlen: torch.Tensor
    tile_seq: torch.Tensor
    tile_row0: torch.Tensor
    n_tiles: int
    want_rows: Optional[torch.Tensor]
    all_decode: bool
    max_ctx: int
    decode_splits: int = 0                      # fixed split count (graph replay), 0 = choose per step
    small_rows: int = 0                         # steps with at most this many rows use the weight-streaming product
    host: Dict[str, list] = field(default_factory=dict)  # host copies for parts written in Python


@dataclass
class _ChunkSeq:
    slot: int
    tokens: Sequence[int]
    start: int                 # position of the first token
    want: List[Tuple[int, int]]  # (row within this sequence's chunk tokens, output row)


class Engine:
    """A model, its cache and workspace on one device.

    max_tokens       the most tokens live sequences hold together (each rounded up to a page)
    max_seqs         number of slots (default: as many as pages, at most 4096)
    max_step_tokens  longer steps are cut into chunks of at most this many tokens
    """

    def __init__(self, model: Model, max_tokens: int, max_seqs: Optional[int] = None,
                 max_step_tokens: int = 8192):
        if not model.bound:
            raise RuntimeError("Engine: bind weights to the model first")
        self.model = model
        self.device = model.device
        self.act_dtype = model.act_dtype
        n_pages = (max_tokens + PAGE - 1) // PAGE
        self.cache = SequenceCache(model.cache_needs(), max_tokens,
                                   max_seqs if max_seqs is not None else min(n_pages, 4096),
                                   model.max_positions, model.act_dtype, self.device)
        self.ws = Workspace(self.device)
        self.max_step_tokens = max(int(max_step_tokens), ATTN_TILE)
        self.vocab_size = model.spec.vocab_size
        self._meta_host: Optional[torch.Tensor] = None
        self._meta_dev: Optional[torch.Tensor] = None
        self._meta_copied = None
        self.small_rows = 64  # rows up to which linears may use this package's weight-streaming kernels
        self.launch_count = 0  # kernels of this package launched (estimate kept by the parts' callers)

    # ---- helpers shared by everything that generates with this engine -------------------- #
    def shared_sampler(self):
        if getattr(self, "_sampler", None) is None:
            from ..sampling.sampler import DeviceSampler
            self._sampler = DeviceSampler(self.device, max(self.cache.n_slots, 64))
        return self._sampler

    def shared_decode_graphs(self):
        if getattr(self, "_graphs", None) is None:
            from .decode_graph import DecodeGraphs
            self._graphs = DecodeGraphs(self, self.shared_sampler())
        return self._graphs

    # ---- slots ---------------------------------------------------------------- #
    def acquire(self, count: int = 1) -> List[int]:
        return self.cache.acquire(count)

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    # ---- the step ---------------------------------------------------------------- #
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run the entries' tokens; return float32 logits [n_wanted, vocab] in the order of
        the entries and of each entry's `want`, or None when nothing is wanted.  The
        result is the caller's own tensor."""
        borrowed = self.step_borrowed(entries)
        return None if borrowed is None else borrowed.clone()

    def step_borrowed(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """As `step`, but the result may alias workspace memory that the next step overwrites."""
        chunks, n_want = self._plan(entries)
        out: Optional[torch.Tensor] = None
        if n_want and len(chunks) > 1:
            out = torch.empty((n_want, self.vocab_size), dtype=torch.float32, device=self.device)
        result = None
        for chunk in chunks:
            logits, out_rows = self._run_chunk(chunk)
            if logits is None:
                continue
            if len(chunks) == 1 and out_rows == list(range(n_want)):
                result = logits
            else:
                if out is None:
                    out = torch.empty((n_want, self.vocab_size), dtype=torch.float32, device=self.device)
                index = torch.tensor(out_rows, dtype=torch.long, device=self.device)
                out.index_copy_(0, index, logits)
                result = out
        return result

    # ---- planning (host only) ------------------------------------------------------ #
    def _plan(self, entries: Sequence[StepEntry]):
        if not entries:
            raise StepError("a step needs at least one entry")
        growth = []
        vocab = self.vocab_size
        for e in entries:
            n = len(e.tokens)
            if n < 1:
                raise StepError(f"slot {e.slot}: a step must bring at least one token")
            lo, hi = min(e.tokens), max(e.tokens)
            if lo < 0 or hi >= vocab:
                raise StepError(f"slot {e.slot}: token {lo if lo < 0 else hi} outside the vocabulary [0, {vocab})")
            for w in e.want:
                if not 0 <= w < n:
                    raise StepError(f"slot {e.slot}: wanted place {w} outside the {n} tokens of this step")
            growth.append((e.slot, n))
        starts = {}
        for slot, _ in growth:
            if not self.cache.is_live(slot):
                raise StepError(f"slot {slot} is not live")
            starts[slot] = self.cache.seq_len[slot]
        try:
            self.cache.reserve(growth)  # all or nothing; raises CacheFull / CacheError
        except CacheError:
            raise
        self.cache.flush()

        chunks: List[List[_ChunkSeq]] = [[]]
        room = self.max_step_tokens
        out_row = 0
        for e in entries:
            n = len(e.tokens)
            wants_by_place: Dict[int, List[int]] = {}
            for w in e.want:
                wants_by_place.setdefault(w, []).append(out_row)
                out_row += 1
            done = 0
            while done < n:
                if room == 0:
                    chunks.append([])
                    room = self.max_step_tokens
                take = min(room, n - done)
                want = [(place - done, row) for place in range(done, done + take)
                        for row in wants_by_place.get(place, [])] if wants_by_place else []
                chunks[-1].append(_ChunkSeq(e.slot, e.tokens[done:done + take], starts[e.slot] + done, want))
                done += take
                room -= take
        return chunks, out_row

    # ---- one chunk ------------------------------------------------------------------- #
    def _meta(self, n_ints: int):
        if self._meta_host is None or self._meta_host.numel() < n_ints:
            size = max(n_ints, 4096)
            pin = self.device.type == "cuda"
            self._meta_host = torch.empty(size, dtype=torch.int32, pin_memory=pin)
            self._meta_dev = torch.empty(size, dtype=torch.int32, device=self.device)
            self._meta_copied = torch.cuda.Event() if pin else None
        elif self._meta_copied is not None:
            # the previous step's copy may still be reading the pinned buffer
            self._meta_copied.synchronize()
        return self._meta_host, self._meta_dev

    def build_state(self, seqs: Sequence[_ChunkSeq], decode_splits: int = 0) -> Tuple[StepState, List[int]]:
        """Pack the chunk's index arrays, copy them to the device, return the step state and
        the output rows of the wanted logits (in the order they will be produced)."""
        n_seqs = len(seqs)
        lens = [len(s.tokens) for s in seqs]
        n_tokens = sum(lens)
        all_decode = all(n == 1 for n in lens)
        tiles_seq: List[int] = []
        tiles_row: List[int] = []
        if not all_decode:
            order = sorted(range(n_seqs), key=lambda i: -(seqs[i].start + lens[i]))  # long contexts first
            for i in order:
                for row0 in range(0, lens[i], ATTN_TILE):
                    tiles_seq.append(i)
                    tiles_row.append(row0)
        n_tiles = len(tiles_seq)
        want_rows: List[int] = []
        out_rows: List[int] = []
        qstart = []
        offset = 0
        for s, n in zip(seqs, lens):
            qstart.append(offset)
            for row, out_row in s.want:
                want_rows.append(offset + row)
                out_rows.append(out_row)
            offset += n
        n_want = len(want_rows)

        total = 3 * n_tokens + 4 * n_seqs + 2 * n_tiles + n_want
        host, dev = self._meta(total)
        h = host.numpy()
        o = 0

        def put(values, count):
            nonlocal o
            h[o:o + count] = values
            view = dev[o:o + count]
            o += count
            return view

        tokens = put(np.concatenate([np.asarray(s.tokens, dtype=np.int32) for s in seqs]), n_tokens)
        tok_pos = put(np.concatenate([np.arange(s.start, s.start + n, dtype=np.int32)
                                      for s, n in zip(seqs, lens)]), n_tokens)
        tok_seq = put(np.repeat(np.arange(n_seqs, dtype=np.int32), lens), n_tokens)
        seq_slot = put([s.slot for s in seqs], n_seqs)
        ctx = [s.start + n for s, n in zip(seqs, lens)]
        seq_ctx = put(ctx, n_seqs)
        seq_qstart = put(qstart, n_seqs)
        seq_qlen = put(lens, n_seqs)
        tile_seq = put(tiles_seq, n_tiles)
        tile_row0 = put(tiles_row, n_tiles)
        want = put(want_rows, n_want) if n_want else None
        dev[:total].copy_(host[:total], non_blocking=True)
        if self._meta_copied is not None:
            self._meta_copied.record()

        state = StepState(ws=self.ws, n_tokens=n_tokens, n_seqs=n_seqs, tokens=tokens, tok_pos=tok_pos,
                          tok_seq=tok_seq, seq_slot=seq_slot, seq_ctx=seq_ctx, seq_qstart=seq_qstart,
                          seq_qlen=seq_qlen, tile_seq=tile_seq, tile_row0=tile_row0, n_tiles=n_tiles,
                          want_rows=want, all_decode=all_decode, max_ctx=max(ctx), decode_splits=decode_splits,
                          small_rows=self.small_rows,
                          host={"slots": [s.slot for s in seqs], "lens": lens, "starts": [s.start for s in seqs]})
        return state, out_rows

    def _run_chunk(self, seqs: Sequence[_ChunkSeq]):
        state, out_rows = self.build_state(seqs)
        logits = self.model.forward(state, self.cache, state.tokens, state.want_rows)
        return logits, out_rows
