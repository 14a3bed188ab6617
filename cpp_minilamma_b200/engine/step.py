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
lengths, wanted rows, the index arrays that parts prepare for their own kernels, and the
block-table rows that changed) are packed into one int32 buffer that crosses to the device
in one copy from pinned memory.  Activations live in a workspace that is reused from layer
to layer and from step to step.  A step therefore allocates nothing, copies one buffer to
the device and none back (the reference counts the same in test/forward_test.cc:412-420);
the exceptions are a step cut into several chunks and wanted rows that are not in order,
which assemble their logits in a tensor of their own.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.paged import PAGE, CacheError, SequenceCache
from ..parts.base import StepShape
from .model import Model



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
        self._zeroed: set = set()
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
            self._zeroed.add(name)
            self.generation += 1
        return self._flat[name][:count].view(shape)

    def rezero(self) -> None:
        """Zero every buffer handed out by `zeros` again (after a kernel that may have left its counters dirty)."""
        for name in self._zeroed:
            self._flat[name].zero_()

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._flat.values())


@dataclass
class StepState:
    """Everything the parts see of a step (device tensors are int32 views of one buffer).

    The fields up to `max_ctx` are the engine's own and the same for every model.  `meta` holds the
    index arrays that parts prepared for this step (`Part.prepare_step`, by the part's
    `step_metadata_key()` and the array's name), `fixed` the launch parameters of a captured step
    (`Part.capture_parameters`, by part), `extras` arrays that the caller of the step sent along."""

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
    want_rows: Optional[torch.Tensor]
    all_decode: bool
    max_ctx: int
    small_rows: int = 0                         # steps with at most this many rows use the weight-streaming product
    shape: Optional[StepShape] = None           # the same step as host lists, for parts written in Python
    meta: Dict[Hashable, Dict[str, torch.Tensor]] = field(default_factory=dict)
    fixed: Dict[Any, Dict[str, int]] = field(default_factory=dict)
    extras: Dict[str, torch.Tensor] = field(default_factory=dict)


def metadata_providers(parts) -> Dict[Hashable, Any]:
    """key -> the first of `parts` with that `step_metadata_key()`: who prepares each kind of index array."""
    providers: Dict[Hashable, Any] = {}
    for part in parts:
        key = part.step_metadata_key()
        if key is not None and key not in providers:
            providers[key] = part
    return providers


def step_arrays(shape: StepShape, tokens, want_rows: Sequence[int], providers: Dict[Hashable, Any],
                extras: Optional[Dict[str, Sequence[int]]] = None) -> List[Tuple[Any, np.ndarray]]:
    """(name, int32 array) for everything the step's kernels index by, in packing order."""
    lens = shape.lens
    n_seqs = shape.n_seqs
    arrays: List[Tuple[Any, np.ndarray]] = [
        ("tokens", np.asarray(tokens, dtype=np.int32)),
        ("tok_pos", np.concatenate([np.arange(s, s + n, dtype=np.int32) for s, n in zip(shape.starts, lens)])),
        ("tok_seq", np.repeat(np.arange(n_seqs, dtype=np.int32), lens)),
        ("seq_slot", np.asarray(shape.slots, dtype=np.int32)),
        ("seq_ctx", np.asarray([s + n for s, n in zip(shape.starts, lens)], dtype=np.int32)),
        ("seq_qstart", np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.int32)),
        ("seq_qlen", np.asarray(lens, dtype=np.int32)),
        ("want_rows", np.asarray(want_rows, dtype=np.int32)),
    ]
    for key, part in providers.items():
        for name, values in part.prepare_step(shape).items():
            arrays.append((("meta", key, name), np.asarray(values, dtype=np.int32).reshape(-1)))
    for name, values in (extras or {}).items():
        arrays.append((("extra", name), np.asarray(values, dtype=np.int32).reshape(-1)))
    return arrays


def state_from_views(ws: Workspace, shape: StepShape, views: Dict[Any, torch.Tensor], small_rows: int) -> StepState:
    state = StepState(ws=ws, n_tokens=shape.n_tokens, n_seqs=shape.n_seqs, tokens=views["tokens"],
                      tok_pos=views["tok_pos"], tok_seq=views["tok_seq"], seq_slot=views["seq_slot"],
                      seq_ctx=views["seq_ctx"], seq_qstart=views["seq_qstart"], seq_qlen=views["seq_qlen"],
                      want_rows=views["want_rows"] if views["want_rows"].shape[0] else None,
                      all_decode=shape.all_decode, max_ctx=shape.max_ctx, small_rows=small_rows, shape=shape)
    for name, view in views.items():
        if isinstance(name, tuple) and name[0] == "meta":
            state.meta.setdefault(name[1], {})[name[2]] = view
        elif isinstance(name, tuple) and name[0] == "extra":
            state.extras[name[1]] = view
    return state


def make_step_state(device, slots: Sequence[int], starts: Sequence[int], lens: Sequence[int], tokens=None,
                    want_rows: Sequence[int] = (), parts=(), ws: Optional[Workspace] = None,
                    small_rows: int = 0) -> StepState:
    """A `StepState` outside an engine, for running a part alone (tests, experiments): the same arrays, packed
    and copied once.  `parts`: the parts that will see the state; their index arrays are prepared."""
    shape = StepShape(list(slots), list(starts), list(lens))
    arrays = step_arrays(shape, tokens if tokens is not None else [0] * shape.n_tokens, want_rows,
                         metadata_providers(parts))
    flat = torch.from_numpy(np.concatenate([a for _, a in arrays])).to(device)
    views, at = {}, 0
    for name, a in arrays:
        views[name] = flat[at:at + a.shape[0]]
        at += a.shape[0]
    return state_from_views(ws or Workspace(device), shape, views, small_rows)


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
        self.max_step_tokens = max(int(max_step_tokens), PAGE)
        self.vocab_size = model.spec.vocab_size
        self.providers = metadata_providers(model.all_parts())
        self._meta_host: Optional[torch.Tensor] = None
        self._meta_dev: Optional[torch.Tensor] = None
        self._meta_copied = None
        self.extras: Dict[str, torch.Tensor] = {}  # device views of the extras that the last step was given
        self.small_rows = 64  # rows up to which linears may use this package's weight-streaming kernels
        self.launch_count = 0  # kernels of this package launched (estimate kept by the parts' callers)

    # ---- helpers shared by everything that generates with this engine -------------------- #
    def shared_sampler(self):
        if getattr(self, "_sampler", None) is None:
            from ..sampling.sampler import DeviceSampler
            from .decode_graph import decode_bucket
            self._sampler = DeviceSampler(self.device, max(decode_bucket(self.cache.n_slots), 64))
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
        self.check_device_error()
        return None if borrowed is None else borrowed.clone()

    def check_device_error(self) -> None:
        """Waits for the device and raises `DeviceKernelError` if a kernel gave up since the flags were
        last read (a bounded wait that ran out).  `step` calls it: its callers read the logits next, so
        the wait costs them nothing they would not pay anyway.  The generation loop does not come here; it
        gets the same flags with the sampled tokens (`DeviceSampler.collect`)."""
        from ..csrc import kernels as K
        mask = K.take_device_error()
        if mask:
            self.after_device_error()
            raise K.DeviceKernelError(K.device_error_message(mask))

    def after_device_error(self) -> None:
        """A kernel that gave up may have left arrival counters non-zero and the workspace half written:
        zero the counters and drop the captured decode graphs, so that later steps start clean."""
        self.ws.rezero()
        if getattr(self, "_graphs", None) is not None:
            self._graphs.drop()

    def step_borrowed(self, entries: Sequence[StepEntry],
                      extras: Optional[Dict[str, Sequence[int]]] = None) -> Optional[torch.Tensor]:
        """As `step`, but the result may alias workspace memory that the next step overwrites, and the
        device's error flags are not looked at.  `extras`: further integer arrays that cross to the device
        with the step's index arrays (the sampler's counters, say); their device views are in
        `self.extras` afterwards."""
        chunks, n_want = self._plan(entries)
        out: Optional[torch.Tensor] = None
        if n_want and len(chunks) > 1:
            out = torch.empty((n_want, self.vocab_size), dtype=torch.float32, device=self.device)
        result = None
        for i, chunk in enumerate(chunks):
            logits, out_rows = self._run_chunk(chunk, extras if i == len(chunks) - 1 else None)
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
        # the block-table rows that changed travel with the first chunk's index arrays (build_state)

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
            if self._meta_copied is not None:
                self._meta_copied.synchronize()
            size = max(2 * n_ints, 4096)
            pin = self.device.type == "cuda"
            self._meta_host = torch.empty(size, dtype=torch.int32, pin_memory=pin)
            self._meta_dev = torch.empty(size, dtype=torch.int32, device=self.device)
            self._meta_copied = torch.cuda.Event() if pin else None
        elif self._meta_copied is not None:
            # the previous step's copy may still be reading the pinned buffer
            self._meta_copied.synchronize()
        return self._meta_host, self._meta_dev

    def build_state(self, seqs: Sequence[_ChunkSeq],
                    extras: Optional[Dict[str, Sequence[int]]] = None) -> Tuple[StepState, List[int]]:
        """Pack the chunk's index arrays and the cache's changed block-table rows, copy them to the
        device (one copy), apply the rows, and return the step state and the output rows of the wanted
        logits (in the order they will be produced)."""
        from ..csrc import kernels as K
        shape = StepShape([s.slot for s in seqs], [s.start for s in seqs], [len(s.tokens) for s in seqs])
        want_rows: List[int] = []
        out_rows: List[int] = []
        offset = 0
        for s, n in zip(seqs, shape.lens):
            for row, out_row in s.want:
                want_rows.append(offset + row)
                out_rows.append(out_row)
            offset += n
        arrays = step_arrays(shape, np.concatenate([np.asarray(s.tokens, dtype=np.int32) for s in seqs]),
                             want_rows, self.providers, extras)
        updates = self.cache.take_table_updates()  # (group, int32 [n, 1 + max_blocks]) per group with changes
        total = sum(a.shape[0] for _, a in arrays) + sum(rows.size for _, rows in updates)
        host, dev = self._meta(total)
        h = host.numpy()
        views: Dict[Any, torch.Tensor] = {}
        at = 0
        for name, a in arrays:
            h[at:at + a.shape[0]] = a
            views[name] = dev[at:at + a.shape[0]]
            at += a.shape[0]
        staged = []
        for group, rows in updates:
            h[at:at + rows.size] = rows.reshape(-1)
            staged.append((group, dev[at:at + rows.size], rows.shape[0]))
            at += rows.size
        dev[:total].copy_(host[:total], non_blocking=True)
        if self._meta_copied is not None:
            self._meta_copied.record()
        for group, region, n_rows in staged:
            K.scatter_rows(group.table_dev, region, n_rows)
        state = state_from_views(self.ws, shape, views, self.small_rows)
        return state, out_rows

    def _run_chunk(self, seqs: Sequence[_ChunkSeq], extras=None):
        state, out_rows = self.build_state(seqs, extras)
        self.extras = state.extras
        logits = self.model.forward(state, self.cache, state.tokens, state.want_rows)
        return logits, out_rows
