"""What a model is made of: specs (data) and part interfaces (code).

A `ModelSpec` is pure data produced by an architecture's builder from its typed
configuration: for each layer the kinds and parameters of its mixer, feed-forward, norms
and block arrangement, and a schedule - the order in which layers run, which may name a
layer twice or let an entry read the cache that another entry writes.  `build_part`
turns a `PartSpec` into an object through the per-role registries below.  No part knows
which model it is in: sizes, constants and tensor names all arrive as parameters.

Roles and their interfaces
  position encoding  `PositionEncoding.tables(device, max_positions)` -> tensors a mixer uses
  norm               `Norm.forward(step, x, delta, rows=None)`  x float32 residual [T, D]
  mixer              `Mixer.cache_need()`, `Mixer.forward(step, h, cache)` -> [T, D]
  feed-forward       `FeedForward.forward(step, h)` -> [T, D]
  block              `Block.forward(step, x, pending, layer, cache)` -> pending delta
A part may offer more than its role asks (see `PreNormed`): the flags `takes_prenormed` and
`adds_residual` of a mixer or feed-forward, `Norm.prenorm_weight`, `Block.first_reader`.  They are off by
default, and a part that leaves them off never meets the objects they bring.
Every part also lists the tensors it loads (`weight_specs`) and receives them by name
(`bind`).  The reference has one hard-wired graph (src/forward.cc:385-414); these seams
are this library's own.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch


# --------------------------------------------------------------------------- #
# specs                                                                        #
# --------------------------------------------------------------------------- #
@dataclass(frozen=True)
class WeightSpec:
    """One tensor a part loads.

    kind: "matrix" follows the run's dtype unless the file stores it in 32-bit (then it
    stays 32-bit); "vector" (norm weights, biases) is always held as float32, which keeps
    every stored value exactly; "int_table" is held as int32.
    init: how the random-weights mode fills it: "normal" N(0, matrix_std), "norm"
    1 + N(0, norm_std), "zeros", "ones".
    """

    name: str
    shape: Tuple[int, ...]
    kind: str = "matrix"
    init: str = "normal"


@dataclass
class PartSpec:
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass
class LayerSpec:
    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Dict[str, PartSpec]


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.  `cache_of` names an earlier entry (by its index in the
    schedule) whose cache this entry reads instead of owning one."""

    layer: int
    cache_of: Optional[int] = None


@dataclass
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    final_norm: PartSpec
    lm_head: PartSpec
    stop_token_ids: List[int] = field(default_factory=list)


# --------------------------------------------------------------------------- #
# cache needs a mixer may declare                                              #
# --------------------------------------------------------------------------- #
@dataclass(frozen=True)
class KVNeed:
    """Keys and values per position: pages of [n_kv_heads, PAGE, head_dim].  `window` > 0
    means only the last `window` positions are ever read."""

    n_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size state per sequence: named tensors of the given shapes, float32, zeroed
    when a slot is handed out."""

    tensors: Tuple[Tuple[str, Tuple[int, ...]], ...]


@dataclass(frozen=True)
class CacheNeed:
    kv: Optional[KVNeed] = None
    state: Optional[StateNeed] = None


# --------------------------------------------------------------------------- #
# a norm folded into the products around it                                    #
# --------------------------------------------------------------------------- #
@dataclass
class PreNormed:
    """Rows of the residual stream on their way through a norm y = x * w / rms(x): `values` [T, D]
    holds x * w, `sumsq` float32 [T, stride] holds `partials` partial sums of x^2 per row.  The product
    that reads them multiplies its result by 1 / sqrt(sum / D + eps), so that no kernel runs for the norm.
    The part that ended the previous sub-layer writes it (it has already added its output to the residual
    stream), `norm` is the norm it was written for, and only a part with `takes_prenormed` is given one."""

    values: torch.Tensor
    sumsq: torch.Tensor
    partials: int
    eps: float
    norm: "Norm"


@dataclass
class ResidualTarget:
    """Offered to a part with `adds_residual`: it may add its output to the float32 residual stream `x`
    itself and return a `PreNormed` for `norm`, the norm that reads the stream next, instead of returning
    the output.  It may also ignore the offer."""

    x: torch.Tensor
    norm: "Norm"


# --------------------------------------------------------------------------- #
# build context and part bases                                                 #
# --------------------------------------------------------------------------- #
@dataclass
class BuildContext:
    hidden_size: int
    act_dtype: torch.dtype  # bfloat16 or float32: activations, cache and (by default) matrices
    device: torch.device
    max_positions: int
    shared: Dict[Any, Any] = field(default_factory=dict)  # tables shared between layers
    multiprocessors: int = 0  # of the device, asked once when the model is built (0: not a CUDA device)


@dataclass
class StepShape:
    """What a step looks like from the host: for each sequence of the batch its slot, the position of its
    first new token and the number of tokens it brings.  Parts read it when they prepare index arrays of
    their own for the step (`Part.prepare_step`); a part written in Python may also walk it in `forward`."""

    slots: List[int]
    starts: List[int]
    lens: List[int]

    @property
    def n_seqs(self) -> int:
        return len(self.slots)

    @property
    def n_tokens(self) -> int:
        return sum(self.lens)

    @property
    def all_decode(self) -> bool:
        return all(n == 1 for n in self.lens)

    @property
    def max_ctx(self) -> int:
        return max(s + n for s, n in zip(self.starts, self.lens))


class WeightStore:
    """Loaded device tensors by name, handed to the parts at bind time.  `take` removes
    the tensor (the part owns it or fuses it away), `get` leaves it for others (tied
    weights).  What is left after binding was loaded for nothing and is dropped."""

    def __init__(self, tensors: Dict[str, torch.Tensor]):
        self._tensors = dict(tensors)

    def has(self, name: str) -> bool:
        return name in self._tensors

    def get(self, name: str) -> torch.Tensor:
        return self._tensors[name]

    def take(self, name: str) -> torch.Tensor:
        return self._tensors.pop(name)

    def names(self):
        return sorted(self._tensors)


class Part:
    role = "part"
    # True when `forward` only enqueues work whose arguments live in device memory at fixed
    # addresses, so that a decode step can be captured in a CUDA graph and replayed.  A part
    # that reads host-side step information (step.shape) or allocates must leave it False.
    capturable = False

    def __init__(self, params: Dict[str, Any], ctx: BuildContext):
        self.params = params
        self.ctx = ctx

    def weight_specs(self) -> List[WeightSpec]:
        return []

    def bind(self, store: "WeightStore") -> None:
        """Take the device tensors named in `weight_specs` from the store (fusing is done here)."""

    def parameter_bytes(self) -> int:
        """Bytes of weights a step reads from this part (for the roofline)."""
        return 0

    # ---- index arrays and launch parameters of the part's own ------------------------------------- #
    def step_metadata_key(self):
        """None, or a hashable key: the part's kernels want index arrays of their own on the device for
        every step (tile lists, work queues ...).  Parts with equal keys share one preparation per step."""
        return None

    def prepare_step(self, shape: "StepShape") -> Dict[str, Any]:
        """name -> sequence of integers for this step.  The engine packs them into the one int32 buffer
        that crosses to the device per step and hands them back as device views in
        `step.meta[key][name]`.  In a step where every sequence brings one token the sizes must depend on
        the number of sequences alone (such steps are replayed from a captured graph)."""
        return {}

    def step_variant(self, shape: "StepShape"):
        """None, or a hashable value when the part launches differently for different kinds of steps of one
        batch size (a list of other length from `prepare_step`, another kernel).  Captured decode steps are
        kept per (batch size, variants of all parts): the part sees only steps of one variant in each."""
        return None

    def capture_parameters(self, batch: int, max_positions: int) -> Dict[str, int]:
        """Launch parameters that must not change between replays of a captured decode step of `batch`
        sequences (a captured graph serves every context length).  The part finds them in
        `step.fixed[self]` during such steps and chooses freely otherwise."""
        return {}


class PositionEncoding(Part):
    role = "position_encoding"

    def tables(self):
        """Device tensors the mixer's kernels read, or None when positions are not encoded."""
        raise NotImplementedError


class Norm(Part):
    role = "norm"

    def forward(self, step, x: torch.Tensor, delta: Optional[torch.Tensor],
                rows: Optional[torch.Tensor] = None, out_name: str = "h") -> torch.Tensor:
        """x += delta (in place, float32), return norm(x) in the activation dtype; with
        `rows` only those rows, x unchanged.  A `PreNormed` made for this norm is handed on as it is."""
        raise NotImplementedError

    def prenorm_weight(self):
        """(weight float32 [D], eps) if the norm is x * weight / sqrt(mean(x^2) + eps) and may be folded
        into the products around it (`PreNormed`), else None."""
        return None


class Mixer(Part):
    role = "mixer"
    takes_prenormed = False  # True: `h` may be a PreNormed
    adds_residual = False    # True: forward has a keyword `into` (a ResidualTarget or None) and may return a PreNormed

    def cache_need(self) -> CacheNeed:
        return CacheNeed()

    def forward(self, step, h: torch.Tensor, cache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    role = "feed_forward"
    takes_prenormed = False  # as for a mixer
    adds_residual = False

    def forward(self, step, h: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """The arrangement of norms, mixer and feed-forward around the residual stream."""

    role = "block"

    def norm_names(self) -> List[str]:
        raise NotImplementedError

    def forward(self, step, x: torch.Tensor, pending: Optional[torch.Tensor], layer, cache):
        """Run one layer on residual x [T, D] (float32).  `pending` is a delta still to be
        added to x (so that the next norm kernel can fuse the add); returns the new pending.
        A block whose `first_reader` is not None also takes the keyword `next_reader` (the first reader
        of the layer that runs next, or None) and may then return, and be given, a `PreNormed`."""
        raise NotImplementedError

    def first_reader(self, layer):
        """(norm, part): the norm that reads the residual stream first in this arrangement and the part that
        takes its output - if the layer before may fold that norm away (`PreNormed`), else None."""
        return None


# --------------------------------------------------------------------------- #
# registries                                                                   #
# --------------------------------------------------------------------------- #
_PARTS: Dict[str, Dict[str, Callable]] = {
    "position_encoding": {}, "norm": {}, "mixer": {}, "feed_forward": {}, "block": {},
    "embedding": {}, "lm_head": {},
}


def register_part(role: str, kind: str, factory: Callable) -> None:
    """`factory(params, ctx)` builds the part.  Registering a kind again replaces it."""
    if role not in _PARTS:
        raise KeyError(f"unknown part role {role!r}; roles: {sorted(_PARTS)}")
    _PARTS[role][kind] = factory


def build_part(role: str, spec: PartSpec, ctx: BuildContext):
    kinds = _PARTS[role]
    if spec.kind not in kinds:
        raise KeyError(f"no {role} of kind {spec.kind!r} is registered; known: {sorted(kinds)}")
    return kinds[spec.kind](spec.params, ctx)


def known_parts(role: str) -> List[str]:
    return sorted(_PARTS[role])
