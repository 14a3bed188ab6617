"""Causal grouped-query attention with a paged key/value cache.

One layer's mixer: fused q/k/v projection, rotary encoding of q and k fused with the
cache write, attention over the cache (prefill tiles or split decode), output
projection.  The arithmetic is the reference's (src/forward.cc:393-408 for the layer,
:265-298 for the scores/softmax/values): head h reads kv head h // (Hq / Hk), scores are
scaled by 1 / sqrt(head_dim) after the dot product, a token attends to itself and all
earlier positions.  A window (not in the reference) limits that to the last w positions.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from ..csrc import kernels as K
from .base import (BuildContext, CacheNeed, KVNeed, Mixer, PartSpec, PreNormed, WeightSpec, register_part)
from .linear import Linear
from .rope import shared_position_encoding

PREFILL_TILE = K.PREFILL_TILE  # query rows per tile of the prefill attention kernels' work list


class Attention(Mixer):
    """params:
      n_heads, n_kv_heads, head_dim     sizes
      window                            0 = all earlier positions
      position                          PartSpec of the position encoding
      names                             {"q","k","v","o"}: tensor name stems (".weight"/".bias" appended)
      qkv_bias, o_bias                  whether the projections carry a bias
      reads_cache_only                  True for an entry that reads another entry's cache:
                                        it has no k/v projection and writes nothing
    """

    capturable = True
    work_list_min_pages = 16  # a piece of a cut sequence is no shorter than this many pages (decode_work_list)

    def __init__(self, params, ctx: BuildContext):
        super().__init__(params, ctx)
        self.n_heads = int(params["n_heads"])
        self.n_kv_heads = int(params["n_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.window = int(params.get("window") or 0)
        self.names = dict(params["names"])
        self.qkv_bias = bool(params.get("qkv_bias", False))
        self.o_bias = bool(params.get("o_bias", False))
        self.reads_cache_only = bool(params.get("reads_cache_only", False))
        self.scale = 1.0 / math.sqrt(self.head_dim)
        if self.head_dim % 16 or not 16 <= self.head_dim <= 256:
            raise ValueError(f"attention: head_dim {self.head_dim} must be a multiple of 16 in [16, 256] "
                             "for the attention kernels")
        if self.n_heads % self.n_kv_heads:
            raise ValueError(f"attention: {self.n_heads} heads are not a multiple of {self.n_kv_heads} kv heads")
        self.position = shared_position_encoding(params.get("position") or PartSpec("none"), ctx)
        self.target_blocks = 2 * max(ctx.multiprocessors, 1)  # decode attention aims at two blocks per multiprocessor
        self.qkv: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.bias: Optional[torch.Tensor] = None
        self.o_bias_t: Optional[torch.Tensor] = None

    # ---- weights ---------------------------------------------------------- #
    def _proj_names(self):
        return ("q",) if self.reads_cache_only else ("q", "k", "v")

    def weight_specs(self) -> List[WeightSpec]:
        D, d = self.ctx.hidden_size, self.head_dim
        rows = {"q": self.n_heads * d, "k": self.n_kv_heads * d, "v": self.n_kv_heads * d}
        specs = []
        for p in self._proj_names():
            specs.append(WeightSpec(self.names[p] + ".weight", (rows[p], D)))
            if self.qkv_bias:
                specs.append(WeightSpec(self.names[p] + ".bias", (rows[p],), kind="vector", init="normal"))
        specs.append(WeightSpec(self.names["o"] + ".weight", (D, self.n_heads * d)))
        if self.o_bias:
            specs.append(WeightSpec(self.names["o"] + ".bias", (D,), kind="vector", init="normal"))
        return specs

    def bind(self, store) -> None:
        mats = [store.take(self.names[p] + ".weight") for p in self._proj_names()]
        if len({m.dtype for m in mats}) > 1:  # a 32-bit tensor stays 32-bit: widen its partners
            mats = [m.float() for m in mats]
        self.qkv = Linear(torch.cat(mats, dim=0) if len(mats) > 1 else mats[0], self.names["q"] + "+k+v")
        del mats
        if self.qkv_bias:
            self.bias = torch.cat([store.take(self.names[p] + ".bias") for p in self._proj_names()]).contiguous()
        self.o = Linear(store.take(self.names["o"] + ".weight"), self.names["o"])
        if self.o_bias:
            self.o_bias_t = store.take(self.names["o"] + ".bias")

    def parameter_bytes(self) -> int:
        return self.qkv.parameter_bytes() + self.o.parameter_bytes()

    def cache_need(self) -> CacheNeed:
        return CacheNeed(kv=KVNeed(self.n_kv_heads, self.head_dim, self.window))

    # ---- step ------------------------------------------------------------- #
    def step_metadata_key(self):
        # attention layers of one shape read the same lists
        return ("attention.step_lists", PREFILL_TILE, self.n_heads, self.n_kv_heads, self.head_dim, self.window)

    def prepare_step(self, shape):
        """The prefill kernels' work lists: one tile of up to PREFILL_TILE query rows per entry, as
        (sequence, first row within the sequence's new tokens), long contexts first so that the longest
        tiles start first; and the same in tiles of twice as many rows, for the kernel that works on those
        (a block per entry: no block is launched only to find that its rows belong to its neighbour).
        Steps of single tokens get the order in which the decode kernel starts its sequences instead: longest
        context first, so that the short ones fill the end of the launch."""
        if shape.all_decode:
            if shape.n_seqs < 2:
                return {}
            work = self.decode_work_list(shape)
            if work is not None:
                return {"decode_work": work}
            return {"decode_order": sorted(range(shape.n_seqs), key=lambda i: -(shape.starts[i] + shape.lens[i]))}
        order = sorted(range(shape.n_seqs), key=lambda i: -(shape.starts[i] + shape.lens[i]))
        lists = {"tile_seq": [], "tile_row0": []}
        wide = []
        for i in order:
            for row0 in range(0, shape.lens[i], PREFILL_TILE):
                lists["tile_seq"].append(i)
                lists["tile_row0"].append(row0)
            for row0 in range(0, shape.lens[i], 2 * PREFILL_TILE):
                wide.append((shape.starts[i] + min(shape.lens[i], row0 + 2 * PREFILL_TILE), i, row0))
        # that kernel walks its list from the back: the tiles that read the most keys come last here
        wide.sort()
        lists["wide_seq"] = [i for _, i, _ in wide]
        lists["wide_row0"] = [row0 for _, _, row0 in wide]
        return lists

    def _decode_pages(self, shape):
        """Pages of keys that each sequence's decode step reads."""
        pages = []
        for start, length in zip(shape.starts, shape.lens):
            ctx = start + length
            first = max(0, ctx - self.window) // K.PAGE if self.window > 0 else 0
            pages.append(max(1, -(-ctx // K.PAGE) - first))
        return pages

    def step_variant(self, shape):
        """"list" for a decode step that runs from a list of (sequence, split) pairs (decode_work_list)."""
        return "list" if shape.all_decode and shape.n_seqs >= 2 and self._wants_work_list(shape) else None

    def _wants_work_list(self, shape) -> bool:
        n = shape.n_seqs
        capacity = K.attention_decode_cluster_capacity(self.ctx.act_dtype, self.head_dim, self.bias is None)
        if capacity is None or n > 32767:
            return False  # the kernel that takes such a list does not run
        splits = self.decode_splits(n, self.ctx.max_positions)
        if splits == 1:
            return True   # too many sequences for a split of each: only a list can cut the long ones
        # A smaller batch gives every sequence the same number of splits inside a cluster, which is the faster
        # merge when the lengths are alike, and still when they are spread (4 sequences of 1,024 to 16,384 tokens:
        # 1.04 ms a step of 8 layers in clusters of 8, 1.09 to 1.20 from the list, whose cut sequences merge
        # through global memory).  When the longest sequence's share is more than three times what an even share
        # of the device would read (or the shortest piece worth cutting), the list wins: 8 sequences of which one
        # has 32,768 tokens 1.25 against 1.58 ms, 16 sequences 1.29 against 2.06.
        pages = self._decode_pages(shape)
        group = self.n_heads // self.n_kv_heads
        items = self.n_kv_heads * (-(-group // 16))
        even = max(self.work_list_min_pages, -(-sum(pages) * items // (2 * capacity[2])))
        return max(pages) > 3 * even * splits

    def decode_work_list(self, shape):
        """For a batch so large that a split of every sequence would not fit the device (decode_splits gives 1),
        or one whose longest sequence is far longer than the rest: the launch as a list of (sequence, split)
        pairs, as many places as sequences and again as many (at least 32) for cuts.  Sequences much longer
        than the rest are cut - one of 32,768 tokens among 63 of a thousand kept its block busy for 280 us while
        the others' took 45 - into pieces of about the length that an even share of the device would read,
        none shorter than 16 pages; the pairs start longest first.  None where the step does not want a list."""
        if not self._wants_work_list(shape):
            return None
        n = shape.n_seqs
        capacity = K.attention_decode_cluster_capacity(self.ctx.act_dtype, self.head_dim, self.bias is None)
        group = self.n_heads // self.n_kv_heads
        items = self.n_kv_heads * (-(-group // 16))
        pages = self._decode_pages(shape)
        extra = max(n, 32)
        resident = 2 * capacity[2]  # blocks that the device holds at once
        per_split = max(self.work_list_min_pages, -(-5 * sum(pages) * items // (4 * resident)))
        while True:
            cuts = [min(K.WORK_LIST_MAX_SPLITS, -(-p // per_split)) for p in pages]
            if sum(cuts) - n <= extra:
                break
            per_split = -(-5 * per_split // 4)
        pairs = sorted(((-(-pages[i] // cuts[i]), -i, s) for i in range(n) for s in range(cuts[i])), reverse=True)
        work = [K.decode_work_entry(-i, s, cuts[-i]) for _, i, s in pairs]
        return work + [-1] * (n + extra - len(work))

    def capture_parameters(self, batch: int, max_positions: int):
        # a captured step serves every context length: the split count follows from the batch size alone
        return {"splits": self.decode_splits(batch, max_positions)}

    def decode_splits(self, n_seqs: int, max_ctx: int) -> int:
        group = self.n_heads // self.n_kv_heads
        heads_per_block = max(1, min(group, 2048 // self.head_dim))
        chunks = -(-group // heads_per_block)
        blocks = max(1, n_seqs * self.n_kv_heads * chunks)
        span = max_ctx if self.window <= 0 else min(max_ctx, self.window + K.PAGE)
        pages = max(1, -(-span // K.PAGE))
        # as many splits as keep every block resident at once (two per multiprocessor) - a second,
        # nearly empty wave costs more than coarser splits - at least one page per split, and at
        # most 16 until a split has 16 pages of its own: the merge grows with the number of splits.
        # The tensor-core kernel applies the same rule to each sequence's own length (a short
        # sequence uses fewer of the offered splits), so a launch captured for the longest
        # context serves the short ones at their own split count.
        by_length = min(pages, max(16, pages // 16))
        splits = max(1, min(self.target_blocks // blocks, by_length))
        # Up to 16 splits the TMA kernel's blocks of one (sequence, kv head) form a cluster, and fewer clusters
        # of s blocks are resident together than 2 x multiprocessors / s blocks are (a cluster stays inside
        # one group of multiprocessors): the most splits whose clusters are all resident at once.
        capacity = K.attention_decode_cluster_capacity(self.ctx.act_dtype, self.head_dim, self.bias is None)
        if capacity is not None:
            fit = [s for s in range(2, min(16, by_length) + 1) if blocks <= capacity[s]]
            return fit[-1] if fit else 1
        return splits

    takes_prenormed = True  # the q/k/v product may read rows whose norm it finishes itself
    adds_residual = True    # the output product may add to the residual stream and prepare the next norm

    def forward(self, step, h, cache, into=None):
        T = (h.values if isinstance(h, PreNormed) else h).shape[0]
        d, Hq, Hk = self.head_dim, self.n_heads, self.n_kv_heads
        act = self.ctx.act_dtype
        if cache.k is None:
            raise RuntimeError("attention: the cache view has no key/value storage")
        qkv = self.qkv.forward(step, h, "qkv")
        cos, sin = self.position.tables()
        out = step.ws.buffer("attn", (T, Hq * d), act)
        splits, scratch, counters, order, work = 1, None, None, None, None
        if step.all_decode:
            lists = step.meta.get(self.step_metadata_key(), {})
            order, work = lists.get("decode_order"), lists.get("decode_work")
            fixed = step.fixed.get(self)
            splits = fixed["splits"] if fixed else self.decode_splits(step.n_seqs, step.max_ctx)
            # room for the most splits that this batch size can ever be given, from its first decode step on, so
            # that no buffer appears or grows (an allocation in the middle of a generation) when the contexts do
            most = max(splits, self.decode_splits(step.n_seqs, self.ctx.max_positions))
            if work is not None:  # every sequence has the number of splits its places of the list say
                splits = most = K.WORK_LIST_MAX_SPLITS
            if most > 1:
                scratch = step.ws.buffer(
                    "attn.scratch", (K.attention_decode_scratch_floats(step.n_seqs, Hq, d, most),), torch.float32)
                # one arrival counter per (sequence, kv head, chunk of 16 heads): the last split merges
                counters = step.ws.zeros("attn.counters", (step.n_seqs * Hk * (-(-(Hq // Hk) // 16)),), torch.int32)
        if (step.all_decode and self.bias is None and qkv.dtype == torch.bfloat16
                and K.attention_decode_fused_supported(act, d)):
            # one launch: rotate q and k, write k and v into the cache, attend
            K.attention_decode_fused(qkv, cos, sin, self.position.interleaved, not self.reads_cache_only,
                                     cache.k, cache.v, step.seq_slot, step.seq_ctx, cache.block_table, scratch, out,
                                     step.n_seqs, Hq, Hk, d, splits, self.window, self.scale, counters=counters,
                                     order=order, work=work)
        else:
            q = step.ws.buffer("q", (T, Hq * d), act)
            K.rope_cache_write(qkv, self.bias, cos, sin, step.tok_pos, step.tok_seq, step.seq_slot,
                               cache.block_table, q, cache.k, cache.v, Hq, Hk, d,
                               self.position.interleaved, write_kv=not self.reads_cache_only)
            if step.all_decode:
                K.attention_decode(q, cache.k, cache.v, step.seq_slot, step.seq_ctx, cache.block_table, scratch, out,
                                   step.n_seqs, Hq, Hk, d, splits, self.window, self.scale, counters=counters,
                                   order=order, work=work)
            else:
                tiles = step.meta[self.step_metadata_key()]
                K.attention_prefill(q, cache.k, cache.v, step.seq_slot, step.seq_ctx, step.seq_qstart, step.seq_qlen,
                                    tiles["tile_seq"], tiles["tile_row0"], cache.block_table, out,
                                    tiles["tile_seq"].shape[0], Hq, Hk, d, self.window, self.scale,
                                    wide_tiles=(tiles["wide_seq"], tiles["wide_row0"]))
        if self.o_bias_t is None:
            return self.o.forward(step, out, "o", into=into)
        o = self.o.forward(step, out, "o")
        K.add_bias(o, self.o_bias_t)
        return o


register_part("mixer", "attention", Attention)
