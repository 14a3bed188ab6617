"""`Model`: a `ModelSpec` made real - parts built, weights bound, one forward over a step.

The forward is the reference's graph (src/forward.cc:432-472: embedding, the layers,
final norm, lm_head) driven by data: it walks the spec's schedule, so the same code runs
a model whose schedule repeats a layer or whose entries share a cache.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from ..parts.base import (Block, BuildContext, CacheNeed, FeedForward, Mixer, ModelSpec, Norm, WeightSpec,
                          WeightStore, build_part)


@dataclass
class Layer:
    block: Block
    mixer: Mixer
    feed_forward: FeedForward
    norms: Dict[str, Norm]

    def parts(self):
        return [self.mixer, self.feed_forward, *self.norms.values()]


class Model:
    def __init__(self, spec: ModelSpec, act_dtype: torch.dtype, device, max_positions: Optional[int] = None):
        self.spec = spec
        self.act_dtype = act_dtype
        self.device = torch.device(device)
        positions = spec.max_positions if max_positions is None else min(spec.max_positions, max_positions)
        multiprocessors = (torch.cuda.get_device_properties(self.device).multi_processor_count
                           if self.device.type == "cuda" else 0)
        self.ctx = BuildContext(spec.hidden_size, act_dtype, self.device, positions, multiprocessors=multiprocessors)
        self.max_positions = positions
        self.embedding = build_part("embedding", spec.embedding, self.ctx)
        self.layers: List[Layer] = []
        for layer_spec in spec.layers:
            block = build_part("block", layer_spec.block, self.ctx)
            missing = [n for n in block.norm_names() if n not in layer_spec.norms]
            if missing:
                raise ValueError(f"block {layer_spec.block.kind!r} needs norms {missing}")
            self.layers.append(Layer(
                block=block,
                mixer=build_part("mixer", layer_spec.mixer, self.ctx),
                feed_forward=build_part("feed_forward", layer_spec.feed_forward, self.ctx),
                norms={name: build_part("norm", s, self.ctx) for name, s in layer_spec.norms.items()}))
        self.final_norm = build_part("norm", spec.final_norm, self.ctx)
        self.lm_head = build_part("lm_head", spec.lm_head, self.ctx)
        for i, entry in enumerate(spec.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule entry {i} names layer {entry.layer}, the model has {len(self.layers)}")
            if entry.cache_of is not None and not 0 <= entry.cache_of < i:
                raise ValueError(f"schedule entry {i} reads the cache of entry {entry.cache_of}, which is not earlier")
        self.bound = False

    # ---- weights ------------------------------------------------------------ #
    def all_parts(self):
        parts = [self.embedding]
        for layer in self.layers:
            parts.extend(layer.parts())
        parts.extend([self.final_norm, self.lm_head])
        return parts

    def weight_specs(self) -> List[WeightSpec]:
        specs: List[WeightSpec] = []
        seen = set()
        for part in self.all_parts():
            for spec in part.weight_specs():
                if spec.name in seen:
                    raise ValueError(f"two parts load the tensor {spec.name!r}")
                seen.add(spec.name)
                specs.append(spec)
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        store = WeightStore(tensors)
        tensors.clear()  # the store holds the only references from here on
        for part in self.all_parts():
            part.bind(store)
        self.bound = True

    def parameter_count(self) -> int:
        total = 0
        for spec in self.weight_specs():
            n = 1
            for dim in spec.shape:
                n *= dim
            total += n
        return total

    def step_weight_bytes(self) -> int:
        """Bytes of weights one decode step reads: every scheduled part once, plus the
        final norm and the head (the embedding rows are negligible)."""
        total = self.final_norm.parameter_bytes() + self.lm_head.parameter_bytes()
        for entry in self.spec.schedule:
            total += sum(p.parameter_bytes() for p in self.layers[entry.layer].parts())
        return total

    def capturable(self) -> bool:
        """Whether a decode step of this model can be captured in a CUDA graph."""
        return all(part.capturable for part in self.all_parts()) and all(l.block.capturable for l in self.layers)

    # ---- cache needs ---------------------------------------------------------- #
    def cache_needs(self) -> List[Tuple[int, Optional[int], CacheNeed]]:
        return [(i, entry.cache_of, self.layers[entry.layer].mixer.cache_need())
                for i, entry in enumerate(self.spec.schedule)]

    # ---- forward ---------------------------------------------------------------- #
    def forward(self, step, cache, tokens: torch.Tensor, want_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Run the step's tokens [T] through every scheduled layer; return float32 logits
        [n_want, vocab] of the rows in `want_rows` (int32), or None when nothing is wanted."""
        if not self.bound:
            raise RuntimeError("the model has no weights bound")
        x = self.embedding.forward(step, tokens)
        pending = None
        schedule = self.spec.schedule
        for i, entry in enumerate(schedule):
            layer = self.layers[entry.layer]
            if layer.block.first_reader(layer) is None:
                pending = layer.block.forward(step, x, pending, layer, cache.view(i))
                continue
            # this arrangement can fold a norm into the products around it: tell it who reads the stream next
            follower = self.layers[schedule[i + 1].layer] if i + 1 < len(schedule) else None
            reader = follower.block.first_reader(follower) if follower else None
            pending = layer.block.forward(step, x, pending, layer, cache.view(i), next_reader=reader)
        if want_rows is None or want_rows.shape[0] == 0:
            return None
        h = self.final_norm.forward(step, x, pending, rows=want_rows, out_name="h_final")
        return self.lm_head.forward(step, h)
