"""Token embedding and the language-model head.

x = E[token, :] (src/forward.cc:198-205) into the float32 residual stream;
logits = lm_head . norm(x), returned as float32 (src/forward.cc:415-424).  A tied head
reuses the embedding matrix (the reference's GGUF loader does so when `output.weight`
is missing, src/gguf_load.cc:406-408).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import kernels as K
from .base import BuildContext, Part, WeightSpec, register_part
from .linear import Linear


class TokenEmbedding(Part):
    """params: vocab, name."""

    capturable = True

    role = "embedding"

    def __init__(self, params, ctx: BuildContext):
        super().__init__(params, ctx)
        self.vocab = int(params["vocab"])
        self.name = params["name"]
        self.table: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name, (self.vocab, self.ctx.hidden_size))]

    def bind(self, store) -> None:
        self.table = store.get(self.name)  # left in the store: a tied head takes it too

    def forward(self, step, tokens: torch.Tensor) -> torch.Tensor:
        x = step.ws.buffer("x", (tokens.shape[0], self.ctx.hidden_size), torch.float32)
        K.embedding(tokens, self.table, x)
        return x


class LMHead(Part):
    """params: vocab, name, tied_to (name of the embedding tensor, or None)."""

    capturable = True

    role = "lm_head"

    def __init__(self, params, ctx: BuildContext):
        super().__init__(params, ctx)
        self.vocab = int(params["vocab"])
        self.name = params["name"]
        self.tied_to = params.get("tied_to")
        self.linear: Optional[Linear] = None

    def weight_specs(self) -> List[WeightSpec]:
        if self.tied_to:
            return []
        return [WeightSpec(self.name, (self.vocab, self.ctx.hidden_size))]

    def bind(self, store) -> None:
        self.linear = Linear(store.get(self.tied_to) if self.tied_to else store.take(self.name),
                             self.tied_to or self.name)

    def parameter_bytes(self) -> int:
        return self.linear.parameter_bytes()

    def forward(self, step, h: torch.Tensor, out_name: str = "logits") -> torch.Tensor:
        return self.linear.forward(step, h, out_name, out_dtype=torch.float32)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("lm_head", "linear_head", LMHead)
