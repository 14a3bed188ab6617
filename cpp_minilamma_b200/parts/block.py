"""Block arrangements: how norms, mixer and feed-forward sit around the residual stream.

`pre_norm` is the reference's layer (src/forward.cc:385-414):
    r = x + mixer(norm_in(x));   x' = r + feed_forward(norm_post(r))
The residual adds are not separate kernels: a part's output stays "pending" until the
next norm, which adds it to the float32 residual and normalises in one pass.
"""
from __future__ import annotations

from typing import List

from .base import Block, register_part


class PreNormBlock(Block):
    capturable = True

    def norm_names(self) -> List[str]:
        return ["input", "post_mixer"]

    def forward(self, step, x, pending, layer, cache):
        h = layer.norms["input"].forward(step, x, pending)
        mixed = layer.mixer.forward(step, h, cache)
        h = layer.norms["post_mixer"].forward(step, x, mixed)
        return layer.feed_forward.forward(step, h)


register_part("block", "pre_norm", PreNormBlock)
