"""Block arrangements: how norms, mixer and feed-forward sit around the residual stream.

`pre_norm` is the reference's layer (src/forward.cc:385-414):
    r = x + mixer(norm_in(x));   x' = r + feed_forward(norm_post(r))
The residual adds are not separate kernels: a part's output stays "pending" until the
next norm, which adds it to the float32 residual and normalises in one pass.  Where the parts on both
sides of a norm offer it, the norm is no kernel either: the part before adds to the residual stream
itself and hands on a `PreNormed`, which the part behind reads (small decode batches).
"""
from __future__ import annotations

from typing import List

from .base import Block, ResidualTarget, register_part


def _offer(x, norm, writer, reader):
    """The ResidualTarget that lets `writer` fold `norm` away for `reader`, or None."""
    if norm is None or not writer.adds_residual or not reader.takes_prenormed or norm.prenorm_weight() is None:
        return None
    return ResidualTarget(x, norm)


class PreNormBlock(Block):
    capturable = True

    def norm_names(self) -> List[str]:
        return ["input", "post_mixer"]

    def first_reader(self, layer):
        return (layer.norms["input"], layer.mixer) if layer.mixer.takes_prenormed else None

    def forward(self, step, x, pending, layer, cache, next_reader=None):
        h = layer.norms["input"].forward(step, x, pending)
        post = layer.norms["post_mixer"]
        into = _offer(x, post, layer.mixer, layer.feed_forward)
        mixed = layer.mixer.forward(step, h, cache, into=into) if into else layer.mixer.forward(step, h, cache)
        h = post.forward(step, x, mixed)
        into = _offer(x, next_reader[0], layer.feed_forward, next_reader[1]) if next_reader else None
        return layer.feed_forward.forward(step, h, into=into) if into else layer.feed_forward.forward(step, h)


register_part("block", "pre_norm", PreNormBlock)
