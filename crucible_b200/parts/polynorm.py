"""Dense feed-forward with the PolyNorm activation: x += act(h Wup^T) Wdown^T,
act(z) = a N(z) + b N(z^2) + c N(z^3) + e with N(v) = v / sqrt(mean(v^2) + eps) over
a token's ff values and powers taken element by element; (a, b, c, e) are the four
numbers of the tensor `act`.  The statistics are 32-bit."""
from __future__ import annotations

import torch

from .. import ops
from ..config.model_config import FeedForwardSpec
from .base import FEED_FORWARDS, FeedForward, TensorDecl


class PolyNormFeedForward(FeedForward):
    can_overwrite = True

    def __init__(self, spec: FeedForwardSpec):
        self.spec = spec
        self.eps = float(spec.option("norm_eps", 1e-6))
        self.up = self.down = self.coef = None

    def tensors(self):
        d, f = self.spec.width, self.spec.intermediate
        return [TensorDecl("up", (f, d)), TensorDecl("down", (d, f)),
                TensorDecl("act", (4,), role="vector", init=("uniform", 0.2, 1.0))]

    def bind(self, tensors, dtype, device):
        self.up, self.down, self.coef = tensors["up"], tensors["down"], tensors["act"]
        ops.declare_weights(self.up, self.down)
        self.dtype = dtype

    def forward(self, ctx, h, residual, accumulate: bool = True):
        t, f = h.shape[0], self.spec.intermediate
        z = ctx.scratch("ffn.z", (t, f), self.dtype)
        ops.linear(h, self.up, z)
        ops.polynorm(z, self.coef, self.eps, z)
        ops.linear(z, self.down, residual, accumulate=accumulate)


class NoFeedForward(FeedForward):
    """A layer without a feed-forward sublayer."""
    absent = True

    def __init__(self, spec: FeedForwardSpec):
        self.spec = spec

    def forward(self, ctx, h, residual, accumulate: bool = True):
        pass


FEED_FORWARDS.register("polynorm", PolyNormFeedForward)
FEED_FORWARDS.register("none", NoFeedForward)
