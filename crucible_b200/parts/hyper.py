"""Hyper-connections: a pre-norm layer whose residual is several streams.

The residual is fp32 [tokens, S, width]; all streams start as the embedding's output.
Sublayer q of a layer (1: mixer, 2: feed-forward, absent if the layer has none) has
weights `hc<q>.in` [S], `hc<q>.mix` [S, S] (indexed [from, to]) and `hc<q>.out` [S]:
    u = sum_s in[s] x_s;   y = sublayer(norm_q(u));
    x_t <- sum_s mix[s, t] x_s + out[t] y     for all t at once, from the old x_s.
The model's result is the sum of the streams.  With one stream, in = out = 1 and
mix = [[1]] this is the plain pre-norm layer, which is what absent weights mean.

One kernel does a sublayer's write together with the read (mixture and norm) of the
sublayer that follows, also across layers: the model tells a layer which layer runs
next (`ctx.norm_after_layer`), and the next layer finds its first read done
(`ctx.streams_read_ahead`).
"""
from __future__ import annotations

import torch

from ..ops import streams as kernels
from .base import ARRANGEMENTS, Arrangement, TensorDecl


class HyperConnections(Arrangement):
    norm_names = ("norm1", "norm2")

    def __init__(self, spec, norms, mixer, feed_forward):
        self.has_ffn = not getattr(feed_forward, "absent", False)
        self.norm_names = ("norm1", "norm2") if self.has_ffn else ("norm1",)
        super().__init__(spec, norms, mixer, feed_forward)
        self.streams = int(spec.option("streams", 1))
        self.learned = bool(spec.option("learned", True))
        self.w = {}

    def tensors(self):
        if not self.learned:
            return []
        s = self.streams
        out = []
        for q in (1, 2) if self.has_ffn else (1,):
            out += [TensorDecl(f"hc{q}.in", (s,), role="vector", init=("normal", 1.0 / s, 0.1)),
                    TensorDecl(f"hc{q}.out", (s,), role="vector", init=("normal", 1.0, 0.1)),
                    TensorDecl(f"hc{q}.mix", (s, s), role="vector", init=("eye", 1.0, 0.05))]
        return out

    def bind(self, tensors, dtype, device):
        self.dtype = dtype
        s = self.streams
        for q in (1, 2) if self.has_ffn else (1,):
            if self.learned:
                self.w[q] = (tensors[f"hc{q}.in"], tensors[f"hc{q}.mix"].contiguous(), tensors[f"hc{q}.out"])
            else:
                self.w[q] = (torch.ones(s, device=device), torch.eye(s, device=device).contiguous(),
                             torch.ones(s, device=device))

    def entry_read(self):
        """(stream weights, norm) of this layer's first read, for the layer before it."""
        return self.w[1][0], self.norms["norm1"]

    def _h(self, ctx, x):
        return ctx.scratch("hyper.h", (x.shape[0], x.shape[2]), self.dtype)

    def _y(self, ctx, x):
        return ctx.scratch("hyper.y", (x.shape[0], x.shape[2]), torch.float32)

    def _sublayer(self, ctx, x, q, h, run, nxt):
        """h: the sublayer's normalised input.  `nxt`: (stream weights, norm) of the read
        that follows, or None.  Returns that read's result, if it was done."""
        _, mix, out_w = self.w[q]
        y = self._y(ctx, x)
        run(h, y)
        if nxt is None:
            kernels.write(x, y, mix, out_w)
            return None
        weights, norm = nxt
        kernels.write(x, y, mix, out_w, next_weights=weights, next_gain=norm.gain,
                      eps=norm.spec.eps, h=h)
        return h

    def forward(self, ctx, x, binding):
        if x.dim() != 3 or x.shape[1] != self.streams:
            raise ValueError(f"this layer's residual is [tokens, {self.streams}, width]")
        h = getattr(ctx, "streams_read_ahead", None)
        ctx.streams_read_ahead = None
        if h is None:
            h = self._h(ctx, x)
            weights, norm = self.entry_read()
            kernels.read(x, weights, norm.gain, norm.spec.eps, h)
        after = getattr(ctx, "norm_after_layer", None)      # the next layer's entry read, if it has one
        after = after if isinstance(after, tuple) and len(after) == 2 and torch.is_tensor(after[0]) else None

        def mixer(h_in, y):
            self._run(ctx, self.mixer, (ctx, h_in, y, binding), y)

        def ffn(h_in, y):
            self._run(ctx, self.feed_forward, (ctx, h_in, y), y)

        if self.has_ffn:
            h = self._sublayer(ctx, x, 1, h, mixer, (self.w[2][0], self.norms["norm2"]))
            ctx.streams_read_ahead = self._sublayer(ctx, x, 2, h, ffn, after)
        else:
            ctx.streams_read_ahead = self._sublayer(ctx, x, 1, h, mixer, after)

    @staticmethod
    def _run(ctx, part, args, y):
        if getattr(part, "can_overwrite", False):
            part.forward(*args, accumulate=False)
        else:
            y.zero_()
            part.forward(*args)

    def entry_norm(self):
        # what the model hands the layer before this one as `ctx.norm_after_layer`
        return self.entry_read()


ARRANGEMENTS.register("hyper_connections", HyperConnections)
