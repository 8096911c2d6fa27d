"""Attention over a cached latent with a rotated key part that all heads share.

q = h Wq^T, head by head [dim unrotated | rot rotated]; h Wdkv^T = [latent: rank | key
part: rot].  c = rmsnorm(latent) * gain; per head the unrotated key is W_uk c and the value
W_uv c; the score of head i is (q_plain_i . k_plain_i + rotate(q_rot_i) . rotate(key part))
* scale, softmax over all earlier tokens, and the head's output times sigmoid(h Wg^T)_i goes
through Wo.  Only [c | rotated key part] is cached, one row per token for all heads.

How it runs: each head's key matrix is folded into its query (q'_i = [W_uk_i^T q_plain_i |
rotated q_rot_i]), so a head's scores over the cache are q'_i . [c | key part]: the paged
attention of `heads` query heads over ONE key head of size rank + rot, whose cached row also
serves as the value; the first `rank` features of the result are sum_j p_j c_j, which W_uv_i
takes to the head's output.  The rotation is the spec's position encoding (`rope_yarn`:
half-split pairs, frequencies blended between the base's and the stretched ones, cos and
sin times a constant).
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.model_config import MixerSpec
from ..ops import latent as kernels
from .base import MIXERS, POSITIONS, CacheNeed, Mixer, TensorDecl


class LatentAttention(Mixer):
    fuses_norm = True          # h goes into products only: few rows are normalised on their way in
    takes_prenormed = False

    def __init__(self, spec: MixerSpec):
        s = self.spec = spec
        self.H, self.D = s.n_heads, s.head_dim
        self.R = int(s.option("rot_dim", 0))
        self.E = int(s.option("value_dim", s.head_dim))
        self.C = int(s.option("kv_rank", 0))
        self.eps = float(s.option("norm_eps", 1e-6))
        self.has_gate = bool(s.option("gate", True))
        if self.H <= 0 or self.D <= 0 or self.E <= 0 or self.C <= 0 or self.R < 0 or self.R % 2:
            raise ValueError("latent attention: positive heads, dim, vdim and kv_rank; an even rot_dim")
        if s.window is not None:
            raise ValueError("latent attention sees every earlier token: it takes no window")
        self.position = (POSITIONS.build(s.position.kind, s.position) if s.position is not None else None)
        if self.position is not None and (not hasattr(self.position, "frequencies")
                                          or self.position.spec.rotary_dim > self.R):
            raise ValueError("latent attention: the rotated part needs a position encoding that gives "
                             "`frequencies()` over at most rot_dim features")
        # of the rot_dim features the encoding's first rotary_dim turn, the rest pass unchanged
        self.turned = self.position.spec.rotary_dim if self.position is not None else 0

    def tensors(self):
        d, H, D, R, E, C = self.spec.width, self.H, self.D, self.R, self.E, self.C
        out = [TensorDecl("q", (H * (D + R), d)), TensorDecl("dkv", (C + R, d)),
               TensorDecl("dkv.norm", (C,), role="vector"), TensorDecl("uk", (H * D, C)),
               TensorDecl("uv", (H * E, C)), TensorDecl("o", (d, H * E))]
        if self.has_gate:
            out.append(TensorDecl("g", (H, d)))
        return out

    def bind(self, tensors, dtype, device):
        H, D, E, C = self.H, self.D, self.E, self.C
        self.w_in = torch.cat([tensors["q"], tensors["dkv"]], 0).contiguous()
        self.w_gate = tensors.get("g") if self.has_gate else None
        self.gain = tensors["dkv.norm"]
        # head i's key matrix transposed: [rank, dim] takes q_plain_i to the latent's space
        self.uk_t = tensors["uk"].view(H, D, C).transpose(1, 2).contiguous()
        self.uv = tensors["uv"].view(H, E, C).contiguous()
        self.w_out = tensors["o"]
        self.dtype = dtype
        ops.declare_weights(self.w_in, self.w_gate, self.uk_t, self.uv, self.w_out)
        if self.position is not None:
            self.position.bind({}, dtype, device)

    def cache_need(self):
        return CacheNeed(kv_heads=1, head_dim=self.C + self.R, window=None, values_are_keys=True)

    def forward(self, ctx, h, residual, binding):
        t, H, D, R, E, C = h.shape[0], self.H, self.D, self.R, self.E, self.C
        hq, row = H * (D + R), C + R
        proj = ctx.scratch("latent.proj", (t, hq + row), self.dtype)
        ops.linear(h, self.w_in, proj)
        cache = ctx.cache(binding.group)
        qx = ctx.scratch("latent.qx", (t, H * row), self.dtype)
        freq, mscale = ((self.position.frequencies()[0], self.position.magnitude()) if self.turned
                        else (None, 1.0))
        kernels.prepare(proj[:, hq:], proj[:, :hq], qx, self.gain, freq, mscale, self.eps, H, D, C, R,
                        self.turned, ctx, cache, binding)
        kernels.heads_linear(proj, D + R, self.uk_t, qx, row)
        ox = ctx.scratch("latent.ox", (t, H * row), self.dtype)
        ops.paged_attention(qx, ox, H, 1, row, self.spec.softmax_scale, None, ctx, cache, binding)
        act = ctx.scratch("latent.act", (t, H * E), self.dtype)
        logit = None
        if self.w_gate is not None:
            logit = ctx.scratch("latent.gate", (t, H), torch.float32)
            ops.linear(h, self.w_gate, logit)
        kernels.heads_linear(ox, row, self.uv, act, E, gate_logit=logit)
        ops.linear(act, self.w_out, residual, accumulate=True, closes=ctx)


MIXERS.register("latent_attention", LatentAttention)
