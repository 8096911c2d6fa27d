"""Mixers with a matrix memory per head instead of a cache of keys.  Their state is
fp32 in the request's state slot (zero when the slot is handed out) and is carried
from step to step, so a prompt may be cut anywhere.

`gated_delta` (the gated delta rule): q, k [G, D] and v [H, E] pass a short causal
convolution per channel (`<tensor>.conv` [channels, taps], the last tap meets the
current token; its last taps - 1 inputs are state) and SiLU; q and k become unit
vectors per head (x / sqrt(sum x^2 + 1e-6)), q times D^-1/2.  Per head, with
beta = sigmoid(h Wb^T) and g = exp(-exp(A_log) * softplus(h Wa^T + dt_bias)):
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.
o / rms(o) * norm [E] * silu(h Wg^T) goes through Wo.  Head i uses q/k head i // (H / G).

`mlstm` (the matrix memory of the xLSTM): q = h Wq^T * D^-1/2, k [H, D], v [H, E];
log gates i = cap * tanh((h Wi^T + bi) / cap), f = logsigmoid(cap * tanh((h Wf^T + bf) / cap));
with m (from 0):  m' = max(f + m, i);  S <- exp(f + m - m') S + exp(i - m') k v^T;
n likewise with k alone;  o = S^T q / (max(|n . q|, exp(-m')) + 1e-6).
o / rms(o) per head, times norm [H * E], times sigmoid(h Wg^T), goes through Wo.
"""
from __future__ import annotations

import torch

from ..config.model_config import MixerSpec
from ..ops import recurrent as kernels
from .base import MIXERS, TensorDecl
from .branch import BranchMixer


def _round16(n: int) -> int:
    return (n + 15) // 16 * 16


class GatedDeltaRule(BranchMixer):
    def __init__(self, spec: MixerSpec):
        s = self.spec = spec
        self.H, self.G, self.D = s.n_heads, s.n_kv_heads, s.head_dim
        self.E = int(s.option("value_dim", s.head_dim))
        self.taps = int(s.option("conv_taps", 4))
        self.eps = float(s.option("norm_eps", 1e-6))
        if self.H <= 0 or self.G <= 0 or self.H % self.G or self.D <= 0 or self.E <= 0 or self.taps < 1:
            raise ValueError("gated_delta: heads must be a multiple of kv_heads; sizes positive")
        if self.D > 256:
            raise ValueError("gated_delta: key size up to 256")
        self.C = 2 * self.G * self.D + self.H * self.E          # channels under the convolution
        self.s_bytes = _round16(4 * self.H * self.D * self.E)
        self.tail_bytes = 4 * (self.taps - 1) * self.C

    def tensors(self):
        d, H, G, D, E = self.spec.width, self.H, self.G, self.D, self.E
        conv = ("uniform", -0.5, 0.5)
        return [TensorDecl("q", (G * D, d)), TensorDecl("k", (G * D, d)), TensorDecl("v", (H * E, d)),
                TensorDecl("q.conv", (G * D, self.taps), role="vector", init=conv),
                TensorDecl("k.conv", (G * D, self.taps), role="vector", init=conv),
                TensorDecl("v.conv", (H * E, self.taps), role="vector", init=conv),
                TensorDecl("b", (H, d)), TensorDecl("a", (H, d)),
                TensorDecl("A_log", (H,), role="vector", init=("uniform", -1.0, 1.0)),
                TensorDecl("dt_bias", (H,), role="vector", init=("uniform", -1.0, 1.0)),
                TensorDecl("norm", (E,), role="vector"),
                TensorDecl("g", (H * E, d)), TensorDecl("o", (d, H * E))]

    def bind(self, tensors, dtype, device):
        self.w_in = torch.cat([tensors["q"], tensors["k"], tensors["v"], tensors["g"]], 0).contiguous()
        self.w_gates = torch.cat([tensors["b"], tensors["a"]], 0).contiguous()
        self.w_out = tensors["o"]
        self.conv_w = torch.cat([tensors["q.conv"], tensors["k.conv"], tensors["v.conv"]], 0).contiguous()
        self.a_log, self.dt_bias, self.gain = tensors["A_log"], tensors["dt_bias"], tensors["norm"]
        self.dtype = dtype
        self._declare()

    def state_bytes(self) -> int:
        return self.s_bytes + self.tail_bytes

    def run_branch(self, ctx, proj, gates, act, out_scale, binding):
        t, H, G, D, E, C = proj.shape[0], self.H, self.G, self.D, self.E, self.C
        state = ctx.state(binding)
        qkv = ctx.scratch("delta.qkv", (t, C), torch.float32)
        beta = ctx.scratch("delta.beta", (t, H), torch.float32)
        decay = ctx.scratch("delta.decay", (t, H), torch.float32)
        o = ctx.scratch("delta.o", (t, H * E), torch.float32)
        kernels.delta_prepare(proj, self.conv_w, self.taps, gates, self.a_log, self.dt_bias, ctx,
                              state, self.s_bytes, qkv, beta, decay, H, G, D, E)
        kernels.conv_tail_update(proj, self.taps, C, ctx, state, self.s_bytes)
        kernels.matrix_memory(kernels.DELTA, qkv, 0, G * D, 2 * G * D, decay, beta, ctx, state, 0, 0,
                              0, o, H, G, D, E)
        kernels.head_norm_gate(o, self.gain, False, proj[:, C:C + H * E], act, kernels.GATE_SILU, H, E,
                               self.eps, out_scale)


class MLSTM(BranchMixer):
    def __init__(self, spec: MixerSpec):
        s = self.spec = spec
        self.H, self.D = s.n_heads, s.head_dim
        self.E = int(s.option("value_dim", s.head_dim))
        self.cap = float(s.option("gate_cap", 15.0))
        self.eps = float(s.option("norm_eps", 1e-6))
        if self.H <= 0 or self.D <= 0 or self.E <= 0 or self.cap <= 0:
            raise ValueError("mlstm: heads, sizes and the gates' cap must be positive")
        if self.D > 256:
            raise ValueError("mlstm: key size up to 256")
        self.s_bytes = _round16(4 * self.H * self.D * self.E)
        self.n_bytes = _round16(4 * self.H * self.D)
        self.m_bytes = _round16(4 * self.H)

    def tensors(self):
        d, H, D, E = self.spec.width, self.H, self.D, self.E
        return [TensorDecl("q", (H * D, d)), TensorDecl("k", (H * D, d)), TensorDecl("v", (H * E, d)),
                TensorDecl("g", (H * E, d)), TensorDecl("o", (d, H * E)),
                TensorDecl("norm", (H * E,), role="vector"),
                TensorDecl("i", (H, d)), TensorDecl("i.b", (H,), role="vector", init=("normal", 0.0, 1.0)),
                TensorDecl("f", (H, d)), TensorDecl("f.b", (H,), role="vector", init=("uniform", 1.0, 4.0))]

    def bind(self, tensors, dtype, device):
        self.w_in = torch.cat([tensors["q"], tensors["k"], tensors["v"], tensors["g"]], 0).contiguous()
        self.w_gates = torch.cat([tensors["i"], tensors["f"]], 0).contiguous()
        self.w_out = tensors["o"]
        self.bias_i, self.bias_f, self.gain = tensors["i.b"], tensors["f.b"], tensors["norm"]
        self.dtype = dtype
        self._declare()

    def state_bytes(self) -> int:
        return self.s_bytes + self.n_bytes + self.m_bytes

    def run_branch(self, ctx, proj, gates, act, out_scale, binding):
        t, H, D, E = proj.shape[0], self.H, self.D, self.E
        C = 2 * H * D + H * E
        state = ctx.state(binding)
        qkv = ctx.scratch("mlstm.qkv", (t, C), torch.float32)
        log_keep = ctx.scratch("mlstm.keep", (t, H), torch.float32)
        log_in = ctx.scratch("mlstm.in", (t, H), torch.float32)
        o = ctx.scratch("mlstm.o", (t, H * E), torch.float32)
        kernels.mlstm_prepare(proj, gates, self.bias_i, self.bias_f, self.cap, qkv, log_keep, log_in,
                              H, D, E)
        kernels.matrix_memory(kernels.MLSTM, qkv, 0, H * D, 2 * H * D, log_keep, log_in, ctx, state, 0,
                              self.s_bytes, self.s_bytes + self.n_bytes, o, H, H, D, E)
        kernels.head_norm_gate(o, self.gain, True, proj[:, C:C + H * E], act, kernels.GATE_SIGMOID, H, E,
                               self.eps, out_scale)


MIXERS.register("gated_delta", GatedDeltaRule)
MIXERS.register("mlstm", MLSTM)
