"""Mixers as branches, and the mixer that runs several of them side by side.

A branch mixer has the form  result = act(h W_in^T, h W_gates^T) W_out^T : one joint
input projection in the engine dtype (`input_weight()`: the rows of q, k, v, output
gate ... stacked), optionally a few gate logits that the recurrence needs in 32 bits
(`gate_weight()`, a product with a float32 result), its own work on those
(`run_branch`: rotation, cache, recurrence, norms, gating; the result, times a scale,
goes into columns it is given), and an output projection (`output_weight()`).

Alone, a branch runs these three products itself.  `ParallelMixer` stacks the input
matrices of its branches and places their output matrices beside one another, so the
whole mixer is still three products: every branch reads its columns of the joint
projection and writes its columns of one activation buffer, scaled by the branch's
weight, and  sum_b scale_b * branch_b(h)  is one product over the stacked columns.
"""
from __future__ import annotations

from dataclasses import replace
from typing import List, Optional

import torch

from .. import ops
from ..config.model_config import MixerSpec
from .base import MIXERS, CacheNeed, Mixer, TensorDecl


class BranchMixer(Mixer):
    can_overwrite = True           # forward(..., accumulate=False) writes the result instead

    dtype = None
    w_in: Optional[torch.Tensor] = None
    w_gates: Optional[torch.Tensor] = None
    w_out: Optional[torch.Tensor] = None

    # -- what a branch says of itself ------------------------------------------------
    def input_weight(self) -> torch.Tensor:
        return self.w_in

    def gate_weight(self) -> Optional[torch.Tensor]:
        return self.w_gates

    def output_weight(self) -> torch.Tensor:
        return self.w_out

    def run_branch(self, ctx, proj: torch.Tensor, gates: Optional[torch.Tensor],
                   act: torch.Tensor, out_scale: float, binding) -> None:
        """proj: [T, rows of input_weight] (a view of columns), gates: float32
        [T, rows of gate_weight] or None; writes act [T, columns of output_weight]."""
        raise NotImplementedError

    # -- alone -------------------------------------------------------------------------
    def _declare(self) -> None:
        ops.declare_weights(self.w_in, self.w_gates, self.w_out)

    def forward(self, ctx, h, residual, binding, accumulate: bool = True):
        run_products(ctx, self, [self], [1.0], [binding], h, residual, accumulate,
                     self.w_in, self.w_gates, self.w_out)


def run_products(ctx, owner, branches: List[BranchMixer], scales, bindings, h, out, accumulate,
                 w_in, w_gates, w_out) -> None:
    t = h.shape[0]
    tag = type(owner).__name__
    dtype = w_in.dtype          # the engine dtype (h may be rows that are not yet normalised)
    proj = ctx.scratch(f"{tag}.proj", (t, w_in.shape[0]), dtype)
    ops.linear(h, w_in, proj)
    gates = None
    if w_gates is not None:
        gates = ctx.scratch(f"{tag}.gates", (t, w_gates.shape[0]), torch.float32)
        ops.linear(h, w_gates, gates)
    act = ctx.scratch(f"{tag}.act", (t, w_out.shape[1]), dtype)
    p = g = a = 0
    for branch, scale, binding in zip(branches, scales, bindings):
        np_, na = branch.input_weight().shape[0], branch.output_weight().shape[1]
        gw = branch.gate_weight()
        ng = gw.shape[0] if gw is not None else 0
        branch.run_branch(ctx, proj[:, p:p + np_], gates[:, g:g + ng] if ng else None,
                          act[:, a:a + na], scale, binding)
        p, g, a = p + np_, g + ng, a + na
    ops.linear(act, w_out, out, accumulate=accumulate)


class ParallelMixer(Mixer):
    """sum_b scale_b * branch_b(h): branches read the same h.  The spec's options give
    `branches`: a tuple of (name, MixerSpec, scale); a branch's tensors are `<name>.<its
    own name>`.  At most one branch may keep a paged cache; each may keep state."""
    can_overwrite = True

    def __init__(self, spec: MixerSpec):
        self.spec = spec
        entries = spec.option("branches")
        if not entries:
            raise ValueError("a parallel mixer needs its branches")
        self.names = [name for name, _, _ in entries]
        self.scales = [float(scale) for _, _, scale in entries]
        self.branches: List[BranchMixer] = [MIXERS.build(s.kind, s) for _, s, _ in entries]
        for name, b in zip(self.names, self.branches):
            if not isinstance(b, BranchMixer):
                raise ValueError(f"branch {name!r} of a parallel mixer is not a branch mixer")
        if sum(b.cache_need() is not None for b in self.branches) > 1:
            raise ValueError("only one branch of a parallel mixer may keep a paged cache")
        self._state_offsets = []
        at = 0
        for b in self.branches:
            self._state_offsets.append(at)
            at += (int(b.state_bytes()) + 15) // 16 * 16
        self._state_total = at
        self.w_in = self.w_gates = self.w_out = None

    def tensors(self):
        return [replace(d, name=f"{name}.{d.name}")
                for name, b in zip(self.names, self.branches) for d in b.tensors()]

    def bind(self, tensors, dtype, device):
        for name, b in zip(self.names, self.branches):
            b.bind({k[len(name) + 1:]: v for k, v in tensors.items() if k.startswith(name + ".")},
                   dtype, device)
        self.w_in = torch.cat([b.input_weight() for b in self.branches], dim=0).contiguous()
        gates = [b.gate_weight() for b in self.branches if b.gate_weight() is not None]
        self.w_gates = torch.cat(gates, dim=0).contiguous() if gates else None
        self.w_out = torch.cat([b.output_weight() for b in self.branches], dim=1).contiguous()
        ops.declare_weights(self.w_in, self.w_gates, self.w_out)

    def cache_need(self) -> Optional[CacheNeed]:
        for b in self.branches:
            if b.cache_need() is not None:
                return b.cache_need()
        return None

    def state_bytes(self) -> int:
        return self._state_total

    def forward(self, ctx, h, residual, binding, accumulate: bool = True):
        bindings = [replace(binding, state_offset=binding.state_offset + off,
                            state_bytes=int(b.state_bytes()))
                    for b, off in zip(self.branches, self._state_offsets)]
        run_products(ctx, self, self.branches, self.scales, bindings, h, residual, accumulate,
                     self.w_in, self.w_gates, self.w_out)


MIXERS.register("parallel", ParallelMixer)
