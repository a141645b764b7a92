"""A short causal convolution over time in front of a mixer.

``InputConv`` wraps any mixer: what the mixer reads, h, is replaced by
h + conv(h), one filter of ``taps`` weights per channel,

    conv(h)_t = sum_j w[:, j] * h_(t - taps + 1 + j)         (zeros before the request's start),

and the last taps - 1 inputs of every request live in a state slot beside the
wrapped mixer's own cache, so that a request may arrive in portions cut
anywhere.  The wrapper reads the float residual rows themselves (``reads_residual``)
and hands the mixer the result in the activation type.
"""
from __future__ import annotations

from typing import Any, Dict, List

import torch

from .. import ops
from ..weights.spec import VECTOR, ParamSpec
from .base import MIXERS, Delta, Mixer, Part, StateSpec


@MIXERS.register("input_conv")
class InputConv(Mixer):
    reads_residual = True

    def __init__(self, inner: Mixer, width: int, taps: int, name: str, residual: bool = True):
        if taps < 1:
            raise ValueError("a convolution needs at least one tap")
        self.inner, self.width, self.taps, self.name, self.residual = inner, width, int(taps), name, residual
        self.w = None

    @property
    def graph_safe(self) -> bool:
        return self.inner.graph_safe

    def children(self) -> List[Part]:
        return [self.inner]

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec(self.name, (self.width, self.taps), VECTOR)]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w = tensors[self.name]

    def cache_spec(self):
        return (StateSpec((self.taps - 1, self.width), torch.float32), self.inner.cache_spec())

    def step_plan(self):
        return self.inner.step_plan()

    def forward(self, h: torch.Tensor, ctx: Any, cache: Any) -> Delta:
        tails, inner_cache = cache
        out = torch.empty(h.shape, dtype=ctx.act_dtype, device=h.device)
        ops.conv_residual(h, self.w, tails.state, out, ctx.positions, ctx.seq_of_token, ctx.q_start, ctx.slots,
                          residual=self.residual)
        return self.inner.forward(out, ctx, inner_cache)

    def param_bytes(self) -> int:
        return (self.w.numel() * 4 if self.w is not None else 0) + self.inner.param_bytes()
