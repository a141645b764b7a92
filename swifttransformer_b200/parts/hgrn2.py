"""The HGRN2 mixer: a gated linear recurrence whose forget gate also decides what is written.

Per head, with q_t = silu(W_q h_t) [dim], v_t = W_v h_t [vdim] and the forget gate
f_t = lower + (1 - lower) * sigmoid(W_f h_t + b_f) [dim]  (``lower`` a per-channel lower bound):

    S_t = diag(f_t) S_{t-1} + (1 - f_t) v_t^T          S: [dim, vdim], zero when a request starts
    o_t = S_t^T q_t

each head's o_t is RMS-normed over vdim with one weight vector shared by the heads, the heads are concatenated
and projected.  S is float32 and lives in a state slot per request; gates, the recurrence and the norm are
float arithmetic, the three projections are one product.
"""
from __future__ import annotations

from typing import Any, Dict, List

import torch

from .. import ops
from ..weights.spec import GAIN, MATRIX, VECTOR, ParamSpec
from .base import MIXERS, Delta, Mixer, StateSpec


@MIXERS.register("hgrn2")
class HGRN2(Mixer):
    """names: {"q","f","v","o"} matrices [out, in], "f_bias" and "lower" [heads * dim], "norm" [vdim]."""

    def __init__(self, hidden: int, num_heads: int, dim: int, vdim: int, eps: float, names: Dict[str, str]):
        self.hidden, self.nh, self.dim, self.vdim, self.eps, self.names = hidden, num_heads, dim, vdim, float(eps), dict(names)
        self.w_qfv = self.w_o = self.f_bias = self.lower = self.norm_w = None

    def param_specs(self) -> List[ParamSpec]:
        n, qw, vw = self.names, self.nh * self.dim, self.nh * self.vdim
        return [ParamSpec(n["q"], (qw, self.hidden), MATRIX), ParamSpec(n["f"], (qw, self.hidden), MATRIX),
                ParamSpec(n["v"], (vw, self.hidden), MATRIX), ParamSpec(n["o"], (self.hidden, vw), MATRIX),
                ParamSpec(n["f_bias"], (qw,), VECTOR), ParamSpec(n["lower"], (qw,), VECTOR),
                ParamSpec(n["norm"], (self.vdim,), GAIN)]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        self.w_qfv = torch.cat([tensors.pop(n[k]) for k in "qfv"], dim=0).contiguous()
        self.w_o = tensors.pop(n["o"])
        self.f_bias, self.lower, self.norm_w = tensors[n["f_bias"]], tensors[n["lower"]], tensors[n["norm"]]

    def cache_spec(self):
        return StateSpec((self.nh, self.dim, self.vdim), torch.float32)

    def forward(self, h: torch.Tensor, ctx: Any, cache: Any) -> Delta:
        qw = self.nh * self.dim
        proj = ops.linear(h, self.w_qfv)
        o = torch.empty((h.shape[0], self.nh * self.vdim), dtype=h.dtype, device=h.device)
        ops.hgrn2_scan(proj, 0, qw, 2 * qw, self.f_bias, self.lower, self.norm_w, self.eps, cache.state, o,
                       ctx.positions, ctx.q_start, ctx.slots, ctx.n_seqs, self.nh, self.dim, self.vdim,
                       scratch=ctx.scratch_f32(h.shape[0] * self.nh * (self.vdim + 2 * self.dim)) if self.dim <= 128 else None)
        return Delta(ops.linear(o, self.w_o))

    def param_bytes(self) -> int:
        return (self.w_qfv.numel() + self.w_o.numel()) * self.w_qfv.element_size()
