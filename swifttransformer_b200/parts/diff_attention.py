"""Differential attention: two softmax maps per head over one set of values.

Per query head h (key/value head g = h // (heads / kv_heads)) and map a = 1, 2:

    q, k, v   = the projections of the mixer's input, each followed by a short causal convolution over time
                (one filter per channel, the last taps - 1 projected rows of a request kept as state)
    q_a, k_a  <- RMS norm over ``dim`` with one weight vector for the queries and one for the keys,
                 then rotation of pairs of dimensions by position (a ``rotary_pairs`` encoding)
    s_a       = cap * tanh(scale * q_a . k_a / cap)
    p_a       = softmax of s_a over the keys the query sees: those of its own block of ``block`` positions
                (counted from position 0 of the request), up to itself
    o         = p_1 V - lam * p_2 V,     lam = exp(lq1 . lk1) - exp(lq2 . lk2) + diff
    out       = o / sqrt(mean(o^2) + eps) * (1 - diff)        per head, over ``vdim``

and the heads' results go through the output projection.  The cache holds, per key/value head and position,
the two maps' keys side by side (2 * dim) and the values (vdim), in pages; a block-diagonal mask lets pages be
given back when the request has moved past their block.  lam is computed once, when the weights are bound.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional

import torch

from .. import ops
from ..weights.spec import MATRIX, VECTOR, GAIN, ParamSpec
from .attention import PagedAttentionPlan
from .base import MIXERS, Delta, Mixer, PagedKVSpec, StateSpec, StepPlan


@MIXERS.register("differential_attention")
class DifferentialAttention(Mixer):
    """names: tensor names of the projections {"q","k","v","o"} ([out, in] matrices; "<q|k|v>.conv" are their
    filters [channels, taps]), of the norm weights {"q_norm","k_norm"} and of the four vectors of lam
    {"lq1","lk1","lq2","lk2"}."""

    def __init__(self, hidden: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, conv_taps: int,
                 scale: float, softcap: float, block: Optional[int], diff: float, eps: float, names: Dict[str, str],
                 qk_position: Any = None, window: Optional[int] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads cannot share {num_kv_heads} key/value heads")
        self.hidden, self.nh, self.nkv, self.dim, self.vdim = hidden, num_heads, num_kv_heads, dim, vdim
        self.taps, self.scale, self.softcap = int(conv_taps), float(scale), float(softcap or 0.0)
        self.block, self.window = (int(block) if block else None), (int(window) if window else None)
        self.diff, self.eps, self.names, self.qk_position = float(diff), float(eps), dict(names), qk_position
        self.qw, self.kw, self.vw = num_heads * 2 * dim, num_kv_heads * 2 * dim, num_kv_heads * vdim
        self.w_qkv = self.w_o = self.conv_w = self.q_norm = self.k_norm = None
        self.lam = 0.0
        self._plan: Optional[PagedAttentionPlan] = None

    def step_plan(self) -> StepPlan:
        # the paged attention's sorting of a step's tokens: portions in tiles, short ones and single tokens as items
        if self._plan is None:
            self._plan = PagedAttentionPlan()
        return self._plan

    def param_specs(self) -> List[ParamSpec]:
        n, specs = self.names, []
        for key, rows in (("q", self.qw), ("k", self.kw), ("v", self.vw)):
            specs.append(ParamSpec(n[key], (rows, self.hidden), MATRIX))
            specs.append(ParamSpec(n[key] + ".conv", (rows, self.taps), VECTOR))
        specs.append(ParamSpec(n["o"], (self.hidden, self.nh * self.vdim), MATRIX))
        specs += [ParamSpec(n["q_norm"], (self.dim,), GAIN), ParamSpec(n["k_norm"], (self.dim,), GAIN)]
        specs += [ParamSpec(n[k], (self.dim,), VECTOR) for k in ("lq1", "lk1", "lq2", "lk2")]
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        self.w_qkv = torch.cat([tensors.pop(n[k]) for k in "qkv"], dim=0).contiguous()
        self.conv_w = torch.cat([tensors.pop(n[k] + ".conv") for k in "qkv"], dim=0).contiguous()
        self.w_o = tensors.pop(n["o"])
        self.q_norm, self.k_norm = tensors[n["q_norm"]], tensors[n["k_norm"]]
        lq1, lk1, lq2, lk2 = (tensors[n[k]].double().cpu() for k in ("lq1", "lk1", "lq2", "lk2"))
        self.lam = math.exp(float((lq1 * lk1).sum())) - math.exp(float((lq2 * lk2).sum())) + self.diff

    def cache_spec(self):
        # the convolution's last inputs (all q | k | v channels), and the pages of keys and values
        return (StateSpec((self.taps - 1, self.qw + self.kw + self.vw), torch.float32),
                PagedKVSpec(self.nkv, 2 * self.dim, self.window, value_dim=self.vdim, block=self.block))

    def forward(self, h: torch.Tensor, ctx: Any, cache: Any) -> Delta:
        tails, kv = cache
        n = h.shape[0]
        proj = ops.linear(h, self.w_qkv)
        q = torch.empty((n, self.qw), dtype=h.dtype, device=h.device)
        # a step of single tokens (decoding): the preparation kernel moves the convolution's state itself
        single = bool(getattr(ctx, "single_tokens", False))
        rot = self.qk_position
        rot_dims = rot.dims if rot is not None else 0
        inv_freq = rot.inv_freq(h.device) if rot is not None else self.q_norm
        ops.diff_qkv_prepare(proj, self.conv_w, tails.state, self.q_norm, self.k_norm, self.eps, inv_freq, rot_dims,
                             q, kv.pool, kv.layer, ctx.positions, ctx.seq_of_token, ctx.q_start, ctx.slots,
                             kv.block_table, self.nh, self.nkv, self.dim, self.vdim, kv.page_size, ctx.status,
                             write_kv=kv.writable, move_state=single and tails.writable)
        if self.taps > 1 and tails.writable and not single:
            ops.conv_state_update(proj, self.qw + self.kw + self.vw, tails.state, ctx.positions, ctx.q_start, ctx.slots,
                                  ctx.n_seqs)
        o = torch.empty((n, self.nh * self.vdim), dtype=h.dtype, device=h.device)
        consts = (self.nh, self.nkv, self.dim, self.vdim, kv.page_size, self.scale, self.softcap, self.block or 0,
                  self.window or 0, self.lam, self.eps, 1.0 - self.diff)
        if ops.diff_attention_tiles_applies(q, self.dim, self.vdim):
            # prompt portions in tiles of query rows on the tensor cores, short portions and single tokens one by one
            plan = ctx.plan(PagedAttentionPlan.name)
            if plan.n_tiles:
                ops.diff_attention_tiles(q, kv.pool, kv.layer, o, plan.tiles, plan.n_tiles, self._plan.tile_rows,
                                         ctx.q_start, ctx.start_pos, ctx.slots, kv.block_table, *consts,
                                         status=ctx.status)
            if plan.n_items:
                ops.diff_attention_single(q, kv.pool, kv.layer, o, ctx.positions, ctx.seq_of_token, ctx.slots,
                                          kv.block_table, *consts, status=ctx.status, items=plan.items,
                                          n_items=plan.n_items)
        else:
            ops.diff_attention_plain(q, kv.pool, kv.layer, o, ctx.positions, ctx.seq_of_token, ctx.slots,
                                     kv.block_table, *consts, status=ctx.status)
        return Delta(ops.linear(o, self.w_o))

    def param_bytes(self) -> int:
        return (self.w_qkv.numel() + self.w_o.numel()) * self.w_qkv.element_size()
