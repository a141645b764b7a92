"""Latent attention: queries through a normed latent, keys and values from one normed latent per token.

With h the mixer's input, H heads, per head ``dim`` unrotated and ``rot`` rotated query/key dimensions, values of
``vdim``, a key/value latent of ``kv_rank`` and a query latent of ``q_rank`` numbers:

    c_q   = rmsnorm(W_dq h) * w_qn                     q = W_uq c_q, per head [dim unrotated | rot rotated]
    [c'|r] = W_dkv h                                   c = rmsnorm(c') * w_kvn  (kv_rank numbers)
    k_rot = rotation of r by position                  one rotated key part of ``rot`` numbers for all heads
    k_h   = Uk_h c,  v_h = Uv_h c                      (W_uk, W_uv laid out head by head)
    s     = scale * (q_h . k_h + q_rot_h . k_rot)      over the keys up to the query's own position
    p     = softmax of s with exp(sink_h) as one more term of the denominator (no key, no value)
    out   = W_o concat_h( sigmoid(W_g h)_h * sum_j p_j v_h,j )

The cache holds per token only [c | k_rot] (kv_rank + rot numbers, whatever the number of heads), in pages.  The
kernels work in the latent space: q_h . k_h = (Uk_h^T q_h) . c, so the query of a head is multiplied by Uk_h^T once
(a product per head), the attention reads the cached rows as keys *and* (their first kv_rank numbers) as values,
and Uv_h is applied to the head's weighted sum of latents afterwards (a product per head).  The gate is a number
per (token, head) and commutes with Uv_h: the attention kernel applies it.  W_dq, W_dkv and W_g are one product.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch

from .. import ops
from ..weights.spec import GAIN, MATRIX, VECTOR, ParamSpec
from .base import MIXERS, Delta, Mixer, PagedKVSpec


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """names: tensor names {"dq", "uq", "dkv", "uk", "uv", "o"} ([out, in] matrices), {"q_norm", "kv_norm"} (the
    latents' norm weights), "sink" ([heads], or absent from the dict: no sink) and "gate" ([heads, hidden], or absent:
    no gate).  ``qk_position``: a ``rotary_halves`` encoding (its ``dims`` <= rot), or None."""

    def __init__(self, hidden: int, num_heads: int, dim: int, rot: int, vdim: int, kv_rank: int, q_rank: int,
                 scale: float, eps: float, names: Dict[str, str], qk_position: Any = None):
        self.hidden, self.nh, self.dim, self.rot, self.vdim = hidden, num_heads, dim, int(rot), vdim
        self.kr, self.qr, self.scale, self.eps, self.names = kv_rank, q_rank, float(scale), float(eps), dict(names)
        self.qk_position = qk_position
        if qk_position is not None and qk_position.dims > self.rot:
            raise ValueError("more rotated dimensions than the rotated part has")
        self.w_in = self.w_uq = self.w_ukt = self.w_uv = self.w_o = self.q_norm = self.kv_norm = self.sink = None

    @property
    def has_gate(self) -> bool:
        return "gate" in self.names

    def param_specs(self) -> List[ParamSpec]:
        n, H = self.names, self.nh
        specs = [ParamSpec(n["dq"], (self.qr, self.hidden), MATRIX), ParamSpec(n["q_norm"], (self.qr,), GAIN),
                 ParamSpec(n["uq"], (H * (self.dim + self.rot), self.qr), MATRIX),
                 ParamSpec(n["dkv"], (self.kr + self.rot, self.hidden), MATRIX), ParamSpec(n["kv_norm"], (self.kr,), GAIN),
                 ParamSpec(n["uk"], (H * self.dim, self.kr), MATRIX), ParamSpec(n["uv"], (H * self.vdim, self.kr), MATRIX),
                 ParamSpec(n["o"], (self.hidden, H * self.vdim), MATRIX)]
        if "sink" in n:
            specs.append(ParamSpec(n["sink"], (H,), VECTOR))
        if self.has_gate:
            specs.append(ParamSpec(n["gate"], (H, self.hidden), MATRIX))
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        n, H = self.names, self.nh
        first = [tensors.pop(n["dq"]), tensors.pop(n["dkv"])] + ([tensors.pop(n["gate"])] if self.has_gate else [])
        self.w_in = torch.cat(first, dim=0).contiguous()
        self.w_uq, self.w_o = tensors[n["uq"]], tensors[n["o"]]
        # Uk_h^T, head by head [kv_rank, dim]: the matrix that takes a head's unrotated query into the latent space
        self.w_ukt = tensors.pop(n["uk"]).view(H, self.dim, self.kr).transpose(1, 2).contiguous()
        self.w_uv = tensors.pop(n["uv"]).view(H, self.vdim, self.kr).contiguous()
        self.q_norm, self.kv_norm = tensors[n["q_norm"]], tensors[n["kv_norm"]]
        self.sink = tensors[n["sink"]] if "sink" in n else None

    def cache_spec(self) -> PagedKVSpec:
        # one row [latent | shared rotated key part] per token; the values are the row's first kv_rank numbers
        return PagedKVSpec(1, self.kr + self.rot, None, value_dim=0)

    def forward(self, h: torch.Tensor, ctx: Any, cache: Any) -> Delta:
        n, H, kd = h.shape[0], self.nh, self.kr + self.rot
        proj = ops.linear(h, self.w_in)
        cq = torch.empty((n, self.qr), dtype=h.dtype, device=h.device)
        rot = self.qk_position
        rot_dims = rot.dims if rot is not None else 0
        inv_freq = rot.inv_freq(h.device) if rot is not None else self.q_norm
        ops.latent_prepare(proj, self.qr, self.q_norm, self.kv_norm, self.eps, inv_freq, rot_dims, cq, cache.pool,
                           cache.layer, ctx.positions, ctx.seq_of_token, ctx.slots, cache.block_table, self.kr, self.rot,
                           cache.page_size, ctx.status, write_kv=cache.writable)
        q = ops.linear(cq, self.w_uq)
        q_lat = torch.empty((n, H * kd), dtype=h.dtype, device=h.device)
        ops.gemm_heads(q, self.w_ukt, q_lat, H, self.dim, self.kr, self.dim + self.rot, kd)
        if self.rot:
            ops.latent_q_rotate(q, q_lat, ctx.positions, inv_freq, rot_dims, H, self.dim, self.rot, self.kr)
        o_lat = torch.empty((n, H * self.kr), dtype=h.dtype, device=h.device)
        gates = proj[:, self.qr + kd:self.qr + kd + H] if self.has_gate else None
        ops.latent_attention(q_lat, cache.pool, cache.layer, o_lat, ctx.positions, ctx.seq_of_token, ctx.slots,
                             cache.block_table, H, self.kr, self.rot, cache.page_size, self.scale, self.sink, gates,
                             status=ctx.status, q_start=ctx.q_start, start_pos=ctx.start_pos, n_seqs=ctx.n_seqs,
                             scratch=ctx.scratch_f32)
        o = torch.empty((n, H * self.vdim), dtype=h.dtype, device=h.device)
        ops.gemm_heads(o_lat, self.w_uv, o, H, self.kr, self.vdim, self.kr, self.vdim)
        return Delta(ops.linear(o, self.w_o))

    def param_bytes(self) -> int:
        mats = (self.w_in, self.w_uq, self.w_ukt, self.w_uv, self.w_o)
        return sum(w.numel() * w.element_size() for w in mats)
