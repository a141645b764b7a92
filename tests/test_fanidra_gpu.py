"""The Fanidra design on the GPU against the plain implementation (tests/plain_fanidra.py).

Mechanisms alone (the kernels driven directly over a small paged cache and state slots, with inputs made so
that a single key or an edge decides the result), then whole models of several small configurations through
the trace replay (whole prompts, token-by-token decoding, portions down to two tokens, mixed batches with
pages and slots used again) and through ``LLMEngine.generate``.
"""
from __future__ import annotations

import json
import os

import numpy as np
import pytest
import torch

import helpers
import plain_fanidra as pf

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
TD = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device="cuda")


def ints(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device="cuda")


def bf16_round(a):
    """float64 array with values that bfloat16 holds exactly."""
    return torch.tensor(np.asarray(a), dtype=torch.float32).to(torch.bfloat16).double().numpy()


class Step:
    """The index arrays of one step for given (slot, start, n) entries, as the step function lays them out,
    with padding tokens at position -1 and padding requests behind."""

    def __init__(self, entries, pad_tokens=0, pad_requests=0):
        pos, seq, q_start, slots = [], [], [0], []
        for i, (slot, start, n) in enumerate(entries):
            pos += list(range(start, start + n))
            seq += [i] * n
            q_start.append(q_start[-1] + n)
            slots.append(slot)
        self.n = len(pos)
        pos += [-1] * pad_tokens
        seq += [0] * pad_tokens
        q_start += [self.n] * pad_requests
        slots += [0] * pad_requests
        self.n_rows, self.n_seqs = len(pos), len(entries) + pad_requests
        self.positions, self.seq, self.q_start, self.slots = ints(pos), ints(seq), ints(q_start), ints(slots)


def portions(total, sizes):
    out, pos, k = [], 0, 0
    while pos < total:
        n = min(sizes[k % len(sizes)], total - pos)
        out.append((pos, n))
        pos += n
        k += 1
    return out


# ------------------------------------------------------------------------------------------ short convolution
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps,sizes", [(3, (5, 1, 2, 1, 1, 9)), (4, (2, 1, 1, 1, 7, 3)), (2, (1,)), (1, (4, 3)), (8, (3, 2, 1, 20))])
def test_conv_residual_in_portions_equals_the_whole(dtype, taps, sizes):
    from swifttransformer_b200 import ops
    rng = np.random.default_rng(taps)
    C, T, slots = 70, 41, 3
    w = bf16_round(rng.normal(size=(C, taps)))
    xs = [rng.normal(size=(T - 3 * r, C)) for r in range(2)]
    state = torch.zeros((slots, taps - 1, C), device="cuda")
    state[1].fill_(7.0)        # a slot nobody uses must stay as it is
    got = [np.zeros_like(x) for x in xs]
    cuts = [portions(len(x), sizes) for x in xs]
    for k in range(max(len(c) for c in cuts)):
        entries, rows = [], []
        for r, slot in ((0, 2), (1, 0)):
            if k < len(cuts[r]):
                start, n = cuts[r][k]
                entries.append((slot, start, n))
                rows.append(xs[r][start:start + n])
        st = Step(entries, pad_tokens=3, pad_requests=2)
        x = dev(np.concatenate(rows + [np.full((3, C), 1e4)]))
        out = torch.zeros((st.n_rows, C), dtype=TD[dtype], device="cuda")
        ops.conv_residual(x, dev(w), state, out, st.positions, st.seq, st.q_start, st.slots)
        o, at = out.float().cpu().numpy(), 0
        for r in (0, 1):
            if k < len(cuts[r]):
                start, n = cuts[r][k]
                got[r][start:start + n] = o[at:at + n]
                at += n
    assert torch.all(state[1] == 7.0)
    tol = 1e-5 if dtype == "float32" else 2e-2
    for r in range(2):
        ref = xs[r].astype(np.float32).astype(np.float64)
        ref = ref + pf.causal_conv(ref, w)
        assert np.abs(got[r] - ref).max() < tol * np.abs(ref).max()


# ------------------------------------------------------------------------------------------ small elementwise
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [37, 320])
def test_norm_add_and_gated_act(dtype, width):
    from swifttransformer_b200 import ops
    rng = np.random.default_rng(width)
    x, y = rng.normal(size=(9, width)), bf16_round(rng.normal(size=(9, width)) * 3)
    xd = dev(x)
    pos = ints([0, 1, 2, -1, 4, 5, 6, 7, 8])
    act = torch.zeros((9, width), dtype=TD[dtype], device="cuda")
    ops.norm_add(xd, dev(y, TD[dtype]), dev([1.7]), 0.3, 1e-3, pos, out_act=act)
    ref = x.astype(np.float32) + 0.3 * pf.scalar_norm(y, 1.7, 1e-3)
    ref[3] = x[3]                   # a padding row is left alone
    assert np.abs(xd.cpu().numpy() - ref).max() < 1e-5
    live = [0, 1, 2, 4, 5, 6, 7, 8]
    tol = 1e-5 if dtype == "float32" else 1e-2
    assert np.all(np.abs(act.float().cpu().numpy()[live] - ref[live]) <= tol * (1 + np.abs(ref[live])))
    gu = bf16_round(rng.normal(size=(5, 2 * width)) * 2)
    out = ops.gated_act(dev(gu, TD[dtype]), "gelu_tanh").float().cpu().numpy()
    ref = pf.gelu_tanh(gu[:, :width]) * gu[:, width:]
    assert np.all(np.abs(out - ref) <= tol * (1 + np.abs(ref)))


# ------------------------------------------------------------------------------------------ the recurrence
@pytest.mark.parametrize("in_registers", [False, True, "gates"])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,d,dv", [(2, 20, 40), (1, 64, 16), (3, 8, 130), (2, 128, 36), (1, 5, 7)])
def test_hgrn2_scan_in_portions_and_token_by_token(dtype, H, d, dv, in_registers, monkeypatch):
    from swifttransformer_b200 import ops
    rng = np.random.default_rng(H * 100 + d)
    T = 75
    zq, zf, v = (bf16_round(rng.normal(size=(T, H * n))) for n in (d, d, dv))
    zf = bf16_round(zf * 3 + 2)                  # gates near one: the state remembers far back
    f_bias, lower = rng.normal(size=H * d) * 0.1, rng.uniform(0, 0.9, size=H * d)
    norm_w = 1 + 0.1 * rng.normal(size=dv)
    ref = pf.gated_recurrence(zq, zf, v, f_bias.astype(np.float32), lower.astype(np.float32),
                              norm_w.astype(np.float32), H, d, dv, 1e-5)
    proj = np.concatenate([zq, zf, v], axis=1)
    if in_registers == "gates":
        monkeypatch.setattr(ops, "HGRN2_GATES_MIN_TOKENS", 3)      # portions of four tokens and more prepare their gates
    for sizes in ((T,), (17, 2, 1, 1, 1, 30, 1, 1), (1,)):
        state = torch.zeros((3, H, d, dv), device="cuda")
        state[0].fill_(3.0)
        got = np.zeros_like(ref)
        for start, n in portions(T, sizes):
            st = Step([(1, start, n)], pad_tokens=2, pad_requests=1)
            rows = dev(np.concatenate([proj[start:start + n], np.full((2, proj.shape[1]), 50.0)]), TD[dtype])
            out = torch.zeros((st.n_rows, H * dv), dtype=TD[dtype], device="cuda")
            ops.hgrn2_scan(rows, 0, H * d, 2 * H * d, dev(f_bias), dev(lower), dev(norm_w), 1e-5, state, out,
                           st.positions, st.q_start, st.slots, st.n_seqs, H, d, dv,
                           scratch=torch.full((st.n_rows * H * (dv + 2 * d),), 9.0, device="cuda") if in_registers else None)
            got[start:start + n] = out.float().cpu().numpy()[:n]
        assert torch.all(state[0] == 3.0) and torch.all(state[2] == 0.0)
        assert np.abs(got - ref).max() < (2e-5 if dtype == "float32" else 3e-2) * np.abs(ref).max(), sizes


def test_hgrn2_padding_request_of_a_decode_step_leaves_slot_zero_alone():
    """A recorded decode step pads with requests of one token at position -1 whose slot index reads 0."""
    from swifttransformer_b200 import ops
    H, d, dv = 2, 8, 8
    state = torch.full((2, H, d, dv), 5.0, device="cuda")
    st = Step([], pad_tokens=2)
    st.q_start, st.slots, st.n_seqs = ints([0, 1, 2]), ints([0, 0]), 2
    rows = torch.ones((2, 2 * H * d + H * dv), device="cuda")
    out = torch.zeros((2, H * dv), device="cuda")
    for scratch in (None, torch.zeros(2 * H * dv, device="cuda")):
        ops.hgrn2_scan(rows, 0, H * d, 2 * H * d, dev(np.zeros(H * d)), dev(np.zeros(H * d)), dev(np.ones(dv)), 1e-5,
                       state, out, st.positions, st.q_start, st.slots, st.n_seqs, H, d, dv, scratch=scratch)
    conv = torch.full((2, 2, 16), 5.0, device="cuda")
    ops.conv_state_update(rows[:, :16].contiguous(), 16, conv, st.positions, st.q_start, st.slots, 2)
    assert torch.all(state == 5.0) and torch.all(conv == 5.0)


# ------------------------------------------------------------------------------------------ differential attention
class PagedHarness:
    """A small paged cache (shuffled pages), state slots and the sequence of kernels the mixer runs."""

    def __init__(self, H, G, d, dv, taps, page_size, dtype, n_slots=3, pages=64, entries=2, seed=0):
        self.H, self.G, self.d, self.dv, self.taps, self.ps, self.dtype = H, G, d, dv, taps, page_size, TD[dtype]
        self.C = (H + G) * 2 * d + G * dv
        self.entry = 1
        self.pool = torch.full((pages, entries, G * page_size * (2 * d + dv)), 1e3, dtype=self.dtype, device="cuda")
        self.max_pages = 64
        self.table = torch.full((n_slots, self.max_pages), -1, dtype=torch.int32, device="cuda")
        self.free = list(np.random.default_rng(seed).permutation(pages))
        self.held = {s: {} for s in range(n_slots)}
        self.state = torch.zeros((n_slots, taps - 1, self.C), device="cuda")
        self.status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def reserve(self, slot, start, n):
        for j in range(start // self.ps, (start + n - 1) // self.ps + 1):
            if j not in self.held[slot]:
                self.held[slot][j] = int(self.free.pop())
                self.table[slot, j] = self.held[slot][j]

    def release(self, slot):
        self.free.extend(self.held[slot].values())
        self.held[slot] = {}
        self.table[slot].fill_(-1)
        self.state[slot].zero_()

    def run(self, entries, rows, p, kernel="plain"):
        """entries: (slot, start, n); rows: the projections of the step's tokens [sum n, C]; p: constants."""
        from swifttransformer_b200 import ops
        for slot, start, n in entries:
            self.reserve(slot, start, n)
        st = Step(entries, pad_tokens=2, pad_requests=1)
        proj = dev(np.concatenate([rows, np.full((2, self.C), 9.0)]), self.dtype)
        q = torch.zeros((st.n_rows, self.H * 2 * self.d), dtype=self.dtype, device="cuda")
        out = torch.zeros((st.n_rows, self.H * self.dv), dtype=self.dtype, device="cuda")
        ops.diff_qkv_prepare(proj, p["conv_w"], self.state, p["q_norm"], p["k_norm"], p["eps"], p["inv_freq"],
                             p["rot_dims"], q, self.pool, self.entry, st.positions, st.seq, st.q_start, st.slots,
                             self.table, self.H, self.G, self.d, self.dv, self.ps, self.status)
        ops.conv_state_update(proj, self.C, self.state, st.positions, st.q_start, st.slots, st.n_seqs)
        consts = (self.H, self.G, self.d, self.dv, self.ps, p["scale"], p["cap"], p["block"], 0, p["lam"], p["eps"],
                  p["out_scale"])
        if kernel == "tiles" and ops.diff_attention_tiles_applies(q, self.d, self.dv):
            # as the mixer does it: portions of 16 tokens and more in tiles of 128 rows, the rest one by one
            tiles, items, first = [], [], 0
            for i, (slot, start, n) in enumerate(entries):
                if n >= 16:
                    tiles += [(i, off) for off in range(0, n, 128)]
                else:
                    items += list(range(first, first + n))
                first += n
            tiles.append((0, 1 << 24))                   # a padding tile
            items += [-1, -1]
            if len(tiles) > 1:
                ops.diff_attention_tiles(q, self.pool, self.entry, out, ints(tiles), len(tiles), 128, st.q_start,
                                         ints([e[1] for e in entries] + [0]), st.slots, self.table, *consts,
                                         status=self.status)
            ops.diff_attention_single(q, self.pool, self.entry, out, st.positions, st.seq, st.slots, self.table, *consts,
                                      status=self.status, items=ints(items), n_items=len(items))
        else:
            ops.diff_attention_plain(q, self.pool, self.entry, out, st.positions, st.seq, st.slots, self.table, *consts,
                                     status=self.status)
        assert int(self.status.item()) == 0
        return out.float().cpu().numpy()[:st.n]


def attention_case(H, G, d, dv, taps, rot_dims, block, cap, seed, T):
    rng = np.random.default_rng(seed)
    C = (H + G) * 2 * d + G * dv
    conv_w = bf16_round(rng.normal(size=(C, taps)) * 0.5)
    conv_w[:, -1] = 1.0
    c = dict(conv_w=conv_w, q_norm=bf16_round(1 + 0.2 * rng.normal(size=d)), k_norm=bf16_round(1 + 0.2 * rng.normal(size=d)),
             eps=1e-5, rot_dims=rot_dims, rot_base=500.0, scale=1.7 / np.sqrt(d), cap=cap, block=block, lam=0.37,
             out_scale=0.6)
    rows = bf16_round(rng.normal(size=(T, C)))
    return c, rows


def on_device(c, rot_base_dims):
    from swifttransformer_b200.parts.position import RotaryPairs
    p = dict(c)
    p["conv_w"], p["q_norm"], p["k_norm"] = dev(c["conv_w"]), dev(c["q_norm"]), dev(c["k_norm"])
    p["inv_freq"] = RotaryPairs(c["rot_dims"], c["rot_base"]).inv_freq("cuda") if c["rot_dims"] else p["q_norm"]
    p["block"] = c["block"] or 0
    return p


def plain_attention(c, rows, H, G, d, dv):
    qw, kw = H * 2 * d, G * 2 * d
    u = pf.causal_conv(rows, c["conv_w"])
    return pf.attend_two_maps(u[:, :qw], u[:, qw:qw + kw], u[:, qw + kw:], H, G, d, dv, c["q_norm"], c["k_norm"], c["eps"],
                              c["rot_dims"], c["rot_base"], c["scale"], c["cap"], c["block"], c["lam"], c["out_scale"])


SHAPES = [  # H, G, d, dv, taps, rot_dims, block, cap, page
    (4, 2, 16, 24, 3, 8, 40, 30.0, 16),
    (2, 2, 32, 16, 2, 32, 16, 0.0, 8),
    (3, 1, 10, 70, 4, 0, None, 5.0, 4),          # sizes the tile kernel does not take
    (1, 1, 64, 128, 1, 64, 100, 50.0, 32),
    (2, 1, 40, 72, 2, 16, 90, 20.0, 16),         # sizes between the tile kernel's rounded ones
    (1, 1, 128, 256, 2, 128, None, 0.0, 64),
]


KERNELS = [("float32", "plain"), ("bfloat16", "plain"), ("bfloat16", "tiles")]


@pytest.mark.parametrize("dtype,kernel", KERNELS)
@pytest.mark.parametrize("shape", SHAPES)
def test_differential_attention_whole_portions_and_decoding(dtype, kernel, shape):
    H, G, d, dv, taps, rot_dims, block, cap, page = shape
    T = 150
    c, rows = attention_case(H, G, d, dv, taps, rot_dims, block, cap, seed=H * 7 + d, T=T)
    ref = plain_attention(c, rows, H, G, d, dv)
    p = on_device(c, None)
    tol = (3e-5 if dtype == "float32" else 4e-2) * np.abs(ref).max()
    hz = PagedHarness(H, G, d, dv, taps, page, dtype, seed=d)
    for slot, sizes in ((0, (T,)), (2, (100, 1, 1, 1, 1, 1, 1)), (0, (3, 2, 37, 1, 2, 50, 2, 2))):
        got = np.zeros_like(ref)
        for start, n in portions(T, sizes):
            got[start:start + n] = hz.run([(slot, start, n)], rows[start:start + n], p, kernel)
        err = np.abs(got - ref).max(axis=1)
        assert err.max() < tol, (sizes, int(np.argmax(err > tol)), float(err.max()))
        hz.release(slot)          # the next case gets these pages and this slot again, with what they held


@pytest.mark.parametrize("dtype,kernel", KERNELS)
def test_differential_attention_batch_of_unequal_requests_equals_each_alone(dtype, kernel):
    H, G, d, dv, taps, rot_dims, block, cap, page = SHAPES[0]
    cases = [attention_case(H, G, d, dv, taps, rot_dims, block, cap, seed=5, T=T) for T in (90, 33, 61)]
    c = cases[0][0]
    p = on_device(c, None)
    refs = [plain_attention(c, rows, H, G, d, dv) for _, rows in cases]
    hz = PagedHarness(H, G, d, dv, taps, page, dtype)
    at = [0, 0, 0]
    got = [np.zeros_like(r) for r in refs]
    plan = [(20, 33, 2), (30, 0, 1), (1, 0, 17), (39, 0, 40), (0, 0, 1)]
    for step in plan:
        entries, parts = [], []
        for r, n in enumerate(step):
            n = min(n, len(refs[r]) - at[r])
            if n:
                entries.append((r, at[r], n))
                parts.append(cases[r][1][at[r]:at[r] + n])
        out, k = hz.run(entries, np.concatenate(parts), p, kernel), 0
        for r, start, n in entries:
            got[r][start:start + n] = out[k:k + n]
            k += n
            at[r] += n
    tol = (3e-5 if dtype == "float32" else 4e-2)
    for r in range(3):
        assert np.abs(got[r][:at[r]] - refs[r][:at[r]]).max() < tol * np.abs(refs[r]).max()


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("dtype,kernel", KERNELS)
def test_one_key_decides_at_block_edges_page_borders_and_far_back(dtype, kernel, decode):
    """The query at position t and the key at position j are scaled so that, if j is visible, map 1 puts all
    its weight on j: the result is then v_j (normalised).  j just inside the query's block, just outside it,
    on either side of a page border, the first key of the sequence, and hundreds of keys back."""
    H, G, d, dv, taps, page = 1, 1, 16, 32, 1, 16
    T = 330
    for block, pairs in ((64, [(70, 64), (70, 63), (127, 64), (128, 127), (128, 128), (65, 64), (64, 63)]),
                         (None, [(329, 0), (329, 1), (300, 15), (300, 16), (300, 17), (329, 328)])):
        for t, j in pairs:
            c, rows = attention_case(H, G, d, dv, taps, 0, block, 0.0, seed=t * 1000 + j, T=T)
            c["lam"], c["scale"] = 0.0, 3.0
            rows = rows * 0.05
            direction = np.zeros(d)
            direction[3] = 1.0
            rows[t, :d] = 50 * direction                 # query of map 1
            rows[j, 2 * d * H:2 * d * H + d] = 50 * direction   # key of map 1
            rows = bf16_round(rows)
            ref = plain_attention(c, rows, H, G, d, dv)
            lo = (t // block) * block if block else 0
            if j >= lo:     # the oracle itself must show the effect, or the case tests nothing
                v = rows[j, -dv:]
                assert np.abs(ref[t] - pf.rms(v, c["eps"]) * c["out_scale"]).max() < 0.05
            p = on_device(c, None)
            hz = PagedHarness(H, G, d, dv, taps, page, dtype, seed=t)
            if decode:
                hz.run([(1, 0, t)], rows[:t], p, kernel)
                got = hz.run([(1, t, 1)], rows[t:t + 1], p, kernel)[0]
            else:
                got = hz.run([(1, 0, t + 1)], rows[:t + 1], p, kernel)[t]
            assert np.abs(got - ref[t]).max() < (1e-4 if dtype == "float32" else 4e-2), (block, t, j)


# ------------------------------------------------------------------------------------------ whole models
def layer_attention(**kw):
    mixer = dict(heads=4, kv_heads=2, dim=16, vdim=24, conv=3, scale=0.25, diff=0.2, softcap=30.0,
                 mask={"size": 40}, rot={"dims": 8, "base": 10000.0})
    mixer.update(kw)
    return {"type": "attention", "mixer": {k: v for k, v in mixer.items() if v is not None}}


def layer_hgrn2(**kw):
    mixer = dict(heads=3, dim=20, vdim=40)
    mixer.update(kw)
    return {"type": "hgrn2", "mixer": mixer}


def with_mlp(layer, ff):
    return dict(layer, mlp={"kind": "dense", "ff": ff} if ff else None)


CONFIGS = {
    # attention and recurrence mixed, grouped heads, a layer without feed-forward, partial rotation
    "mix": dict(cfg=dict(architecture="Fanidra", vocab=300, width=96, norm={"eps": 1e-6}, residual_mult=0.5,
                         embedding={"scale": 3.0}, canon={"taps": 4},
                         layers=[with_mlp(layer_attention(), 160), with_mlp(layer_hgrn2(), None),
                                 with_mlp(layer_attention(heads=2, kv_heads=2, dim=32, vdim=16, conv=2,
                                                          mask={"size": 16}, rot={"dims": 32, "base": 100.0},
                                                          softcap=None), 64),
                                 with_mlp(layer_hgrn2(heads=1, dim=64, vdim=16), 200)]),
                seed=3, std=0.08, page_size=16),
    # only recurrences: no page group at all, no input convolution, no embedding scale
    "rec": dict(cfg=dict(architecture="Fanidra", vocab=200, width=64, norm={"eps": 1e-5},
                         layers=[with_mlp(layer_hgrn2(heads=2, dim=16, vdim=32), 96),
                                 with_mlp(layer_hgrn2(heads=4, dim=8, vdim=8), 96)]),
                seed=4, std=0.1, page_size=8),
    # one key/value head, no mask (all keys stay), no rotation, odd sizes, pages of 4
    "att": dict(cfg=dict(architecture="Fanidra", vocab=257, width=72, norm={"eps": 1e-4}, residual_mult=1.0,
                         embedding={"scale": 0.5}, canon={"taps": 2},
                         layers=[with_mlp(layer_attention(heads=3, kv_heads=1, dim=10, vdim=70, conv=4, mask=None,
                                                          rot=None, softcap=5.0, diff=0.45, scale=0.6), 100),
                                 with_mlp(layer_attention(heads=1, kv_heads=1, dim=24, vdim=24, conv=1,
                                                          mask={"size": 7}, rot={"dims": 24, "base": 50.0}), None)]),
                seed=5, std=0.1, page_size=4),
}


@pytest.fixture(scope="module")
def fanidra_dirs(tmp_path_factory):
    from swifttransformer_b200.config import FanidraConfig
    from swifttransformer_b200.models import write_random_model
    root = tmp_path_factory.mktemp("fanidra")
    out = {}
    for name, c in CONFIGS.items():
        out[name] = write_random_model(str(root / name), FanidraConfig.from_dict(c["cfg"]), seed=c["seed"], std=c["std"])
    return out


_PLAIN = {}


def plain_logits(model_dir, tokens):
    key = (model_dir, tuple(tokens))
    if key not in _PLAIN:
        if model_dir not in _PLAIN:
            _PLAIN[model_dir] = pf.load_model(model_dir)
        cfg, w = _PLAIN[model_dir]
        _PLAIN[key] = pf.forward(cfg, w, tokens)
    return _PLAIN[key]


def requests_for(name, lengths=(150, 1, 23, 97, 64)):
    vocab = CONFIGS[name]["cfg"]["vocab"]
    return {f"r{i}": helpers.random_tokens(vocab, n, seed=10 * i + len(name)) for i, n in enumerate(lengths)}


def compare(model_dir, reqs, got, dtype, what):
    tol = {"float32": 3e-5, "bfloat16": 5e-2}[dtype]
    for rid, toks in reqs.items():
        ref = plain_logits(model_dir, toks)
        assert got[rid].shape == ref.shape, (what, rid)
        scale = np.abs(ref).max()
        bad = helpers.first_bad(got[rid], ref, tol * scale)
        assert bad is None, f"{what}/{dtype}: request {rid} first differs at position {bad[0]} of {len(toks)} by {bad[1]:.3e} of {scale:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("schedule", ["whole", "decode", "portions", "mixed"])
def test_replay_matches_plain(fanidra_dirs, name, dtype, schedule):
    from swifttransformer_b200.engine.replay import TraceSession
    reqs = requests_for(name)
    steps = {"whole": helpers.trace_whole, "decode": lambda r: helpers.trace_decode_tail(r, tail=45),
             "portions": helpers.trace_portions, "mixed": lambda r: helpers.trace_mixed(r, seed=1, max_live=3)}[schedule](reqs)
    need = helpers.live_token_need(steps)
    s = TraceSession(fanidra_dirs[name], dtype, need, page_size=CONFIGS[name]["page_size"], max_requests=3)
    got = helpers.replay(s, steps)
    compare(fanidra_dirs[name], reqs, got, dtype, f"{name}/{schedule}")
    s.cache.check()
    assert all(g.pool.num_held == 0 for g in s.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
def test_recorded_and_eager_steps_agree(fanidra_dirs, dtype):
    from swifttransformer_b200.engine.replay import TraceSession
    reqs = requests_for("mix", lengths=(70, 9))
    steps = helpers.trace_mixed(reqs, seed=2, max_live=2)
    outs = []
    for graphs in (True, False):
        s = TraceSession(fanidra_dirs["mix"], dtype, helpers.live_token_need(steps), max_requests=2)
        s.runner.use_cuda_graphs = graphs
        outs.append(helpers.replay(s, steps))
    # a recorded step has a padded shape, and the kernels choose their forms by shape (how many lanes share a column
    # of the recurrence's state, which product kernel): the sums are the same, their order need not be
    for rid in reqs:
        tol = 1e-5 if dtype == "float32" else 2e-2
        assert np.abs(outs[0][rid] - outs[1][rid]).max() < tol * np.abs(outs[1][rid]).max()


def test_block_mask_gives_pages_back_while_a_request_runs(fanidra_dirs):
    """With a block-diagonal mask no query reads before its block: a long request holds pages for little more
    than one block and a portion, and pages are used again within the request."""
    from swifttransformer_b200.engine.replay import TraceSession
    name = "mix"
    toks = helpers.random_tokens(CONFIGS[name]["cfg"]["vocab"], 400, seed=9)
    s = TraceSession(fanidra_dirs[name], "float32", 448, max_requests=1)
    rows, peak = [], 0
    for start, n in portions(400, (30, 1, 1, 25)):
        out = s.run_step([dict(id="a", tokens=toks[start:start + n], want=list(range(n)))])
        rows.append(out.cpu().numpy().copy())
        peak = max(peak, max(g.pool.num_held for g in s.cache.groups))
    s.check()
    assert peak * 16 <= 40 + 30 + 2 * 16
    got = np.concatenate(rows)
    ref = plain_logits(fanidra_dirs[name], toks)
    assert np.abs(got - ref).max() < 3e-5 * np.abs(ref).max()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mix", "rec"])
def test_greedy_generation_through_the_engine(fanidra_dirs, name, dtype):
    from swifttransformer_b200.engine.engine import LLMEngine
    from swifttransformer_b200.sampling.sampler import SamplingParams
    vocab = CONFIGS[name]["cfg"]["vocab"]
    prompts = [helpers.random_tokens(vocab, n, seed=n) for n in (5, 31, 1, 18, 44, 9)]
    eng = LLMEngine(fanidra_dirs[name], dtype=dtype, page_size=CONFIGS[name]["page_size"], num_pages=24,
                    max_num_seqs=3, max_batch_tokens=48, chunk_size=20, max_seq_len=256)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=12, temperature=0.0))
    cfg, w = pf.load_model(fanidra_dirs[name])
    for prompt, out in zip(prompts, outs):
        toks = list(prompt)
        tokens = list(out.output if hasattr(out, "output") else out)
        assert len(tokens) == 12
        for k, tok in enumerate(tokens):
            logits = pf.forward(cfg, w, toks)[-1]
            best = int(np.argmax(logits))
            if tok != best:
                # a near tie may fall either way in bfloat16; anything else is a fault
                gap = logits[best] - logits[tok]
                assert dtype == "bfloat16" and gap < 0.05 * np.abs(logits).max(), (name, k, tok, best, gap)
            toks.append(tok)


# ------------------------------------------------------------------------------------------ the programs
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_run_gpt_takes_a_fanidra_folder(fanidra_dirs, tmp_path):
    import subprocess
    import sys
    vocab = CONFIGS["mix"]["cfg"]["vocab"]
    prompts = [helpers.random_tokens(vocab, n, 70 + n) for n in (6, 21)]
    inp = tmp_path / "in.txt"
    inp.write_text("\n".join(" ".join(map(str, p)) for p in prompts) + "\n")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "run_gpt"), fanidra_dirs["mix"], "any", "fp32", str(inp),
                        "--max_decoding_step", "5", "--num_total_blocks", "32"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    cfg, w = pf.load_model(fanidra_dirs["mix"])
    lines = [l for l in r.stdout.splitlines() if l.startswith("[")]
    assert len(lines) == 2
    for line, p in zip(lines, prompts):
        got = [int(t) for t in line.split(")")[1].split("(")[0].split()]
        toks = list(p)
        for tok in got:
            assert tok == int(np.argmax(pf.forward(cfg, w, toks)[-1]))
            toks.append(tok)
        assert len(got) == 5


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_run_program_with_four_slots(fanidra_dirs, tmp_path, dtype):
    """bin/trace_run with its defaults (four request slots, pages of 16): six requests, at most four live, so slots and
    pages are handed out again; every wanted row against the plain implementation."""
    import subprocess
    import sys
    name = "mix"
    reqs = requests_for(name, lengths=(50, 1, 33, 70, 18, 40))
    steps = helpers.trace_mixed(reqs, seed=3, max_live=4)
    out = tmp_path / "out"
    p = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", fanidra_dirs[name], "--dtype", dtype,
                          "--out", str(out), "--max-tokens", str(helpers.live_token_need(steps))],
                         stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    got = {rid: [] for rid in reqs}
    vocab = CONFIGS[name]["cfg"]["vocab"]
    for i, st in enumerate(steps):
        p.stdin.write(json.dumps(dict(st, step=i)) + "\n")
        p.stdin.flush()
        assert p.stdout.readline().strip() == f"done {i}", p.stderr.read()[-2000:]
        arr = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, vocab)
        k = 0
        for e in st["entries"]:
            got[e["id"]].append(arr[k:k + len(e["want"])])
            k += len(e["want"])
        assert k == len(arr)
    p.stdin.close()
    assert p.wait(timeout=120) == 0
    compare(fanidra_dirs[name], reqs, {rid: np.concatenate(v) for rid, v in got.items()}, dtype, "trace_run")
