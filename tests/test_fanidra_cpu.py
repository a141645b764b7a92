"""The Fanidra design's host side on the CPU: configuration, tensor names, cache needs, page release under a
block-diagonal mask.  (What runs kernels is in test_fanidra_gpu.py.)"""
from __future__ import annotations

import json

import pytest
import torch

from swifttransformer_b200.cache.manager import CacheManager, PagedCacheView, StateView
from swifttransformer_b200.config import ConfigError, FanidraConfig, load_config
from swifttransformer_b200.models import build_model_def, write_random_model
from swifttransformer_b200.parts.base import PagedKVSpec, StateSpec


def raw_config():
    att = {"type": "attention", "mlp": {"kind": "dense", "ff": 40},
           "mixer": dict(heads=4, kv_heads=2, dim=8, vdim=12, conv=3, scale=0.3, diff=0.2, softcap=10.0,
                         mask={"size": 20}, rot={"dims": 4, "base": 100.0})}
    rec = {"type": "hgrn2", "mlp": None, "mixer": dict(heads=2, dim=6, vdim=10)}
    return dict(architecture="Fanidra", vocab=50, width=24, norm={"eps": 1e-5}, residual_mult=0.5,
                embedding={"scale": 3.0}, canon={"taps": 4}, layers=[att, rec, att])


def test_config_round_trip_and_registry(tmp_path):
    cfg = FanidraConfig.from_dict(raw_config())
    assert cfg.canon_taps == 4 and cfg.embedding_scale == 3.0 and len(cfg.layers) == 3
    write_random_model(str(tmp_path), cfg, seed=0, std=0.1)
    again = load_config(str(tmp_path))
    assert isinstance(again, FanidraConfig) and again == FanidraConfig.from_dict(json.loads(json.dumps(cfg.to_dict())))


@pytest.mark.parametrize("change,word", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["layers"][0].update(type="window"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=5), "rot.dims"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "mlp.kind"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
])
def test_config_errors_name_the_key(change, word):
    raw = raw_config()
    change(raw)
    with pytest.raises(ConfigError) as e:
        FanidraConfig.from_dict(raw)
    assert word in str(e.value)


def test_tensor_names_shapes_and_cache_needs():
    mdef = build_model_def(FanidraConfig.from_dict(raw_config()))
    specs = {s.name: tuple(s.shape) for s in mdef.param_specs()}
    assert specs["embed"] == (50, 24) and specs["head"] == (50, 24) and specs["final.norm"] == ()
    assert specs["l0.mix.q"] == (4 * 2 * 8, 24) and specs["l0.mix.k"] == (2 * 2 * 8, 24) and specs["l0.mix.v"] == (2 * 12, 24)
    assert specs["l0.mix.q.conv"] == (64, 3) and specs["l0.mix.o"] == (24, 48) and specs["l0.canon1"] == (24, 4)
    assert specs["l1.mix.f.b"] == (12,) and specs["l1.mix.norm"] == (10,) and specs["l1.mix.o"] == (24, 20)
    assert "l1.norm2" not in specs and "l1.mlp.gate" not in specs and "l2.norm2" in specs
    needs = mdef.cache_specs()
    conv, (tails, pages) = needs[0]
    assert conv == StateSpec((3, 24)) and tails == StateSpec((2, 64 + 32 + 24))
    assert pages == PagedKVSpec(2, 16, None, value_dim=12, block=20)
    assert needs[1] == (StateSpec((3, 24)), StateSpec((2, 6, 10)))


def test_nested_cache_entries_share_a_pool_and_keep_their_states():
    mdef = build_model_def(FanidraConfig.from_dict(raw_config()))
    m = CacheManager(mdef.cache_specs(), torch.float32, "cpu", page_size=4, num_pages=16, max_seqs=2, max_seq_len=64)
    assert len(m.groups) == 1 and m.groups[0].kv.shape == (16, 2, 2 * 4 * (16 + 12))
    conv, (tails, pages) = m.entries()[0].view()
    assert isinstance(conv, StateView) and isinstance(tails, StateView) and isinstance(pages, PagedCacheView)
    assert conv.state.shape == (2, 3, 24) and tails.state.shape == (2, 2, 120) and pages.layer == 0
    assert m.entries()[2].view()[1][1].layer == 1 and m.entries()[2].view()[1][1].pool is pages.pool
    rec = m.entries()[1].view()[1]
    assert rec.state.shape == (2, 2, 6, 10)
    s = m.alloc_slot()
    rec.state[s].fill_(1.0)
    m.free_slot(s)
    assert m.alloc_slot() == s and float(rec.state[s].abs().sum()) == 0.0      # a slot is zero when handed out again


def test_block_mask_releases_the_pages_before_the_block():
    m = CacheManager([PagedKVSpec(1, 8, None, value_dim=4, block=20)], torch.float32, "cpu", page_size=4,
                     num_pages=12, max_seqs=1, max_seq_len=200)
    s = m.alloc_slot()
    g = m.groups[0]
    held = []
    for start in range(0, 100, 7):
        assert m.reserve(s, start, start + 7)
        m.commit(s, start + 7)
        held.append(g.pool.num_held)
        first_needed = ((start + 7) // 20 * 20) // 4
        assert min(g.pages[s]) >= first_needed
    assert max(held) <= (20 + 7) // 4 + 2      # one block and one portion, never the whole request
    m.check()
    assert g.peak_pages(100, 7) <= 8
