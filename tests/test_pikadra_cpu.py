"""The Pikadra design's host side on the CPU: configuration, order of layer runs, tensor names, cache needs.
(What runs kernels is in test_pikadra_gpu.py.)"""
from __future__ import annotations

import json

import pytest

from swifttransformer_b200.config import ConfigError, PikadraConfig, load_config
from swifttransformer_b200.models import build_model_def, write_random_model
from swifttransformer_b200.parts.base import PagedKVSpec

import plain_pikadra as pp


def mixer(heads=3, dim=6, rot_dim=4, vdim=10, kv_rank=14, q_rank=9, dims=None):
    return dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=0.3,
                rot={"dims": rot_dim if dims is None else dims, "base": 100.0})


def raw_config():
    dense = {"type": "latent_attention", "mixer": mixer(), "mlp": {"kind": "dense", "ff": 20}}
    moe = {"type": "latent_attention", "mixer": mixer(heads=2, kv_rank=8),
           "mlp": {"kind": "moe", "expert": {"ff": 12}, "router": {"experts": 5, "top": 2}, "shared": {"ff": 16}}}
    bare = {"type": "latent_attention", "mixer": mixer(dims=2), "mlp": None}
    return dict(architecture="Pikadra", vocab=50, width=24, norm={"eps": 1e-5}, embedding={"scale": 3.0},
                logit_scale=0.5, logit_softcap=20.0, loop={"start": 1, "stop": 3, "times": 3},
                layers=[dense, moe, bare, dense])


def test_config_round_trip_and_registry(tmp_path):
    cfg = PikadraConfig.from_dict(raw_config())
    assert cfg.loop == (1, 3, 3) and cfg.embedding_scale == 3.0 and cfg.logit_softcap == 20.0 and len(cfg.layers) == 4
    write_random_model(str(tmp_path), cfg, seed=0, std=0.1)
    again = load_config(str(tmp_path))
    assert isinstance(again, PikadraConfig) and again == PikadraConfig.from_dict(json.loads(json.dumps(cfg.to_dict())))
    # the oracle reads the same folder
    cfg2, w = pp.load_model(str(tmp_path))
    assert w["loop.in"].shape == (24, 48) and "head" not in w and cfg2["loop"]["times"] == 3


def test_what_the_file_does_not_mention_does_not_exist():
    raw = raw_config()
    for key in ("loop", "logit_softcap", "logit_scale", "embedding"):
        raw.pop(key)
    raw["layers"][1]["mlp"].pop("shared")
    cfg = PikadraConfig.from_dict(raw)
    assert cfg.loop is None and cfg.logit_softcap == 0.0 and cfg.logit_scale == 1.0 and cfg.embedding_scale == 1.0
    mdef = build_model_def(cfg)
    names = {s.name for s in mdef.param_specs()}
    assert "loop.in" not in names and "l1.mlp.shared.gate" not in names and "l1.mlp.shared.sg" not in names
    assert [st.block for st in mdef.layer_order] == [0, 1, 2, 3]


@pytest.mark.parametrize("change,word", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["layers"][0].update(type="window"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=6), "rot.dims"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "mlp.kind"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=6), "router.top"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
])
def test_config_errors_name_the_key(change, word):
    raw = raw_config()
    change(raw)
    with pytest.raises(ConfigError) as e:
        PikadraConfig.from_dict(raw)
    assert word in str(e.value)


def test_layer_runs_tensor_names_and_cache_needs():
    cfg = PikadraConfig.from_dict(raw_config())
    assert cfg.layer_runs() == pp.layer_runs(raw_config())
    mdef = build_model_def(cfg)
    specs = {s.name: tuple(s.shape) for s in mdef.param_specs()}
    assert specs["embed"] == (50, 24) and specs["final.norm"] == (24,) and specs["loop.step"] == (3, 24)
    assert specs["l0.mix.dq"] == (9, 24) and specs["l0.mix.uq"] == (3 * 10, 9) and specs["l0.mix.dkv"] == (18, 24)
    assert specs["l0.mix.uk"] == (18, 14) and specs["l0.mix.uv"] == (30, 14) and specs["l0.mix.o"] == (24, 30)
    assert specs["l0.mix.sink"] == (3,) and specs["l0.mix.g"] == (3, 24) and specs["l0.mix.dkv.norm"] == (14,)
    assert specs["l1.mlp.router"] == (5, 24) and specs["l1.mlp.e4.down"] == (24, 12) and specs["l1.mlp.shared.sg"] == (1, 24)
    assert "l2.mlp.gate" not in specs and specs["l3.mlp.up"] == (20, 24)
    # layer 0, then three passes over layers 1 and 2, each opened by the reentry block (index 4), then layer 3
    assert [(st.block, st.turn) for st in mdef.layer_order] == [(0, 0), (4, 0), (1, 0), (2, 0), (4, 1), (1, 0), (2, 0),
                                                                 (4, 2), (1, 0), (2, 0), (3, 0)]
    # every run of a layer has a cache entry of its own: one row [latent | shared rotated part] per token
    entries = [st.cache for st in mdef.layer_order if st.cache >= 0]
    assert entries == list(range(8))
    needs = mdef.cache_specs()
    assert needs[0] == PagedKVSpec(1, 14 + 4, None, value_dim=0) and needs[1] == PagedKVSpec(1, 8 + 4, None, value_dim=0)
    assert needs[1] == needs[3] == needs[5] and needs[2] == needs[4] == needs[0]
