"""The Mokalorn configuration, its model as data, and what its layers ask of the cache manager (no GPU)."""
import copy

import pytest
import torch

from mokalorn_configs import MOK_A, MOK_B, MOK_C, MOK_D

from tiny_transformer_inference_engine_b200 import ModelConfig
from tiny_transformer_inference_engine_b200.cache import CacheManager
from tiny_transformer_inference_engine_b200.config import ConfigError
from tiny_transformer_inference_engine_b200.config.mokalorn_config import MokalornConfig
from tiny_transformer_inference_engine_b200.models.model import Model
from tiny_transformer_inference_engine_b200.parts.base import PagedKVNeed, FixedStateNeed
from tiny_transformer_inference_engine_b200.parts.wkv import padded_keys
from tiny_transformer_inference_engine_b200.registry import model_spec
from tiny_transformer_inference_engine_b200.weights import random_tensors, write_random_model, read_safetensors


def test_architecture_picks_the_config_class_and_round_trips(tmp_path):
    cfg = ModelConfig.from_dict(MOK_A)
    assert isinstance(cfg, MokalornConfig)
    assert (cfg.vocab_size, cfg.d_model, cfg.norm_eps, cfg.embedding_scale, cfg.logit_softcap) == (131, 64, 1e-5, 4.0, 10.0)
    write_random_model(cfg, 3, str(tmp_path))
    again = ModelConfig.from_json(str(tmp_path))
    assert again == cfg and again.to_dict() == cfg.to_dict()
    stored = read_safetensors(str(tmp_path))
    assert set(stored) == set(Model(model_spec(cfg)).param_specs())
    assert ModelConfig.from_dict(MOK_D).logit_softcap is None


def test_tensor_names_and_shapes():
    specs = {k: tuple(v[2].shape) for k, v in Model(model_spec(ModelConfig.from_dict(MOK_A))).param_specs().items()}
    assert specs["embed"] == (131, 64) and specs["head"] == (131, 64) and specs["final.norm"] == (64,)
    # the first attention has no value projection; its gate is as large as the concatenated heads
    assert specs["l0.mix.q"] == (64, 64) and specs["l0.mix.k"] == (32, 64) and "l0.mix.v" not in specs
    assert specs["l0.mix.q.norm"] == (16,) and specs["l0.mix.k.norm"] == (16,)
    assert specs["l0.mix.g"] == (64, 64) and specs["l0.mix.o"] == (64, 64)
    # the second has one, at a value size of its own
    assert specs["l2.mix.q"] == (72, 64) and specs["l2.mix.k"] == (24, 64) and specs["l2.mix.v"] == (20, 64)
    assert specs["l2.mix.g"] == (60, 64) and specs["l2.mix.o"] == (64, 60) and specs["l2.mix.q.norm"] == (24,)
    assert "l2.norm2" not in specs and not any(k.startswith("l2.mlp") for k in specs)           # a layer without a feed-forward
    # retention: key and value sizes differ
    assert specs["l1.mix.q"] == (32, 64) and specs["l1.mix.k"] == (32, 64) and specs["l1.mix.v"] == (48, 64)
    assert specs["l1.mix.g"] == (48, 64) and specs["l1.mix.o"] == (64, 48)
    assert not any(k.startswith("l1.mix.") and k.endswith(".norm") for k in specs)              # its head norm has no weight
    # the router scores identity experts too; they have no tensors
    assert specs["l0.mlp.router"] == (7, 64) and specs["l0.mlp.correction"] == (7,)
    assert specs["l0.mlp.e4.gate"] == (40, 64) and specs["l0.mlp.e4.up"] == (40, 64) and specs["l0.mlp.e4.down"] == (64, 40)
    assert "l0.mlp.e5.gate" not in specs
    only_identity = {k for k in Model(model_spec(ModelConfig.from_dict(MOK_D))).param_specs() if k.startswith("l2.mlp.")}
    assert only_identity == {"l2.mlp.router", "l2.mlp.correction"}


def test_cache_needs():
    model = Model(model_spec(ModelConfig.from_dict(MOK_A)))
    needs = model.cache_needs()
    assert needs[0] == [PagedKVNeed(2, 16, None, None, chunk=11)] and needs[4] == needs[0]
    assert needs[2] == [PagedKVNeed(1, 32, None, None)]                       # keys of 24 and values of 20 in rows of 32
    assert needs[1] == [FixedStateNeed((2, 24, padded_keys(16)), "float32")]
    assert needs[3] == [FixedStateNeed((3, 8, padded_keys(24)), "float32")]


def test_pages_of_past_chunks_go_back():
    """Two groups: the chunked layers' (pages leave when the chunk of the next token starts behind them) and the causal
    layer's (every page stays)."""
    model = Model(model_spec(ModelConfig.from_dict(MOK_A)))
    mgr = CacheManager(model.cache_needs(), model.run_order, 4, 24, 2, "float32", "cpu")
    chunked = [i for i, g in enumerate(mgr.groups) if g.need.chunk == 11]
    causal = [i for i, g in enumerate(mgr.groups) if g.need.chunk is None]
    assert len(chunked) == 1 and len(causal) == 1
    mgr.admit("r")
    mgr.extend("r", 0, 30)                       # one step: positions 0..29 still read chunks 0, 1 and 2 in this step
    assert all(p != 0 for p in mgr.table(chunked[0], "r"))
    mgr.extend("r", 30, 31)                      # position 30 is in chunk 2 (22..32): keys before 22 are past, pages 0..4 hold 0..19
    assert [p != 0 for p in mgr.table(chunked[0], "r")] == [False] * 5 + [True] * 3
    assert all(p != 0 for p in mgr.table(causal[0], "r")) and len(mgr.table(causal[0], "r")) == 8
    mgr.extend("r", 31, 34)                      # 33 opens chunk 3, but 31 and 32 of this step still read chunk 2
    assert [p != 0 for p in mgr.table(chunked[0], "r")] == [False] * 5 + [True] * 4
    mgr.extend("r", 34, 35)
    assert [p != 0 for p in mgr.table(chunked[0], "r")] == [False] * 8 + [True]
    mgr.check()
    mgr.release("r")
    mgr.check()
    assert mgr.num_free_pages == mgr.num_usable_pages


@pytest.mark.parametrize("edit,text", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=24), "values are the keys"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5, 1.5]), "decay"),
    (lambda c: c["layers"][2]["mixer"]["q_temp"].update(every=0), "q_temp.every"),
    (lambda c: c["layers"][2]["mixer"]["q_temp"].pop("coef"), "coef"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "unknown"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=8), "top"),
    (lambda c: c["layers"][0]["mlp"]["expert"].pop("ff"), "ff"),
    (lambda c: c.pop("embedding"), "embedding"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.update(layers=[]), "at least one"),
])
def test_bad_configs_are_refused(edit, text):
    cfg = copy.deepcopy(MOK_A)
    edit(cfg)
    with pytest.raises(ConfigError, match=text):
        ModelConfig.from_dict(cfg)


@pytest.mark.parametrize("cfg", [MOK_A, MOK_B, MOK_C, MOK_D])
def test_every_configuration_builds(cfg):
    model = Model(model_spec(ModelConfig.from_dict(cfg)))
    assert len(model.cache_needs()) == len(cfg["layers"])


def test_random_weights_are_reproducible():
    cfg = ModelConfig.from_dict(MOK_B)
    a, b = random_tensors(cfg, 5), random_tensors(cfg, 5)
    assert all(torch.equal(a[k], b[k]) for k in a)
