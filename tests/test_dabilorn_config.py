"""The Dabilorn configuration, its model as data, its rescaled rotation frequencies, and what its layers ask of the cache
manager (no GPU)."""
import copy

import pytest
import torch

import plain_dabilorn as pd
from dabilorn_configs import ALL, DAB_A, DAB_B, DAB_C, DAB_D, DAB_E, yarn

from tiny_transformer_inference_engine_b200 import ModelConfig
from tiny_transformer_inference_engine_b200.cache import CacheManager
from tiny_transformer_inference_engine_b200.config import ConfigError
from tiny_transformer_inference_engine_b200.config.dabilorn_config import DabilornConfig
from tiny_transformer_inference_engine_b200.models.model import Model
from tiny_transformer_inference_engine_b200.parts.base import PagedKVNeed, FixedStateNeed, PartSpec
from tiny_transformer_inference_engine_b200.parts.wkv import padded_keys
from tiny_transformer_inference_engine_b200.registry import model_spec, build_part
from tiny_transformer_inference_engine_b200.weights import random_tensors, write_random_model, read_safetensors


def test_architecture_picks_the_config_class_and_round_trips(tmp_path):
    cfg = ModelConfig.from_dict(DAB_A)
    assert isinstance(cfg, DabilornConfig)
    assert (cfg.vocab_size, cfg.d_model, cfg.norm_eps, cfg.canon_taps) == (131, 64, 1e-5, 3)
    write_random_model(cfg, 3, str(tmp_path))
    again = ModelConfig.from_json(str(tmp_path))
    assert again == cfg and again.to_dict() == cfg.to_dict()
    stored = read_safetensors(str(tmp_path))
    assert set(stored) == set(Model(model_spec(cfg)).param_specs())
    assert ModelConfig.from_dict(DAB_D).canon_taps is None and "canon" not in ModelConfig.from_dict(DAB_D).to_dict()


def test_tensor_names_and_shapes():
    specs = {k: tuple(v[2].shape) for k, v in Model(model_spec(ModelConfig.from_dict(DAB_A))).param_specs().items()}
    assert specs["embed"] == (131, 64) and specs["embed.norm"] == (64,) and specs["final.norm"] == (64,) and "head" not in specs
    for i in range(5):
        assert specs[f"l{i}.norm1"] == (64,) and specs[f"l{i}.ls1"] == (64,) and specs[f"l{i}.canon1"] == (64, 3)
    # sigmoid attention: one norm weight per channel of the whole projection, a bias per head, a gate per value
    assert specs["l0.mix.q"] == (64, 64) and specs["l0.mix.k"] == (32, 64) and specs["l0.mix.v"] == (48, 64)
    assert specs["l0.mix.q.norm"] == (64,) and specs["l0.mix.k.norm"] == (32,) and specs["l0.mix.pb"] == (4,)
    assert specs["l0.mix.g"] == (96, 64) and specs["l0.mix.o"] == (64, 96)
    # time mixing
    assert specs["l1.mix.w1"] == (8, 64) and specs["l1.mix.w2"] == (32, 8) and specs["l1.mix.u"] == (2, 16) and specs["l1.mix.mu.w"] == (64,)
    # latent attention: queries through a latent of their own; the latent and one rotated key part come out of dkv
    assert specs["l2.mix.dq"] == (40, 64) and specs["l2.mix.dq.norm"] == (40,) and specs["l2.mix.uq"] == (3 * 20, 40)
    assert specs["l2.mix.dkv"] == (32, 64) and specs["l2.mix.dkv.norm"] == (24,)
    assert specs["l2.mix.uk"] == (36, 24) and specs["l2.mix.uv"] == (60, 24) and specs["l2.mix.g"] == (60, 64) and specs["l2.mix.o"] == (64, 60)
    assert "l2.mix.q" not in specs
    assert "l2.norm2" not in specs and "l2.ls2" not in specs and not any(k.startswith("l2.mlp") for k in specs)   # no feed-forward
    # experts without a gate matrix; the shared expert and its gate
    assert specs["l0.mlp.router"] == (5, 64) and specs["l0.mlp.e4.up"] == (40, 64) and specs["l0.mlp.e4.down"] == (64, 40)
    assert "l0.mlp.e4.gate" not in specs and "l0.mlp.e5.up" not in specs
    assert specs["l0.mlp.shared.up"] == (24, 64) and specs["l0.mlp.shared.down"] == (64, 24) and specs["l0.mlp.shared.sg"] == (1, 64)
    assert not any(k.startswith("l1.mlp.shared") for k in specs)
    no_conv = Model(model_spec(ModelConfig.from_dict(DAB_D))).param_specs()
    assert not any(k.endswith("canon1") for k in no_conv)


def test_cache_needs():
    needs = Model(model_spec(ModelConfig.from_dict(DAB_A))).cache_needs()
    tail = FixedStateNeed((2, 64), "float32")                               # the last taps - 1 stream rows, in every layer
    assert all(n[0] == tail for n in needs)
    assert needs[0][1:] == [PagedKVNeed(2, 32, None, None, chunk=11)]         # keys of 16 and values of 24 in rows of 32
    assert needs[1][1:] == [FixedStateNeed((2, 16, padded_keys(16)), "float32"), FixedStateNeed((64,), "float32")]
    assert needs[2][1:] == [PagedKVNeed(1, 32, None, None, planes=1)]         # the latent (24) and the rotated part (8): one plane
    assert needs[3][1:] == [PagedKVNeed(1, 32, None, None, chunk=32)]
    one_tap = Model(model_spec(ModelConfig.from_dict(DAB_B))).cache_needs()
    assert not any(isinstance(n, FixedStateNeed) and n.shape == (0, 50) for e in one_tap for n in e)
    assert one_tap[0] == [PagedKVNeed(1, 32, None, None, planes=1)]
    assert Model(model_spec(ModelConfig.from_dict(DAB_D))).cache_needs()[1] == [PagedKVNeed(2, 32, None, None)]     # no mask: every page stays


def test_pages_of_past_chunks_go_back():
    model = Model(model_spec(ModelConfig.from_dict(DAB_A)))
    mgr = CacheManager(model.cache_needs(), model.run_order, 4, 24, 2, "float32", "cpu")
    chunked = [i for i, g in enumerate(mgr.groups) if g.need.chunk == 11]
    causal = [i for i, g in enumerate(mgr.groups) if g.need.chunk is None]
    assert len(chunked) == 1 and len(causal) == 1                               # (both latent layers share the causal group)
    mgr.admit("r")
    mgr.extend("r", 0, 30)
    mgr.extend("r", 30, 31)                      # position 30 is in chunk 2 (22..32): pages 0..4 hold 0..19
    assert [p != 0 for p in mgr.table(chunked[0], "r")] == [False] * 5 + [True] * 3
    assert all(p != 0 for p in mgr.table(causal[0], "r")) and len(mgr.table(causal[0], "r")) == 8
    mgr.release("r")
    mgr.check()
    assert mgr.num_free_pages == mgr.num_usable_pages


@pytest.mark.parametrize("rot", [
    {"base": 50.0, "dims": 8, "scaling": yarn(4.0, 64, 8.0, 1.0)},
    {"base": 5e5, "dims": 12, "scaling": yarn(3.0, 1024, 16.0, 2.0)},          # the ramp ends inside the pairs
    {"base": 10.0, "dims": 6, "scaling": yarn(8.0, 32, 4.0, 0.5)},
    {"base": 1e4, "dims": 64, "scaling": yarn(16.0, 4096, 32.0, 1.0)},
    {"base": 1e4, "dims": 4, "scaling": yarn(3.0, 8, 1.0, 1.0)},               # lo == hi: the 0.001 floor decides
    {"base": 300.0, "dims": 10}])
def test_rescaled_frequencies_and_magnitude(rot):
    sc = rot.get("scaling")
    scaling = None if sc is None else dict(sc, kind="yarn")
    part = build_part("position", PartSpec("rope", "", {"dim": rot["dims"], "base": rot["base"], "style": "interleaved", "scaling": scaling}))
    f, mag = pd.frequencies(rot)
    got = part.frequencies().double()
    assert torch.allclose(got, torch.tensor(f, dtype=torch.float64), rtol=1e-6, atol=0)
    assert abs(part.magnitude - mag) < 1e-12
    if sc is not None:
        plain = torch.tensor([rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)], dtype=torch.float64)
        assert mag > 1.0 and (got <= plain * (1 + 1e-6)).all() and (got >= plain / sc["factor"] * (1 - 1e-6)).all()
        assert not torch.allclose(got, plain, rtol=1e-3)                        # the rescaling changes something


@pytest.mark.parametrize("edit,text", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(scaling=yarn(2.0, 64, 8.0, 1.0)), "rescaled"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"].pop("dim"), "dim"),
    (lambda c: c["layers"][2]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["layers"][2]["mixer"].update(rot_dim=7), "rot_dim"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=4), "rot.dims"),
    (lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].pop("slow"), "slow"),
    (lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].update(factor=0), "factor"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "unknown"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=8), "top"),
    (lambda c: c["layers"][0]["mlp"]["expert"].pop("ff"), "ff"),
    (lambda c: c["layers"][0]["mlp"]["shared"].pop("ff"), "ff"),
    (lambda c: c["canon"].update(taps=0), "canon.taps"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.update(layers=[]), "at least one"),
])
def test_bad_configs_are_refused(edit, text):
    cfg = copy.deepcopy(DAB_A)
    edit(cfg)
    with pytest.raises(ConfigError, match=text):
        ModelConfig.from_dict(cfg)


@pytest.mark.parametrize("name", sorted(ALL))
def test_every_configuration_builds(name):
    cfg = ALL[name]
    model = Model(model_spec(ModelConfig.from_dict(cfg)))
    assert len(model.cache_needs()) == len(cfg["layers"])


def test_decay_rank_left_to_the_weight_file():
    cfg = copy.deepcopy(DAB_E)
    del cfg["layers"][2]["mixer"]["decay_rank"]
    specs = Model(model_spec(ModelConfig.from_dict(cfg))).param_specs()
    assert tuple(specs["l2.mix.w1"][2].shape) == (-1, 48) and tuple(specs["l2.mix.w2"][2].shape) == (48, -1)
    with pytest.raises(ValueError, match="leaves a size"):
        random_tensors(ModelConfig.from_dict(cfg), 1)


def test_random_weights_are_reproducible():
    cfg = ModelConfig.from_dict(DAB_B)
    a, b = random_tensors(cfg, 5), random_tensors(cfg, 5)
    assert all(torch.equal(a[k], b[k]) for k in a)
