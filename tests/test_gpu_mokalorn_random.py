"""Mokalorn configurations drawn at random (layer order, sizes, head counts, chunks, rotated values, temperatures, decays, experts
and constants) through the engine in four cuts and both dtypes, against the plain implementation."""
import random

import pytest

import trace_util as tu
from mokalorn_configs import attn, attn2, ret, moe, layer, model
from test_gpu_mokalorn import weights_for, engine_for, requests, expected_for, check

pytestmark = pytest.mark.gpu


def draw(seed):
    r = random.Random(seed)
    width = r.choice([24, 40, 56, 64, 72, 96, 128])
    layers = []
    for _ in range(r.randint(2, 6)):
        kind = r.choice(["attention", "attention_2", "retention"])
        if kind == "retention":
            heads, dim = r.choice([1, 2, 3, 4]), r.choice([4, 8, 12, 16, 24, 32, 64, 72])
            rot = None if r.random() < 0.25 else {"base": r.choice([10.0, 1e3, 1e4, 5e5]), "dims": r.choice([d for d in (2, 4, 8, dim) if d <= dim])}
            mixer = ret(heads, dim, r.choice([4, 8, 10, 16, 24, 40, 64]), [r.choice([1.0, 0.999, 0.97, 0.9, 0.7, 0.3]) for _ in range(heads)], rot)
        else:
            kv = r.choice([1, 2, 3])
            heads = kv * r.choice([1, 2, 4])
            dim = r.choice([4, 8, 10, 16, 24, 32, 64, 128])
            scale = r.choice([1.0, 0.5, 2.0]) * dim ** -0.5
            if kind == "attention":
                rot = None if r.random() < 0.2 else {"base": r.choice([20.0, 1e3, 1e4, 2e4]), "dims": r.choice([d for d in (2, 4, 8, 16, dim) if d <= dim])}
                chunk = None if r.random() < 0.15 else r.choice([1, 2, 5, 8, 13, 16, 24, 33, 64, 96, 300])
                mixer = attn(heads, kv, dim, scale, chunk=chunk, rot=rot)
            else:
                q_temp = None if r.random() < 0.25 else (r.choice([0.1, 0.5, 1.0, -0.2]), r.choice([1, 3, 8, 32, 100]))
                mixer = attn2(heads, kv, dim, r.choice([4, 8, 12, 16, 32, 64, 128]), scale, q_temp=q_temp)
        if r.random() < 0.2:
            mlp = None
        else:
            experts, identity = r.choice([0, 1, 2, 3, 5, 8, 12]), r.choice([0, 0, 1, 2, 3])
            if experts + identity == 0:
                identity = 1
            mlp = moe(experts, identity, r.randint(1, min(4, experts + identity)), r.choice([8, 16, 24, 40, 64]), r.choice([0.5, 1.0, 3.0, 7.0]))
        layers.append(layer(kind, mixer, mlp))
    return model(r.choice([50, 97, 128, 300]), width, r.choice([1e-6, 1e-5, 1e-3]), r.choice([0.5, 1.0, 4.0, 16.0]),
                 r.choice([None, 5.0, 30.0]), layers)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 8])
def test_random_configuration(seed, dtype):
    cfg = draw(seed)
    w = weights_for(cfg, 100 + seed)
    reqs = requests(cfg, [1, 2, 45, 130, 19, 77], seed=seed)
    exp = expected_for(cfg, w, reqs, dtype)
    page = random.Random(seed).choice([2, 4, 8, 16])
    for cut in (tu.whole, tu.prefill_then_decode, tu.portions, tu.mixed):
        steps = cut(reqs)
        tokens = tu.max_live_tokens(steps, rounding=page)
        eng = engine_for(cfg, w, dtype, page=page, pages=tokens // page + 2)
        check(tu.run_steps(eng, steps), exp, dtype)
