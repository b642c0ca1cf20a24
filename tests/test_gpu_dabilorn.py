"""The Dabilorn design in the engine against the plain implementation (plain_dabilorn.py): each mechanism alone, whole
prompts, decoding through the cache and the state slots, portions down to two tokens, mixed batches with pages and slots
used again, keys at the edges of chunks and pages and far back, other sizes, and greedy generation through the scheduler."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_dabilorn as pd
import trace_util as tu

from tiny_transformer_inference_engine_b200 import Engine, ModelConfig, EngineConfig, CacheConfig, SchedulerConfig, SamplingParams
from tiny_transformer_inference_engine_b200.parts.base import PartSpec, StepContext, PagedKVView, FixedStateView
from tiny_transformer_inference_engine_b200.registry import build_part
from tiny_transformer_inference_engine_b200.weights import random_tensors
from tiny_transformer_inference_engine_b200.models.dabilorn import _mixer, _ffn, _norm       # config.json's layer entry -> the part

from dabilorn_configs import ALL as CONFIGS, DAB_A, DAB_B, DAB_C, DAB_D, DAB_E, attn, latent, yarn

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def ops():
    from tiny_transformer_inference_engine_b200.ops import get_ops
    return get_ops(DEV)


def weights_for(cfg, seed, store="float32", sharp=True):
    """Random weights large enough that every mechanism matters: peaked attention, head biases and gates away from zero, layer
    scales and convolution taps of a size, router logits of a few units (the sub-layers read the stream itself, whose size
    grows from layer to layer: the router's rows are kept small so that the scores stay away from 1 and from each other)."""
    w = random_tensors(ModelConfig.from_dict(cfg), seed, std=0.08, perturb_norms=True, store_dtype=store)
    g = torch.Generator().manual_seed(seed + 1)
    for k in w:
        if sharp and k.endswith((".mix.q", ".mix.k", ".mix.uq", ".mix.dkv")):
            w[k] = w[k] * 3.0
        if sharp and k.endswith(".up"):
            w[k] = w[k] * 4.0
        if k.endswith(".mlp.router"):
            w[k] = w[k] * (0.6 / (w[k].float().std() * cfg["width"] ** 0.5))
        if k.endswith((".q.norm", ".k.norm", ".dq.norm", ".dkv.norm", ".ls1", ".ls2")):
            w[k] = (1.0 + torch.randn(w[k].shape, generator=g) * 0.3).to(w[k].dtype)
    return w


def engine_for(cfg, w, dtype, page=16, pages=64, max_seqs=4, budget=64, graphs=False):
    ec = EngineConfig(dtype=dtype, device=DEV, use_cuda_graphs=graphs,
                      cache=CacheConfig(block_size=page, num_gpu_blocks=pages),
                      sched=SchedulerConfig(max_num_seqs=max_seqs, max_num_batched_tokens=budget))
    return Engine(ModelConfig.from_dict(cfg), w, ec)


def requests(cfg, lens, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for i, n in enumerate(lens)}


def expected_for(cfg, w, reqs, dtype):
    ww = {k: (v.to(torch.bfloat16).double() if dtype == "bfloat16" and v.dtype.is_floating_point else v) for k, v in w.items()}
    return {rid: pd.forward(cfg, ww, toks) for rid, toks in reqs.items()}


def check(got, exp, dtype, tail16=0.15, worst32=1e-4):
    """32-bit: every place within 1e-4 of the row's largest logit.  bfloat16: these models are narrow and their weights are
    scaled up so that gates and routers bite; the sub-layers read the stream itself (nothing norms their input), an expert
    squares what it activates (a relative error doubles there) and the sigmoid weights of a chunk add up without a
    normalisation, so rounding alone moves a typical row by 2 to 4 % and a router's choice between two close experts, flipped
    by the rounding, moves one by tens of percent; the run is held to the typical error (every mechanism alone is held to
    its largest error in both dtypes below).  ``tail16``: what nine rows in ten stay below in bfloat16; ``worst32``: the bound on
    the worst row in 32-bit."""
    errs = []
    for (rid, pos), row in got.items():
        ref = exp[rid][pos]
        errs.append((((row.double() - ref).abs().max() / ref.abs().max()).item(), rid, pos))
    errs.sort(reverse=True)
    if dtype == "float32":
        assert errs[0][0] < worst32 and errs[len(errs) // 2][0] < 2e-5, errs[:3]
    else:
        n = len(errs)
        assert all(e[0] == e[0] for e in errs), "a NaN among the logits"
        assert errs[n // 2][0] < 6e-2 and errs[n // 10][0] < tail16, (errs[n // 2], errs[n // 10], errs[:3])


# ------------------------------------------------------------------------------------------ the whole model, four cuts
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_schedules_against_plain_model(name, dtype):
    cfg = CONFIGS[name]
    w = weights_for(cfg, 5 + ord(name))
    reqs = requests(cfg, [1, 2, 37, 70, 101, 23], seed=3)
    exp = expected_for(cfg, w, reqs, dtype)
    page = {"A": 16, "B": 8, "C": 4, "D": 2, "E": 16}[name]
    for cut in (tu.whole, tu.prefill_then_decode, tu.portions, tu.mixed):
        steps = cut(reqs)
        tokens = tu.max_live_tokens(steps, rounding=page)
        eng = engine_for(cfg, w, dtype, page=page, pages=tokens // page + 2)        # no slack: pages and slots are used again
        check(tu.run_steps(eng, steps), exp, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_wider_model_with_long_prompts_on_pages_of_16(dtype):
    """Six layers at head sizes of 64 (the tensor-core kernels' sizes on pages of 16 keys), prompts of several hundred tokens, a
    chunk that no page edge meets: whole, with a decoded tail, and mixed on a pool without slack.  The weights are the plain
    random ones (not sharpened): over six layers and hundreds of positions a model of this design has tokens at which rounding is
    magnified a hundredfold (the plain implementation run in 32-bit against itself in 64-bit shows the same rows: 7e-4 at one
    token of 700), so the worst row in 32-bit is held to 2e-3 and the typical row to 2e-5."""
    from dabilorn_configs import layer, moe, wkv, model
    cfg = model(200, 256, 1e-5, 3, [
        layer("latent_attention", latent(4, 64, 32, 64, 96, 80, 0.1, base=1e4, scaling=yarn(4.0, 256, 16.0, 1.0)), moe(6, 2, 64, shared=96)),
        layer("attention", attn(8, 2, 64, 64, 0.125, chunk=80, rot={"base": 5e4, "dims": 32}), moe(6, 2, 64, shared=96)),
        layer("wkv", wkv(4, 64, 12), moe(6, 2, 64, shared=96)),
        layer("attention", attn(4, 4, 64, 64, 0.125, chunk=208, rot={"base": 5e4, "dims": 64}), moe(6, 2, 64, shared=96)),
        layer("latent_attention", latent(4, 64, 32, 64, 96, 80, 0.1, base=1e4, scaling=yarn(4.0, 256, 16.0, 1.0)), moe(6, 2, 64, shared=96)),
        layer("wkv", wkv(4, 64, 12))])
    w = weights_for(cfg, 61, sharp=False)
    reqs = requests(cfg, [700, 333, 41, 290], seed=6)
    exp = expected_for(cfg, w, reqs, dtype)
    for cut in (tu.whole, tu.prefill_then_decode, tu.mixed):
        steps = cut(reqs)
        tokens = tu.max_live_tokens(steps, rounding=16)
        eng = engine_for(cfg, w, dtype, page=16, pages=tokens // 16 + 2, budget=1024)
        check(tu.run_steps(eng, steps), exp, dtype, worst32=2e-3)


def test_long_decode_past_chunks_and_pages():
    """A short prompt, then 150 tokens one by one: chunk edges (every 11 and every 32 positions) and many page edges pass under
    decoded tokens, the convolution's rows, the previous token's input and the time mixing's state are carried 150 times."""
    cfg = DAB_A
    w = weights_for(cfg, 77)
    reqs = requests(cfg, [160], seed=9)
    exp = expected_for(cfg, w, reqs, "float32")
    steps = tu.prefill_then_decode(reqs, tail=150)
    eng = engine_for(cfg, w, "float32", page=8, pages=24)
    check(tu.run_steps(eng, steps), exp, "float32")


def test_batch_of_unequal_requests_equals_each_alone():
    cfg = DAB_A
    w = weights_for(cfg, 21)
    reqs = requests(cfg, [3, 50, 1, 29], seed=4)
    eng = engine_for(cfg, w, "float32", pages=40)
    alone = tu.run_steps(eng, tu.whole(reqs))
    together = tu.run_steps(eng, [{"entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in reqs.items()],
                                   "end": list(reqs)}])
    for key, row in alone.items():
        assert (row - together[key]).abs().max() <= 2e-5 * row.abs().max(), key


def test_slots_and_pages_used_again_carry_nothing_over():
    """Two state slots and pages for one long request: the same request replayed after others have used (and dirtied) its slot
    and pages gives the same logits to the bit."""
    cfg = DAB_A
    w = weights_for(cfg, 23)
    reqs = requests(cfg, [40, 33, 40], seed=8)
    reqs["r2"] = list(reqs["r0"])
    eng = engine_for(cfg, w, "float32", page=8, pages=8, max_seqs=2)
    got = tu.run_steps(eng, tu.portions(reqs))
    for pos in range(40):
        assert torch.equal(got[("r0", pos)], got[("r2", pos)]), pos
    check(got, expected_for(cfg, w, reqs, "float32"), "float32")


def test_first_tokens_of_a_sequence():
    """Requests of one and two tokens, alone and beside a longer one, and the first positions of a prompt asked for one by one:
    position 0 sees itself only, the convolution finds zeros before it, the states start at zero."""
    for cfg_, page in ((DAB_B, 2), (DAB_C, 4)):
        w = weights_for(cfg_, 41)
        reqs = requests(cfg_, [1, 2, 3, 30], seed=5)
        exp = expected_for(cfg_, w, reqs, "float32")
        eng = engine_for(cfg_, w, "float32", page=page, pages=40)
        check(tu.run_steps(eng, tu.whole(reqs)), exp, "float32")
        check(tu.run_steps(eng, tu.prefill_then_decode(reqs, tail=29)), exp, "float32")
        steps = [{"entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in reqs.items()], "end": list(reqs)}]
        check(tu.run_steps(eng, steps), exp, "float32")


@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_scheduler(graphs):
    cfg = dict(DAB_A, max_seq_len=256)
    w = weights_for(cfg, 31)
    prompts = [[5, 9, 2], list(range(10, 41)), [7]]
    want = []
    for p in prompts:
        toks = list(p)
        for _ in range(14):                                           # past a chunk edge for every prompt
            toks.append(int(torch.argmax(pd.forward(cfg, w, toks)[-1])))
        want.append(toks[len(p):])
    eng = engine_for(cfg, w, "float32", pages=40, max_seqs=4, budget=16, graphs=graphs)
    got = eng.generate(prompts, SamplingParams(max_new_tokens=14, greedy=True))
    assert got == want


def test_command_line_and_trace_runner_with_a_model_folder(tmp_path):
    """A folder written in the random-weights mode (bfloat16 on disk), generated from by the command line and replayed by the
    trace runner: the architecture is picked from config.json by both."""
    import numpy as np
    from safetensors.torch import load_file
    from tiny_transformer_inference_engine_b200 import write_random_model
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = dict(DAB_E, max_seq_len=96)
    folder = write_random_model(ModelConfig.from_dict(cfg), 13, str(tmp_path / "model"), std=0.08, perturb_norms=True, store_dtype="bfloat16")
    w = load_file(os.path.join(folder, "model.safetensors"))
    prompt = [4, 60, 7, 7, 23]
    run = subprocess.run([sys.executable, "-m", "tiny_transformer_inference_engine_b200", "--model", folder, "--tokens", "6", "--greedy",
                          "--dtype", "float32", "--num-gpu-blocks", "16", "--prompt-ids", ",".join(map(str, prompt))],
                         cwd=root, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    toks = list(prompt)
    for _ in range(6):
        toks.append(int(torch.argmax(pd.forward(cfg, w, toks)[-1])))
    assert json.loads(run.stdout.strip().split("\n")[-1])["generated_ids"] == toks[len(prompt):]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:7], "want": [0, 6]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[7:9], "want": [1]}, {"id": "b", "tokens": toks[:3], "want": []}], "end": ["a"]},
             {"step": 2, "entries": [{"id": "b", "tokens": toks[3:4], "want": [0]}], "end": ["b"]}]
    out = tmp_path / "out"
    run = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", str(out), "--max-tokens", "128"],
                         input="\n".join(json.dumps(s) for s in steps) + "\n", cwd=root, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    assert [l for l in run.stdout.split("\n") if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    exp = pd.forward(cfg, w, toks)
    for name, rows in (("0.f32", [0, 6]), ("1.f32", [8]), ("2.f32", [3])):
        got = torch.from_numpy(np.fromfile(str(out / name), dtype="<f4").reshape(len(rows), cfg["vocab"]))
        assert ((got.double() - exp[rows]).abs().max() / exp[rows].abs().max()).item() < 1e-4, name


# ------------------------------------------------------------------------------------------ each mechanism alone
def ctx_for(ops, dtype, seqs, tables, slots=None):
    pos = [s + i for s, n in seqs for i in range(n)]
    tseq = [i for i, (_, n) in enumerate(seqs) for _ in range(n)]
    qsl = [0]
    for _, n in seqs:
        qsl.append(qsl[-1] + n)
    t = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    return StepContext(ops=ops, dtype=dtype, device=torch.device(DEV), num_tokens=len(pos), num_seqs=len(seqs),
                       max_q_len=max(n for _, n in seqs), max_kv_len=max(s + n for s, n in seqs), token_ids=t([0] * len(pos)),
                       positions=t(pos), token_seq=t(tseq), query_start_loc=t(qsl), seq_lens=t([s + n for s, n in seqs]),
                       slot_ids=t(slots if slots is not None else list(range(len(seqs)))), logit_rows=t([0]), num_logit_rows=0,
                       block_tables={0: tables})


def rel(a, b):
    return ((a.double().cpu() - b.double()).abs().max() / b.double().abs().max()).item()


def part_with_weights(category, spec, dtype, ops, seed, scale=0.15, scales=None, edit=None):
    """The part with random tensors (matrices as the run's dtype stores them) and the same tensors in float64 for the plain
    implementation, under the names of the model folder without the part's prefix."""
    part = build_part(category, spec)
    part.bind(ops, DT[dtype], torch.device(DEV))
    g = torch.Generator().manual_seed(seed)
    w, specs = {}, {}
    for p in [part] + [c for c in part.children()]:
        for k, ps in p.param_specs().items():
            specs[(p, k)] = ps
    for (p, k), ps in specs.items():
        t = torch.randn(ps.shape, generator=g) * (scales or {}).get(k, scale)
        if ps.init == "ones":
            t = 1.0 + t
        full = k if p is part else f"{p.prefix[len(part.prefix):].lstrip('.')}.{k}".lstrip(".")
        w[full] = t.to(DT[dtype]).float() if ps.storage != "vector" else t
    if edit is not None:
        edit(w)
    for p in [part] + [c for c in part.children()]:
        rels = {}
        for k, ps in p.param_specs().items():
            full = k if p is part else f"{p.prefix[len(part.prefix):].lstrip('.')}.{k}".lstrip(".")
            rels[k] = (w[full].to(DT[dtype]) if ps.storage != "vector" else w[full]).to(DEV)
        if rels:
            p.load(rels)
    return part, {k: v.double() for k, v in w.items()}


def run_paged(part, ops, dtype, x, cuts, page, table, pool_pages, planes=2):
    """One request through an attention part in steps of ``cuts`` tokens, from pages that hold noise where nothing was stored.
    ``planes`` 1: keys and values are one array (a latent cache)."""
    need = part.cache_needs()[0]
    pages = [torch.randn(pool_pages, need.num_kv_heads, page, need.head_dim, device=DEV).to(DT[dtype]) for _ in range(planes)]
    outs, start = [], 0
    for n in cuts:
        ctx = ctx_for(ops, DT[dtype], [(start, n)], table)
        o = part.forward(x[start:start + n].to(DEV), ctx, PagedKVView(pages[0], pages[-1], table, page))
        outs.append(o.sum(0) if o.dim() == 3 else o.float())
        start += n
    return torch.cat(outs)


def attention_layer(chunk=None, rot=None, heads=3, kv_heads=1, dim=20, vdim=28, scale=0.21):
    return {"type": "attention", "mixer": attn(heads, kv_heads, dim, vdim, scale, chunk=chunk, rot=rot)}


TABLE = [[9, 2, 7, 1, 3, 6, 11, 4, 8, 5, 10, 12]]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("chunk", [1, 3, 4, 7, 16, 200, None])
def test_sigmoid_attention_alone(ops, dtype, chunk):
    """Whole, in portions and token by token from the pages; chunks of one key, inside a page, a page wide, across pages, wider
    than the prompt, and none; grouped heads; part of every head rotated in half-split pairs; a value size above the key size;
    biases that move the weights; weights that are not normalised (a row's output grows with the keys it sees)."""
    L = attention_layer(chunk=chunk, rot={"base": 50.0, "dims": 6}, heads=4, kv_heads=2)
    part, w = part_with_weights("mixer", _mixer(L, "a", 72, 2e-5), dtype, ops, 1, scales={"pb": 1.5})
    S, page = 45, 4
    x = torch.randn(S, 72, generator=torch.Generator().manual_seed(2)).to(DT[dtype])
    exp = pd.attention(x.double(), w, "", L["mixer"], 2e-5)
    nobias = pd.attention(x.double(), dict(w, pb=w["pb"] * 0), "", L["mixer"], 2e-5)
    assert (nobias - exp).abs().max() > 1e-2 * exp.abs().max()
    table = torch.tensor(TABLE, dtype=torch.int32, device=DEV)
    for cuts in ([S], [10, 2, 33], [1] * S, [3, 1, 1, 17, 2, 21]):
        got = run_paged(part, ops, dtype, x, cuts, page, table, 14)
        assert rel(got, exp) < (3e-5 if dtype == "float32" else 3e-2), (cuts, chunk)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,rot", [(8, 2, 64, 64, 16), (2, 2, 128, 128, 128), (4, 1, 32, 48, 0), (3, 3, 48, 16, 48)])
def test_sigmoid_attention_at_tensor_core_sizes(ops, dtype, heads, kv_heads, dim, vdim, rot):
    """Head sizes the tile-loop kernel takes in bfloat16: prompt portions of several row tiles, portions behind a filled cache,
    decoded tokens; the norm over the whole projection with a weight per channel."""
    L = attention_layer(chunk=70, rot={"base": 500.0, "dims": rot} if rot else None, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim,
                        scale=dim ** -0.5)
    part, w = part_with_weights("mixer", _mixer(L, "a", 96, 1e-6), dtype, ops, 3, scales={"q.norm": 0.4, "k.norm": 0.4, "pb": 1.0})
    S, page = 200, 16
    x = torch.randn(S, 96, generator=torch.Generator().manual_seed(4)).to(DT[dtype])
    exp = pd.attention(x.double(), w, "", L["mixer"], 1e-6)
    table = (torch.randperm(14, generator=torch.Generator().manual_seed(5)) + 1).to(torch.int32).to(DEV)[None]
    for cuts in ([S], [130, 70], [69, 2, 100] + [1] * 29):
        got = run_paged(part, ops, dtype, x, cuts, page, table, 16)
        assert rel(got, exp) < (3e-5 if dtype == "float32" else 3e-2), cuts[:3]


@pytest.mark.parametrize("page", [16, 64])
@pytest.mark.parametrize("chunk", [None, 200, 64])
@pytest.mark.parametrize("heads,kv_heads,dim", [(8, 1, 128), (16, 2, 64), (4, 4, 128)])
def test_sigmoid_attention_on_the_tcgen05_kernels(ops, heads, kv_heads, dim, chunk, page):
    """Pages of 16 and 64 keys and head sizes of 64 and 128 in bfloat16: prompt portions of several hundred rows take the tcgen05
    kernels (one and two query tiles per CTA), decoded tokens behind a long cache take the one-tile kernel with the key range
    cut into pieces, some of which hold no visible key of a chunked row."""
    L = attention_layer(chunk=chunk, rot={"base": 1e4, "dims": 32}, heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=dim ** -0.5)
    part, w = part_with_weights("mixer", _mixer(L, "a", 96, 1e-6), "bfloat16", ops, 21, scales={"q.norm": 0.4, "k.norm": 0.4, "pb": 1.0})
    S = 1100
    x = torch.randn(S, 96, generator=torch.Generator().manual_seed(22)).to(torch.bfloat16)
    exp = pd.attention(x.double(), w, "", L["mixer"], 1e-6)
    npages = -(-S // page) + 1
    table = (torch.randperm(npages, generator=torch.Generator().manual_seed(23)) + 1).to(torch.int32).to(DEV)[None]
    kernels = set()
    plan = ops.attention_plan

    def noting(*a, **k):
        out = plan(*a, **k)
        kernels.add(out[0] + ("+pieces" if out[1] > 1 else ""))
        return out

    ops.attention_plan = noting
    try:
        for cuts in ([S], [600, 500], [1068] + [1] * 32, [300, 40, 760]):
            got = run_paged(part, ops, "bfloat16", x, cuts, page, table, npages + 2).cpu().double()
            err = (got - exp).abs().max(dim=-1).values / exp.abs().max(dim=-1).values.clamp_min(exp.abs().max() * 0.05)
            assert err.max() < 3e-2, (cuts[:3], int(err.argmax()), err.max())
    finally:
        ops.attention_plan = plan
    assert any(k.startswith("tc") for k in kernels), kernels


def loud_key(x, key_at, gain=40.0):
    """Makes the token at ``key_at`` one that every later query notices: its input row is scaled up, which the norms undo for the
    key's size but not for its direction, and the value it brings is large."""
    x = x.clone()
    x[key_at] *= gain
    return x


def test_chunk_edge_shows(ops):
    """One token brings a value far larger than the others'; every later query of its chunk must carry it and the first query
    of the next chunk must not: a chunk one position longer or shorter, or chunks counted from the cut, move the edge."""
    chunk, S, key_at = 9, 40, 20                                       # chunk 2 holds 18..26
    L = attention_layer(chunk=chunk, rot={"base": 30.0, "dims": 4}, heads=2, kv_heads=1, dim=8, vdim=8)
    part, w = part_with_weights("mixer", _mixer(L, "a", 72, 2e-5), "float32", ops, 5)
    x = loud_key(torch.randn(S, 72, generator=torch.Generator().manual_seed(6)) * 0.3, key_at)
    m = L["mixer"]
    exp = pd.attention(x.double(), w, "", m, 2e-5)
    for other in (chunk - 1, chunk + 1):                              # the oracle itself tells the sizes apart at the edge
        diff = pd.attention(x.double(), w, "", dict(m, mask={"size": other}), 2e-5)
        assert (exp[24:29] - diff[24:29]).abs().max() > 1e-2 * exp.abs().max()
    table = torch.tensor([[3, 1, 2, 5, 4, 6, 7, 8, 9, 10]], dtype=torch.int32, device=DEV)
    for cuts in ([S], [26, 1, 1, 12], [27, 13], [21, 2, 2, 2, 2, 11], [19, 1] + [1] * 20):
        got = run_paged(part, ops, "float32", x, cuts, 4, table, 12).cpu().double()
        assert (got - exp).abs().max() < 3e-5 * exp.abs().max(), cuts


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sigmoid_weights_over_hundreds_of_keys_add_up(ops, dtype):
    """No mask: 700 keys weigh in, each by its own sigmoid, so the output is a sum that no normalisation bounds.  Decoded tokens
    and short portions behind a long cache run with the key range cut over CTAs, whose pieces must simply add; the third
    token's value is large, so dropping an early page shows."""
    S, key_at, page = 700, 2, 16
    L = attention_layer(heads=4, kv_heads=2, dim=16, vdim=16, scale=0.25, rot={"base": 1e4, "dims": 16})
    part, w = part_with_weights("mixer", _mixer(L, "a", 72, 2e-5), dtype, ops, 7, scales={"pb": 1.0})
    x = loud_key(torch.randn(S, 72, generator=torch.Generator().manual_seed(8)) * 0.3, key_at, gain=100.0).to(DT[dtype])
    exp = pd.attention(x.double(), w, "", L["mixer"], 2e-5)
    gone = x.clone(); gone[key_at] = 0
    without = pd.attention(gone.double(), w, "", L["mixer"], 2e-5)
    assert (exp[-1] - without[-1]).abs().max() > 0.05 * exp[-1].abs().max()
    perm = torch.randperm(S // page + 1, generator=torch.Generator().manual_seed(9)) + 1
    table = perm.to(torch.int32).to(DEV)[None]
    for cuts in ([S], [650] + [1] * 50, [300, 2, 398]):
        got = run_paged(part, ops, dtype, x, cuts, page, table, S // page + 3).cpu().double()
        tol = 3e-5 if dtype == "float32" else 3e-2
        assert ((got - exp).abs().max(dim=-1).values < tol * exp.abs().max(dim=-1).values.clamp_min(exp.abs().max() * 0.05)).all(), cuts[:3]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", [
    dict(heads=3, dim=12, rot_dim=8, vdim=20, kv_rank=24, q_rank=40, scale=0.2, base=50.0, scaling=yarn(4.0, 64, 8.0, 1.0)),
    dict(heads=2, dim=10, rot_dim=2, vdim=14, kv_rank=18, q_rank=60, scale=0.4, base=30.0),
    dict(heads=5, dim=8, rot_dim=0, vdim=8, kv_rank=16, q_rank=16, scale=0.35),
    dict(heads=4, dim=32, rot_dim=32, vdim=32, kv_rank=88, q_rank=64, scale=0.12, base=1e5, scaling=yarn(2.0, 128, 16.0, 2.0)),
    dict(heads=2, dim=64, rot_dim=16, vdim=64, kv_rank=48, q_rank=32, scale=0.1, base=1e4, scaling=yarn(3.0, 40, 4.0, 1.0))])
def test_latent_attention_alone(ops, dtype, case):
    """Queries through their own normed latent, keys and values from the cached latent and the shared rotated part, rescaled
    frequencies with their magnitude, a gate per value; whole, in portions and token by token."""
    L = {"type": "latent_attention", "mixer": latent(**case)}
    part, w = part_with_weights("mixer", _mixer(L, "a", 72, 2e-5), dtype, ops, 11, scales={"dq.norm": 0.3, "dkv.norm": 0.3})
    S, page = 45, 4
    x = torch.randn(S, 72, generator=torch.Generator().manual_seed(12)).to(DT[dtype])
    exp = pd.latent_attention(x.double(), w, "", L["mixer"], 2e-5)
    if case.get("scaling"):                                           # the rescaling matters here: without it the outputs differ
        m2 = dict(L["mixer"], rot={k: v for k, v in L["mixer"]["rot"].items() if k != "scaling"})
        assert (pd.latent_attention(x.double(), w, "", m2, 2e-5) - exp).abs().max() > 1e-3 * exp.abs().max()
    table = torch.tensor(TABLE, dtype=torch.int32, device=DEV)
    for cuts in ([S], [10, 2, 33], [1] * S, [3, 1, 1, 17, 2, 21]):
        got = run_paged(part, ops, dtype, x, cuts, page, table, 14, planes=1)
        assert rel(got, exp) < (3e-5 if dtype == "float32" else 3e-2), (cuts, case)


def test_latent_attention_reaches_a_far_key(ops):
    """Causal softmax over 700 latents on many pages: the third token is made the key every query prefers and its value is
    large, so every later output carries it whether the query comes in a prompt or alone."""
    S, key_at, page = 700, 2, 16
    L = {"type": "latent_attention", "mixer": latent(2, 16, 8, 12, 24, 20, 0.25, base=1e4, scaling=yarn(2.0, 256, 16.0, 1.0))}
    part, w = part_with_weights("mixer", _mixer(L, "a", 72, 2e-5), "float32", ops, 13)
    x = torch.randn(S, 72, generator=torch.Generator().manual_seed(14)) * 0.3
    x[key_at] = x[key_at] * 30.0
    exp = pd.latent_attention(x.double(), w, "", L["mixer"], 2e-5)
    gone = x.clone(); gone[key_at] = 0
    without = pd.latent_attention(gone.double(), w, "", L["mixer"], 2e-5)
    assert (exp[-1] - without[-1]).abs().max() > 0.02 * exp[-1].abs().max()
    perm = torch.randperm(S // page + 1, generator=torch.Generator().manual_seed(9)) + 1
    table = perm.to(torch.int32).to(DEV)[None]
    for cuts in ([S], [650] + [1] * 50, [300, 2, 398]):
        got = run_paged(part, ops, "float32", x, cuts, page, table, S // page + 3, planes=1).cpu().double()
        assert ((got - exp).abs().max(dim=-1).values < 3e-5 * exp.abs().max(dim=-1).values.clamp_min(exp.abs().max() * 0.05)).all(), cuts[:3]


def run_recurrent(ops, part, xs, cuts, dtype, states, slots):
    """Two requests of unequal length in one batch per cut, in slots that are not in order."""
    done, outs = [0, 0], [[], []]
    for n in cuts:
        seqs, rows = [], []
        for i, x in enumerate(xs):
            k = min(n, x.shape[0] - done[i])
            if k > 0:
                seqs.append((done[i], k)); rows.append(i)
        if not seqs:
            continue
        ctx = ctx_for(ops, DT[dtype], seqs, None, slots=[slots[i] for i in rows])
        xin = torch.cat([xs[i][done[i]:done[i] + k] for i, (_, k) in zip(rows, seqs)]).to(DEV)
        y = part.forward(xin, ctx, [FixedStateView(s) for s in states])
        y = y.sum(0) if y.dim() == 3 else y.float()
        at = 0
        for i, (_, k) in zip(rows, seqs):
            outs[i].append(y[at:at + k]); at += k; done[i] += k
    return [torch.cat(o) for o in outs]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dim,rank,S", [(2, 32, 8, 40), (3, 12, 5, 70), (2, 64, 4, 120)])
def test_time_mixing_alone(ops, dtype, heads, dim, rank, S):
    """Whole, in portions down to one token and token by token; decays between 0 and 1, a bonus that matters."""
    d = 40
    L = {"type": "wkv", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank}}
    part, w = part_with_weights("mixer", _mixer(L, "a", d, 1e-5), dtype, ops, 4, scale=0.3, scales={"w2": 1.0, "w0": 0.7, "u": 0.8})
    g = torch.Generator().manual_seed(6)
    xs = [torch.randn(S, d, generator=g).to(DT[dtype]), torch.randn(S // 2 + 1, d, generator=g).to(DT[dtype])]
    exps = [pd.wkv(x.double(), w, "", L["mixer"], 1e-5) for x in xs]
    for cuts in ([S], [1] * 12 + [S - 12], [2, 1, 3, S - 6], [S - 1, 1]):
        states = [torch.zeros(4, *need.shape, device=DEV) for need in part.cache_needs()]
        outs = run_recurrent(ops, part, xs, cuts, dtype, states, slots=[2, 0])
        for i in range(2):
            assert rel(outs[i], exps[i]) < (3e-5 if dtype == "float32" else 3e-2), (cuts, i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T", [1, 5, 130])
@pytest.mark.parametrize("experts,top,shared", [(5, 2, 24), (4, 1, None), (1, 1, 8), (6, 6, 16), (12, 3, 40)])
def test_experts_weighted_on_their_input(ops, dtype, T, experts, top, shared):
    """One to many tokens (the weight-streaming and the many-rows products); one, several and all experts per token; with and
    without the gated shared expert.  The weight on the input is not the weight on the output: the oracle is told apart from it."""
    f = {"kind": "moe", "expert": {"ff": 40}, "router": {"experts": experts, "top": top}}
    if shared:
        f["shared"] = {"ff": shared}

    def spread(w):                                                     # router scores away from 1/2, 1 and each other; activations of a size
        w["router"] = w["router"] * 1.5
        for k in w:
            if k.endswith(".up"):
                w[k] = w[k] * 3.0

    part, w = part_with_weights("ffn", _ffn(f, "f", 48), dtype, ops, 9, scale=0.3, edit=spread)
    x = torch.randn(T, 48, generator=torch.Generator().manual_seed(T)).to(DT[dtype])
    exp = pd.moe(x.double(), w, "", f)
    s = pd.sigmoid(x.double() @ w["router"].T)
    on_output = torch.zeros_like(exp)
    for t in range(T):
        for e in torch.topk(s[t], top).indices.tolist():
            on_output[t] += s[t, e] * pd.expert(x[t:t + 1].double(), w, f"e{e}.")[0]
    if shared:
        on_output = on_output + pd.expert(x.double(), w, "shared.") * pd.sigmoid(x.double() @ w["shared.sg"].T)
    assert T == 1 or (on_output - exp).abs().max() > 1e-2 * exp.abs().max()
    y = part.forward(x.to(DEV), None)
    assert y.dtype == torch.float32
    if dtype == "float32":
        assert rel(y, exp) < 2e-5
    else:                                                              # a choice between two close scores may flip on a few rows
        err = ((y.double().cpu() - exp).abs().max(dim=-1).values / exp.abs().max())
        assert (err > 2e-2).sum() <= max(1, T // 25), err.max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d,taps", [(40, 1), (50, 2), (64, 4), (72, 7)])
def test_stream_convolution_and_its_state(ops, dtype, d, taps):
    """h = x + conv(x) over the 32-bit stream, two requests side by side in slots out of order, in cuts shorter than the taps
    (the state row keeps the newest of its old rows), from state rows that hold zeros for a new request only."""
    g = torch.Generator().manual_seed(d + taps)
    wt = torch.randn(d, taps, generator=g) * 0.5
    conv_w = wt.t().contiguous().clone()
    conv_w[taps - 1] += 1.0
    conv_w = conv_w.to(DEV)
    xs = [torch.randn(33, d, generator=g), torch.randn(9, d, generator=g)]
    exps = [x.double() + pd.time_conv(x.double(), wt.double()) for x in xs]
    slots = [2, 0]
    for cuts in ([33], [1] * 33, [2, 1, 1, 3, 26], [taps, 1, 2, 30]):
        state = torch.randn(4, max(taps - 1, 1), d, device=DEV)
        for s in slots:
            state[s] = 0
        done, outs = [0, 0], [[], []]
        for n in cuts:
            seqs, rows = [], []
            for i, x in enumerate(xs):
                k = min(n, x.shape[0] - done[i])
                if k > 0:
                    seqs.append((done[i], k)); rows.append(i)
            if not seqs:
                continue
            ctx = ctx_for(ops, DT[dtype], seqs, None, slots=[slots[i] for i in rows])
            resid = torch.cat([xs[i][done[i]:done[i] + k] for i, (_, k) in zip(rows, seqs)]).to(DEV)
            fused = n == 1                                              # one token per request: the kernel advances the state rows itself
            h = ops.stream_conv(resid, conv_w, taps, state if taps > 1 else None, ctx.token_seq, ctx.query_start_loc, ctx.slot_ids, DT[dtype],
                                update_tail=fused)
            if not fused:
                ops.conv_tail_update(resid, d, taps, state, ctx.query_start_loc, ctx.slot_ids, ctx.num_seqs)
            at = 0
            for i, (_, k) in zip(rows, seqs):
                outs[i].append(h[at:at + k].float()); at += k; done[i] += k
        for i in range(2):
            assert rel(torch.cat(outs[i]), exps[i]) < (1e-6 if dtype == "float32" else 5e-3), (cuts, i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d", [40, 50, 384, 9000])
def test_norm_on_a_sublayer_output_with_layer_scale(ops, dtype, d):
    """x <- x + ls * LN(delta) * w over the 32-bit stream: the moments are delta's alone; delta in the compute dtype, in 32-bit and
    as partial sums; the copy in the compute dtype is of the new x."""
    part, w = part_with_weights("norm", _norm("", "n", d, 1e-5, scale="ls"), dtype, ops, d, scale=0.4)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(7, d, generator=g)
    for form in ("compute", "float32", "partial"):
        delta = torch.randn(7, d, generator=g) * 3.0 + 1.0
        if form == "compute":
            delta = delta.to(DT[dtype])
            given, total = delta.to(DEV), delta.double()
        elif form == "float32":
            given, total = delta.to(DEV), delta.double()
        else:
            parts = torch.randn(3, 7, d, generator=g)
            given, total = parts.to(DEV), parts.double().sum(0)
        exp = x.double() + pd.layer_norm(total, w["n"], 1e-5) * w["ls"]
        resid = x.clone().to(DEV)
        out = part.add_normed(resid, given)
        assert rel(resid, exp) < 5e-6
        assert rel(out, exp) < (5e-6 if dtype == "float32" else 5e-3)
