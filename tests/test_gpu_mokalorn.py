"""The Mokalorn design in the engine against the plain implementation (plain_mokalorn.py): each mechanism alone, whole
prompts, decoding through the cache and the state slots, portions down to two tokens, mixed batches with pages and slots
used again, keys at the edges of chunks and pages and far back, other sizes, and greedy generation through the scheduler."""
import pytest
import torch

import plain_mokalorn as pm
import trace_util as tu

from tiny_transformer_inference_engine_b200 import Engine, ModelConfig, EngineConfig, CacheConfig, SchedulerConfig, SamplingParams
from tiny_transformer_inference_engine_b200.parts.base import PartSpec, StepContext, PagedKVView, FixedStateView
from tiny_transformer_inference_engine_b200.registry import build_part
from tiny_transformer_inference_engine_b200.weights import random_tensors

from mokalorn_configs import ALL as CONFIGS, MOK_A, MOK_B, MOK_C, MOK_D

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def ops():
    from tiny_transformer_inference_engine_b200.ops import get_ops
    return get_ops(DEV)


def weights_for(cfg, seed, store="float32"):
    """Random weights large enough that every mechanism matters: peaked attention, gates away from 1/2, clamps that bite,
    router logits of a few units (scores away from each other, so that no two tie) and corrections that change the choice."""
    w = random_tensors(ModelConfig.from_dict(cfg), seed, std=0.08, perturb_norms=True, store_dtype=store)
    g = torch.Generator().manual_seed(seed + 1)
    for k in w:
        if k.endswith((".mix.q", ".mix.k")):
            w[k] = w[k] * 3.0
        if k.endswith((".gate", ".up")):
            w[k] = w[k] * 4.0
        if k.endswith(".mlp.router"):
            w[k] = w[k] * (3.0 / (w[k].float().std() * cfg["width"] ** 0.5))
        if k.endswith(".mlp.correction"):
            w[k] = (torch.randn(w[k].shape, generator=g) * 0.15).to(w[k].dtype)
        if k.endswith((".q.norm", ".k.norm")):
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
    return {rid: pm.forward(cfg, ww, toks) for rid, toks in reqs.items()}


def check(got, exp, dtype):
    """32-bit: every place within 1e-4 of the row's largest logit.  bfloat16: these models are narrow and their weights are
    scaled up so that clamps, gates and routers bite, so rounding alone moves a typical row by 1 to 2 % and a router's choice
    between two close experts, flipped by the rounding, moves one by tens of percent; the run is held to the typical error
    (every mechanism alone is held to its largest error in both dtypes below)."""
    errs = []
    for (rid, pos), row in got.items():
        ref = exp[rid][pos]
        errs.append((((row.double() - ref).abs().max() / ref.abs().max()).item(), rid, pos))
    errs.sort(reverse=True)
    if dtype == "float32":
        assert errs[0][0] < 1e-4, errs[:3]
    else:
        n = len(errs)
        assert all(e[0] == e[0] for e in errs), "a NaN among the logits"
        assert errs[n // 2][0] < 3e-2 and errs[n // 10][0] < 8e-2, (errs[n // 2], errs[n // 10], errs[:3])


# ------------------------------------------------------------------------------------------ the whole model, four cuts
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_schedules_against_plain_model(name, dtype):
    cfg = CONFIGS[name]
    w = weights_for(cfg, 5 + ord(name))
    reqs = requests(cfg, [1, 2, 37, 70, 101, 23], seed=3)
    exp = expected_for(cfg, w, reqs, dtype)
    page = {"A": 16, "B": 8, "C": 4, "D": 2}[name]
    for cut in (tu.whole, tu.prefill_then_decode, tu.portions, tu.mixed):
        steps = cut(reqs)
        tokens = tu.max_live_tokens(steps, rounding=page)
        eng = engine_for(cfg, w, dtype, page=page, pages=tokens // page + 2)        # no slack: pages and slots are used again
        check(tu.run_steps(eng, steps), exp, dtype)


def test_long_decode_past_chunks_and_pages():
    """A short prompt, then 150 tokens one by one: chunk edges (every 11 positions), many page edges and three steps of the
    query temperature pass under decoded tokens, and the retention state is carried 150 times."""
    cfg = MOK_A
    w = weights_for(cfg, 77)
    reqs = requests(cfg, [160], seed=9)
    exp = expected_for(cfg, w, reqs, "float32")
    steps = tu.prefill_then_decode(reqs, tail=150)
    eng = engine_for(cfg, w, "float32", page=8, pages=24)
    check(tu.run_steps(eng, steps), exp, "float32")


def test_batch_of_unequal_requests_equals_each_alone():
    cfg = MOK_A
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
    cfg = MOK_A
    w = weights_for(cfg, 23)
    reqs = requests(cfg, [40, 33, 40], seed=8)
    reqs["r2"] = list(reqs["r0"])
    eng = engine_for(cfg, w, "float32", page=8, pages=8, max_seqs=2)
    got = tu.run_steps(eng, tu.portions(reqs))
    for pos in range(40):
        assert torch.equal(got[("r0", pos)], got[("r2", pos)]), pos
    check(got, expected_for(cfg, w, reqs, "float32"), "float32")


@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_scheduler(graphs):
    cfg = dict(MOK_A, max_seq_len=256)
    w = weights_for(cfg, 31)
    prompts = [[5, 9, 2], list(range(10, 41)), [7]]
    want = []
    for p in prompts:
        toks = list(p)
        for _ in range(14):                                           # past a chunk edge for every prompt
            toks.append(int(torch.argmax(pm.forward(cfg, w, toks)[-1])))
        want.append(toks[len(p):])
    eng = engine_for(cfg, w, "float32", pages=40, max_seqs=4, budget=16, graphs=graphs)
    got = eng.generate(prompts, SamplingParams(max_new_tokens=14, greedy=True))
    assert got == want


def test_command_line_and_trace_runner_with_a_model_folder(tmp_path):
    """A folder written in the random-weights mode (bfloat16 on disk), generated from by the command line and replayed by the
    trace runner: the architecture is picked from config.json by both."""
    import json, os, subprocess, sys
    import numpy as np
    from safetensors.torch import load_file
    from tiny_transformer_inference_engine_b200 import write_random_model
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = dict(MOK_B, max_seq_len=96)
    folder = write_random_model(ModelConfig.from_dict(cfg), 13, str(tmp_path / "model"), std=0.08, perturb_norms=True, store_dtype="bfloat16")
    w = load_file(os.path.join(folder, "model.safetensors"))
    prompt = [4, 90, 7, 7, 23]
    run = subprocess.run([sys.executable, "-m", "tiny_transformer_inference_engine_b200", "--model", folder, "--tokens", "6", "--greedy",
                          "--dtype", "float32", "--num-gpu-blocks", "16", "--prompt-ids", ",".join(map(str, prompt))],
                         cwd=root, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    toks = list(prompt)
    for _ in range(6):
        toks.append(int(torch.argmax(pm.forward(cfg, w, toks)[-1])))
    assert json.loads(run.stdout.strip().split("\n")[-1])["generated_ids"] == toks[len(prompt):]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:7], "want": [0, 6]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[7:9], "want": [1]}, {"id": "b", "tokens": toks[:3], "want": []}], "end": ["a"]},
             {"step": 2, "entries": [{"id": "b", "tokens": toks[3:4], "want": [0]}], "end": ["b"]}]
    out = tmp_path / "out"
    run = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", str(out), "--max-tokens", "128"],
                         input="\n".join(json.dumps(s) for s in steps) + "\n", cwd=root, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    assert [l for l in run.stdout.split("\n") if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    exp = pm.forward(cfg, w, toks)
    for name, rows in (("0.f32", [0, 6]), ("1.f32", [8]), ("2.f32", [3])):
        got = torch.from_numpy(np.fromfile(str(out / name), dtype="<f4").reshape(len(rows), cfg["vocab"]))
        assert ((got.double() - exp[rows]).abs().max() / exp[rows].abs().max()).item() < 1e-4, name


# ------------------------------------------------------------------------------------------ each mechanism alone
from tiny_transformer_inference_engine_b200.models.mokalorn import _mixer, _ffn        # config.json's layer entry -> the part


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


def part_with_weights(category, spec, dtype, ops, seed, scale=0.15, edit=None):
    """The part with random tensors (matrices as the run's dtype stores them) and the same tensors in float64 for the plain
    implementation, under the names of the model folder without the part's prefix."""
    part = build_part(category, spec)
    part.bind(ops, DT[dtype], torch.device(DEV))
    g = torch.Generator().manual_seed(seed)
    w = {}
    for k, ps in part.param_specs().items():
        t = torch.randn(ps.shape, generator=g) * scale
        if ps.init == "ones":
            t = 1.0 + t
        w[k] = t.to(DT[dtype]).float() if ps.storage != "vector" else t
    if edit is not None:
        edit(w)
    part.load({k: (w[k].to(DT[dtype]) if ps.storage != "vector" else w[k]).to(DEV) for k, ps in part.param_specs().items()})
    return part, {k: v.double() for k, v in w.items()}


def run_attention(part, ops, dtype, x, cuts, page, table, pool_pages):
    """One request through the part in steps of ``cuts`` tokens, from pages that hold noise where nothing was stored."""
    pages = [torch.randn(pool_pages, part.num_kv_heads, page, part.padded_dim, device=DEV).to(DT[dtype]) for _ in range(2)]
    outs, start = [], 0
    for n in cuts:
        ctx = ctx_for(ops, DT[dtype], [(start, n)], table)
        o = part.forward(x[start:start + n].to(DEV), ctx, PagedKVView(pages[0], pages[1], table, page))
        outs.append(o.sum(0) if o.dim() == 3 else o.float())
        start += n
    return torch.cat(outs)


def attention_layer(kind, chunk=None, rot=None, q_temp=None, heads=3, kv_heads=1, dim=20, vdim=28, scale=0.21):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim if kind == "attention" else vdim, "scale": scale}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if rot is not None:
        m["rot"] = rot
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return {"type": kind, "mixer": m}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("chunk", [1, 3, 4, 7, 16, 200])
def test_chunked_attention_alone(ops, dtype, chunk):
    """Whole, in portions and token by token from the pages; chunks of one key, inside a page, a page wide, across pages, wider
    than the prompt; part of every head rotated; the values are the keys as projected."""
    L = attention_layer("attention", chunk=chunk, rot={"base": 50.0, "dims": 6}, heads=4, kv_heads=2)
    part, w = part_with_weights("mixer", _mixer(L, "a", 72, 2e-5), dtype, ops, 1)
    S, page = 45, 4
    x = torch.randn(S, 72, generator=torch.Generator().manual_seed(2)).to(DT[dtype])
    exp = pm.attention(x.double(), w, "", L["mixer"], 2e-5, "attention")
    table = torch.tensor([[9, 2, 7, 1, 3, 6, 11, 4, 8, 5, 10, 12]], dtype=torch.int32, device=DEV)
    for cuts in ([S], [10, 2, 33], [1] * S, [3, 1, 1, 17, 2, 21]):
        got = run_attention(part, ops, dtype, x, cuts, page, table, 14)
        assert rel(got, exp) < (3e-5 if dtype == "float32" else 3e-2), (cuts, chunk)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("q_temp", [None, (0.7, 5), (1.5, 1), (-0.3, 16)])
def test_causal_attention_with_query_temperature_alone(ops, dtype, q_temp):
    """A value size of its own (above the key size), no rotation, every key visible; the temperature steps at positions
    ``every - 1``, ``2 every - 1``, ... whatever the cut."""
    L = attention_layer("attention_2", q_temp=q_temp)
    part, w = part_with_weights("mixer", _mixer(L, "a", 72, 2e-5), dtype, ops, 3)
    S, page = 45, 4
    x = torch.randn(S, 72, generator=torch.Generator().manual_seed(4)).to(DT[dtype])
    exp = pm.attention(x.double(), w, "", L["mixer"], 2e-5, "attention_2")
    if q_temp is not None:                                            # the temperature matters here: without it the outputs differ
        plain = pm.attention(x.double(), w, "", {k: v for k, v in L["mixer"].items() if k != "q_temp"}, 2e-5, "attention_2")
        assert (plain - exp).abs().max() > 1e-3 * exp.abs().max()
    table = torch.tensor([[9, 2, 7, 1, 3, 6, 11, 4, 8, 5, 10, 12]], dtype=torch.int32, device=DEV)
    for cuts in ([S], [4, 1, 40], [1] * S, [15, 2, 28]):
        got = run_attention(part, ops, dtype, x, cuts, page, table, 14)
        assert rel(got, exp) < (3e-5 if dtype == "float32" else 3e-2), (cuts, q_temp)


def loud_key(w, x, key_at, gain=40.0):
    """Makes the token at ``key_at`` a key that every query prefers: its input row is scaled up, which the key norm undoes for
    the key's size but not for its direction, and the (raw) value it brings is large."""
    x = x.clone()
    x[key_at] *= gain
    return x


def test_chunk_edge_shows(ops):
    """One token brings a value far larger than the others'; every later query of its chunk must carry it and the first query
    of the next chunk must not: a chunk one position longer or shorter, or chunks counted from the cut, move the edge."""
    chunk, S, key_at = 9, 40, 20                                       # chunk 2 holds 18..26
    L = attention_layer("attention", chunk=chunk, rot={"base": 30.0, "dims": 4}, heads=2, kv_heads=1, dim=8)
    part, w = part_with_weights("mixer", _mixer(L, "a", 72, 2e-5), "float32", ops, 5)
    x = loud_key(w, torch.randn(S, 72, generator=torch.Generator().manual_seed(6)) * 0.3, key_at)
    m = L["mixer"]
    exp = pm.attention(x.double(), w, "", m, 2e-5, "attention")
    for other in (chunk - 1, chunk + 1):                              # the oracle itself tells the sizes apart at the edge
        diff = pm.attention(x.double(), w, "", dict(m, mask={"size": other}), 2e-5, "attention")
        assert (exp[24:29] - diff[24:29]).abs().max() > 1e-2 * exp.abs().max()
    gone = x.clone(); gone[key_at] = 0
    moved = (pm.attention(gone.double(), w, "", m, 2e-5, "attention") - exp).abs().max(dim=-1).values
    assert moved[key_at:27].min() > 0.1 * exp.abs().max() and moved[27:].max() == 0      # 26 still sees the loud value, 27 opens a chunk
    table = torch.tensor([[3, 1, 2, 5, 4, 6, 7, 8, 9, 10]], dtype=torch.int32, device=DEV)
    for cuts in ([S], [26, 1, 1, 12], [27, 13], [21, 2, 2, 2, 2, 11], [19, 1] + [1] * 20):
        got = run_attention(part, ops, "float32", x, cuts, 4, table, 12).cpu().double()
        assert (got - exp).abs().max() < 3e-5 * exp.abs().max(), cuts


def test_far_key_among_hundreds(ops):
    """Causal attention over 700 keys on many pages: the third token's value is large, so every later output carries it whether
    the query comes in a prompt or alone, and a kernel that drops early pages or splits the keys wrongly shows."""
    S, key_at, page = 700, 2, 16
    L = attention_layer("attention_2", q_temp=(0.4, 64), heads=2, kv_heads=1, dim=16, vdim=12)
    part, w = part_with_weights("mixer", _mixer(L, "a", 72, 2e-5), "float32", ops, 7)
    x = loud_key(w, torch.randn(S, 72, generator=torch.Generator().manual_seed(8)) * 0.3, key_at, gain=400.0)
    exp = pm.attention(x.double(), w, "", L["mixer"], 2e-5, "attention_2")
    gone = x.clone(); gone[key_at] = 0
    without = pm.attention(gone.double(), w, "", L["mixer"], 2e-5, "attention_2")
    assert (exp[-1] - without[-1]).abs().max() > 0.5 * exp[-1].abs().max()      # the far value is most of the last output
    perm = torch.randperm(S // page + 1, generator=torch.Generator().manual_seed(9)) + 1
    table = perm.to(torch.int32).to(DEV)[None]
    for cuts in ([S], [650] + [1] * 50, [300, 2, 398]):
        got = run_attention(part, ops, "float32", x, cuts, page, table, S // page + 3).cpu().double()
        assert ((got - exp).abs().max(dim=-1).values < 3e-5 * exp.abs().max(dim=-1).values).all(), cuts[:3]     # row by row


def retention_layer(heads, dim, vdim, decay, rot=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot is not None:
        m["rot"] = rot
    return {"type": "retention", "mixer": m}


def run_retention(part, ops, dtype, xs, cuts, slots, state_rows):
    """Several requests side by side through the part, each step bringing up to ``n`` tokens of every request that has some
    left; the state rows start with noise where a new request must find zeros only after the engine cleared them, so the
    rows in ``slots`` are zeroed here and the others must stay as they are."""
    H, Dv, Dp = part.num_heads, part.vdim, part.cache_needs()[0].shape[-1]
    state = torch.randn(state_rows + 1, H, Dv, Dp, device=DEV)
    for s in slots:
        state[s] = 0
    before = state.clone()
    done, outs = [0] * len(xs), [[] for _ in xs]
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
        y = part.forward(xin, ctx, [FixedStateView(state)])
        y = y.sum(0) if y.dim() == 3 else y.float()
        at = 0
        for i, (_, k) in zip(rows, seqs):
            outs[i].append(y[at:at + k]); at += k; done[i] += k
    for r in range(state_rows):
        if r not in slots:
            assert torch.equal(state[r], before[r]), r                 # a slot nobody holds is not touched
    return [torch.cat(o) for o in outs]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dim,vdim,decay,rot", [
    (2, 16, 24, (0.9, 0.97), {"base": 50.0, "dims": 16}),               # every key value rotated
    (3, 24, 8, (0.5, 1.0, 0.999), {"base": 1e4, "dims": 6}),            # part of a head; a head that forgets nothing
    (1, 20, 20, (0.0,), None),                                          # no rotation; a state that keeps only the last token
    (4, 64, 64, (0.99, 0.9, 0.8, 0.96875), {"base": 1e6, "dims": 64}),
    (2, 6, 130, (0.95, 0.75), {"base": 7.0, "dims": 2}),                # a value size above the threads of a warp, not a multiple of 4
])
def test_retention_alone(ops, dtype, heads, dim, vdim, decay, rot):
    """Whole, in portions down to two tokens and token by token; two requests whose slots are not in order."""
    L = retention_layer(heads, dim, vdim, decay, rot)
    part, w = part_with_weights("mixer", _mixer(L, "a", 40, 3e-5), dtype, ops, 4, scale=0.3)
    g = torch.Generator().manual_seed(6)
    S = 75
    xs = [torch.randn(S, 40, generator=g).to(DT[dtype]), torch.randn(S // 2 + 1, 40, generator=g).to(DT[dtype])]
    exps = [pm.retention(x.double(), w, "", L["mixer"], 3e-5) for x in xs]
    for cuts in ([S], [1] * 12 + [S - 12], [2, 1, 3, S - 6], [S - 1, 1], [1] * S):
        outs = run_retention(part, ops, dtype, xs, cuts, slots=[2, 0], state_rows=4)
        for i in range(2):
            if dtype == "float32" or 0.0 not in decay:
                assert rel(outs[i], exps[i]) < (3e-5 if dtype == "float32" else 3e-2), (cuts[:4], i)
            else:
                # a head that keeps only the last token reads out (q_t . k_t) v_t and the head norm divides by its size: where
                # q_t . k_t nearly cancels, the rounding of the projections to bfloat16 decides the row (its sign, even)
                err = (outs[i].double().cpu() - exps[i]).abs().max(dim=-1).values / exps[i].abs().max()
                assert (err > 3e-2).sum() <= 3, (cuts[:4], i, err.max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dim,vdim,decay", [
    (4, 16, 12, (1.0, 0.99, 0.6, 0.0)),
    (2, 64, 40, (0.999, 0.9)),
    (2, 128, 20, (0.97, 1.0)),
    (1, 160, 24, (0.95,)),
    (2, 48, 8, (0.5, 0.98)),                                            # padded to 64 channels
])
def test_retention_long_prompts_in_parts(ops, dtype, heads, dim, vdim, decay):
    """Prompts long enough that a step walks them in parts (two launches): a long request beside a short one and beside one
    of a single token, whole and cut so that later steps are short again; heads that forget nothing, little, fast and
    everything; a state that the step finds filled (the second and third cut)."""
    L = retention_layer(heads, dim, vdim, decay, {"base": 200.0, "dims": 8})
    part, w = part_with_weights("mixer", _mixer(L, "a", 40, 1e-5), dtype, ops, 14, scale=0.3)
    g = torch.Generator().manual_seed(15)
    lens = (1500, 90, 1)
    xs = [(torch.randn(n, 40, generator=g) * 0.5).to(DT[dtype]) for n in lens]
    state = part.cache_needs()[0].shape
    assert ops.retention_parts(sum(lens), 3, state[0] * state[1] * state[2]) > 1 and ops.retention_parts(700 + 90 + 1, 3) > 1
    assert ops.retention_parts(sum(lens), 3, 1 << 20) == 1 and ops.retention_parts(300, 3) == 1
    exps = [pm.retention(x.double(), w, "", L["mixer"], 1e-5) for x in xs]
    for cuts in ([1500], [700, 800], [3, 1400, 1, 96]):
        outs = run_retention(part, ops, dtype, xs, cuts, slots=[1, 3, 0], state_rows=4)
        for i in range(3):
            err = (outs[i].double().cpu() - exps[i]).abs().max(dim=-1).values / exps[i].abs().max()
            if dtype == "float32":
                assert err.max() < 5e-5, (cuts, i, int(err.argmax()))
            else:                                                      # (the head that keeps nothing: see test_retention_alone)
                assert (err > 3e-2).sum() <= len(err) // 100 + 1, (cuts, i, err.max())


def test_retention_keeps_a_far_token_by_its_decay(ops):
    """One early token brings a large key and value.  The head that does not decay still reads it 400 tokens later (whole, in
    portions and decoded), the head with a decay of 0.9 has lost it: the two heads' outputs are told apart before the head norm
    would hide the size, by comparing with the plain recurrence."""
    L = retention_layer(2, 8, 8, (1.0, 0.9), {"base": 100.0, "dims": 4})
    part, w = part_with_weights("mixer", _mixer(L, "a", 40, 1e-6), "float32", ops, 11, scale=0.3)
    S = 420
    x = torch.randn(S, 40, generator=torch.Generator().manual_seed(12)) * 0.2
    x[3] *= 60.0
    exp = pm.retention(x.double(), w, "", L["mixer"], 1e-6)
    gone = x.clone(); gone[3] = 0
    assert (pm.retention(gone.double(), w, "", L["mixer"], 1e-6)[-1] - exp[-1]).abs().max() > 1e-2 * exp.abs().max()
    for cuts in ([S], [400] + [1] * 20, [64, 2, 300, 54]):
        out = run_retention(part, ops, "float32", [x], cuts, slots=[1], state_rows=2)[0]
        assert rel(out, exp) < 5e-5, cuts[:3]


@pytest.mark.parametrize("experts,identity,top", [(5, 2, 3), (4, 0, 1), (1, 3, 2), (0, 2, 1), (2, 1, 3), (12, 2, 4), (40, 0, 8)])
def test_router_choices(ops, experts, identity, top):
    """Softmax over all experts, identity experts included; the correction moves the choice and not the weights; every expert
    chosen; one expert."""
    E = experts + identity
    g = torch.Generator().manual_seed(E * 10 + top)
    logits = torch.randn(333, E, generator=g) * 2
    corr = torch.randn(E, generator=g) * 0.2
    idx, wts = ops.moe_route(logits.to(DEV), 1, 1, 1, top, 1.0, False, score="softmax", correction=corr.to(DEV))
    s = torch.softmax(logits.double(), dim=-1)
    want = torch.topk(s + corr.double(), top, dim=-1).indices
    assert torch.equal(idx.cpu().long().sort(dim=-1).values, want.sort(dim=-1).values)
    assert rel(wts, torch.gather(s, 1, idx.cpu().long())) < 1e-6
    plain = torch.topk(s, top, dim=-1).indices                       # the correction changes some choices, or the test shows nothing
    assert top == E or not torch.equal(plain.sort(dim=-1).values, want.sort(dim=-1).values)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T", [1, 5, 130])
@pytest.mark.parametrize("experts,identity,top", [(5, 2, 3), (1, 3, 2), (0, 2, 1), (6, 0, 2)])
def test_moe_alone(ops, dtype, T, experts, identity, top):
    f = {"kind": "moe", "expert": {"ff": 40, "limit": 0.8}, "router": {"experts": experts, "identity": identity, "top": top}}

    def spread(w):                                                     # router logits of a few units, clamps that bite
        w["router"] = w["router"] * 6.0
        for k in w:
            if k.endswith((".gate", ".up")):
                w[k] = w[k] * 3.0

    part, w = part_with_weights("ffn", _ffn(f, "f", 48), dtype, ops, 9, scale=0.3, edit=spread)
    x = torch.randn(T, 48, generator=torch.Generator().manual_seed(T)).to(DT[dtype])
    exp = pm.moe(x.double(), w, "", f)
    if experts:
        assert (x.double() @ w["e0.gate"].T).abs().max() > 0.8
    y = part.forward(x.to(DEV), None)
    assert y.dtype == torch.float32
    if dtype == "float32":
        assert rel(y, exp) < 2e-5
    else:                                                              # a choice between two close scores may flip on a few rows
        err = ((y.double().cpu() - exp).abs().max(dim=-1).values / exp.abs().max())
        assert (err > 2e-2).sum() <= max(1, T // 25), err.max()


def test_first_tokens_of_a_sequence():
    """Requests of one and two tokens, alone and beside a longer one, and the first three positions of a prompt asked for one by
    one: position 0 sees itself only, the state starts at zero, the temperature is 1 where ``(p + 1) < every``."""
    cfg = MOK_B
    w = weights_for(cfg, 41)
    reqs = requests(cfg, [1, 2, 3, 30], seed=5)
    exp = expected_for(cfg, w, reqs, "float32")
    eng = engine_for(cfg, w, "float32", page=2, pages=40)
    check(tu.run_steps(eng, tu.whole(reqs)), exp, "float32")
    check(tu.run_steps(eng, tu.prefill_then_decode(reqs, tail=29)), exp, "float32")
    steps = [{"entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in reqs.items()], "end": list(reqs)}]
    check(tu.run_steps(eng, steps), exp, "float32")
