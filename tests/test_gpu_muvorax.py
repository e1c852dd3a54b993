"""The Muvorax decoder on the GPU against the plain statement in plain_muvorax.py: each mechanism
alone, the residual stream layer by layer, whole prompts against token-by-token decoding and
against portions, unequal batches, slots and pages used again, far keys and page borders, the first
tokens, long decoding, other sizes, greedy generation through the entry point. Configurations and
weights are made here; weights are larger than a trained model's so that every branch moves the
logits."""
import json
import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_muvorax as plain

pytestmark = pytest.mark.gpu

TOL_F32 = 2e-4       # of a row's largest logit
TOL_BF16 = 6e-2
YARN = {"factor": 4.0, "fast": 16.0, "original": 64, "slow": 2.0}


def latent(heads=3, dim=8, rot_dim=4, vdim=12, rank=20, scale=0.4, base=100.0, dims=None, scaling=None, kv_from=None):
    rot = {"base": base, "dims": rot_dim if dims is None else dims}
    if scaling is not None:
        rot["scaling"] = scaling
    m = {"dim": dim, "heads": heads, "kv_rank": rank, "rot": rot, "rot_dim": rot_dim, "scale": scale, "vdim": vdim}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def lightning(heads=3, dim=8, vdim=12, decay=(0.5, 0.9, 0.99)):
    return {"type": "lightning", "mixer": {"decay": list(decay), "dim": dim, "heads": heads, "vdim": vdim}}


def mamba(inner=40, state=6, dt_rank=5, conv=3):
    return {"type": "mamba1", "mixer": {"conv": conv, "dt_rank": dt_rank, "inner": inner, "state": state}}


def dense(ff):
    return {"ff": ff, "kind": "dense"}


def moe(ff=24, experts=8, top=2, count=2, keep=1, scale=1.5):
    return {"expert": {"ff": ff}, "kind": "moe", "router": {"experts": experts, "groups": {"count": count, "keep": keep}, "scale": scale,
                                                            "top": top}}


def with_ff(layer, mlp):
    return dict(layer, mlp=mlp)


def config(layers, width=64, vocab=96, eps=1e-6):
    return {"architecture": "Muvorax", "layers": [dict({"mlp": None}, **l) for l in layers], "norm": {"eps": eps}, "vocab": vocab,
            "width": width}


# Sizes that differ from one another in every number. A: every kind of layer once or twice, a layer
# reading another's latent with other head counts, a layer without a feed-forward. B: ten heads (two
# groups of the attention kernel's warps), a latent that is no multiple of 32, value columns that are
# no multiple of 4, one tap, a rotation of fewer dims than the rotated part and without rescaling,
# nine experts in three groups of which two are kept. C: one group of experts, one expert a token,
# decays of exactly 0 and 1, many states per channel.
CFG_A = config([with_ff(lightning(), moe()), with_ff(latent(scaling=YARN), dense(80)), with_ff(mamba(), moe(16, 6, 3, 3, 2, 0.7)),
                latent(5, 6, 4, 10, 20, 0.3, scaling=YARN, kv_from=1), with_ff(lightning(2, 16, 4, (0.2, 0.999)), dense(40))])
CFG_B = config([with_ff(latent(10, 12, 8, 6, 72, 0.25, 5000.0, dims=6), moe(40, 9, 3, 3, 2, 2.5)), mamba(56, 17, 3, 1),
                with_ff(lightning(2, 40, 50, (0.97, 0.6)), dense(72)), with_ff(latent(4, 16, 8, 20, 72, 0.2, 5000.0, dims=6, kv_from=0),
                                                                               moe(8, 4, 1, 1, 1, 1.0))],
               width=96, vocab=130, eps=1e-5)
CFG_C = config([with_ff(mamba(24, 40, 8, 4), moe(12, 5, 1, 1, 1, 3.0)), with_ff(lightning(4, 4, 24, (0.0, 1.0, 0.8, 0.95)), moe(20, 4, 4, 2, 2, 1.0)),
                with_ff(latent(1, 20, 2, 32, 130, 0.5, 20.0), dense(24))], width=40, vocab=77)


# widths that are multiples of nothing: every vector path has to step aside
CFG_D = config([with_ff(latent(3, 5, 2, 3, 9, 0.6, 30.0), moe(6, 3, 2, 1, 1, 1.2)), with_ff(mamba(10, 1, 1, 2), dense(14)),
                with_ff(lightning(1, 5, 7, (0.9,)), moe(10, 6, 1, 3, 1, 0.5)), latent(1, 3, 2, 5, 9, 0.4, 30.0, kv_from=0),
                mamba(6, 3, 2, 5)], width=50, vocab=61)


def random_weights(cfg, seed, std=0.25):
    """Weights by tensor name for `cfg`, bfloat16-representable (the folder stores bfloat16)."""
    from scriptling_llm_lib_b200 import models  # noqa: F401
    from scriptling_llm_lib_b200.config.registry import architecture_for
    from scriptling_llm_lib_b200.engine.model import DecoderModel
    arch = architecture_for("Muvorax")
    specs = DecoderModel(arch.layout(arch.config_class.from_dict(cfg, "test"))).tensor_specs()
    g = torch.Generator().manual_seed(seed)
    W = {}
    for s in specs:
        t = torch.randn(s.shape, generator=g)
        if s.init == "norm_weight":
            t = 1.0 + 0.2 * t
        elif s.init == "slope":
            t = 0.8 + 0.1 * t
        elif s.init == "matrix":
            t = t * std * (4.0 / math.sqrt(s.shape[-1]))
        elif s.init == "bias":
            t = 0.3 * t
        else:
            t = 0.5 * t
        W[s.name] = t.to(torch.bfloat16)
    W["embed"] = torch.randn(W["embed"].shape, generator=g).to(torch.bfloat16)
    return W


def write_folder(path, cfg, W):
    from scriptling_llm_lib_b200.weights.safetensors_io import write_safetensors
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(path / "model.safetensors", W)
    return path


def ids(n, vocab, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, n)]


def engine(folder, dtype="float32", max_tokens=2048, max_seqs=8, **kw):
    from scriptling_llm_lib_b200.engine.step import Engine
    return Engine.from_folder(folder, dtype, max_tokens=max_tokens, max_seqs=max_seqs, **kw)


def run(eng, pieces):
    """Feed one sequence in the given pieces; logits of every position [T, vocab]."""
    from scriptling_llm_lib_b200.engine.step import StepEntry
    seq = eng.open()
    out = []
    for p in pieces:
        out.append(eng.step([StepEntry(seq, list(p), list(range(len(p))))]))
    eng.check_errors()
    seq.close()
    return torch.cat(out).cpu().double()


def cut(tokens, sizes):
    out, at = [], 0
    for s in sizes:
        out.append(tokens[at:at + s])
        at += s
    if at < len(tokens):
        out.append(tokens[at:])
    return [p for p in out if p]


def rel(got, want):
    return float(((got - want).abs().amax(-1) / want.abs().amax(-1).clamp_min(1e-30)).max())


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("muvorax")
    out = {}
    for name, cfg, seed in (("A", CFG_A, 1), ("B", CFG_B, 2), ("C", CFG_C, 3), ("D", CFG_D, 4)):
        W = random_weights(cfg, seed)
        out[name] = (write_folder(root / name, cfg, W), cfg, W)
    return out


def plain_logits(cfg, W, tokens, rnd=plain.ident, layers_out=None):
    return plain.PlainMuvorax(cfg, W, rnd).forward(tokens, layers_out)


# --------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_a_whole_prompt_equals_the_plain_statement_in_32_bit(folders, name):
    folder, cfg, W = folders[name]
    tokens = ids(90, cfg["vocab"], 10)
    want = plain_logits(cfg, W, tokens)
    got = run(engine(folder), [tokens])
    assert rel(got, want) < TOL_F32


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_bfloat16_stays_near_the_plain_statement_that_rounds_where_the_engine_stores(folders, name):
    folder, cfg, W = folders[name]
    tokens = ids(70, cfg["vocab"], 11)
    want = plain_logits(cfg, W, tokens)
    want16 = plain_logits(cfg, W, tokens, rnd=plain.bf16_round)
    eng = engine(folder, "bfloat16")
    got = run(eng, [tokens])
    assert rel(got, want16) < TOL_BF16 and rel(got, want) < 2 * TOL_BF16
    step = run(eng, [tokens[:50]] + [[t] for t in tokens[50:]])
    assert rel(step, got) < TOL_BF16


def test_the_residual_stream_after_every_layer(folders):
    from scriptling_llm_lib_b200.engine.step import StepEntry
    folder, cfg, W = folders["A"]
    tokens = ids(37, cfg["vocab"], 12)
    want = []
    plain_logits(cfg, W, tokens, layers_out=want)
    eng = engine(folder)
    seq = eng.open()
    arr = np.asarray(tokens, dtype=np.int64)
    eng.cache.reserve([(seq.slot, len(tokens))])
    ctx = eng._context([StepEntry(seq, tokens, [])], arr, [len(tokens)], [0], [])
    x = eng.model.embedding.forward(ctx.token_ids, ctx)
    delta = None
    for i, e in enumerate(eng.layout.schedule):
        delta = eng.model.blocks[e.layer].forward(x, delta, ctx, e.cache_unit, e.writes_cache)
        y = delta.y.double()
        y = y.sum(0) if y.dim() == 3 else y
        w, b, a = delta.norm.terms()
        full = x.double() + torch.tanh(a * y) * w.double() + b.double()
        assert float((full.cpu() - want[i]).abs().max()) < 1e-4 * float(want[i].abs().max()), f"layer {i}"
    seq.close()


@pytest.mark.parametrize("layer", [lightning(), latent(scaling=YARN), mamba(), with_ff(lightning(1, 4, 4, (0.9,)), moe()),
                                   with_ff(mamba(8, 2, 1, 2), dense(48)), latent(2, 4, 0, 8, 6, 1.0, dims=0), mamba(20, 12, 4, 3),
                                   mamba(12, 70, 2, 2)],
                         ids=["lightning", "latent", "scan", "experts", "dense", "latent-without-rotation", "scan-12-states", "scan-70-states"])
def test_each_mechanism_alone(tmp_path, layer):
    cfg = config([layer], width=32, vocab=50)
    W = random_weights(cfg, 5, std=0.4)
    folder = write_folder(tmp_path / "m", cfg, W)
    tokens = ids(45, 50, 13)
    want = plain_logits(cfg, W, tokens)
    eng = engine(folder)
    assert rel(run(eng, [tokens]), want) < TOL_F32
    assert rel(run(eng, [tokens[:20]] + [[t] for t in tokens[20:]]), want) < TOL_F32


@pytest.mark.parametrize("rank,heads,dtype", [(160, 2, "float32"), (264, 9, "float32"), (512, 3, "float32"), (256, 4, "bfloat16")])
def test_wide_latents_token_by_token(tmp_path, rank, heads, dtype):
    """Latents of several hundred: every lane of the attention kernel owns several groups of columns."""
    cfg = config([latent(heads, 8, 8, 8, rank, 0.5, 1000.0), with_ff(latent(2, 4, 8, 12, rank, 0.3, 1000.0, kv_from=0), dense(16))],
                 width=32, vocab=40)
    W = random_weights(cfg, 9, std=0.4)
    folder = write_folder(tmp_path / "m", cfg, W)
    tokens = ids(75, 40, 21)
    eng = engine(folder, dtype)
    got = run(eng, [tokens[:3]] + [[t] for t in tokens[3:]])
    if dtype == "float32":
        assert rel(got, plain_logits(cfg, W, tokens)) < TOL_F32
    else:
        assert rel(got, plain_logits(cfg, W, tokens, rnd=plain.bf16_round)) < TOL_BF16


# --------------------------------------------------------------------------- cutting, batches, slots
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_token_by_token_and_portions_equal_the_whole_prompt(folders, name):
    folder, cfg, W = folders[name]
    tokens = ids(150, cfg["vocab"], 14)
    want = plain_logits(cfg, W, tokens)
    eng = engine(folder)
    for sizes in ([1] * 150, [2] * 75, [3, 2, 31, 33, 1, 64], [64, 64], [63, 2, 63], [100] + [1] * 50):
        got = run(eng, cut(tokens, sizes))
        assert rel(got, want) < TOL_F32, sizes


def test_unequal_requests_in_a_batch_equal_each_alone_and_slots_are_used_again(folders):
    from scriptling_llm_lib_b200.engine.step import StepEntry
    folder, cfg, W = folders["B"]
    V = cfg["vocab"]
    reqs = [ids(n, V, 20 + i) for i, n in enumerate((70, 3, 129, 1, 40))]
    prompt = [60, 2, 100, 1, 33]
    want = [plain_logits(cfg, W, r) for r in reqs]
    eng = engine(folder, max_seqs=6)
    for round_ in range(3):                     # the same slots and pages again, after other requests held them
        seqs = [eng.open() for _ in reqs]
        out = eng.step([StepEntry(s, r[:p], list(range(p))) for s, r, p in zip(seqs, reqs, prompt)]).cpu().double()
        got, at = [[] for _ in reqs], 0
        for i, p in enumerate(prompt):
            got[i].append(out[at:at + p])
            at += p
        pos = list(prompt)
        live = [i for i in range(len(reqs)) if pos[i] < len(reqs[i])]
        for i in range(len(reqs)):
            if i not in live:
                seqs[i].close()
        while live:
            out = eng.step([StepEntry(seqs[i], [reqs[i][pos[i]]], [0]) for i in live]).cpu().double()
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
                pos[i] += 1
                if pos[i] == len(reqs[i]):
                    seqs[i].close()
            live = [i for i in live if pos[i] < len(reqs[i])]
        for i in range(len(reqs)):
            assert rel(torch.cat(got[i]), want[i]) < TOL_F32, (round_, i)
        reqs, prompt, want = reqs[::-1], prompt[::-1], want[::-1]
    assert eng.cache.slots.n_held == 0 and all(g.pool.n_held == 0 for g in eng.cache.groups)


def test_the_first_tokens_of_a_sequence(folders):
    folder, cfg, W = folders["A"]
    eng = engine(folder)
    for n in (1, 2, 3, 4):
        tokens = ids(n, cfg["vocab"], 30 + n)
        want = plain_logits(cfg, W, tokens)
        assert rel(run(eng, [tokens]), want) < TOL_F32
        assert rel(run(eng, [[t] for t in tokens]), want) < TOL_F32


def test_long_decoding_keeps_the_states(folders):
    folder, cfg, W = folders["C"]
    tokens = ids(260, cfg["vocab"], 15)
    want = plain_logits(cfg, W, tokens)
    got = run(engine(folder), [tokens[:5]] + [[t] for t in tokens[5:]])
    assert rel(got, want) < TOL_F32


# --------------------------------------------------------------------------- far keys and page borders
def test_one_loud_key_far_back_and_at_page_borders(tmp_path):
    """One key that carries every later row. A token of its own (the last id) lights channel 0 of the
    stream, the down-projection turns that into the latent's first component, head 0's first key dim
    reads it, and every query has a constant there: so wherever that token stands, at the first
    position, far back, or on either side of a page border, the rows behind it take their output from
    its cached latent; in a prompt and token by token."""
    cfg = config([with_ff(latent(2, 8, 4, 8, 12, 2.0, 50.0), dense(32))], width=32, vocab=40)
    W = random_weights(cfg, 7, std=0.5)
    loud = 39
    W["embed"][:, 0] = 0.0
    W["embed"][loud, 0] = 8.0
    for name, v0, v1 in (("l0.norm1", 1.0, 0.0), ("l0.norm1.b", 0.0, 1.0)):       # channel 0 passes, channel 1 is the constant 1
        W[name][0], W[name][1] = v0, v1
    W["l0.mix.dkv"][0, :] = 0.0
    W["l0.mix.dkv"][0, 0] = 10.0
    W["l0.mix.dkv.norm"][0] = 1.0
    W["l0.mix.uk"][0, :] = 0.0
    W["l0.mix.uk"][0, 0] = 1.0
    W["l0.mix.q"][0, :] = 0.0
    W["l0.mix.q"][0, 1] = 5.0
    folder = write_folder(tmp_path / "m", cfg, W)
    eng = engine(folder)
    base = ids(200, 39, 16)                          # never the loud token
    other = plain_logits(cfg, W, base)
    for p in (0, 1, 63, 64, 65, 127, 128, 150):
        tokens = list(base)
        tokens[p] = loud
        want = plain_logits(cfg, W, tokens)
        assert rel(want[190:], other[190:]) > 100 * TOL_F32         # the far key shows in the last rows
        assert rel(run(eng, [tokens]), want) < TOL_F32
        assert rel(run(eng, [tokens[:170]] + [[t] for t in tokens[170:]]), want) < TOL_F32


def test_a_slowly_decaying_head_remembers_the_first_token(tmp_path):
    cfg = config([lightning(2, 8, 8, (1.0, 0.5))], width=24, vocab=30)
    W = random_weights(cfg, 8, std=0.5)
    folder = write_folder(tmp_path / "m", cfg, W)
    eng = engine(folder)
    a = ids(140, 30, 17)
    b = [(a[0] + 3) % 30] + a[1:]
    wa, wb = plain_logits(cfg, W, a), plain_logits(cfg, W, b)
    assert rel(wa[130:], wb[130:]) > 10 * TOL_F32
    for tokens, want in ((a, wa), (b, wb)):
        assert rel(run(eng, [tokens]), want) < TOL_F32
        assert rel(run(eng, [tokens[:33]] + [[t] for t in tokens[33:]]), want) < TOL_F32


# --------------------------------------------------------------------------- kernels by themselves
def test_the_router_against_the_plain_choice():
    from scriptling_llm_lib_b200.csrc.bindings import KernelSet
    k = KernelSet(torch.float32).mix
    g = torch.Generator().manual_seed(3)
    for E, groups, keep, top in ((8, 2, 1, 2), (12, 4, 2, 3), (6, 1, 1, 6), (9, 9, 3, 3), (64, 8, 3, 6), (5, 5, 5, 1)):
        h = torch.randn(50, 24, generator=g)
        wr = torch.randn(E, 24, generator=g)
        corr = torch.randn(E, generator=g) * 1.5          # corrections large enough to make choice scores negative
        Wd = {"r.router": wr.double(), "r.correction": corr.double()}
        want_idx, want_w = plain.route(h.double(), Wd, "r.", {"experts": E, "top": top, "scale": 1.7, "groups": {"count": groups, "keep": keep}})
        idx = torch.empty((50, top), dtype=torch.int32, device="cuda")
        wgt = torch.empty((50, top), dtype=torch.float32, device="cuda")
        k.moe_route((h @ wr.T).cuda().contiguous(), corr.cuda(), idx, wgt, groups, keep, top, 1.7)
        for t in range(50):
            got = dict(zip(idx[t].tolist(), wgt[t].tolist()))
            want = dict(zip(want_idx[t].tolist(), want_w[t].tolist()))
            assert set(got) == set(want), (E, t)
            assert all(abs(got[e] - want[e]) < 1e-5 for e in want)


def test_linear_attention_in_pieces_against_the_recurrence():
    from scriptling_llm_lib_b200.csrc.bindings import KernelSet
    k = KernelSet(torch.float32).mix
    g = torch.Generator().manual_seed(4)
    H, D, V = 3, 10, 22
    lens = [1, 31, 32, 33, 70, 4]
    T = sum(lens)
    proj = torch.randn(T, 2 * H * D + H * V + 5, generator=g)
    decay = torch.tensor([0.3, 0.95, 1.0])
    start = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    state0 = torch.randn(len(lens) + 2, H, D, V, generator=g) * 0.3
    ctx = SimpleNamespace(seq_start=torch.from_numpy(start).cuda(), slots=torch.tensor([5, 0, 3, 1, 6, 2], dtype=torch.int32).cuda(),
                          n_seqs=len(lens), max_new=max(lens), engine=SimpleNamespace(sm_count=148))
    st = state0.clone().cuda()
    o = torch.empty((T, H * V), dtype=torch.float32, device="cuda")
    k.lin_attn_decay(proj.cuda(), 0, H * D, 2 * H * D, decay.cuda(), st, ctx, o, H, D, V)
    p = proj.double()
    q = plain.silu(p[:, :H * D]).view(T, H, D)
    kk = plain.silu(p[:, H * D:2 * H * D]).view(T, H, D)
    v = plain.silu(p[:, 2 * H * D:2 * H * D + H * V]).view(T, H, V)
    for b, slot in enumerate([5, 0, 3, 1, 6, 2]):
        for h in range(H):
            S = state0[slot, h].double()
            for t in range(start[b], start[b + 1]):
                S = float(decay[h]) * S + torch.outer(kk[t, h], v[t, h])
                want = S.T @ q[t, h]
                assert float((o[t].cpu().double().view(H, V)[h] - want).abs().max()) < 1e-4 * max(1.0, float(want.abs().max()))
            assert float((st[slot, h].cpu().double() - S).abs().max()) < 1e-4 * max(1.0, float(S.abs().max()))
    assert torch.equal(st[4].cpu(), state0[4])          # a slot no sequence of the step holds is left alone


def test_the_norm_adds_a_normed_addend_and_keeps_the_sum():
    from scriptling_llm_lib_b200.csrc.bindings import KernelSet
    for dtype in (torch.float32, torch.bfloat16):
        k = KernelSet(dtype).mix
        g = torch.Generator().manual_seed(5)
        x = torch.randn(9, 50, generator=g)
        parts = torch.randn(3, 9, 50, generator=g)
        pw, pb, w, b = (torch.randn(50, generator=g) for _ in range(4))
        want_x = x.double() + torch.tanh(0.7 * parts.double().sum(0)) * pw.double() + pb.double()
        want = torch.tanh(1.3 * want_x) * w.double() + b.double()
        xd = x.clone().cuda()
        out = torch.empty((9, 50), dtype=dtype, device="cuda")
        k.dyt_add_norm(xd, parts.cuda(), (pw.cuda(), pb.cuda(), 0.7), None, w.cuda(), b.cuda(), 1.3, out)
        assert float((xd.cpu().double() - want_x).abs().max()) < 1e-5
        assert float((out.cpu().double() - want).abs().max()) < (1e-5 if dtype == torch.float32 else 3e-2)
        rows = torch.tensor([7, 2], dtype=torch.int32).cuda()
        x2 = x.clone().cuda()
        out2 = torch.empty((2, 50), dtype=dtype, device="cuda")
        one = parts[0].to(dtype)
        k.dyt_add_norm(x2, one.cuda(), None, rows, w.cuda(), b.cuda(), 1.3, out2)
        want2 = torch.tanh(1.3 * (x.double() + one.double())[[7, 2]]) * w.double() + b.double()
        assert torch.equal(x2.cpu(), x)                  # picked rows: the stream is left as it was
        assert float((out2.cpu().double() - want2).abs().max()) < (1e-5 if dtype == torch.float32 else 3e-2)


def test_experts_one_by_one_and_grouped_agree(folders):
    """A step of few rows runs every (token, expert) pair by itself, a longer one groups them by expert."""
    folder, cfg, W = folders["A"]
    tokens = ids(80, cfg["vocab"], 18)
    eng = engine(folder)
    whole = run(eng, [tokens])                       # 80 rows x 2 experts: grouped
    small = run(eng, cut(tokens, [7] * 12))          # 7 rows a step: one by one
    assert rel(small, whole) < TOL_F32


# --------------------------------------------------------------------------- the entry point
def test_greedy_generation_through_the_entry_point(folders):
    from scriptling_llm_lib_b200 import llm
    folder, cfg, W = folders["A"]
    prompt = ids(21, cfg["vocab"], 19)
    for dtype in ("float32", "bfloat16"):
        out = llm.generate(str(folder), prompt, max_tokens=12, strategy="greedy", dtype=dtype)
        tokens = list(prompt)
        for t in out:
            lg = plain_logits(cfg, W, tokens)[-1]
            top2 = lg.topk(2).values
            if dtype == "float32" or float(top2[0] - top2[1]) > 0.2 * float(lg.abs().max()):
                assert int(lg.argmax()) == t
            tokens.append(t)
        assert len(out) == 12


def test_random_weights_mode_and_the_command_line(tmp_path):
    import subprocess
    import sys
    from pathlib import Path
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(CFG_B))
    eng = engine(f"random:{cfg_path}:3", "bfloat16")
    got = run(eng, [ids(40, CFG_B["vocab"], 1)])
    assert torch.isfinite(got).all() and float(got.abs().max()) > 0
    root = Path(__file__).resolve().parent.parent
    r = subprocess.run([sys.executable, "-m", "scriptling_llm_lib_b200", "-model", f"random:{cfg_path}:3", "-prompt", "1,2,3",
                        "-tokens", "4"], cwd=root, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
