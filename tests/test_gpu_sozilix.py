"""The Sozilix decoder on the GPU against the plain statement in plain_sozilix.py: each mechanism
alone, whole prompts against token-by-token decoding and against portions, unequal batches, slots
and pages used again, window and page borders, other sizes, greedy generation through the entry
point. Configurations and weights are made here; weights are larger than a trained model's so that
every branch moves the logits."""
import json
import math

import numpy as np
import pytest
import torch

import plain_sozilix as plain

pytestmark = pytest.mark.gpu

TOL_F32 = 2e-4       # of a row's largest logit
TOL_BF16 = 6e-2


def attention(heads=4, kv_heads=2, dim=16, vdim=8, window=5, rot=8, base=100.0, scale=0.3):
    return {"dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": window}, "rot": {"base": base, "dims": rot},
            "scale": scale, "vdim": vdim}


def delta(heads=2, kv_heads=1, dim=8, vdim=24, conv=2):
    return {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim}


def parallel(left=None, right=None, left_scale=1.3, right_scale=0.4, ff=None):
    return {"type": "parallel", "mixer": {"left": left or attention(), "right": right or delta(), "left_scale": left_scale,
                                          "right_scale": right_scale}, "mlp": None if ff is None else {"ff": ff, "kind": "dense"}}


def rglru(width=48, blocks=3, conv=4, ff=None):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv},
            "mlp": None if ff is None else {"ff": ff, "kind": "dense"}}


def config(layers, width=64, vocab=96, taps=3, mult=0.5, eps=1e-6):
    return {"architecture": "Sozilix", "canon": {"taps": taps}, "layers": layers, "norm": {"eps": eps}, "residual_mult": mult,
            "vocab": vocab, "width": width}


# sizes that differ from one another in every number; B has keys and values of one width (64: the
# attention kernels that the library's other models use), a window beyond a page and heads that
# share nothing; C has widths off every power of two, one tap, one block.
CFG_A = config([rglru(ff=80), parallel(), rglru(width=32, blocks=1, conv=2), parallel(ff=72)])
CFG_B = config([parallel(attention(2, 2, 64, 64, 70, 64, 10000.0, 0.125), delta(3, 3, 16, 16, 4), 0.7, 1.1, ff=96), rglru(64, 4, 3)],
               width=96, vocab=130, taps=2, mult=1.0, eps=1e-5)
CFG_C = config([parallel(attention(3, 1, 24, 40, 9, 6, 50.0, 0.2), delta(4, 2, 20, 12, 1), 1.0, 1.0), rglru(40, 2, 1, ff=56)],
               width=72, vocab=77, taps=1, mult=0.3)
# keys and values both 128 wide (the other width of the tensor-core attention kernels), a delta rule with wide keys
CFG_D = config([rglru(56, 7, 2), parallel(attention(4, 1, 128, 128, 90, 32, 1000.0, 0.09), delta(2, 2, 160, 24, 3), 0.9, 0.8, ff=64)],
               width=80, vocab=101, taps=5, mult=0.7, eps=1e-5)


def random_weights(cfg, seed, std=0.25):
    """Weights by tensor name for `cfg`, bfloat16-representable (the folder stores bfloat16)."""
    from scriptling_llm_lib_b200 import models  # noqa: F401
    from scriptling_llm_lib_b200.config.registry import architecture_for
    from scriptling_llm_lib_b200.engine.model import DecoderModel
    arch = architecture_for("Sozilix")
    specs = DecoderModel(arch.layout(arch.config_class.from_dict(cfg, "test"))).tensor_specs()
    g = torch.Generator().manual_seed(seed)
    W = {}
    for s in specs:
        t = torch.randn(s.shape, generator=g)
        if s.init == "norm_weight":
            t = 1.0 + 0.2 * t
        elif s.init in ("log_rate",):
            t = 0.5 * t
        elif s.init == "matrix":
            t = t * std * (4.0 / math.sqrt(s.shape[-1]))
        elif s.init == "gate_matrix":
            t = t * (2.0 / math.sqrt(s.shape[-1]))
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


def run(eng, pieces, want_all=True):
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


def close(got, want, tol):
    worst = float(((got - want).abs().amax(-1) / want.abs().amax(-1)).max())
    assert worst <= tol, f"largest difference {worst:.3e} of a row's largest logit (allowed {tol:.1e})"


# ------------------------------------------------------------------ mechanisms alone
ALONE = {
    "attention": config([parallel(left_scale=1.0, right_scale=0.0)]),
    "attention_one_head_per_group": config([parallel(attention(3, 3, 8, 16, 4, 2, 7.0, 0.5), left_scale=1.0, right_scale=0.0)]),
    "attention_no_rotation_long_window": config([parallel(attention(2, 1, 16, 16, 1000, 0, 10.0, 0.25), left_scale=1.0, right_scale=0.0)]),
    "delta_rule": config([parallel(left_scale=0.0, right_scale=1.0)]),
    "delta_rule_heads_of_their_own": config([parallel(right=delta(3, 3, 12, 8, 3), left_scale=0.0, right_scale=1.0)]),
    "delta_rule_wide_keys": config([parallel(right=delta(2, 1, 80, 40, 2), left_scale=0.0, right_scale=1.0)], width=48),
    "rglru": config([rglru()]),
    "rglru_one_block_one_tap": config([rglru(40, 1, 1)], taps=1),
    "feed_forward_and_convolution": config([rglru(16, 2, 2, ff=88)], taps=5),
}


@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone_whole_and_token_by_token(tmp_path, name):
    cfg = ALONE[name]
    W = random_weights(cfg, 11)
    d = write_folder(tmp_path / "m", cfg, W)
    toks = ids(37, cfg["vocab"], 5)
    want = plain.forward(toks, W, cfg)
    eng = engine(d)
    close(run(eng, [toks]), want, TOL_F32)
    close(run(eng, [[t] for t in toks]), want, TOL_F32)
    close(run(engine(d, "bfloat16"), [toks[:20]] + [[t] for t in toks[20:]]), want, TOL_BF16)


def test_the_residual_stream_after_every_layer(tmp_path):
    """The stream itself, layer by layer: a model cut after layer i with a final norm of ones and the
    identity as head returns the stream's rows, centred and scaled."""
    W = random_weights(CFG_A, 3)
    width = CFG_A["width"]
    toks = ids(19, width, 1)
    for i in range(len(CFG_A["layers"])):
        cfg = dict(CFG_A, layers=CFG_A["layers"][:i + 1], vocab=width)
        Wi = {k: v for k, v in W.items() if k.startswith(tuple(f"l{j}." for j in range(i + 1)))}
        Wi["embed"] = W["embed"][:width].clone() if W["embed"].shape[0] >= width else torch.randn(width, width).to(torch.bfloat16)
        Wi["final.norm"] = torch.ones(width, dtype=torch.bfloat16)
        Wi["head"] = torch.eye(width, dtype=torch.bfloat16)
        streams = []
        want = plain.forward(toks, Wi, cfg, streams)
        x = streams[-1]
        ref = (x - x.mean(-1, keepdim=True)) / torch.sqrt(x.var(-1, unbiased=False, keepdim=True) + cfg["norm"]["eps"])
        assert float((want - ref).abs().max()) < 1e-9
        got = run(engine(write_folder(tmp_path / f"m{i}", cfg, Wi)), cut(toks, [6, 1, 5]))
        close(got, ref, TOL_F32)


# ------------------------------------------------------------------ whole models
@pytest.mark.parametrize("cfg,seed", [(CFG_A, 1), (CFG_B, 2), (CFG_C, 3), (CFG_D, 4)])
def test_prompt_portions_and_decoding_agree_with_the_plain_model(tmp_path, cfg, seed):
    W = random_weights(cfg, seed)
    d = write_folder(tmp_path / "m", cfg, W)
    toks = ids(150, cfg["vocab"], seed)
    want = plain.forward(toks, W, cfg)
    eng = engine(d)
    close(run(eng, [toks]), want, TOL_F32)
    for sizes in ([2] * 10 + [3, 64, 1, 2], [63, 2, 64], [1, 1, 126], [128]):
        close(run(eng, cut(toks, sizes)), want, TOL_F32)
    close(run(eng, [toks[:7]] + [[t] for t in toks[7:]]), want, TOL_F32)          # long decoding over page and window borders
    e16 = engine(d, "bfloat16")
    close(run(e16, [toks]), want, TOL_BF16)
    close(run(e16, cut(toks, [70, 2, 5]) ), want, TOL_BF16)
    close(run(e16, [toks[:66]] + [[t] for t in toks[66:]]), want, TOL_BF16)


@pytest.mark.parametrize("dtype,tol", [("float32", TOL_F32), ("bfloat16", TOL_BF16)])
@pytest.mark.parametrize("cfg", [CFG_A, CFG_B])
def test_a_batch_of_unequal_requests_equals_each_alone(tmp_path, cfg, dtype, tol):
    from scriptling_llm_lib_b200.engine.step import StepEntry
    W = random_weights(cfg, 7)
    d = write_folder(tmp_path / "m", cfg, W)
    lens = [1, 70, 5, 129, 33]
    n_dec = 9
    prompts = [ids(n + n_dec, cfg["vocab"], 100 + n) for n in lens]
    want = [plain.forward(p, W, cfg) for p in prompts]
    eng = engine(d, dtype, max_seqs=8)
    seqs = [eng.open() for _ in prompts]
    got = [[] for _ in prompts]
    out = eng.step([StepEntry(s, p[:n], list(range(n))) for s, p, n in zip(seqs, prompts, lens)])
    at = 0
    for i, n in enumerate(lens):
        got[i].append(out[at:at + n])
        at += n
    live = list(range(len(prompts)))
    for k in range(n_dec):
        if k == 4:                              # two requests end early; the batch shrinks
            for i in (1, 3):
                seqs[i].close()
                live.remove(i)
        out = eng.step([StepEntry(seqs[i], [prompts[i][lens[i] + k]], [0]) for i in live])
        for j, i in enumerate(live):
            got[i].append(out[j:j + 1])
    eng.check_errors()
    for i in range(len(prompts)):
        g = torch.cat(got[i]).cpu().double()
        close(g, want[i][:g.shape[0]], tol)


def test_slots_and_pages_used_again_start_from_nothing(tmp_path):
    """A sequence that takes over a slot and pages another one used must not see its state, its
    convolutions' last inputs or its keys."""
    from scriptling_llm_lib_b200.engine.step import StepEntry
    cfg = CFG_A
    W = random_weights(cfg, 9)
    d = write_folder(tmp_path / "m", cfg, W)
    eng = engine(d, max_tokens=256, max_seqs=2)
    a, b = ids(130, cfg["vocab"], 1), ids(90, cfg["vocab"], 2)
    want_b = plain.forward(b, W, cfg)
    for _ in range(3):
        s = eng.open()
        eng.step([StepEntry(s, a[:100], [])])
        for t in a[100:]:
            eng.step([StepEntry(s, [t], [0])])
        slot = s.slot
        s.close()
        close(run(eng, cut(b, [3, 64])), want_b, TOL_F32)
        s2 = eng.open()
        assert s2.slot == slot
        s2.close()
    assert eng.cache.slots.n_held == 0 and all(g.pool.n_held == 0 for g in eng.cache.groups)


def test_a_window_gives_its_pages_back_while_decoding(tmp_path):
    from scriptling_llm_lib_b200.engine.step import StepEntry
    cfg = config([parallel(attention(2, 1, 16, 32, 66, 4, 30.0, 0.25))], width=32, vocab=50)
    W = random_weights(cfg, 4)
    d = write_folder(tmp_path / "m", cfg, W)
    toks = ids(300, cfg["vocab"], 8)
    want = plain.forward(toks, W, cfg)
    eng = engine(d, max_tokens=64 * 5, max_seqs=1)
    s = eng.open()
    got = [eng.step([StepEntry(s, toks[:100], list(range(100)))])]
    for t in toks[100:]:
        got.append(eng.step([StepEntry(s, [t], [0])]))
        assert eng.cache.groups[0].pool.n_held <= 3      # a window of 66 never spans more than three pages: older ones return
    close(torch.cat(got).cpu().double(), want, TOL_F32)


# ------------------------------------------------------------------ attention: one key that matters
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd,vd,window", [(16, 8, 70), (24, 40, 64), (48, 128, 129), (32, 32, 1), (8, 16, 0)])
def test_attention_sees_the_window_s_first_key_and_not_the_one_before(dtype, hd, vd, window):
    """Among hundreds of keys one is made to stand out, once just inside the window (at a page
    border where the window allows) and once just outside: the row's output is that key's value, or
    has nothing of it. Pages are scattered over the store."""
    from scriptling_llm_lib_b200.csrc.bindings import KernelSet
    k = KernelSet(dtype).seq
    H, G, T, PAGE = 4, 2, 333, 64
    dev = "cuda:0"
    g = torch.Generator().manual_seed(hd * 1000 + vd)
    n_pages = -(-T // PAGE)
    order = torch.randperm(n_pages + 3, generator=g)[:n_pages].to(torch.int32)
    q = (0.1 * torch.randn(T, H, hd, generator=g))
    kk = (0.1 * torch.randn(T, G, hd, generator=g))
    v = torch.randn(T, G, vd, generator=g)
    pos = torch.arange(T)
    w = window if window > 0 else T
    inside = pos - (w - 1)                      # the oldest key a row sees
    probe_rows = [r for r in (w - 1, w, 200, 255, 256, T - 1) if 0 <= r < T and inside[r] >= 0]
    for case in ("inside", "outside"):
        qq, kc = q.clone(), kk.clone()
        loud = []
        for r in probe_rows:
            j = int(inside[r]) - (1 if case == "outside" else 0)
            if j < 0:
                continue
            qq[r] = 0.0
            qq[r, :, hd - 1] = 6.0
            kc[j, :, hd - 1] = 6.0             # score 36 against about 0 for every other key
            loud.append(j)
        qkv = torch.cat([qq.reshape(T, -1), kc.reshape(T, -1), v.reshape(T, -1)], dim=1).to(dtype).to(dev).contiguous()
        kp = torch.zeros(n_pages + 3, G, PAGE, hd, dtype=dtype, device=dev)
        vp = torch.zeros(n_pages + 3, G, PAGE, vd, dtype=dtype, device=dev)
        tok_pos = pos.to(torch.int32).to(dev)
        tok_seq = torch.zeros(T, dtype=torch.int32, device=dev)
        table = order.view(1, -1).to(dev).contiguous()
        k.kv_store(qkv, tok_pos, tok_seq, table, None, kp, vp, H, G, hd, vd, 0, True, None)
        out = torch.empty(T, H * vd, dtype=dtype, device=dev)
        k.attn_wide_value(qkv, out, tok_pos, tok_seq, table, kp, vp, H, G, hd, vd, window, 1.0)
        out = out.float().cpu().view(T, H, vd)
        # the plain answer for all rows
        qd, kd, vdd = qkv[:, :H * hd].float().cpu().view(T, H, hd).double(), kc.to(dtype).double(), v.to(dtype).double()
        for h in range(H):
            s = qd[:, h] @ kd[:, h // (H // G)].T
            seen = (pos[:, None] - pos[None, :] >= 0) & (pos[:, None] - pos[None, :] < w)
            p = torch.softmax(s.masked_fill(~seen, float("-inf")), -1)
            ref = p @ vdd[:, h // (H // G)]
            tol = 1e-5 if dtype == torch.float32 else 2e-2
            assert float((out[:, h].double() - ref).abs().max()) <= tol * float(ref.abs().max())
        for r in probe_rows:
            j = int(inside[r])
            if case == "inside" and sum(j <= x <= r for x in loud) == 1:       # the one loud key in sight is the oldest
                assert float((out[r, 0].double() - vdd[j, 0]).abs().max()) < 0.05 * float(vdd[j, 0].abs().max()) + 0.02


def test_values_are_cached_with_unit_root_mean_square_and_keys_rotated():
    from scriptling_llm_lib_b200.csrc.bindings import KernelSet
    k = KernelSet(torch.float32).seq
    H, G, hd, vd, T, rot = 2, 2, 12, 20, 70, 6
    dev = "cuda:0"
    g = torch.Generator().manual_seed(1)
    qkv = torch.randn(T, (H + G) * hd + G * vd, generator=g)
    pos = torch.arange(5, 5 + T)
    ang = pos.double()[:, None] * (30.0 ** (-2.0 * torch.arange(rot // 2).double() / rot))[None, :]
    table = torch.zeros(5 + T, rot // 2, 2)
    table[5:] = torch.stack([torch.cos(ang), torch.sin(ang)], -1).float()
    kp = torch.zeros(3, G, 64, hd, device=dev)
    vp = torch.zeros(3, G, 64, vd, device=dev)
    bt = torch.tensor([[2, 0]], dtype=torch.int32, device=dev)
    dq = qkv.to(dev).contiguous()
    k.kv_store(dq, pos.to(torch.int32).to(dev), torch.zeros(T, dtype=torch.int32, device=dev), bt, table.to(dev), kp, vp, H, G,
               hd, vd, rot, True, 1e-3)
    want_q = plain.rotate_interleaved(qkv[:, :H * hd].double().view(T, H, hd), pos, rot, 30.0)
    want_k = plain.rotate_interleaved(qkv[:, H * hd:(H + G) * hd].double().view(T, G, hd), pos, rot, 30.0)
    want_v = plain.rms_unit(qkv[:, (H + G) * hd:].double().view(T, G, vd), 1e-3)
    assert float((dq[:, :H * hd].cpu().double().view(T, H, hd) - want_q).abs().max()) < 1e-5
    for t in (0, 58, 59, 69):
        p = int(pos[t])
        page = int(bt[0, p // 64])
        assert float((kp[page, :, p % 64].cpu().double() - want_k[t]).abs().max()) < 1e-5
        assert float((vp[page, :, p % 64].cpu().double() - want_v[t]).abs().max()) < 1e-5


# ------------------------------------------------------------------ kernels of the recurrent parts
class _Ctx:
    def __init__(self, lens, slots, dev):
        start = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        self.seq_start = torch.from_numpy(start).to(dev)
        self.tok_seq = torch.from_numpy(np.repeat(np.arange(len(lens), dtype=np.int32), lens)).to(dev)
        self.slots = torch.tensor(slots, dtype=torch.int32, device=dev)
        self.n_seqs, self.max_new = len(lens), max(lens)


@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_the_short_convolution_carries_its_last_inputs_across_steps(taps):
    from scriptling_llm_lib_b200.csrc.bindings import KernelSet
    k = KernelSet(torch.float32).seq
    dev, C = "cuda:0", 37
    g = torch.Generator().manual_seed(taps)
    w, bias, ib = torch.randn(C, taps, generator=g), torch.randn(C, generator=g), torch.randn(C, generator=g)
    xs = [torch.randn(n, C, generator=g) for n in (23, 9)]
    want = [plain.silu(plain.causal_conv(x.double() + ib.double(), w.double(), bias.double()) + x.double() + ib.double()) for x in xs]
    state = torch.full((4, max(taps - 1, 1), C), 7.0, device=dev)[:, :taps - 1].contiguous() if taps > 1 else None
    if state is not None:
        state[1].zero_()
        state[3].zero_()
    got = [[], []]
    at = [0, 0]
    for sizes in ([1, 2], [2, 1], [5, 3], [1, 1], [14, 2]):           # both sequences in every step, unequal pieces
        x = torch.cat([xs[i][at[i]:at[i] + n] for i, n in enumerate(sizes)]).to(dev).contiguous()
        y = torch.empty_like(x)
        k.causal_conv(x, w.to(dev), state, _Ctx(sizes, [3, 1], dev), y, taps, in_bias=ib.to(dev), out_bias=bias.to(dev),
                      add_input=True, act="silu")
        o = 0
        for i, n in enumerate(sizes):
            got[i].append(y[o:o + n].cpu())
            o += n
            at[i] += n
    for i in range(2):
        assert float((torch.cat(got[i]).double() - want[i]).abs().max()) < 1e-5


@pytest.mark.parametrize("center", [True, False])
def test_the_norm_adds_weighted_addends_in_float(center):
    from scriptling_llm_lib_b200.csrc.bindings import KernelSet
    k = KernelSet(torch.bfloat16).seq
    dev, T, d = "cuda:0", 9, 70
    g = torch.Generator().manual_seed(2)
    x = torch.randn(T, d, generator=g) * 3 + 5.0
    a1, a2 = torch.randn(T, d, generator=g).to(torch.bfloat16), torch.randn(T, d, generator=g)
    w = (1 + 0.1 * torch.randn(d, generator=g)).to(torch.bfloat16)
    v = x.double() + 0.3 * a1.double() - 1.7 * a2.double()
    want = plain.layer_norm(v, w.double(), 1e-5) if center else plain.rms_unit(v, 1e-5) * w.double()
    xd = x.to(dev)
    y = torch.empty(T, d, dtype=torch.float32, device=dev)
    k.add_norm(xd, [(a1.to(dev), 0.3), (a2.to(dev), -1.7)], None, w.to(dev), y, 1e-5, center)
    assert float((y.cpu().double() - want).abs().max()) < 1e-5
    assert float((xd.cpu().double() - v).abs().max()) < 1e-5
    rows = torch.tensor([4, 0], dtype=torch.int32, device=dev)
    y2 = torch.empty(2, d, dtype=torch.bfloat16, device=dev)
    k.add_norm(xd, [], rows, w.to(dev), y2, 1e-5, center)
    assert float((y2.cpu().double() - want[[4, 0]]).abs().max()) < 3e-2


def test_the_delta_rule_forgets_by_its_decay_and_overwrites_along_a_key():
    """With beta = 1 and decay = 1, writing value v along a unit key k and reading with q = k returns v;
    writing again along the same key replaces it; with decay g the old content is read g times weaker."""
    from scriptling_llm_lib_b200.csrc.bindings import KernelSet
    k = KernelSet(torch.float32).seq
    dev, H, G, dk, dv = "cuda:0", 2, 1, 8, 40
    e0, e1 = torch.zeros(dk), torch.zeros(dk)
    e0[0], e1[3] = 1.0, 1.0
    qk = torch.stack([torch.cat([e0, e0]), torch.cat([e0, e1]), torch.cat([e0, e0]), torch.cat([e1, e1])]).to(dev).contiguous()
    g = torch.Generator().manual_seed(0)
    v = torch.randn(4, H * dv, generator=g).to(dev)
    # beta | decay | k . q of the row
    bd = torch.tensor([[1, 1, 1, 1, 1], [1, 1, 0.5, 0.25, 0], [1, 1, 1, 1, 1], [0, 0, 1, 1, 1]], dtype=torch.float32, device=dev)
    state = torch.zeros(3, H, dk, dv, device=dev)
    o = torch.empty(4, H * dv, device=dev)
    k.delta_rule(qk, v, bd, state, _Ctx([4], [2], dev), o, H, G, dk, dv)
    o, v = o.cpu().view(4, H, dv), v.cpu().view(4, H, dv)
    assert torch.allclose(o[0], v[0], atol=1e-6)                                   # written and read at once
    assert torch.allclose(o[1, 0], 0.5 * v[0, 0], atol=1e-6) and torch.allclose(o[1, 1], 0.25 * v[0, 1], atol=1e-6)
    assert torch.allclose(o[2], v[2], atol=1e-6)                                   # the same key again: replaced
    assert torch.allclose(o[3], v[1], atol=1e-6)                                   # beta 0 writes nothing; the other key still holds
    assert float(state[:2].abs().max()) == 0.0 and float(state[2].abs().max()) > 0


# ------------------------------------------------------------------ generation
@pytest.mark.parametrize("cfg,seed", [(CFG_A, 21), (CFG_B, 22)])
def test_greedy_generation_through_the_entry_point(tmp_path, cfg, seed):
    from scriptling_llm_lib_b200 import llm
    llm.unload()
    W = random_weights(cfg, seed)
    d = write_folder(tmp_path / "m", cfg, W)
    prompts = [ids(n, cfg["vocab"], 40 + n) for n in (5, 67, 1, 20)]
    n_new = 10

    def greedy(p):
        out = []
        for _ in range(n_new):
            out.append(int(plain.forward(list(p) + out, W, cfg)[-1].argmax()))
        return out
    want = [greedy(p) for p in prompts]
    got = llm.generate(str(d), prompts, n_new, "greedy", stop_ids=[], dtype="float32")
    assert got == want
    assert llm.generate(str(d), prompts[1], n_new, "greedy", stop_ids=[], dtype="float32") == want[1]
    got16 = llm.generate(str(d), prompts, n_new, "greedy", stop_ids=[], dtype="bfloat16")
    for p, g in zip(prompts, got16):           # every token is a maximum of the plain logits on its own path, within rounding
        for i, t in enumerate(g):
            lg = plain.forward(list(p) + g[:i], W, cfg)[-1]
            assert float(lg.max() - lg[t]) <= TOL_BF16 * float(lg.abs().max())
    llm.unload()


def test_random_weights_mode_and_the_command_line(tmp_path):
    """A model that exists only as a configuration and a seed equals the folder random-weights mode writes for
    it, and the command line generates from either."""
    import subprocess
    import sys
    from pathlib import Path
    from scriptling_llm_lib_b200 import llm
    llm.unload()
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(CFG_C))
    folder = llm.random_model(str(cfg_path), 5, tmp_path / "m")
    prompt = ids(9, CFG_C["vocab"], 3)
    a = llm.generate(str(folder), prompt, 6, "greedy", stop_ids=[], dtype="float32")
    b = llm.generate(f"random:{cfg_path}:5", prompt, 6, "greedy", stop_ids=[], dtype="float32")
    assert a == b and len(a) == 6
    root = Path(__file__).resolve().parent.parent
    out = subprocess.run([sys.executable, str(root / "bin" / "sllm-b200"), "-model", str(tmp_path / "m2"), "-random", str(cfg_path),
                          "-seed-weights", "5", "-prompt", ",".join(map(str, prompt)), "-tokens", "6", "-dtype", "float32", "-stop", ""],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    assert [int(t) for t in out.stdout.replace(",", " ").split()] == a
    llm.unload()
