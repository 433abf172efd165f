"""Bulodra on the device against the plain implementation: every mechanism alone (kernels, then
one-layer models), the stream after every layer, whole prompts, token-by-token decoding,
portions, unequal batches, reused slots and pages, window edges, sinks, far keys, long decoding,
greedy generation through the entry point, the command line and the trace replay program."""
import json
import math

import numpy as np
import pytest
import torch

import plain_bulodra as pb
import sonicboom_b200 as sb
from sonicboom_b200 import llm, ops
from sonicboom_b200.cache.kv import Cache, KVNeed
from sonicboom_b200.engine.step import StepEntry, StepPlan
from sonicboom_b200.parts.rotary import frequency_table, yarn_frequencies
from test_gpu_generate import replay
from bulodra_util import (CONFIGS, attention, attention_2, calm_tokens, dense, latent, layer, model, moe, rot, tokens,
                          write_model)

pytestmark = pytest.mark.gpu
# The largest root mean square of a row's difference, over the root mean square of the whole
# reference (a request's logits).  The plain implementation is float64; bfloat16 rounds to 2^-9.
TOL = {"float32": 3e-5, "bfloat16": 8e-2}
DTYPES = ["float32", "bfloat16"]
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
SEEN = {}
F = torch.float64


def rel_err(got, ref):
    ref = ref.to(F)
    ref = ref.reshape(-1, ref.shape[-1])
    d = got.to(F).cpu().reshape(ref.shape) - ref
    return float(d.pow(2).mean(-1).sqrt().max() / ref.pow(2).mean().sqrt().clamp_min(1e-30))


def model_err(got, ref, dtype):
    e = rel_err(got, ref)
    SEEN[dtype] = max(SEEN.get(dtype, 0.0), e)
    return e


def teardown_module(module):
    print("largest row errors of whole models:", {k: f"{v:.2e}" for k, v in SEEN.items()})


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, cfg in CONFIGS.items():
        d = tmp_path_factory.mktemp(f"bulodra{name}")
        out[name] = (d,) + write_model(d, cfg, seed=60 + ord(name))
    return out


@pytest.fixture(scope="module")
def engines(folders):
    made = {}

    def get(name, dtype, max_tokens=2048):
        key = (name, dtype)
        if key not in made:
            made[key] = sb.load_model(folders[name][0], dtype=dtype)
        return sb.Engine(made[key], max_tokens=max_tokens)
    return get


def run_cuts(engine, toks, cuts):
    """Logits at every position of one request fed in portions of the given sizes."""
    s = engine.open()
    outs, at = [], 0
    for n in cuts:
        outs.append(engine.step([(s, toks[at:at + n], list(range(n)))]).float().cpu())
        at += n
    assert at == len(toks)
    engine.close(s)
    return torch.cat(outs)


# ------------------------------------------------------------------ mechanisms alone: kernels
def test_norm_add_leaves_the_stream_in_the_other_dtype():
    g = torch.Generator().manual_seed(1)
    for rows, width in ((1, 8), (7, 44), (40, 1000), (3, 4096)):
        y, x = torch.randn(rows, width, generator=g) * 2, torch.randn(rows, width, generator=g)
        w = torch.randn(width, generator=g)
        ref = x.double() + pb.rms(y.double(), 1e-5) * w.double()
        out = torch.empty(rows, width, device="cuda")
        copy = torch.empty(rows, width, device="cuda", dtype=torch.bfloat16)
        ops.norm_add(y.cuda(), x.cuda(), w.cuda(), 1e-5, out, (None, 0.0, copy))
        assert rel_err(out, ref) < 2e-6 and torch.equal(copy, out.bfloat16())
        xc = x.cuda()
        assert torch.equal(ops.norm_add(y.cuda(), xc, w.cuda(), 1e-5, xc), out)          # in place, nothing along
        nw = torch.randn(width, generator=g)
        normed = torch.empty(rows, width, device="cuda")
        ops.norm_add(y.cuda(), x.cuda(), w.cuda(), 1e-5, torch.empty_like(out), (nw.cuda(), 1e-3, normed))
        assert rel_err(normed, pb.rms(ref, 1e-3) * nw.double()) < 1e-5


def test_gelu_gate_and_scale_and_norm_of_a_row_prefix():
    g = torch.Generator().manual_seed(2)
    for rows, ff in ((3, 8), (9, 304), (2, 20), (70, 7)):
        gu = torch.randn(rows, 2 * ff, generator=g) * 3
        ref = pb.gelu_tanh(gu[:, :ff].double()) * gu[:, ff:].double()
        out = ops.gated_act(gu.cuda(), ops.GATE_GELU_TANH, torch.empty(rows, ff, device="cuda"))
        assert rel_err(out, ref) < 2e-6
        if ff % 8 == 0:
            mixed = torch.stack([gu[:, :ff].view(rows, ff // 8, 8), gu[:, ff:].view(rows, ff // 8, 8)], 2).reshape(rows, 2 * ff)
            assert torch.equal(ops.gated_act(mixed.cuda(), ops.GATE_GELU_TANH, torch.empty(rows, ff, device="cuda"), True), out)
        silu = ops.gated_act(gu.cuda(), ops.GATE_SILU, torch.empty(rows, ff, device="cuda"))
        assert rel_err(silu, gu[:, :ff].double() * torch.sigmoid(gu[:, :ff].double()) * gu[:, ff:].double()) < 2e-6
    x = torch.randn(5, 33, generator=g)
    assert rel_err(ops.scale(x.cuda(), 0.3), x.double() * 0.3) < 1e-7
    wide, w = torch.randn(6, 52, generator=g), torch.randn(20, generator=g)
    out = ops.rmsnorm(wide.cuda(), w.cuda(), 1e-5, torch.empty(6, 20, device="cuda"), width=20)
    assert rel_err(out, pb.rms(wide[:, :20].double(), 1e-5) * w.double()) < 2e-6


@pytest.mark.parametrize("experts,top,groups,scale", [(6, 2, (3, 2), 1.7), (8, 3, (4, 3), 0.8), (4, 2, (2, 1), 2.2),
                                                      (5, 1, None, 1.0), (64, 6, (8, 4), 2.0), (6, 3, (6, 4), 1.0),
                                                      (12, 12, (3, 3), 1.0), (40, 4, (1, 1), 1.0)])
def test_router_scores_groups_and_weights(experts, top, groups, scale):
    g = torch.Generator().manual_seed(experts * 7 + top)
    rows = 50
    z = torch.randn(rows, experts, generator=g) * 2
    z[3] = z[3, 0]                                  # every score the same: the lowest indices win
    z[4, :] = torch.tensor([1.0, -1.0] * experts)[:experts]
    corr = torch.randn(experts, generator=g) * 0.3
    corr[-1] -= 3.0                                 # a choice score below zero
    r = {"experts": experts, "top": top, "scale": scale}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    ids = torch.empty(rows, top, dtype=torch.int32, device="cuda")
    w = torch.empty(rows, top, device="cuda")
    ops.moe_route_scored(z.cuda(), corr.cuda(), top, ids, w, groups=groups or (1, 1), group_top=2, scale=scale)
    for t in range(rows):
        chosen, weights, gap = pb.route(z[t].double(), corr.double(), r)
        if gap > 1e-5 or t in (3, 4):
            assert ids[t].tolist() == chosen, t
            assert torch.allclose(w[t].cpu().double(), torch.tensor(weights, dtype=F), rtol=1e-5), t
    none = torch.empty_like(w)
    ops.moe_route_scored(z.cuda(), None, top, ids, none, groups=groups or (1, 1), scale=scale, renormalize=True)
    assert torch.allclose(none.sum(-1).cpu(), torch.full((rows,), scale), rtol=1e-5)


def attend(dtype, seqs, hq, hkv, dim, vdim, window, scale, rotation, head_norm, norm_w, sink, softcap, gate_w,
           kernel="auto", eps=1e-5, cuts=None):
    """Projection rows of several sequences (float32 [n, q | gate | k | v]) through `attn_prep`, the
    attention kernels and `attn_unrotate`; a sequence may come in portions (`cuts`)."""
    hd = (max(dim, vdim) + 15) // 16 * 16
    cache = Cache([KVNeed(hkv, hd, window)], [None], 4096, DT[dtype], "cuda")
    slots = [cache.open() for _ in seqs]
    gw = hq if gate_w else 0
    if rotation.get("scaling"):
        f, mag = yarn_frequencies(rotation["base"], rotation["dims"], *[rotation["scaling"][k] for k in ("factor", "original", "fast", "slow")])
        table = torch.from_numpy(f.astype(np.float32)).cuda()
    else:
        table, mag = frequency_table(rotation["base"], rotation["dims"], "cuda"), 1.0
    outs = [[] for _ in seqs]
    at = [0] * len(seqs)
    for step in (cuts or [[x.shape[0] for x in seqs]]):
        live = [(i, n) for i, n in enumerate(step) if n]
        for i, n in live:
            cache.reserve(slots[i], cache.length(slots[i]) + n)
        plan = StepPlan(cache, [StepEntry(slots[i], [0] * n, []) for i, n in live], "cuda")
        proj = torch.cat([seqs[i][at[i]:at[i] + n] for i, n in live]).cuda()
        g, storage = plan.groups[0], cache.groups[0].entry_storage(0)
        q = torch.empty(proj.shape[0], hq, hd, dtype=DT[dtype], device="cuda")
        k_off = hq * dim + gw
        ops.attn_prep(proj, 0, k_off, k_off + hkv * dim, hq, hkv, dim, vdim, hd, rotation["dims"], False, table, None,
                      norm_w[0].cuda() if norm_w else None, norm_w[1].cuda() if norm_w else None, eps,
                      plan.row_seq, plan.row_pos, g.page_off, g.page_ids, g.page_size, storage, q,
                      head_norm=head_norm, rot_scale=mag)
        out = torch.empty(proj.shape[0], hq * hd, dtype=DT[dtype], device="cuda")
        ops.attention(q, out, plan, 0, storage, hq, hkv, hd, window, scale, kernel=kernel,
                      sink=sink.cuda() if sink is not None else None, softcap=softcap)
        if hd != vdim or gw:
            out = ops.attn_unrotate(out, torch.empty(proj.shape[0], hq * vdim, dtype=DT[dtype], device="cuda"), hq, hd,
                                    vdim, False, None, plan.row_pos, gate=(proj, hq * dim) if gw else None)
        out = out.float().cpu()
        row = 0
        for i, n in live:
            outs[i].append(out[row:row + n])
            row += n
            at[i] += n
            cache.advance(slots[i], cache.length(slots[i]) + n)
    return [torch.cat(o) for o in outs]


def attend_ref(x, hq, hkv, dim, vdim, window, scale, rotation, head_norm, norm_w, sink, softcap, gate_w, eps=1e-5):
    """The same on one whole sequence with the plain implementation's functions."""
    x = x.double()
    T = x.shape[0]
    gw = hq if gate_w else 0
    q = x[:, :hq * dim].reshape(T, hq, dim)
    k = x[:, hq * dim + gw:hq * dim + gw + hkv * dim].reshape(T, hkv, dim)
    v = x[:, hq * dim + gw + hkv * dim:].reshape(T, hkv, vdim)
    pos = list(range(T))
    if head_norm == "before":
        q, k = pb.rms(q, eps) * norm_w[0].double(), pb.rms(k, eps) * norm_w[1].double()
    q, k = pb.rotate(q, pos, rotation), pb.rotate(k, pos, rotation)
    if head_norm == "after":
        q, k = pb.rms(q, eps), pb.rms(k, eps)
    vis = pb.causal(T, window)
    out = torch.zeros(T, hq, vdim, dtype=F)
    for h in range(hq):
        s = (q[:, h] @ k[:, h // (hq // hkv)].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        o = pb.softmax_rows(s, vis, sink[h].double() if sink is not None else None) @ v[:, h // (hq // hkv)]
        out[:, h] = o * torch.sigmoid(x[:, hq * dim + h:hq * dim + h + 1]) if gw else o
    return out.reshape(T, hq * vdim)


ATTEND = [
    # hq, hkv, dim, vdim, window, rotation, head_norm, sink, softcap, gate
    (4, 2, 16, 24, 9, rot(10000.0, 8), "after", False, 5.0, True),
    (6, 3, 64, 32, 0, rot(100000.0, 32, (8.0, 64, 4.0, 0.5)), "before", True, 0.0, False),
    (2, 1, 64, 64, 70, rot(200000.0, 24), "after", False, 20.0, True),
    (8, 2, 128, 128, 100, rot(70000.0, 64), "after", False, 12.0, True),
    (3, 3, 8, 8, 3, rot(50.0, 2), "after", False, 1.5, False),
    (4, 1, 96, 96, 0, rot(300000.0, 64, (6.0, 256, 16.0, 2.0)), "before", True, 0.0, False),
    (2, 2, 48, 40, 33, rot(1000.0, 0), None, True, 4.0, True),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", range(len(ATTEND)))
def test_attention_rows_with_head_norms_cap_sink_and_gate(dtype, case):
    """Every attention kernel family: the plain one, the mma.sync ones, and at head sizes 64 and 128
    the tensor-memory prompt kernel and the TMA decode kernel; whole, in portions and one by one."""
    hq, hkv, dim, vdim, window, rotation, head_norm, has_sink, softcap, gate = ATTEND[case]
    g = torch.Generator().manual_seed(100 + case)
    width = hq * dim + (hq if gate else 0) + hkv * (dim + vdim)
    seqs = [torch.randn(n, width, generator=g) * 1.5 for n in (150, 37, 1)]
    norm_w = (torch.randn(dim, generator=g) * 0.2 + 1, torch.randn(dim, generator=g) * 0.2 + 1) if head_norm == "before" else None
    sink = torch.randn(hq, generator=g) + 1.0 if has_sink else None
    scale = 2.0 / math.sqrt(dim)
    args = (hq, hkv, dim, vdim, window, scale, rotation, head_norm, norm_w, sink, softcap, gate)
    refs = [attend_ref(x, *args) for x in seqs]
    tol = 2e-5 if dtype == "float32" else 3e-2
    kernels = ["auto"] if dtype == "float32" else ["auto", "plain", "mma"] + (["tma"] if max(dim, vdim) in (64, 128) else [])
    for kernel in kernels:
        for cuts in (None, [[100, 30, 0], [2, 7, 1], [48, 0, 0]], [[140, 36, 1]] + [[1, 1 if i == 0 else 0, 0] for i in range(10)]):
            outs = attend(dtype, seqs, *args, kernel=kernel, cuts=cuts)
            for o, r in zip(outs, refs):
                assert rel_err(o, r) < tol, (kernel, cuts and cuts[1])


# ------------------------------------------------------------------ mechanisms alone: one-layer models
ONE_LAYER = {
    "attention": layer("attention", attention(4, 2, 16, 24, rot(20000.0, 12, (3.0, 48, 6.0, 0.5)), scale=0.4)),
    "attention, plain rotation of the whole head": layer("attention", attention(2, 1, 32, 32, rot(100.0, 32))),
    "latent attention": layer("latent_attention", latent(3, 16, 8, 12, 24, 20, rot(5000.0, 8, (4.0, 32, 8.0, 1.0)))),
    "latent attention, few turned dimensions": layer("latent_attention", latent(2, 8, 16, 16, 16, 40, rot(300.0, 6))),
    "latent attention, more heads than one decode call takes": layer("latent_attention", latent(20, 8, 8, 8, 24, 16, rot(1000.0, 8))),
    "capped attention in a window": layer("attention_2", attention_2(4, 2, 16, 8, rot(10000.0, 8), 9, 5.0, scale=0.6)),
    "capped attention, no window": layer("attention_2", attention_2(2, 2, 16, 16, rot(10000.0, 16), 0, 3.0, scale=0.9)),
    "dense feed-forward": layer("attention_2", attention_2(1, 1, 16, 16, rot(10.0, 4), 2, 9.0), dense(56)),
    "dense feed-forward, odd size": layer("attention_2", attention_2(1, 1, 16, 16, rot(10.0, 4), 2, 9.0), dense(29)),
    "experts in groups": layer("attention_2", attention_2(1, 1, 16, 16, rot(10.0, 4), 2, 9.0),
                               moe(9, 3, 24, 1.2, groups=(3, 2), scale=1.4, shared=(16, 0.9))),
    "experts, no groups, no shared expert": layer("attention_2", attention_2(1, 1, 16, 16, rot(10.0, 4), 2, 9.0),
                                                  moe(4, 2, 11, 0.6, scale=3.0)),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(ONE_LAYER))
def test_each_mechanism_in_a_model_of_its_own(tmp_path, name, dtype):
    cfg, tensors = write_model(tmp_path / "one", model(90, 48, [ONE_LAYER[name]], mult=0.6, logit_scale=0.8), seed=len(name))
    toks, ref = calm_tokens(cfg, tensors, 75, 9)
    engine = sb.Engine(sb.load_model(tmp_path / "one", dtype=dtype), max_tokens=512)
    for cuts in ([75], [70, 1, 1, 1, 1, 1], [3, 2, 61, 9]):
        assert model_err(run_cuts(engine, toks, cuts), ref, dtype) < TOL[dtype], cuts


def test_the_stream_after_every_layer(folders, engines):
    _, cfg, tensors = folders["A"]
    toks = tokens(cfg, 50, 3)
    streams = []
    pb.forward(cfg, tensors, toks, layers_out=streams)
    engine = engines("A", "float32")
    seen = []
    for b in engine.model.blocks:
        inner = b.forward
        b.forward = lambda x, ctx, inner=inner: (lambda y: (seen.append(y.clone()), y)[1])(inner(x, ctx))
    try:
        run_cuts(engine, toks, [50])
    finally:
        for b in engine.model.blocks:
            del b.forward
    assert len(seen) == len(streams)
    for got, ref in zip(seen, streams):
        assert rel_err(got, ref) < 1e-5


# ------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_decoding_and_portions(folders, engines, name, dtype):
    _, cfg, tensors = folders[name]
    toks, ref = calm_tokens(cfg, tensors, 171, 5, key=name)
    engine = engines(name, dtype)
    whole = run_cuts(engine, toks, [171])
    assert model_err(whole, ref, dtype) < TOL[dtype]
    # the first tokens of a sequence one by one, then the rest; most of it at once, then one by one
    # over two page borders (64, 128) and every window's edge; portions down to two tokens
    for cuts in ([1, 1, 1, 168], [40] + [1] * 131, [2, 3, 62, 2, 59, 7, 17, 19], [64, 64, 43], [170, 1]):
        got = run_cuts(engine, toks, cuts)
        assert model_err(got, ref, dtype) < TOL[dtype], cuts
        if dtype == "float32":
            assert rel_err(got, whole) < 1e-5, cuts       # rounding: few rows run other kernels
    engine.cache.check()
    assert engine.free_pages() == engine.cache.n_pages


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_unequal_batch_equals_each_alone_and_slots_are_reused(folders, engines, name, dtype):
    from gpu_util import batch_unequal
    _, cfg, tensors = folders[name]
    reqs, refs = zip(*[calm_tokens(cfg, tensors, n, 10 + n, key=name) for n in (1, 70, 131, 23)])
    engine = engines(name, dtype, max_tokens=512)
    # twice in the same engine: the second pass reuses the slots and pages of the first
    for _ in range(2):
        outs = batch_unequal(engine, reqs, [1, 40, 100, 23])
        for o, r in zip(outs, refs):
            assert model_err(o, r, dtype) < TOL[dtype]
        engine.cache.check()
    alone = [run_cuts(engine, r, [k] + [1] * (len(r) - k)) for r, k in zip(reqs, [1, 40, 100, 23])]
    if dtype == "float32":
        for o, a in zip(outs, alone):
            assert rel_err(o, a) < 1e-5
    # a sequence that ends early gives its slot to a new one while the others go on
    a, b = engine.open(), engine.open()
    engine.step([(a, reqs[1][:30], []), (b, reqs[2][:50], [])])
    engine.close(a)
    c = engine.open()
    assert c == a
    lg = engine.step([(b, reqs[2][50:60], list(range(10))), (c, reqs[3], list(range(23)))]).float().cpu()
    assert rel_err(lg[:10], refs[2][50:60]) < TOL[dtype] and rel_err(lg[10:], refs[3]) < TOL[dtype]
    engine.close(b), engine.close(c)


def sharp_model():
    """Large score scales, so that a few keys carry a row's sum: a window one key off, a sink left
    out or a far key lost moves the logits by a large multiple of the tolerance."""
    return model(80, 48, [
        layer("attention_2", attention_2(2, 1, 16, 16, rot(10000.0, 8), window=13, softcap=40.0, scale=1.2)),
        layer("attention", attention(2, 2, 16, 16, rot(10000.0, 16, (4.0, 64, 8.0, 1.0)), scale=0.7), dense(32)),
        layer("attention_2", attention_2(2, 2, 32, 32, rot(40000.0, 16), window=70, softcap=25.0, scale=0.5)),
        layer("latent_attention", latent(2, 16, 8, 16, 24, 16, rot(10000.0, 8), scale=0.5)),
    ], mult=1.0, logit_scale=1.0)


def sharpen(t):
    for i in range(4):
        t[f"l{i}.mix.o"] *= 3.0
    t["l1.mix.sink"] = t["l1.mix.sink"] * 0.0 + 6.0
    t["l3.mix.sink"] = t["l3.mix.sink"] * 0.0 + 2.0


@pytest.mark.parametrize("dtype", DTYPES)
def test_window_edges_sinks_and_far_keys_show(tmp_path, dtype):
    cfg, tensors = write_model(tmp_path / "w", sharp_model(), seed=9, edit=sharpen)
    toks = tokens(cfg, 420, 21)
    ref = pb.forward(cfg, tensors, toks)
    shows = 300 * TOL["float32"]
    for which in (0, 2):
        for delta in (1, -1):
            other = json.loads(json.dumps(cfg))
            other["layers"][which]["mixer"]["mask"]["size"] += delta
            assert rel_err(pb.forward(other, tensors, toks)[100:], ref[100:]) > shows, (which, delta)
    for which in (1, 3):
        no_sink = dict(tensors)
        no_sink[f"l{which}.mix.sink"] = tensors[f"l{which}.mix.sink"] - 40.0
        assert rel_err(pb.forward(cfg, no_sink, toks), ref) > shows, which
    far = list(toks)
    far[3] = (toks[3] + 1) % cfg["vocab"]
    assert rel_err(pb.forward(cfg, tensors, far)[400:], ref[400:]) > shows
    engine = sb.Engine(sb.load_model(tmp_path / "w", dtype=dtype), max_tokens=1024)
    for cuts in ([420], [380] + [1] * 40, [12, 2, 50, 356], [13] + [1] * 120 + [287], [5, 200, 215]):
        assert rel_err(run_cuts(engine, toks, cuts), ref) < TOL[dtype], cuts[:4]


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_gives_pages_back(folders, engines, dtype):
    """Six hundred tokens one by one: the windows pass over many pages, which are given back; the
    layers without a window keep theirs."""
    _, cfg, tensors = folders["B"]
    toks, ref = calm_tokens(cfg, tensors, 600, 77, key="B")
    engine = engines("B", dtype, max_tokens=704)
    s = engine.open()
    engine.step([(s, toks[:5], [])])
    rows = []
    for i in range(5, 600):
        lg = engine.step([(s, [toks[i]], [0] if i % 7 == 0 or i > 590 else [])])
        if lg is not None:
            rows.append((i, lg.float().cpu()[0]))
    engine.close(s)
    got = torch.stack([r for _, r in rows])
    assert rel_err(got, ref[[i for i, _ in rows]]) < TOL[dtype]
    engine.cache.check()
    assert engine.free_pages() == engine.cache.n_pages


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_greedy_generation_through_the_entry_point(folders, name, dtype):
    """`llm.generate_batch`: the scheduler's batches, the captured decode step with the remembered
    token in it, and slots given to the next batch."""
    d, cfg, tensors = folders[name]
    m = llm.model_load(d, dtype=dtype)
    assert m.arch == "Bulodra" and m.vocab_size == cfg["vocab"]
    prompts = [tokens(cfg, n, 30 + n) for n in (3, 66, 20, 1)]
    n_new = 12
    outs = llm.generate_batch(m, prompts, max_tokens=n_new)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for i, t in enumerate(o):
            gaps = []
            logits = pb.forward(cfg, tensors, seq, gaps=gaps)[-1]
            best = int(torch.argmax(logits))
            if t != best:
                top2 = torch.topk(logits, 2).values
                margin = float(top2[0] - top2[1]) / float(logits.abs().max())
                close_call = min((min(g) for g in gaps), default=1.0) < 0.05
                assert dtype == "bfloat16" and (margin < 2 * TOL[dtype] or close_call), (i, o, margin)
                break
            seq.append(t)
    alone = [llm.generate_batch(m, [p], max_tokens=n_new)[0] for p in prompts]
    small = llm.generate_batch(m, prompts, max_tokens=n_new, max_cache_tokens=192)     # more than one batch
    if dtype == "float32":
        assert alone == outs and small == outs
    s = llm.session_new(m, 128)
    assert llm.generate_tokens(s, prompts[2], n_new) == alone[2]
    s.free()


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_program(folders, tmp_path, dtype):
    d, cfg, tensors = folders["B"]
    (a, ra), (b, rb) = calm_tokens(cfg, tensors, 75, 1, key="B"), calm_tokens(cfg, tensors, 30, 2, key="B")
    ra, rb = ra.numpy(), rb.numpy()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": [0, 69]},
                                     {"id": "b", "tokens": b[:29], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[70:71], "want": [0]},
                                     {"id": "b", "tokens": b[29:], "want": [0]}], "end": ["b"]}]
    steps += [{"step": i - 69, "entries": [{"id": "a", "tokens": [a[i]], "want": [0] if i % 2 else []}],
               "end": ["a"] if i == 74 else []} for i in range(71, 75)]
    got = replay(d, dtype, steps, tmp_path / "out", 256)
    V = cfg["vocab"]
    want = {0: ra[[0, 69]], 1: np.stack([ra[70], rb[29]]), 2: ra[71:72], 4: ra[73:74]}
    assert set(got) == set(want)
    for k, ref in want.items():
        assert np.abs(got[k].reshape(-1, V) - ref).max() / np.abs(ra).max() < TOL[dtype], k


def test_command_line_generates(folders, tmp_path):
    """`python -m sonicboom_b200 generate` on a Bulodra folder: greedy tokens as the plain
    implementation's."""
    import subprocess
    import sys
    from conftest import ROOT
    d, cfg, tensors = folders["A"]
    prompts = [tokens(cfg, n, 50 + n) for n in (7, 33)]
    f = tmp_path / "prompts.txt"
    f.write_text("".join(" ".join(map(str, p)) + "\n" for p in prompts))
    base = [sys.executable, "-m", "sonicboom_b200", "generate", "-m", str(d), "--tokens", str(f), "-n", "6",
            "--dtype", "float32"]
    r = subprocess.run(base, capture_output=True, text=True, cwd=ROOT, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    got = [[int(t) for t in line.split()] for line in r.stdout.strip().splitlines()]
    assert got == [pb.greedy_generate(cfg, tensors, p, 6) for p in prompts]
