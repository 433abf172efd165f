"""Leguvik on the device against the plain implementation: every mechanism alone (kernels, then
one-layer models), whole prompts, token-by-token decoding, portions, unequal batches, reused
slots, pages and state rows, window edges and kept first keys, far tokens, long decoding, greedy
generation through the entry point, the command line and the trace replay program."""
import json

import numpy as np
import pytest
import torch

import plain_leguvik as pl
import sonicboom_b200 as sb
from sonicboom_b200 import llm, ops
from sonicboom_b200.cache.kv import Cache, KVNeed, StateNeed
from sonicboom_b200.engine.step import StepEntry, StepPlan
from test_gpu_generate import replay
from leguvik_util import CONFIGS, attention, delta, layer, model, moe, ssm, tokens, write_model

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


CLOSE = {}                # id of a reference -> rows that a close call of a router may have moved
CLOSE_GAP, CLOSE_REACH = 0.02, 4


def reference(cfg, tensors, toks):
    """The plain implementation's logits.  It also notes where a router's choice was close (the
    gap to the best expert not chosen below CLOSE_GAP, a few times what bfloat16 rounding moves
    a logit by): there the bfloat16 model may choose another expert, which is no fault; the input
    convolutions spread the difference over the next rows (CLOSE_REACH rows are excused), and what
    the recurrent states carry on from there stays within the tolerance."""
    gaps = []
    ref = pl.forward(cfg, tensors, toks, gaps=gaps)
    close = torch.zeros(len(toks), dtype=torch.bool)
    for t in (torch.nonzero(torch.stack(gaps).min(0).values < CLOSE_GAP).flatten().tolist() if gaps else []):
        close[t:t + CLOSE_REACH] = True
    CLOSE[id(ref)] = (ref, close)
    return ref


def model_err(got, ref, dtype):
    """The largest row error; in bfloat16 over the rows that no close router call excuses (at least
    half of them, and the excused rows stay within ten times the tolerance)."""
    refd = ref.to(F).reshape(-1, ref.shape[-1])
    rows = (got.to(F).cpu().reshape(refd.shape) - refd).pow(2).mean(-1).sqrt() / refd.pow(2).mean().sqrt().clamp_min(1e-30)
    if dtype == "bfloat16" and id(ref) in CLOSE:
        close = CLOSE[id(ref)][1]
        assert int(close.sum()) * 2 <= close.numel() and float(rows.max()) < 10 * TOL[dtype]
        rows = rows[~close]
    e = float(rows.max())
    SEEN[dtype] = max(SEEN.get(dtype, 0.0), e)
    return e


def teardown_module(module):
    print("largest row errors of whole models:", {k: f"{v:.2e}" for k, v in SEEN.items()})


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, cfg in CONFIGS.items():
        d = tmp_path_factory.mktemp(f"leguvik{name}")
        out[name] = (d,) + write_model(d, cfg, seed=40 + ord(name))
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


def plan_for(cache, slots, lens):
    for s, n in zip(slots, lens):
        cache.reserve(s, cache.length(s) + n)
    return StepPlan(cache, [StepEntry(s, [0] * n, []) for s, n in zip(slots, lens)], "cuda")


def done(cache, slots, lens):
    for s, n in zip(slots, lens):
        cache.advance(s, cache.length(s) + n)


# ------------------------------------------------------------------ mechanisms alone: kernels
def test_layer_norm_rows():
    g = torch.Generator().manual_seed(1)
    for rows, width in ((1, 8), (7, 44), (40, 1000), (3, 5000)):
        x = torch.randn(rows, width, generator=g) * 3 + 1.5
        w = torch.randn(width, generator=g)
        ref = pl.layer_norm(x.double(), w.double(), 1e-5)
        out = ops.layernorm(x.cuda(), w.cuda(), 1e-5, torch.empty(rows, width, device="cuda"))
        assert rel_err(out, ref) < 2e-6
        out16 = ops.layernorm(x.cuda(), w.bfloat16().cuda(), 1e-5,
                              torch.empty(rows, width, device="cuda", dtype=torch.bfloat16))
        assert rel_err(out16.float(), pl.layer_norm(x.double(), w.bfloat16().double(), 1e-5)) < 1e-2
        pick = torch.tensor([rows - 1, 0], dtype=torch.int32)
        some = ops.layernorm(x.cuda(), w.cuda(), 1e-5, torch.empty(2, width, device="cuda"), pick.cuda())
        assert torch.equal(some, out[pick.long()])


def test_pair_embedding_and_the_token_it_remembers():
    g = torch.Generator().manual_seed(2)
    vocab, width, buckets, mp, mc = 50, 24, 13, 31, 5
    table, pair = torch.randn(vocab, width, generator=g), torch.randn(buckets + 1, width, generator=g)
    seqs = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in (9, 1, 30)]
    refs = [pl.embed(s, table, pair, buckets, mp, mc) for s in seqs]
    cache = Cache([None], [None], 256, torch.float32, "cuda", model_state={"prev_token": StateNeed((), torch.int32)})
    prev = cache.state[("model", "prev_token")]
    slots = [cache.open() for _ in seqs]
    got = [[] for _ in seqs]
    fed = [0, 0, 0]
    for lens in ([4, 1, 2], [1, 0, 1], [4, 0, 27]):
        live = [i for i, n in enumerate(lens) if n]
        entries = [StepEntry(slots[i], seqs[i][fed[i]:fed[i] + lens[i]], []) for i in live]
        for e in entries:
            cache.reserve(e.slot, cache.length(e.slot) + len(e.tokens))
        plan = StepPlan(cache, entries, "cuda")
        x = torch.empty(plan.n_rows, width, device="cuda")
        ops.embed_pair(plan, prev, table.cuda(), pair.cuda(), buckets, mp, mc, x)
        ops.keep_last_token(plan, prev)
        at = 0
        for i in live:
            got[i].append(x[at:at + lens[i]].cpu())
            at += lens[i]
            cache.advance(slots[i], cache.length(slots[i]) + lens[i])
            fed[i] += lens[i]
    for i in range(3):
        assert rel_err(torch.cat(got[i]), refs[i]) < 1e-7
    # a slot that is used again starts with the first token's row, whatever it remembered
    cache.close(slots[0])
    s = cache.open()
    assert s == slots[0]
    cache.reserve(s, 3)
    plan = StepPlan(cache, [StepEntry(s, seqs[2][:3], [])], "cuda")
    x = ops.embed_pair(plan, prev, table.cuda(), pair.cuda(), buckets, mp, mc, torch.empty(3, width, device="cuda"))
    assert rel_err(x, refs[2][:3]) < 1e-7


@pytest.mark.parametrize("taps", [1, 2, 4, 9])
def test_convolution_over_time_carries_its_last_inputs(taps):
    g = torch.Generator().manual_seed(3)
    C, pad = 37, 5
    w, b = torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
    seqs = [torch.randn(n, pad + C, generator=g) for n in (20, 3, 11)]
    for act, add, bias in (("silu", False, b), ("none", True, None)):
        def ref_of(x):
            y = pl.causal_conv(x[:, pad:].double(), w.double(), None if bias is None else bias.double())
            return pl.silu(y) if act == "silu" else y + x[:, pad:].double()
        refs = [ref_of(x) for x in seqs]
        need = {"c": StateNeed((taps - 1, C), torch.float32)} if taps > 1 else None
        cache = Cache([None], [need], 256, torch.float32, "cuda")
        state = cache.state[(0, "c")] if taps > 1 else None
        slots = [cache.open() for _ in seqs]
        # slots in another order than the rows; portions of one, two and many tokens
        order = [2, 0, 1]
        got = [[] for _ in seqs]
        fed = [0, 0, 0]
        for lens in ([2, 1, 1], [1, 1, 1], [1, 1, 2], [16, 0, 7]):
            live = [i for i in order if lens[i]]
            plan = plan_for(cache, [slots[i] for i in live], [lens[i] for i in live])
            x = torch.cat([seqs[i][fed[i]:fed[i] + lens[i]] for i in live]).cuda()
            out = torch.full((x.shape[0], C + 2), 7.0, device="cuda")
            ops.causal_conv(x, pad, C, w.cuda(), None if bias is None else bias.cuda(), plan, state, out, out_off=2,
                            act=act, add_input=add)
            assert bool((out[:, :2] == 7.0).all())
            at = 0
            for i in live:
                got[i].append(out[at:at + lens[i], 2:].cpu())
                at += lens[i]
                fed[i] += lens[i]
            done(cache, [slots[i] for i in live], [lens[i] for i in live])
        for i in range(3):
            assert rel_err(torch.cat(got[i]), refs[i]) < 2e-6, (taps, act, i)


def delta_reference(r, k, v, w, a, key_eps):
    """[T, H, K] each, float64: outputs of the delta rule from a zero state."""
    T, H, K = r.shape
    S = torch.zeros(H, K, K, dtype=F)
    o = torch.zeros(T, H, K, dtype=F)
    for t in range(T):
        for h in range(H):
            u = k[t, h] / torch.sqrt((k[t, h] ** 2).sum() + key_eps)
            S[h] = w[t, h][:, None] * S[h] - torch.outer(a[t, h] * u, u @ S[h]) + torch.outer(k[t, h], v[t, h])
            o[t, h] = S[h].T @ r[t, h]
    return o


@pytest.mark.parametrize("heads,dim,rank,extra", [(1, 16, 3, 3), (3, 24, 5, 3), (2, 40, 8, 0), (2, 64, 4, 3), (2, 64, 4, 0),
                                                  (1, 128, 16, 0), (1, 256, 8, 0), (2, 10, 2, 1), (3, 100, 4, 0)])
def test_delta_rule_kernels(heads, dim, rank, extra):
    """`extra` unused columns: rows of a multiple of four floats are copied in pieces of four."""
    g = torch.Generator().manual_seed(heads * 100 + dim)
    hk, scale, key_eps = heads * dim, 0.6, 1e-6
    lens = (90, 1, 12)                                   # the long one: more token groups than the kernel stages
    projs = [torch.randn(n, 5 * hk + rank + extra, generator=g) for n in lens]          # r k v g a z1 and unused columns
    w2, w0, ab = (torch.randn(hk, rank, generator=g), torch.randn(hk, generator=g), torch.randn(hk, generator=g))
    refs = []
    for p in projs:
        d = p.double()
        r, k, v = (d[:, i * hk:(i + 1) * hk].reshape(-1, heads, dim) for i in range(3))
        a = torch.sigmoid(d[:, 4 * hk:5 * hk] + ab.double()).reshape(-1, heads, dim)
        w = torch.exp(-scale * torch.sigmoid(torch.tanh(d[:, 5 * hk:5 * hk + rank]) @ w2.double().T + w0.double()))
        refs.append(delta_reference(r, k, v, w.reshape(-1, heads, dim), a, key_eps))
    cache = Cache([None], [StateNeed((heads, dim, dim), torch.float32)], 256, torch.float32, "cuda")
    slots = [cache.open() for _ in lens]
    got = [[] for _ in lens]
    fed = [0, 0, 0]
    for step in ([10, 1, 2], [1, 0, 1], [2, 0, 9], [77, 0, 0]):
        live = [i for i in (1, 2, 0) if step[i]]
        plan = plan_for(cache, [slots[i] for i in live], [step[i] for i in live])
        proj = torch.cat([projs[i][fed[i]:fed[i] + step[i]] for i in live]).cuda()
        aux = torch.empty(proj.shape[0], 3, hk, device="cuda")
        ops.delta_prep(proj, hk, 4 * hk, 5 * hk, heads, dim, w2.cuda(), w0.cuda(), ab.cuda(), scale, key_eps, aux)
        o = torch.empty(proj.shape[0], heads, dim, device="cuda")
        ops.delta_scan(proj, 0, hk, 2 * hk, aux, plan, heads, dim, cache.state[0], o)
        at = 0
        for i in live:
            got[i].append(o[at:at + step[i]].cpu())
            at += step[i]
            fed[i] += step[i]
        done(cache, [slots[i] for i in live], [step[i] for i in live])
    for i in range(3):
        assert rel_err(torch.cat(got[i]).reshape(lens[i], -1), refs[i].reshape(lens[i], -1)) < 2e-5, i


def sigmoid_attend(dtype, seqs, hq, hkv, dim, vdim, window, keep_first, scale, softcap, bias, cuts=None):
    """Projection rows of several sequences (float32 [n, q | k | v]) through `attn_prep` and the
    logistic attention kernel, each sequence in the given portions; returns [rows, hq * vdim] a sequence."""
    hd = max(dim, vdim)
    cache = Cache([KVNeed(hkv, hd, window, keep_first if window else 0)], [None], 2048, DT[dtype], "cuda")
    slots = [cache.open() for _ in seqs]
    cuts = cuts or [[x.shape[0]] for x in seqs]
    outs = [[] for _ in seqs]
    fed = [0] * len(seqs)
    for step in range(max(len(c) for c in cuts)):
        live = [i for i in range(len(seqs)) if step < len(cuts[i])]
        lens = [cuts[i][step] for i in live]
        plan = plan_for(cache, [slots[i] for i in live], lens)
        proj = torch.cat([seqs[i][fed[i]:fed[i] + n] for i, n in zip(live, lens)]).cuda()
        g, storage = plan.groups[0], cache.groups[0].entry_storage(0)
        q = torch.empty(proj.shape[0], hq, hd, dtype=DT[dtype], device="cuda")
        ops.attn_prep(proj, 0, hq * dim, (hq + hkv) * dim, hq, hkv, dim, vdim, hd, 0, False, None, None, None, None,
                      0.0, plan.row_seq, plan.row_pos, g.page_off, g.page_ids, g.page_size, storage, q)
        out = torch.empty(proj.shape[0], hq * hd, dtype=DT[dtype], device="cuda")
        ops.attention_sigmoid(q, out, plan, 0, storage, hq, hkv, hd, window, keep_first, scale, softcap,
                              None if bias is None else bias.cuda())
        out = out.view(-1, hq, hd)[:, :, :vdim].float().cpu()
        at = 0
        for i, n in zip(live, lens):
            outs[i].append(out[at:at + n].reshape(n, -1))
            at += n
            fed[i] += n
        done(cache, [slots[i] for i in live], lens)
    cache.check()
    return [torch.cat(o) for o in outs]


def sigmoid_attention_reference(x, hq, hkv, dim, vdim, window, keep_first, scale, softcap, bias):
    x = x.double()
    T = x.shape[0]
    q = x[:, :hq * dim].reshape(T, hq, dim)
    k = x[:, hq * dim:(hq + hkv) * dim].reshape(T, hkv, dim)
    v = x[:, (hq + hkv) * dim:].reshape(T, hkv, vdim)
    out = torch.zeros(T, hq, vdim, dtype=F)
    for i in range(T):
        for j in range(i + 1):
            if not (window == 0 or i - j < window or j < keep_first):
                continue
            for h in range(hq):
                s = float(q[i, h] @ k[j, h // (hq // hkv)]) * scale
                if softcap:
                    s = softcap * np.tanh(s / softcap)
                out[i, h] += v[j, h // (hq // hkv)] / (1.0 + np.exp(-(s + (float(bias[h]) if bias is not None else 0.0))))
    return out.reshape(T, hq * vdim)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,dim,vdim,window,keep_first,softcap", [
    (2, 1, 16, 16, 7, 3, 4.0),          # a window with kept first keys
    (4, 2, 8, 24, 70, 0, 0.0),          # values wider than keys; a window over a page border; no cap
    (3, 3, 40, 12, 5, 9, 50.0),         # more kept keys than the window is long
    (2, 2, 64, 64, 0, 0, 10.0),         # no window at all
    (1, 1, 128, 128, 1, 66, 0.0),       # a window of the query's own key; kept keys over a page border
    (4, 2, 64, 64, 70, 5, 6.0),         # several blocks of rows on tensor cores; a window over page borders
    (8, 2, 128, 128, 30, 70, 0.0),      # kept keys over a page border that the window has left behind
    (2, 1, 64, 40, 65, 64, 9.0),        # a page of kept keys, then the window's pages
])
def test_logistic_attention_kernel(dtype, hq, hkv, dim, vdim, window, keep_first, softcap):
    g = torch.Generator().manual_seed(hq * 10 + dim)
    wide = (hq + hkv) * dim + hkv * vdim
    seqs = [torch.randn(n, wide, generator=g) for n in (150, 1, 37)]
    bias = torch.randn(hq, generator=g)
    refs = [sigmoid_attention_reference(x, hq, hkv, dim, vdim, window, keep_first, dim ** -0.5, softcap, bias)
            for x in seqs]
    tol = 2e-5 if dtype == "float32" else 2e-2
    args = (hq, hkv, dim, vdim, window, keep_first, dim ** -0.5, softcap, bias)
    for cuts in (None, [[100] + [1] * 50, [1], [2, 3, 30, 2]], [[1] * 10 + [140], [1], [37]]):
        got = sigmoid_attend(dtype, seqs, *args, cuts=cuts)
        for o, r in zip(got, refs):
            assert rel_err(o, r) < tol, cuts
    if bias is not None:
        got = sigmoid_attend(dtype, seqs[2:], hq, hkv, dim, vdim, window, keep_first, dim ** -0.5, softcap, None)
        assert rel_err(got[0], sigmoid_attention_reference(seqs[2], *args[:-1], None)) < tol


def test_experts_are_chosen_and_weighted():
    g = torch.Generator().manual_seed(5)
    for rows, experts, top in ((1, 1, 1), (9, 5, 2), (300, 12, 4), (40, 7, 7), (5, 64, 3)):
        z = torch.randn(rows, experts, generator=g)
        z[0, :] = 0.25                                   # a tie across the row: the lower index wins
        if experts > 2:
            z[-1, experts - 1] = z[-1, 0] = 5.0
        ids = torch.empty(rows, top, dtype=torch.int32, device="cuda")
        wts = torch.empty(rows, top, device="cuda")
        ops.moe_route(z.cuda(), top, ids, wts)
        for r in range(rows):
            order = sorted(range(experts), key=lambda e: (-float(z[r, e]), e))[:top]
            assert ids[r].tolist() == order
            ref = torch.softmax(z[r, order].double(), 0)
            assert float((wts[r].cpu().double() - ref).abs().max()) < 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,width,ff,experts,top", [(1, 32, 16, 3, 1), (45, 44, 10, 5, 2), (300, 64, 72, 12, 3),
                                                       (70, 128, 200, 4, 4), (8, 256, 64, 40, 2), (600, 64, 40, 3, 2),
                                                       (130, 72, 24, 2, 1)])
def test_experts_feed_forward_kernels(dtype, rows, width, ff, experts, top):
    g = torch.Generator().manual_seed(rows + ff)
    h = torch.randn(rows, width, generator=g).to(DT[dtype])
    up = (torch.randn(experts, 2, ff, width, generator=g) * width ** -0.5).to(DT[dtype])
    down = (torch.randn(experts, width, ff, generator=g) * ff ** -0.5).to(DT[dtype])
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(rows)]).int()
    if experts - 2 >= top and rows > 1:
        ids[: rows // 2, 0] = 1                          # an expert that many rows choose, and experts nobody does
        ids[: rows // 2, 1:] = torch.stack([torch.randperm(experts - 2, generator=g)[:top - 1] + 2
                                            for _ in range(rows // 2)]).int()
    wts = torch.rand(rows, top, generator=g)
    x0 = torch.randn(rows, width, generator=g)
    limit = 0.8
    ref = x0.double().clone()
    for r in range(rows):
        for k in range(top):
            e = int(ids[r, k])
            ref[r] += float(wts[r, k]) * pl.clamped_glu(h[r:r + 1].double(), up[e, 0].double(), up[e, 1].double(),
                                                        down[e].double(), limit)[0]
    x = ops.moe_experts(h.cuda(), ids.cuda(), wts.cuda(), up.cuda(), down.cuda(), limit, pl.GLU_SLOPE, x0.cuda())
    assert rel_err(x, ref) < (2e-6 if dtype == "float32" else 1e-2)
    # a row's result does not depend on what else the step holds: the first rows alone, to the bit
    n = max(1, rows // 3)
    alone = ops.moe_experts(h[:n].cuda(), ids[:n].cuda(), wts[:n].cuda(), up.cuda(), down.cuda(), limit,
                            pl.GLU_SLOPE, x0[:n].cuda())
    assert torch.equal(alone, x[:n])


# ------------------------------------------------------------------ mechanisms alone: one-layer models
ONE_LAYER = {
    "ssm": model(64, 32, [layer("ssm", ssm(2, 8, 16))], taps=0, bigram=None),
    "ssm_groups_and_norm_parts": model(64, 48, [layer("ssm", ssm(6, 12, 8, groups=3, norm_groups=4, conv=4))], taps=0),
    "ssm_one_tap": model(64, 32, [layer("ssm", ssm(1, 64, 64, conv=1))], taps=0, bigram=None),
    "ssm_128": model(64, 32, [layer("ssm", ssm(2, 64, 128, groups=2, norm_groups=2, conv=2))], taps=2),
    "delta": model(64, 32, [layer("delta", delta(2, 16, rank=3))], taps=0, bigram=None),
    "delta_64": model(64, 40, [layer("delta", delta(1, 64, rank=8))], taps=3),
    "attention": model(64, 32, [layer("attention", attention(2, 1, 16, 16, window=11, keep_first=4, softcap=3.0))],
                       taps=0, bigram=None),
    "attention_wide_values": model(64, 32, [layer("attention", attention(3, 3, 8, 40, window=200))], taps=0),
    "attention_without_a_mask": model(64, 32, [layer("attention", attention(2, 1, 64, 64, window=0, softcap=4.0))], taps=2),
    "attention_shared_keys": model(64, 32, [layer("attention", attention(4, 2, 32, 16, window=30, keep_first=2)),
                                            layer("attention", attention(4, 2, 32, 16, window=8, keep_first=12,
                                                                         scale=0.4, softcap=8.0, kv_from=0))], taps=0),
    "experts": model(64, 32, [layer("delta", delta(1, 16), moe(6, 2, 24, 0.9, shared=(16, 1.3)))], taps=0, bigram=None),
    "experts_all_chosen_no_shared": model(64, 32, [layer("ssm", ssm(1, 16, 8), moe(3, 3, 40, 2.0))], taps=0),
    "one_expert": model(64, 32, [layer("ssm", ssm(1, 16, 8), moe(1, 1, 8, 0.5, shared=(8, 0.5)))], taps=0),
    "input_convolutions": model(64, 32, [layer("delta", delta(1, 16), moe(2, 1, 8, 1.0))], taps=5, bigram=None),
    "pair_embedding": model(64, 32, [layer("ssm", ssm(1, 16, 8))], taps=0, bigram=(7, 3, 1)),
    # widths and inner sizes that are no multiple of 8: the plain products in both dtypes
    "odd_sizes": model(61, 44, [layer("attention", attention(3, 1, 12, 6, window=30, keep_first=1), moe(3, 2, 10, 1.0)),
                                layer("ssm", ssm(3, 10, 7, conv=3), moe(2, 1, 9, 1.0, shared=(5, 1.0))),
                                layer("delta", delta(3, 20, rank=2))], taps=2),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(ONE_LAYER))
def test_each_mechanism_in_a_model_of_its_own(tmp_path, name, dtype):
    cfg, tensors = write_model(tmp_path / name, ONE_LAYER[name], seed=7)
    toks = tokens(cfg, 90, 3)
    ref = reference(cfg, tensors, toks)
    engine = sb.Engine(sb.load_model(tmp_path / name, dtype=dtype), max_tokens=256)
    assert model_err(run_cuts(engine, toks, [90]), ref, dtype) < TOL[dtype]
    assert model_err(run_cuts(engine, toks, [50] + [1] * 40), ref, dtype) < TOL[dtype]
    assert model_err(run_cuts(engine, toks, [1, 1, 2, 86]), ref, dtype) < TOL[dtype]


def test_the_stream_after_every_layer(folders, engines):
    """float32: the residual stream after every layer against the plain implementation's."""
    _, cfg, tensors = folders["A"]
    toks = tokens(cfg, 40, 8)
    streams = []
    pl.forward(cfg, tensors, toks, streams)
    engine = engines("A", "float32")
    seen = []
    blocks = engine.model.blocks
    originals = [b.forward for b in blocks]
    for b, orig in zip(blocks, originals):
        b.forward = lambda x, ctx, orig=orig: (lambda y: (seen.append(y.clone()), y)[1])(orig(x, ctx))
    try:
        run_cuts(engine, toks, [40])
    finally:
        for b in blocks:
            del b.forward
    assert len(seen) == len(streams) == len(cfg["layers"])
    for i, (got, ref) in enumerate(zip(seen, streams)):
        assert rel_err(got, ref) < 1e-5, i


def test_the_rank_of_the_decay_map_may_come_from_the_file(tmp_path):
    cfg, tensors = write_model(tmp_path / "m", ONE_LAYER["delta"], seed=3, drop_rank=True)
    assert "decay_rank" not in cfg["layers"][0]["mixer"]
    toks = tokens(cfg, 30, 1)
    engine = sb.Engine(sb.load_model(tmp_path / "m", dtype="float32"), max_tokens=128)
    assert rel_err(run_cuts(engine, toks, [30]), pl.forward(cfg, tensors, toks)) < TOL["float32"]


# ------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_decoding_and_portions(folders, engines, name, dtype):
    _, cfg, tensors = folders[name]
    toks = tokens(cfg, 171, 5)
    ref = reference(cfg, tensors, toks)
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
    reqs = [tokens(cfg, n, 10 + n) for n in (1, 70, 131, 23)]
    refs = [reference(cfg, tensors, r) for r in reqs]
    engine = engines(name, dtype, max_tokens=512)
    # twice in the same engine: the second pass reuses the slots, pages and state rows of the first
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


@pytest.mark.parametrize("dtype", DTYPES)
def test_window_edges_and_kept_first_keys_show(tmp_path, dtype):
    """Queries scaled up and head biases pushed down so that a few keys carry a row's sum: were a
    window one key too long or too short, or one kept first key more or fewer in sight, logits
    would move by 0.07 to 0.8 of their size: thousands of times the float32 tolerance in every layer,
    several times the bfloat16 tolerance in the first."""
    base = model(80, 48, [
        layer("attention", attention(2, 1, 16, 16, window=13, keep_first=5, scale=1.0)),
        layer("attention", attention(2, 2, 32, 32, window=70, keep_first=3, scale=1.0, softcap=25.0), moe(3, 1, 12, 1.0)),
        layer("attention", attention(2, 1, 16, 16, window=29, keep_first=66, scale=1.0, kv_from=0)),
    ], taps=2)

    def sharpen(t):
        for i in range(3):
            t[f"l{i}.mix.q"] *= 3.0
            t[f"l{i}.mix.pb"] = t[f"l{i}.mix.pb"] * 0.0 - 2.0
            t[f"l{i}.mix.o"] *= (1.0, 4.0, 8.0)[i]
    cfg, tensors = write_model(tmp_path / "w", base, seed=9, edit=sharpen)
    toks = tokens(cfg, 200, 21)
    ref = pl.forward(cfg, tensors, toks)
    tol = TOL[dtype] * (1.5 if dtype == "bfloat16" else 1.0)
    for which in range(3):
        for key in ("size", "keep_first"):
            for delta_ in (1, -1):
                other = json.loads(json.dumps(cfg))
                other["layers"][which]["mixer"]["mask"][key] += delta_
                moved = rel_err(pl.forward(other, tensors, toks)[100:], ref[100:])
                assert moved > 1500 * TOL["float32"], (which, key, delta_)
    engine = sb.Engine(sb.load_model(tmp_path / "w", dtype=dtype), max_tokens=512)
    for cuts in ([200], [60] + [1] * 140, [12, 2, 50, 136], [13] + [1] * 187, [4, 1, 1, 60, 3, 131]):
        assert rel_err(run_cuts(engine, toks, cuts), ref) < tol, cuts


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_token_stays_in_the_states(tmp_path, dtype):
    """Decays close to one: four hundred tokens later the logits still depend on the fourth token
    through the state-space layer's and the delta rule's states, by a large multiple of the
    float32 tolerance, which is where a lost or reset state would show."""
    base = model(70, 32, [layer("ssm", ssm(2, 16, 16, conv=2)), layer("delta", delta(1, 16, rank=4))], taps=2)

    def slow(t):
        t["l0.mix.A_log"] -= 7.0
        t["l0.mix.o"] *= 3.0
        t["l1.mix.w0"] -= 9.0
        t["l1.mix.a.b"] -= 6.0
    cfg, tensors = write_model(tmp_path / "far", base, seed=11, edit=slow)
    toks = tokens(cfg, 420, 2)
    other = list(toks)
    other[3] = (toks[3] + 1) % cfg["vocab"]
    ref = pl.forward(cfg, tensors, toks)
    assert rel_err(pl.forward(cfg, tensors, other)[400:], ref[400:]) > 300 * TOL["float32"]
    engine = sb.Engine(sb.load_model(tmp_path / "far", dtype=dtype), max_tokens=512)
    for cuts in ([420], [380] + [1] * 40, [5, 200, 215]):
        assert rel_err(run_cuts(engine, toks, cuts)[400:], ref[400:]) < TOL[dtype], cuts


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_keeps_state_and_kept_pages(folders, engines, dtype):
    """Six hundred tokens one by one: the windows pass over many pages (which are given back, but
    for those of the kept first keys), the recurrences' states are carried all the way."""
    _, cfg, tensors = folders["B"]
    toks = tokens(cfg, 600, 77)
    ref = pl.forward(cfg, tensors, toks)
    engine = engines("B", dtype, max_tokens=384)        # far fewer pages than 600 tokens would hold
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
    """`llm.generate_batch`: the scheduler's batches, the captured decode step with the
    recurrences' states, the convolutions' inputs and the remembered token in it, and slots
    given to the next batch."""
    d, cfg, tensors = folders[name]
    m = llm.model_load(d, dtype=dtype)
    assert m.arch == "Leguvik" and m.vocab_size == cfg["vocab"]
    prompts = [tokens(cfg, n, 30 + n) for n in (3, 66, 20, 1)]
    n_new = 12
    outs = llm.generate_batch(m, prompts, max_tokens=n_new)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for i, t in enumerate(o):
            logits = pl.forward(cfg, tensors, seq)[-1]
            best = int(torch.argmax(logits))
            if t != best:
                top2 = torch.topk(logits, 2).values
                margin = float(top2[0] - top2[1]) / float(logits.abs().max())
                assert dtype == "bfloat16" and margin < 2 * TOL[dtype], (i, o, margin)
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
    a, b = tokens(cfg, 75, 1), tokens(cfg, 30, 2)
    ra, rb = pl.forward(cfg, tensors, a).numpy(), pl.forward(cfg, tensors, b).numpy()
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
    """`python -m sonicboom_b200 generate` on a Leguvik folder: greedy tokens as the plain
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
    assert got == [pl.greedy_generate(cfg, tensors, p, 6) for p in prompts]
