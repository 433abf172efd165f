"""A plain, slow Bulodra in float64 on the CPU: one function per mechanism, written from the
design's equations and sharing nothing with the package.  A model is the config.json dictionary
plus a dict of tensors by name.  Sequences are independent, so there is no batch anywhere; every
attention walks its keys in the most literal way.
"""
from __future__ import annotations

import math

import torch

F = torch.float64
GLU_SLOPE = 1.702          # of the experts' gate
YARN_MAGNITUDE = 0.1       # cos and sin grow by 0.1 ln(factor) + 1
RAMP_FLOOR = 0.001


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    return [buckets if t == 0 else (int(tokens[t - 1]) * mul_prev + int(tok) * mul_cur) % buckets
            for t, tok in enumerate(tokens)]


def embed(tokens, table, pair_table, b):
    idx = torch.tensor(list(tokens), dtype=torch.long)
    rows = torch.tensor(bigram_rows(tokens, b["buckets"], b["mul_prev"], b["mul_cur"]))
    return table[idx].to(F) + pair_table[rows].to(F)


def frequencies(rot):
    """(per-pair frequencies, magnitude of cos and sin) of a rotation record {base, dims, scaling?}."""
    n, base = rot["dims"], float(rot["base"])
    f = [base ** (-2.0 * i / n) for i in range(n // 2)]
    sc = rot.get("scaling")
    if sc is None:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def dim_of(turns):
        return n * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(sc["slow"]))), n - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, RAMP_FLOOR), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, YARN_MAGNITUDE * math.log(factor) + 1.0


def rotate(x, positions, rot):
    """x [T, heads, d]: the first rot.dims values of every head turn, pair (i, i + dims/2)."""
    n = rot["dims"]
    if n == 0:
        return x.clone()
    f, mag = frequencies(rot)
    half = n // 2
    a = torch.tensor(list(positions), dtype=F).view(-1, 1, 1) * torch.tensor(f, dtype=F).view(1, 1, half)
    c, s = torch.cos(a) * mag, torch.sin(a) * mag
    u, v = x[:, :, :half], x[:, :, half:n]
    return torch.cat([u * c - v * s, v * c + u * s, x[:, :, n:]], dim=-1)


def softmax_rows(scores, visible, sink=None):
    """scores [T, T] of one head, visible [T, T] bool; an optional sink joins every row's
    denominator as exp(sink).  Returns the weights (rows need not sum to one with a sink)."""
    s = scores.masked_fill(~visible, -math.inf)
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.clamp(m, min=float(sink))
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(float(sink) - m)
    return e / den


def causal(T, window=0):
    i = torch.arange(T).view(T, 1)
    j = torch.arange(T).view(1, T)
    vis = j <= i
    return vis & (i - j < window) if window else vis


def attention(h, get, m, eps):
    """Grouped-query attention with biases, per-head norms of q and k before the rotation, a sink."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ get("q").T + get("q.b")).view(T, H, d)
    k = (h @ get("k").T + get("k.b")).view(T, G, d)
    v = (h @ get("v").T + get("v.b")).view(T, G, dv)
    q = rms(q, eps) * get("q.norm")
    k = rms(k, eps) * get("k.norm")
    pos = list(range(T))
    q, k = rotate(q, pos, m["rot"]), rotate(k, pos, m["rot"])
    vis = causal(T)
    out = torch.zeros(T, H, dv, dtype=F)
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * m["scale"]
        out[:, hh] = softmax_rows(s, vis, get("sink")[hh]) @ v[:, g]
    return out.reshape(T, H * dv) @ get("o").T


def latent_attention(h, get, m, eps):
    """Queries through a normed latent; keys and values from a normed latent c plus one rotated
    key part that all heads share; a sink."""
    T = h.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms(h @ get("dq").T, eps) * get("dq.norm")
    q = (cq @ get("uq").T).view(T, H, d + r)
    kv = h @ get("dkv").T
    c = rms(kv[:, :rank], eps) * get("dkv.norm")
    pos = list(range(T))
    kr = rotate(kv[:, rank:].reshape(T, 1, r), pos, m["rot"])[:, 0]
    qr = rotate(q[:, :, d:].clone(), pos, m["rot"])
    kn = (c @ get("uk").T).view(T, H, d)
    val = (c @ get("uv").T).view(T, H, dv)
    vis = causal(T)
    out = torch.zeros(T, H, dv, dtype=F)
    for hh in range(H):
        s = (q[:, hh, :d] @ kn[:, hh].T + qr[:, hh] @ kr.T) * m["scale"]
        out[:, hh] = softmax_rows(s, vis, get("sink")[hh]) @ val[:, hh]
    return out.reshape(T, H * dv) @ get("o").T


def attention_2(h, get, m, eps):
    """Grouped-query attention without biases: rotation, then unit root mean square per head,
    capped scores, a sliding window, a gate per head on the result."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ get("q").T).view(T, H, d)
    k = (h @ get("k").T).view(T, G, d)
    v = (h @ get("v").T).view(T, G, dv)
    pos = list(range(T))
    q, k = rms(rotate(q, pos, m["rot"]), eps), rms(rotate(k, pos, m["rot"]), eps)
    cap = m.get("softcap") or 0.0
    vis = causal(T, m["mask"]["size"] if m.get("mask") else 0)
    gate = torch.sigmoid(h @ get("g").T)
    out = torch.zeros(T, H, dv, dtype=F)
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * m["scale"]
        if cap:
            s = cap * torch.tanh(s / cap)
        out[:, hh] = (softmax_rows(s, vis) @ v[:, g]) * gate[:, hh:hh + 1]
    return out.reshape(T, H * dv) @ get("o").T


MIXERS = {"attention": attention, "latent_attention": latent_attention, "attention_2": attention_2}


def dense_ff(h, get):
    return (gelu_tanh(h @ get("gate").T) * (h @ get("up").T)) @ get("down").T


def expert(h, get, limit):
    g = torch.clamp(h @ get("gate").T, max=limit)
    u = torch.clamp(h @ get("up").T, -limit, limit)
    return (g * torch.sigmoid(GLU_SLOPE * g) * (u + 1.0)) @ get("down").T


def route(z, correction, r):
    """z [experts] router logits of one token -> (chosen experts, their weights, margin).  The margin
    is how far the choice is from falling another way: the last chosen expert's choice score above
    the best one left out, and the last kept group's score above the best group left out."""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(z)
    choice = s + correction
    groups = r.get("groups")
    allowed = list(range(E))
    gap = math.inf
    if groups is not None:
        n, per = groups["count"], E // groups["count"]
        score = []
        for gi in range(n):
            part = sorted((float(x) for x in choice[gi * per:(gi + 1) * per]), reverse=True)
            score.append(sum(part[:2]))
        ranked = sorted(range(n), key=lambda gi: (-score[gi], gi))
        best = ranked[:groups["keep"]]
        if len(ranked) > groups["keep"]:
            gap = score[ranked[groups["keep"] - 1]] - score[ranked[groups["keep"]]]
        allowed = [e for e in range(E) if e // per in best]
    order = sorted(allowed, key=lambda e: (-float(choice[e]), e))
    chosen = order[:top]
    if len(order) > top:
        gap = min(gap, float(choice[order[top - 1]] - choice[order[top]]))
    return chosen, [float(s[e]) * r["scale"] for e in chosen], gap


def moe_ff(h, get, mlp, gaps=None):
    T = h.shape[0]
    r = mlp["router"]
    z = h @ get("router").T
    out = torch.zeros(T, h.shape[1], dtype=F)
    sent = {}                                   # expert -> [(token, weight)]
    for t in range(T):
        chosen, weights, gap = route(z[t], get("correction"), r)
        if gaps is not None:
            gaps.append(gap)
        for e, w in zip(chosen, weights):
            sent.setdefault(e, []).append((t, w))
    for e, pairs in sent.items():
        rows = torch.tensor([t for t, _ in pairs])
        y = expert(h[rows], lambda n, e=e: get(f"e{e}.{n}"), mlp["expert"]["limit"])
        out[rows] += torch.tensor([w for _, w in pairs], dtype=F).view(-1, 1) * y
    if mlp.get("shared") is not None:
        out = out + expert(h, lambda n: get("shared." + n), mlp["shared"]["limit"])
    return out


def forward(cfg, tensors, tokens, layers_out=None, gaps=None):
    """Logits [T, vocab] of one sequence; `layers_out` (a list) receives the stream after every
    layer, `gaps` (a list) one list per mixture layer of every token's routing margin."""
    W = {n: t.to(F) for n, t in tensors.items()}
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    x = embed(tokens, W["embed"], W["bigram"], cfg["embedding"]["bigram"])
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        y = MIXERS[L["type"]](x, lambda n: W[p + "mix." + n], L["mixer"], eps)
        x = x + mult * (rms(y, eps) * W[p + "norm1"])
        mlp = L.get("mlp")
        if mlp is not None:
            get = lambda n: W[p + "mlp." + n]
            if mlp["kind"] == "dense":
                y = dense_ff(x, get)
            else:
                g = [] if gaps is not None else None
                y = moe_ff(x, get, mlp, g)
                if gaps is not None:
                    gaps.append(g)
            x = x + mult * (rms(y, eps) * W[p + "norm2"])
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms(x, eps) * W["final.norm"]) @ W["head"].T * cfg["logit_scale"]


def greedy_generate(cfg, tensors, prompt, n_new):
    seq, out = list(prompt), []
    for _ in range(n_new):
        out.append(int(torch.argmax(forward(cfg, tensors, seq)[-1])))
        seq.append(out[-1])
    return out
