"""A plain, slow Leguvik in float64 on the CPU: one function per mechanism, written from the
design's equations and sharing nothing with the package.  A model is a dict of tensors by name
plus the config.json dictionary.  Every function walks a sequence token by token (or key by key)
in the most literal way; sequences are independent, so there is no batch anywhere.
"""
from __future__ import annotations

import math

import torch

F = torch.float64
GLU_SLOPE = 1.702
UNIT_KEY_EPS = 1e-6


def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def causal_conv(h, w, bias=None):
    """h [T, C], w [C, taps]: y_t = sum_j w[:, j] h_(t - taps + 1 + j), zeros before the start."""
    T, C = h.shape
    taps = w.shape[1]
    y = torch.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * h[s]
        if bias is not None:
            y[t] += bias
    return y


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.log1p(torch.exp(-x.abs())) + torch.clamp(x, min=0)


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(buckets if t == 0 else (int(tokens[t - 1]) * mul_prev + int(tok) * mul_cur) % buckets)
    return rows


def embed(tokens, table, bigram, buckets, mul_prev, mul_cur):
    idx = torch.tensor(list(tokens), dtype=torch.long)
    return table[idx].to(F) + bigram[torch.tensor(bigram_rows(tokens, buckets, mul_prev, mul_cur))].to(F)


def mamba2(h, get, m, eps):
    """m: heads, vdim, state, groups, norm_groups (the conv's taps are the stored tensor's)."""
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    T = h.shape[0]
    proj = h @ get("in").T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, get("conv"), get("conv.b")))
    x, B, C = xbc[:, :inner], xbc[:, inner:inner + G * N], xbc[:, inner + G * N:]
    dt = softplus(dt + get("dt_bias"))
    A = torch.exp(get("A_log"))
    D = get("D")
    y = torch.zeros(T, inner, dtype=F)
    S = torch.zeros(H, N, P, dtype=F)
    for t in range(T):
        for hh in range(H):
            g = hh // (H // G)
            xt = x[t, hh * P:(hh + 1) * P]
            Bt, Ct = B[t, g * N:(g + 1) * N], C[t, g * N:(g + 1) * N]
            S[hh] = torch.exp(-A[hh] * dt[t, hh]) * S[hh] + dt[t, hh] * torch.outer(Bt, xt)
            y[t, hh * P:(hh + 1) * P] = S[hh].T @ Ct + D[hh] * xt
    y = y * silu(z)
    ng = m["norm_groups"]
    y = rms(y.view(T, ng, inner // ng), eps).reshape(T, inner) * get("norm")
    return y @ get("o").T


def general_delta(h, get, m, eps):
    H, K = m["heads"], m["dim"]
    T = h.shape[0]
    r, k, v = h @ get("r").T, h @ get("k").T, h @ get("v").T
    w = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ get("w1").T) @ get("w2").T + get("w0")))
    a = torch.sigmoid(h @ get("a").T + get("a.b"))
    o = torch.zeros(T, H, K, dtype=F)
    S = torch.zeros(H, K, K, dtype=F)           # [key channel, value channel]
    for t in range(T):
        for hh in range(H):
            sl = slice(hh * K, (hh + 1) * K)
            kt, vt, rt, wt, at = k[t, sl], v[t, sl], r[t, sl], w[t, sl], a[t, sl]
            u = kt / torch.sqrt((kt * kt).sum() + UNIT_KEY_EPS)
            old = S[hh]
            S[hh] = wt[:, None] * old - torch.outer(at * u, u @ old) + torch.outer(kt, vt)
            o[t, hh] = S[hh].T @ rt
    o = rms(o, eps).reshape(T, H * K) * get("norm") * torch.sigmoid(h @ get("g").T)
    return o @ get("o").T


def visible(i, j, size, keep_first):
    """Whether the query at position i sees the key at position j."""
    return j <= i and (i - j < size or j < keep_first)


def sigmoid_attention(h, get, m, keys=None, values=None):
    """Returns (output, keys, values); `keys` / `values` given: another layer's are used."""
    H, G, K, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ get("q").T).view(T, H, K)
    if keys is None:
        keys, values = (h @ get("k").T).view(T, G, K), (h @ get("v").T).view(T, G, V)
    cap, pb = m.get("softcap", 0.0), get("pb")
    out = torch.zeros(T, H, V, dtype=F)
    for i in range(T):
        mask = m.get("mask") or {"size": T}                     # no mask: every earlier key
        seen = [j for j in range(T) if visible(i, j, mask["size"], mask.get("keep_first", 0))]
        for hh in range(H):
            g = hh // (H // G)
            s = (keys[seen, g] @ q[i, hh]) * m["scale"]
            if cap:
                s = cap * torch.tanh(s / cap)
            out[i, hh] = torch.sigmoid(s + pb[hh]) @ values[seen, g]
    return out.reshape(T, H * V) @ get("o").T, keys, values


def clamped_glu(h, gate, up, down, limit):
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, -limit, limit)
    return (g * torch.sigmoid(GLU_SLOPE * g) * (u + 1)) @ down.T


def moe(h, get, m, gaps=None):
    """`gaps` (a list) receives, per token, the gap between the last chosen logit and the largest one
    that was not chosen (infinite when every expert is chosen)."""
    E, top = m["router"]["experts"], m["router"]["top"]
    T = h.shape[0]
    z = h @ get("router").T + get("router.b")
    if gaps is not None:
        ranked = z.sort(dim=1, descending=True).values
        gaps.append(ranked[:, top - 1] - ranked[:, top] if top < E else torch.full((T,), float("inf"), dtype=F))
    out = torch.zeros(T, get("e0.down").shape[0], dtype=F)
    for t in range(T):
        order = sorted(range(E), key=lambda e: (-float(z[t, e]), e))[:top]
        wts = torch.softmax(torch.stack([z[t, e] for e in order]), 0)
        for wt, e in zip(wts, order):
            out[t] += wt * clamped_glu(h[t:t + 1], get(f"e{e}.gate"), get(f"e{e}.up"), get(f"e{e}.down"),
                                       m["expert"]["limit"])[0]
    if m.get("shared"):
        out += clamped_glu(h, get("shared.gate"), get("shared.up"), get("shared.down"), m["shared"]["limit"])
    return out


def forward(cfg, tensors, tokens, streams=None, gaps=None):
    """float64 logits [T, vocab] of one sequence; `streams` (a list) receives the residual stream
    after every layer, `gaps` (a list) every experts layer's router gaps per token (see `moe`)."""
    def getter(prefix):
        return lambda name: tensors[prefix + name].to(F)
    eps = cfg["norm"]["eps"]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        x = embed(tokens, tensors["embed"], tensors["bigram"], bg["buckets"], bg["mul_prev"], bg["mul_cur"])
    else:
        x = tensors["embed"][torch.tensor(list(tokens), dtype=torch.long)].to(F)
    canon = "canon" in cfg
    kept = {}
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = L["mixer"]
        h = layer_norm(x, tensors[p + "norm1"].to(F), eps)
        if canon:
            h = h + causal_conv(h, tensors[p + "canon1"].to(F))
        get = getter(p + "mix.")
        if L["type"] == "mamba2":
            x = x + mamba2(h, get, m, eps)
        elif L["type"] == "general_delta":
            x = x + general_delta(h, get, m, eps)
        elif L["type"] == "attention":
            src = m.get("kv_from")
            y, k, v = sigmoid_attention(h, get, m, *(kept[src] if src is not None else (None, None)))
            kept[i] = (k, v)
            x = x + y
        else:
            raise ValueError(L["type"])
        if L.get("mlp") is not None:
            h = layer_norm(x, tensors[p + "norm2"].to(F), eps)
            if canon:
                h = h + causal_conv(h, tensors[p + "canon2"].to(F))
            x = x + moe(h, getter(p + "mlp."), L["mlp"], gaps)
        if streams is not None:
            streams.append(x.clone())
    hn = layer_norm(x, tensors["final.norm"].to(F), eps)
    logits = hn @ tensors["head"].to(F).T
    cap = cfg.get("logit_softcap", 0.0)
    return cap * torch.tanh(logits / cap) if cap else logits


def greedy_generate(cfg, tensors, prompt, n_new):
    seq = list(prompt)
    for _ in range(n_new):
        seq.append(int(torch.argmax(forward(cfg, tensors, seq)[-1])))
    return seq[len(prompt):]
