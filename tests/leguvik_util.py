"""Small Leguvik configurations for the tests, and model folders made from them.

The configurations differ from each other in every size and option: layer order, state-space
layers with one and with several groups and norm parts, convolutions of 2, 3 and 4 taps, delta-rule
heads of 16, 24 and 40 channels, attention with value heads narrower and wider than the keys, windows
shorter and longer than the kept first tokens (and no kept tokens at all), a layer that reads another
layer's keys under a mask of its own, experts of which 1, 2 or all are chosen, with and without a
shared expert, layers without a feed-forward, widths that are no multiple of 8."""
import json
from pathlib import Path

import torch


def attention(heads, kv_heads, dim, vdim, window, keep_first=0, scale=None, softcap=0.0, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": scale if scale is not None else dim ** -0.5, "softcap": softcap}
    if window:                                               # window 0: config.json has no mask
        m["mask"] = {"size": window, "keep_first": keep_first}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def ssm(heads, vdim, state, groups=1, norm_groups=1, conv=3):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}


def delta(heads, dim, rank=4):
    return {"heads": heads, "dim": dim, "decay_rank": rank}


def moe(experts, top, ff, limit=1.5, shared=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared is not None:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


KINDS = {"attention": "attention", "ssm": "mamba2", "delta": "general_delta"}


def layer(kind, mixer, mlp=None):
    return {"type": KINDS[kind], "mixer": mixer, "mlp": mlp}


def model(vocab, width, layers, taps=3, bigram=(97, 31, 5), cap=12.0, eps=1e-5):
    d = {"architecture": "Leguvik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if taps:
        d["canon"] = {"taps": taps}
    if bigram:
        d["embedding"] = {"bigram": dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))}
    if cap:
        d["logit_softcap"] = cap
    return d


CONFIGS = {
    # values wider than keys; a reader of layer 0's keys with a longer window and no kept tokens;
    # two groups and two norm parts; a layer without a feed-forward; all experts chosen
    "A": model(211, 64, [
        layer("attention", attention(4, 2, 16, 24, window=9, keep_first=3, scale=0.3, softcap=5.0),
              moe(5, 2, 24, 1.5, shared=(40, 1.0))),
        layer("ssm", ssm(4, 12, 16, groups=2, norm_groups=2, conv=4), moe(3, 1, 20, 0.8)),
        layer("delta", delta(2, 16, rank=4)),
        layer("attention", attention(4, 2, 16, 24, window=20, keep_first=0, scale=0.2, kv_from=0),
              moe(4, 4, 16, 2.0, shared=(8, 3.0))),
        layer("ssm", ssm(3, 8, 24, groups=1, norm_groups=3, conv=2), moe(6, 3, 12, 1.0)),
    ], taps=3),
    # more kept tokens than the window is long, and a window over a page border; head size 64;
    # delta heads of 40 channels; a width that is no multiple of 8; two taps; no logit cap
    "B": model(150, 44, [
        layer("delta", delta(3, 40, rank=6), moe(2, 1, 10, 1.0, shared=(18, 2.0))),
        layer("attention", attention(2, 1, 64, 32, window=70, keep_first=75, scale=0.1, softcap=30.0), moe(7, 2, 9, 1.2)),
        layer("ssm", ssm(2, 20, 8, groups=2, norm_groups=1, conv=3)),
        layer("attention", attention(3, 3, 8, 8, window=1, keep_first=1, scale=0.5), moe(3, 2, 16, 0.7)),
    ], taps=2, bigram=(53, 11, 3), cap=0.0, eps=1e-6),
}
INIT = dict(std=0.08, bias_std=0.3, norm_std=0.2)


def write_model(path, cfg, seed, edit=None, drop_rank=False):
    """A model folder with seeded random weights; `edit(tensors)` may change them (float32 in,
    stored as bfloat16).  With `drop_rank` config.json does not state the rank of a decay's
    low-rank map.  Returns (config as written, float32 tensors as stored)."""
    import plain_model as pm
    from sonicboom_b200 import write_random_model
    from sonicboom_b200.weights.safetensors_io import write_safetensors
    path = Path(path)
    write_random_model(path, cfg, seed=seed, **INIT)
    _, tensors = pm.read_model_dir(path)
    for name in tensors:
        if name.endswith(".A_log") or name.endswith(".dt_bias"):
            tensors[name] = tensors[name] - 1.0           # decays that stay well below one token's step
        if name.endswith(".router"):
            tensors[name] = tensors[name] * 4.0           # routers that prefer some experts clearly
    if edit is not None:
        edit(tensors)
    stored = {n: t.to(torch.bfloat16) for n, t in tensors.items()}
    write_safetensors(path / "model.safetensors",
                      [(n, t.dtype, tuple(t.shape), (lambda t=t: t)) for n, t in stored.items()])
    if drop_rank:
        cfg = json.loads(json.dumps(cfg))
        for L in cfg["layers"]:
            L["mixer"].pop("decay_rank", None)
    (path / "config.json").write_text(json.dumps(cfg))
    return cfg, {n: t.float() for n, t in stored.items()}


def tokens(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()
