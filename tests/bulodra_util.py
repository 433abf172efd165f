"""Small Bulodra configurations for the tests, and model folders made from them.

The configurations differ from each other in every size and option: layer order, value heads
narrower and wider than the keys, one to three key/value heads, rotated prefixes shorter than the
head and as long as it, stretched and plain rotations, latents narrower and wider than the heads,
cache rows of a size the tensor-memory kernels take (64) and of sizes they do not, windows of one
key, of a few and over a page border, layers without a feed-forward, dense feed-forwards whose size
is and is not a multiple of 8, experts in one, two, three and four groups of which one to three are
kept, with and without a shared expert, a width that is no multiple of 8, a stream multiplier and a
logit scale of one and of other values."""
import json
from pathlib import Path

import torch


def rot(base, dims, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def attention(heads, kv_heads, dim, vdim, rotation, scale=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rotation,
            "scale": scale if scale is not None else dim ** -0.5}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, rotation, scale=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
            "rot": rotation, "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}


def attention_2(heads, kv_heads, dim, vdim, rotation, window, softcap, scale=None):
    m = attention(heads, kv_heads, dim, vdim, rotation, scale)
    m["softcap"] = softcap
    if window:
        m["mask"] = {"size": window}
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit=1.5, groups=None, scale=1.0, shared=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "router": router, "expert": {"ff": ff, "limit": limit}}
    if shared is not None:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def model(vocab, width, layers, bigram=(97, 29, 7), mult=0.7, logit_scale=1.5, eps=1e-5):
    return {"architecture": "Bulodra", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "residual_mult": mult, "logit_scale": logit_scale,
            "embedding": {"bigram": dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))}, "layers": layers}


CONFIGS = {
    # values wider than keys (padded cache rows), a window of 9, six experts in three groups of which
    # two are kept; a query latent wider than a head; a stretched rotation over a head's whole
    # size; a window of one key and no feed-forward; fewer rotated dimensions than rot_dim and a
    # dense feed-forward whose size is no multiple of 8
    "A": model(211, 64, [
        layer("attention_2", attention_2(4, 2, 16, 24, rot(10000.0, 8), window=9, softcap=5.0, scale=0.3),
              moe(6, 2, 24, 1.5, groups=(3, 2), scale=1.7, shared=(40, 1.0))),
        layer("latent_attention", latent(3, 16, 8, 12, 24, 20, rot(5000.0, 8, (4.0, 32, 8.0, 1.0))), dense(40)),
        layer("attention", attention(4, 2, 16, 16, rot(20000.0, 16, (3.0, 48, 6.0, 0.5)), scale=0.2),
              moe(5, 1, 20, 0.8)),
        layer("attention_2", attention_2(2, 2, 32, 16, rot(1000.0, 32), window=1, softcap=2.0)),
        layer("latent_attention", latent(2, 8, 8, 16, 16, 8, rot(300.0, 4)), dense(20)),
    ]),
    # head size 64 (the tensor-memory kernels) with three key/value heads and half the head rotated
    # by a stretched rotation; a window over a page border; a latent whose cache row is 64 wide;
    # eight experts in four groups of which three are kept, three chosen; a width that is no multiple
    # of 8; a stream multiplier and a logit scale of one
    "B": model(150, 44, [
        layer("attention", attention(6, 3, 64, 32, rot(100000.0, 32, (8.0, 64, 4.0, 0.5)), scale=0.1),
              moe(8, 3, 10, 1.0, groups=(4, 3), scale=0.8, shared=(18, 2.0))),
        layer("attention_2", attention_2(2, 1, 64, 64, rot(200000.0, 24), window=70, softcap=20.0, scale=0.11),
              moe(4, 2, 9, 1.2, groups=(2, 1), scale=2.2)),
        layer("latent_attention", latent(2, 24, 16, 20, 48, 12, rot(10000.0, 16, (2.0, 128, 16.0, 2.0))), dense(16)),
        layer("attention_2", attention_2(3, 3, 8, 8, rot(50.0, 2), window=3, softcap=1.5, scale=0.5), moe(3, 2, 16, 0.7)),
    ], bigram=(53, 11, 3), mult=1.0, logit_scale=1.0, eps=1e-6),
}
INIT = dict(std=0.08, bias_std=0.3, norm_std=0.2)


def write_model(path, cfg, seed, edit=None):
    """A model folder with seeded random weights; `edit(tensors)` may change them (float32 in,
    stored as bfloat16).  Returns (config as written, float32 tensors as stored)."""
    import plain_model as pm
    from sonicboom_b200 import write_random_model
    from sonicboom_b200.weights.safetensors_io import write_safetensors
    path = Path(path)
    write_random_model(path, cfg, seed=seed, **INIT)
    _, tensors = pm.read_model_dir(path)
    for name in tensors:
        if name.endswith(".router"):
            tensors[name] = tensors[name] * 3.0           # routers that prefer some experts clearly
        if name.endswith(".sink"):
            tensors[name] = tensors[name] + 1.0           # sinks that take a fair share of a row
    if edit is not None:
        edit(tensors)
    stored = {n: t.to(torch.bfloat16) for n, t in tensors.items()}
    write_safetensors(path / "model.safetensors",
                      [(n, t.dtype, tuple(t.shape), (lambda t=t: t)) for n, t in stored.items()])
    (path / "config.json").write_text(json.dumps(cfg))
    return cfg, {n: t.float() for n, t in stored.items()}


def tokens(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


ROUTER_MARGIN = 0.02
_CALM = {}


def calm_tokens(cfg, tensors, n, seed, key=None, margin=ROUTER_MARGIN):
    """`n` seeded random tokens at none of which a router's choice is a close call (the last chosen
    expert's choice score is at least `margin` above the best one left out, and the last kept group's
    score at least `margin` above the best group left out), so that rounding cannot
    send a token to other experts than the plain implementation does.  A position's routing depends on
    the tokens up to it only: the first close call's token is drawn again until none is left.  Returns
    (tokens, the plain implementation's logits)."""
    import plain_bulodra as pb
    k = (key, n, seed, margin)
    if key is not None and k in _CALM:
        return _CALM[k]
    g = torch.Generator().manual_seed(seed)
    toks = torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()
    for _ in range(20 * n):
        gaps = []
        ref = pb.forward(cfg, tensors, toks, gaps=gaps)
        close = [t for t in range(n) if any(layer_gaps[t] < margin for layer_gaps in gaps)]
        if not close:
            break
        toks[close[0]] = int(torch.randint(0, cfg["vocab"], (1,), generator=g))
    else:
        raise AssertionError("no tokens without a close router call were found")
    if key is not None:
        _CALM[k] = (toks, ref)
    return toks, ref
