"""Bulodra without a device: configuration keys and their errors, the parts a configuration
becomes, the tensor list, the stretched rotation's frequencies, and properties of the plain
implementation's own mechanisms."""
import copy
import json
import math

import pytest
import torch

import plain_bulodra as pb
from bulodra_util import CONFIGS, attention, attention_2, calm_tokens, dense, latent, layer, model, moe, rot, write_model
from sonicboom_b200.config import BulodraConfig, ConfigError, spec_from_config_dict
from sonicboom_b200.models import tensor_requests
from sonicboom_b200.parts.rotary import yarn_frequencies


@pytest.mark.parametrize("name", list(CONFIGS))
def test_round_trip_and_parts(name):
    cfg = CONFIGS[name]
    c, spec = spec_from_config_dict(cfg)
    assert isinstance(c, BulodraConfig) and BulodraConfig.from_dict(c.to_dict()) == c
    assert BulodraConfig.from_dict(json.loads(json.dumps(c.to_dict()))) == c
    assert spec.architecture == "Bulodra" and len(spec.layers) == len(cfg["layers"])
    assert spec.logit_scale == cfg["logit_scale"] and spec.pair_embedding.buckets == cfg["embedding"]["bigram"]["buckets"]
    for L, raw in zip(spec.layers, cfg["layers"]):
        assert L.arrangement == "output_norm" and L.mixer_norm is None and L.mixer_post_norm is not None
        assert dict(L.params)["residual_mult"] == cfg["residual_mult"]
        assert (L.feed_forward is None) == (raw["mlp"] is None) == (L.feed_forward_post_norm is None)
        p = dict(L.mixer.params)
        if raw["type"] == "latent_attention":
            assert L.mixer.kind == "latent_attention" and p["q_rank"] == raw["mixer"]["q_rank"] and p["sink"] == "sink"
            assert L.mixer.position.head_dim == raw["mixer"]["rot_dim"]
        elif raw["type"] == "attention":
            assert L.mixer.kind == "window_attention" and p["head_norm"][0] == "before" and L.mixer.window == 0
            assert p["bias"] == ("q.b", "k.b", "v.b") and "softcap" not in p and "gate" not in p
        else:
            assert p["head_norm"] == ("after",) and p["gate"] == "g" and "sink" not in p and "bias" not in p
            assert L.mixer.window == raw["mixer"]["mask"]["size"] and p["softcap"] == raw["mixer"]["softcap"]
        assert L.mixer.position.kind == ("rope_halves_yarn" if "scaling" in raw["mixer"]["rot"] else "rope_halves")
        assert L.mixer.scale == raw["mixer"]["scale"]


def test_tensor_list():
    _, spec = spec_from_config_dict(CONFIGS["A"])
    names = {r.name: tuple(r.shape) for r in tensor_requests(spec) if not r.optional}
    assert names["embed"] == (211, 64) and names["bigram"] == (98, 64) and names["head"] == (211, 64)
    assert names["l0.mix.g"] == (4, 64) and names["l0.mix.q"] == (64, 64) and names["l0.mix.v"] == (48, 64)
    assert names["l0.mlp.correction"] == (6,) and names["l0.mlp.e5.down"] == (64, 24) and names["l0.mlp.shared.up"] == (40, 64)
    assert "l0.mlp.router.b" not in names and "l0.mix.sink" not in names and "l0.mix.q.b" not in names
    assert names["l1.mix.dq"] == (20, 64) and names["l1.mix.dq.norm"] == (20,) and names["l1.mix.uq"] == (72, 20)
    assert names["l1.mix.dkv"] == (32, 64) and names["l1.mix.dkv.norm"] == (24,) and names["l1.mix.uk"] == (48, 24)
    assert names["l1.mix.uv"] == (36, 24) and names["l1.mix.sink"] == (3,) and names["l1.mlp.gate"] == (40, 64)
    assert names["l2.mix.q.b"] == (64,) and names["l2.mix.k.b"] == (32,) and names["l2.mix.q.norm"] == (16,)
    assert names["l2.mix.k.norm"] == (16,) and names["l2.mix.sink"] == (4,)
    assert "l3.norm2" not in names and "l3.norm1" in names and names["final.norm"] == (64,)


@pytest.mark.parametrize("edit,key", [
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d["norm"].pop("eps"), "norm.eps"),
    (lambda d: d.pop("embedding"), "embedding"),
    (lambda d: d["embedding"]["bigram"].pop("mul_cur"), "embedding.bigram.mul_cur"),
    (lambda d: d["layers"][0].update(type="attention_3"), "layers[0].type"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "layers[0].mixer.kv_heads"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=7), "layers[0].mixer.rot.dims"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=18), "layers[0].mixer.rot.dims"),
    (lambda d: d["layers"][1]["mixer"].pop("q_rank"), "layers[1].mixer.q_rank"),
    (lambda d: d["layers"][1]["mixer"]["rot"]["scaling"].pop("fast"), "layers[1].mixer.rot.scaling.fast"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=7), "layers[0].mlp.router.top"),
    (lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(count=4), "layers[0].mlp.router.groups"),
    (lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(keep=1, count=6), "layers[0].mlp.router.groups"),
    (lambda d: d["layers"][1]["mlp"].update(kind="sparse"), "layers[1].mlp.kind"),
    (lambda d: d["layers"][0]["mlp"]["expert"].pop("limit"), "layers[0].mlp.expert.limit"),
])
def test_errors_name_the_key(edit, key):
    d = copy.deepcopy(CONFIGS["A"])
    edit(d)
    with pytest.raises(ConfigError) as e:
        spec_from_config_dict(d)
    assert key in str(e.value)


@pytest.mark.parametrize("base,n,scaling", [(10000.0, 8, (4.0, 32, 8.0, 1.0)), (300000.0, 64, (6.0, 256, 16.0, 2.0)),
                                            (2e6, 48, (3.0, 1024, 24.0, 1.5)), (50.0, 2, (16.0, 8, 1.0, 0.25)),
                                            (20000.0, 16, (3.0, 48, 6.0, 0.5))])
def test_stretched_rotation_frequencies(base, n, scaling):
    f, mag = yarn_frequencies(base, n, *scaling)
    ref, ref_mag = pb.frequencies({"base": base, "dims": n,
                                   "scaling": dict(zip(("factor", "original", "fast", "slow"), scaling))})
    assert len(f) == n // 2 and mag == pytest.approx(ref_mag, rel=1e-15) and mag == pytest.approx(0.1 * math.log(scaling[0]) + 1)
    assert all(a == pytest.approx(b, rel=1e-13) for a, b in zip(f, ref))
    plain = [base ** (-2.0 * i / n) for i in range(n // 2)]
    assert all(p / scaling[0] * (1 - 1e-12) <= a <= p * (1 + 1e-12) for a, p in zip(f, plain))   # between stretched and plain
    assert f[0] == pytest.approx(plain[0]) or n == 2                  # the fastest pair keeps its frequency


def test_rotation_turns_pairs_half_a_prefix_apart():
    x = torch.randn(5, 2, 12, dtype=torch.float64)
    r = {"base": 100.0, "dims": 8}
    y = pb.rotate(x, [0, 1, 2, 7, 30], r)
    assert torch.equal(y[0], x[0]) and torch.equal(y[:, :, 8:], x[:, :, 8:])
    a = 7 * 100.0 ** (-2.0 * 1 / 8)
    assert float(y[3, 1, 1]) == pytest.approx(float(x[3, 1, 1] * math.cos(a) - x[3, 1, 5] * math.sin(a)))
    assert float(y[3, 1, 5]) == pytest.approx(float(x[3, 1, 5] * math.cos(a) + x[3, 1, 1] * math.sin(a)))
    assert torch.allclose(y.pow(2).sum(-1), x.pow(2).sum(-1))                       # lengths stay
    stretched = pb.rotate(x, [0, 1, 2, 7, 30], dict(r, scaling={"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0}))
    mag = 0.1 * math.log(4.0) + 1.0
    assert torch.allclose(stretched[:, :, :8].pow(2).sum(-1), x[:, :, :8].pow(2).sum(-1) * mag ** 2)


def test_a_sink_only_shrinks_the_weights():
    s = torch.randn(6, 6, dtype=torch.float64)
    vis = pb.causal(6)
    w, w_sink = pb.softmax_rows(s, vis), pb.softmax_rows(s, vis, sink=0.3)
    assert torch.allclose(w.sum(-1), torch.ones(6, dtype=torch.float64))
    ratio = w_sink[vis] / w[vis]
    assert bool((ratio < 1).all()) and torch.allclose(w_sink.sum(-1) + torch.exp(0.3 - torch.logsumexp(
        torch.cat([s.masked_fill(~vis, -math.inf), torch.full((6, 1), 0.3, dtype=torch.float64)], 1), 1)), torch.ones(6, dtype=torch.float64))
    assert bool((pb.causal(6, 2).sum(-1) == torch.tensor([1, 2, 2, 2, 2, 2])).all())


def test_the_router_keeps_to_the_best_groups():
    r = {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}}
    z = torch.tensor([2.0, -3.0, 1.0, 0.9, -5.0, 1.5], dtype=torch.float64)       # the best single expert sits in group 0 ...
    corr = torch.zeros(6, dtype=torch.float64)
    chosen, weights, gap = pb.route(z, corr, r)
    assert chosen == [2, 3]                                                      # ... but group 1 has the best pair
    assert weights == pytest.approx([2.0 * float(torch.sigmoid(z[2])), 2.0 * float(torch.sigmoid(z[3]))])
    corr[1] = 5.0                                                                 # a correction moves the choice, not the weight
    chosen, weights, _ = pb.route(z, corr, r)
    assert chosen == [1, 0] and weights[0] == pytest.approx(2.0 * float(torch.sigmoid(z[1])))
    corr[:] = -7.0                                                                # negative choice scores: the others are out, not zero
    assert pb.route(z, corr, r)[0] == [2, 3]
    assert pb.route(z, torch.zeros(6, dtype=torch.float64), {"experts": 6, "top": 2, "scale": 1.0})[0] == [0, 5]


def test_calm_tokens_have_no_close_router_call(tmp_path):
    cfg, tensors = write_model(tmp_path / "m", CONFIGS["A"], seed=3)
    toks, ref = calm_tokens(cfg, tensors, 40, 5)
    gaps = []
    again = pb.forward(cfg, tensors, toks, gaps=gaps)
    assert torch.equal(again, ref) and len(gaps) == 2 and min(min(g) for g in gaps) >= 0.02
    assert ref.shape == (40, cfg["vocab"]) and bool(torch.isfinite(ref).all())
