"""Leguvik without a device: configuration keys and their errors, the schedule and cache needs a
layer that reads another layer's keys makes, the tensors a model asks for, and properties of the
plain implementation's mechanisms."""
import json

import pytest
import torch

import plain_leguvik as pl
from leguvik_util import CONFIGS, attention, delta, layer, model, moe, ssm
from sonicboom_b200.config import ConfigError, LeguvikConfig, spec_from_config_dict
from sonicboom_b200.models import tensor_requests

F = torch.float64


def test_round_trip_and_registry():
    for cfg in CONFIGS.values():
        c, spec = spec_from_config_dict(cfg)
        assert isinstance(c, LeguvikConfig) and LeguvikConfig.from_dict(c.to_dict()) == c
        assert spec.architecture == "Leguvik" and spec.vocab == cfg["vocab"] and len(spec.schedule) == len(cfg["layers"])


def test_a_reader_of_another_layers_keys_owns_no_cache():
    _, spec = spec_from_config_dict(CONFIGS["A"])
    assert [e.cache_from for e in spec.schedule] == [None, None, None, 0, None]
    names = {r.name for r in tensor_requests(spec)}
    assert "l0.mix.k" in names and "l3.mix.q" in names and "l3.mix.k" not in names and "l3.mix.v" not in names
    assert "l2.mlp.router" not in names and "l2.norm2" not in names           # a layer without a feed-forward
    assert "l3.mlp.shared.gate" in names and "l1.mlp.shared.gate" not in names


def test_tensor_names_and_shapes():
    _, spec = spec_from_config_dict(CONFIGS["A"])
    req = {r.name: tuple(r.shape) for r in tensor_requests(spec)}
    assert req["embed"] == (211, 64) and req["bigram"] == (98, 64) and req["final.norm"] == (64,)
    assert req["l0.canon1"] == (64, 3) and req["l0.canon2"] == (64, 3)
    assert req["l0.mix.q"] == (64, 64) and req["l0.mix.k"] == (32, 64) and req["l0.mix.v"] == (48, 64)
    assert req["l0.mix.pb"] == (4,) and req["l0.mix.o"] == (64, 96)
    assert req["l0.mlp.router"] == (5, 64) and req["l0.mlp.e4.gate"] == (24, 64) and req["l0.mlp.shared.down"] == (64, 40)
    inner, gn = 4 * 12, 2 * 16
    assert req["l1.mix.in"] == (2 * inner + 2 * gn + 4, 64) and req["l1.mix.conv"] == (inner + 2 * gn, 4)
    assert req["l1.mix.A_log"] == (4,) and req["l1.mix.norm"] == (inner,) and req["l1.mix.o"] == (64, inner)
    assert req["l2.mix.w1"] == (4, 64) and req["l2.mix.w2"] == (32, 4) and req["l2.mix.a.b"] == (32,)
    # without a stated rank the decay map's two matrices are asked for with that size left open
    cfg = json.loads(json.dumps(CONFIGS["A"]))
    del cfg["layers"][2]["mixer"]["decay_rank"]
    req = {r.name: tuple(r.shape) for r in tensor_requests(spec_from_config_dict(cfg)[1])}
    assert req["l2.mix.w1"] == (-1, 64) and req["l2.mix.w2"] == (32, -1)


def test_what_config_json_leaves_out_does_not_exist():
    bare = model(50, 32, [layer("ssm", ssm(2, 8, 8))], taps=0, bigram=None, cap=0.0)
    c, spec = spec_from_config_dict(bare)
    assert c.canon_taps == 0 and c.bigram is None and c.logit_softcap == 0.0
    names = {r.name for r in tensor_requests(spec)}
    assert not any("canon" in n or n == "bigram" or ".mlp." in n for n in names)
    open_ = model(50, 32, [layer("attention", attention(2, 1, 8, 8, window=0))])
    c, _ = spec_from_config_dict(open_)
    assert c.layers[0].mixer.window == 0 and "mask" not in c.to_dict()["layers"][0]["mixer"]
    assert LeguvikConfig.from_dict(c.to_dict()) == c


@pytest.mark.parametrize("path,value,match", [
    (("layers", 0, "type"), "conv", r"layers\[0\].type"),
    (("layers", 0, "mixer", "kv_heads"), 3, r"layers\[0\].mixer.kv_heads"),
    (("layers", 0, "mixer", "mask", "keep_first"), -1, r"keep_first"),
    (("layers", 1, "mixer", "groups"), 3, r"layers\[1\].mixer.groups"),
    (("layers", 1, "mixer", "norm_groups"), 5, r"layers\[1\].mixer.norm_groups"),
    (("layers", 0, "mlp", "router", "top"), 6, r"layers\[0\].mlp.router.top"),
    (("layers", 0, "mlp", "kind"), "dense", r"layers\[0\].mlp.kind"),
    (("layers", 3, "mixer", "kv_from"), 1, r"layers\[3\].mixer.kv_from"),
    (("layers", 3, "mixer", "kv_from"), 3, r"layers\[3\].mixer.kv_from"),
    (("layers", 3, "mixer", "vdim"), 16, r"layers\[3\].mixer.kv_from"),
    (("norm", "eps"), -1.0, r"norm.eps"),
    (("width",), 0, r"width"),
])
def test_errors_name_the_key(path, value, match):
    cfg = json.loads(json.dumps(CONFIGS["A"]))
    at = cfg
    for p in path[:-1]:
        at = at[p]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=match):
        spec_from_config_dict(cfg)


# ------------------------------------------------------------------ the plain implementation's mechanisms
def test_layer_norm_takes_the_mean_off_and_convolution_is_causal():
    g = torch.Generator().manual_seed(0)
    x, w = torch.randn(5, 16, generator=g, dtype=F), torch.randn(16, generator=g, dtype=F)
    assert torch.allclose(pl.layer_norm(x + 3.0, w, 0.0), pl.layer_norm(x, w, 0.0))
    assert torch.allclose(pl.layer_norm(2.0 * x, w, 0.0), pl.layer_norm(x, w, 0.0))
    h, cw = torch.randn(9, 4, generator=g, dtype=F), torch.randn(4, 3, generator=g, dtype=F)
    y = pl.causal_conv(h, cw)
    later = h.clone()
    later[6:] += 1.0
    assert torch.equal(pl.causal_conv(later, cw)[:6], y[:6])                   # nothing comes from ahead
    assert torch.allclose(y[0], cw[:, 2] * h[0]) and torch.allclose(y[2], (cw * h[:3].T).sum(1))


def test_pair_rows_hash_two_neighbours_and_the_first_token_has_a_row_of_its_own():
    rows = pl.bigram_rows([3, 5, 5, 0], 11, 7, 2)
    assert rows == [11, (3 * 7 + 5 * 2) % 11, (5 * 7 + 5 * 2) % 11, (5 * 7) % 11]


def test_window_with_kept_first_keys():
    seen = [[j for j in range(i + 1) if pl.visible(i, j, 3, 2)] for i in range(7)]
    assert seen[2] == [0, 1, 2] and seen[4] == [0, 1, 2, 3, 4] and seen[5] == [0, 1, 3, 4, 5] and seen[6] == [0, 1, 4, 5, 6]
    assert [j for j in range(7) if pl.visible(6, j, 3, 0)] == [4, 5, 6]


def test_delta_rule_without_removal_or_decay_is_a_running_sum_of_outer_products():
    g = torch.Generator().manual_seed(1)
    width, heads, dim, T = 12, 2, 4, 6
    t = {n: torch.randn(heads * dim, width, generator=g, dtype=F) * 0.3 for n in ("r", "k", "v", "g", "a")}
    t.update({"w1": torch.zeros(2, width, dtype=F), "w2": torch.zeros(heads * dim, 2, dtype=F),
              "w0": torch.full((heads * dim,), -60.0, dtype=F),           # decays of exp(-c sigmoid(-60)) = 1
              "a.b": torch.full((heads * dim,), -60.0, dtype=F),          # removal rates of 0
              "norm": torch.ones(heads * dim, dtype=F), "o": torch.eye(heads * dim, dtype=F)[:width].T.contiguous()})
    t["a"].zero_()
    h = torch.randn(T, width, generator=g, dtype=F)
    y = pl.general_delta(h, lambda n: t[n], {"heads": heads, "dim": dim}, 0.0) @ torch.linalg.pinv(t["o"]).T
    r, k, v = (h @ t[n].T for n in ("r", "k", "v"))
    for hd in range(heads):
        sl = slice(hd * dim, (hd + 1) * dim)
        o = torch.stack([sum(v[j, sl] * (k[j, sl] @ r[i, sl]) for j in range(i + 1)) for i in range(T)])
        want = o / o.pow(2).mean(-1, keepdim=True).sqrt() * torch.sigmoid(h @ t["g"].T)[:, sl]
        assert torch.allclose(y[:, sl], want, atol=1e-9)


def test_all_experts_chosen_is_a_softmax_over_all_of_them():
    g = torch.Generator().manual_seed(2)
    width, E, ff = 8, 3, 5
    t = {"router": torch.randn(E, width, generator=g, dtype=F), "router.b": torch.randn(E, generator=g, dtype=F)}
    for e in range(E):
        t.update({f"e{e}.gate": torch.randn(ff, width, generator=g, dtype=F), f"e{e}.up": torch.randn(ff, width, generator=g, dtype=F),
                  f"e{e}.down": torch.randn(width, ff, generator=g, dtype=F)})
    h = torch.randn(4, width, generator=g, dtype=F)
    gaps = []
    y = pl.moe(h, lambda n: t[n], moe(E, E, ff, 1.5), gaps)
    p = torch.softmax(h @ t["router"].T + t["router.b"], -1)
    want = sum(p[:, e:e + 1] * pl.clamped_glu(h, t[f"e{e}.gate"], t[f"e{e}.up"], t[f"e{e}.down"], 1.5) for e in range(E))
    assert torch.allclose(y, want) and bool(torch.isinf(gaps[0]).all())
    one = []
    pl.moe(h, lambda n: t[n], moe(E, 1, ff, 1.5), one)
    z = (h @ t["router"].T + t["router.b"]).sort(-1, descending=True).values
    assert torch.allclose(one[0], z[:, 0] - z[:, 1])


def test_clamped_gate_saturates_at_its_limit():
    h = torch.tensor([[100.0], [-100.0]], dtype=F)
    one = torch.ones(1, 1, dtype=F)
    y = pl.clamped_glu(h, one, one, one, 2.0)
    assert torch.allclose(y[0], 2.0 * torch.sigmoid(torch.tensor([pl.GLU_SLOPE * 2.0], dtype=F)) * 3.0)
    assert abs(float(y[1])) < 1e-30
