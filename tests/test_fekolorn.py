"""The Fekolorn design without a GPU: its configuration (every key, optional keys absent, refusals), the model a
configuration is turned into (part kinds, which layer is the source of mixed values, pages and state per entry, tensor
names), the distance buckets of the bias table, and the plain implementation's own properties (tests/plain_fekolorn.py
is the oracle of the GPU tests, so what it computes is pinned here by hand-made cases)."""
import copy
import math

import numpy as np
import pytest
import torch

import plain_fekolorn as P
from fekolorn_configs import FEKOLORN, write_fekolorn_model
from llm_rs_b200.config import ConfigError, FekolornConfig, load_config, resolve_architecture
from llm_rs_b200.parts import DecoderModel
from llm_rs_b200.parts.scored_attention import distance_bucket

F64 = torch.float64


# ---- configuration ------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", list(FEKOLORN))
def test_config_round_trip(name):
    raw = FEKOLORN[name][0]
    cfg = FekolornConfig.from_dict(raw)
    again = FekolornConfig.from_dict(cfg.to_dict())
    assert again == cfg
    assert resolve_architecture(raw).config_cls is FekolornConfig


def test_optional_keys_switch_their_mechanism_off():
    raw = {"architecture": "Fekolorn", "vocab": 9, "width": 8, "norm": {"eps": 1e-6},
           "layers": [{"type": "attention", "mixer": {"heads": 2, "dim": 4, "scale": 0.5}, "mlp": None}]}
    cfg = FekolornConfig.from_dict(raw)
    m = cfg.layers[0].mixer
    assert (m.kv_heads, m.vdim, m.window, m.bias_rows, m.v_mix, m.rot_dims) == (2, 4, 0, 0, False, 0)
    assert cfg.streams == 1 and not cfg.hyper and cfg.pairs is None and cfg.embedding_scale == 1.0
    assert cfg.layers[0].mlp is None
    spec = resolve_architecture(raw).build_spec(cfg)
    names = {s.name for s in DecoderModel(spec).weight_specs()}
    assert "bigram" not in names and not any(".hc" in n or n.endswith(".rel") or n.endswith(".vmix") for n in names)
    assert "l0.norm2" not in names and "l0.norm1" in names and "l0.mix.sink" in names


@pytest.mark.parametrize("change,message", [
    (lambda r: r.pop("vocab"), "vocab"),
    (lambda r: r["layers"][0].update(type="conv"), "type"),
    (lambda r: r["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda r: r["layers"][1]["mixer"].update(bias_rows=1), "bias"),
    (lambda r: r["layers"][1]["mixer"].update(bias_max=2), "bias"),
    (lambda r: r["layers"][0]["mixer"]["left"].update(rot={"base": 10.0, "dims": 7}), "rot.dims"),
    (lambda r: r["layers"][0]["mixer"]["right"].pop("conv"), "conv"),
    (lambda r: r["layers"][0]["mixer"].pop("left"), "left"),
    (lambda r: r["layers"][2]["mixer"].update(vdim=4), "v_mix"),
    (lambda r: r["layers"][0].update(mlp={"kind": "moe", "ff": 3}), "dense"),
    (lambda r: r.update(streams=0), "streams"),
])
def test_config_refusals(change, message):
    raw = copy.deepcopy(FEKOLORN["A"][0])
    change(raw)
    with pytest.raises(ConfigError, match=message):
        FekolornConfig.from_dict(raw)


def test_tensor_shapes_decide_what_the_keys_leave_open(tmp_path):
    """Rows of the bias table, sinks and hyper-connection tensors are read from the folder."""
    path = write_fekolorn_model("D", str(tmp_path))
    entry, cfg = load_config(path)
    assert cfg.hyper and cfg.streams == 1
    assert not cfg.layers[0].mixer.left.sink and cfg.layers[1].mixer.sink
    assert cfg.layers[1].mixer.bias_rows == 3
    path = write_fekolorn_model("E", str(tmp_path))
    entry, cfg = load_config(path)
    assert not cfg.hyper
    assert [l.mixer.bias_rows for l in cfg.layers if l.type == "attention"] == [2, 9]


# ---- the model a configuration becomes -------------------------------------------------------------------
def test_spec_of_a_configuration():
    raw = FEKOLORN["A"][0]
    spec = resolve_architecture(raw).build_spec(FekolornConfig.from_dict(raw))
    assert [l.mixer.kind for l in spec.layers] == ["parallel", "scored_attention", "scored_attention", "parallel"]
    assert all(l.block.kind == "hyper" and l.block.params["streams"] == 2 for l in spec.layers)
    assert spec.layers[2].feed_forward is None and spec.layers[2].feed_forward_norm is None
    kinds = [l.mixer.params.get("v_mix") or l.mixer.params["left"].params["v_mix"] for l in spec.layers]
    assert kinds == ["none", "source", "mixed", "mixed"]
    left = spec.layers[0].mixer.params["left"].params
    assert (left["qk_norm"], left["v_norm"], left["mask"], left["rot_dims"]) == ("none", "head_unit", "causal", 8)
    alone = spec.layers[1].mixer.params
    assert (alone["qk_norm"], alone["v_norm"], alone["mask"], alone["mask_size"], alone["bias_rows"]) == \
        ("whole", "none", "window", 20, 8)
    assert spec.embedding.kind == "pair_embedding" and spec.embedding.params["streams"] == 2
    model = DecoderModel(spec)
    needs = model.cache_needs()
    assert [n[0].kind for n in needs] == ["full", "window", "window", "window"]
    assert needs[0][0].planes == (16, 8) and needs[1][0].window == 20
    assert set(needs[0][1].tensors) == {"gated_delta.state", "gated_delta.conv", "embedding.previous_token"}
    assert needs[0][1].tensors["gated_delta.state"] == (4, 16, 8) and needs[0][1].tensors["gated_delta.conv"] == (3, 96)
    assert needs[1][1] is None and set(needs[3][1].tensors) == {"gated_delta.state", "gated_delta.conv"}
    names = {s.name: s.shape for s in model.weight_specs()}
    assert names["l0.mix.left.q"] == (64, 64) and names["l0.mix.right.v.conv"] == (32, 4) and names["l0.hc2.mix"] == (2, 2)
    assert names["l1.mix.rel"] == (8, 4) and names["l1.norm1"] == () and names["bigram"] == (102, 64)
    assert names["l0.mlp.act"] == (4,) and names["l0.mix.right.norm"] == (8,) and "l2.hc2.in" not in names


def test_a_parallel_mixer_plans_for_its_sides():
    raw = FEKOLORN["D"][0]
    model = DecoderModel(resolve_architecture(raw).build_spec(FekolornConfig.from_dict(raw)))
    mixer = model.blocks[0].mixer
    keys = [k for k, _ in mixer.planners()]
    assert keys == [mixer.left.plan_key()] and mixer.right.plan_key() is None
    assert mixer.cache_need() == mixer.left.cache_need() and mixer.right.cache_need() is None


# ---- distance buckets --------------------------------------------------------------------------------------
@pytest.mark.parametrize("rows,reach", [(16, 240), (8, 64), (6, 5), (3, 9), (2, 3), (9, 4.5), (32, 4096), (11, 1000)])
def test_distance_buckets(rows, reach):
    half = rows // 2
    got = [distance_bucket(n, rows, reach) for n in range(int(reach) + 50)]
    assert got == [P.distance_bucket(n, rows, reach) for n in range(int(reach) + 50)]
    assert got[:half] == list(range(half)) and got[half] == half
    assert all(b >= a for a, b in zip(got, got[1:])) and max(got) == rows - 1
    assert all(b == rows - 1 for n, b in enumerate(got) if n >= reach)
    by_hand = [n for n in range(half, int(reach)) if half * (reach / half) ** ((got[n] - half + 1) / (rows - half)) < n * (1 - 1e-9)]
    assert not by_hand, "a distance lies beyond its bucket's upper edge"


# ---- the plain implementation's own properties ---------------------------------------------------------------
def _attention_weights(g, D, m, p="m."):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    r = lambda *s: torch.randn(*s, generator=g, dtype=F64)
    w = {p + "q": r(H * d, D), p + "k": r(G * d, D), p + "v": r(G * dv, D), p + "o": r(D, H * dv),
         p + "q.norm": 1 + 0.2 * r(H * d), p + "k.norm": 1 + 0.2 * r(G * d), p + "sink": r(H), p + "vmix": torch.tensor(0.4, dtype=F64)}
    if "bias_max" in m:
        w[p + "rel"] = r(m["bias_rows"], H)
    return w


def test_a_token_outside_the_window_has_no_influence():
    g = torch.Generator().manual_seed(0)
    m = {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 6, "scale": 0.3, "mask": {"size": 5}, "bias_max": 20, "bias_rows": 6}
    w = _attention_weights(g, 12, m)
    x = torch.randn(20, 12, generator=g, dtype=F64)
    y, _ = P.softmax_mixer(x, m, w, "m.", 1e-6, torch.arange(20), True, False)
    x2 = x.clone()
    x2[7] += 3.0
    y2, _ = P.softmax_mixer(x2, m, w, "m.", 1e-6, torch.arange(20), True, False)
    assert torch.equal(y[12:], y2[12:]) and not torch.allclose(y[11], y2[11]) and torch.equal(y[:7], y2[:7])


def test_the_sink_only_takes_weight_away():
    g = torch.Generator().manual_seed(1)
    m = {"heads": 2, "kv_heads": 2, "dim": 4, "vdim": 4, "scale": 0.5}
    w = _attention_weights(g, 8, m)
    w["m.o"] = torch.eye(8, dtype=F64)
    x = torch.randn(6, 8, generator=g, dtype=F64)
    pos = torch.arange(6)
    with_sink, _ = P.softmax_mixer(x, m, w, "m.", 1e-6, pos, False, False)
    w2 = dict(w)
    del w2["m.sink"]
    without, _ = P.softmax_mixer(x, m, w2, "m.", 1e-6, pos, False, False)
    ratio = (with_sink / without).view(6, 2, 4)
    assert torch.allclose(ratio, ratio[..., :1].expand_as(ratio)) and (ratio < 1).all() and (ratio > 0).all()
    # the first token sees itself alone: its weight is 1 / (1 + exp(sink - score))
    q, k = (x[0] @ w["m.q"].T).view(2, 4), (x[0] @ w["m.k"].T).view(2, 4)
    s = (q * k).sum(-1) * 0.5
    assert torch.allclose(ratio[0, :, 0], 1 / (1 + torch.exp(w["m.sink"] - s)))


def test_the_bias_is_added_per_bucket_and_head_after_the_scale():
    g = torch.Generator().manual_seed(2)
    m = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 3, "scale": 0.0, "bias_max": 12, "bias_rows": 4}
    w = _attention_weights(g, 5, m)
    del w["m.sink"]
    w["m.o"] = torch.eye(3, dtype=F64)
    x = torch.randn(9, 5, generator=g, dtype=F64)
    y, v = P.softmax_mixer(x, m, w, "m.", 1e-6, torch.arange(9), True, False)
    # a scale of zero leaves the bias alone: weights softmax(rel[bucket(i - j)])
    i = 8
    buckets = [P.distance_bucket(i - j, 4, 12) for j in range(9)]
    assert buckets == [3, 3, 3, 3, 2, 2, 2, 1, 0]      # 2 + floor(2 ln(n / 2) / ln 6): distance 5 is the first in row 3
    a = torch.softmax(w["m.rel"][buckets, 0], dim=0)
    assert torch.allclose(y[i], (a[:, None] * v[:, 0]).sum(0))


def test_values_are_normed_per_head_and_mixed_with_the_first_layers():
    g = torch.Generator().manual_seed(3)
    m = {"heads": 2, "kv_heads": 2, "dim": 4, "vdim": 6, "scale": 0.4, "v_mix": True}
    w = _attention_weights(g, 7, m)
    x = torch.randn(5, 7, generator=g, dtype=F64)
    _, v = P.softmax_mixer(x, m, w, "m.", 1e-6, torch.arange(5), False, True)
    assert torch.allclose((v * v).mean(-1), torch.ones(5, 2, dtype=F64), atol=1e-5)
    first = torch.randn(5, 2, 6, generator=g, dtype=F64)
    _, mixed = P.softmax_mixer(x, m, w, "m.", 1e-6, torch.arange(5), False, False, v_first=first)
    assert torch.allclose(mixed, 0.6 * (x @ w["m.v"].T).view(5, 2, 6) + 0.4 * first)


def test_rotation_by_halves_keeps_the_rest():
    x = torch.arange(12, dtype=F64).view(1, 1, 12).repeat(3, 1, 1)
    y = P.rotate_halves(x, torch.tensor([0, 1, 5]), 4, 100.0)
    assert torch.equal(y[0], x[0]) and torch.equal(y[:, :, 4:], x[:, :, 4:])
    a0, a1 = 5.0, 5.0 * 100.0 ** -0.5
    want = [0 * math.cos(a0) - 2 * math.sin(a0), 1 * math.cos(a1) - 3 * math.sin(a1),
            2 * math.cos(a0) + 0 * math.sin(a0), 3 * math.cos(a1) + 1 * math.sin(a1)]
    assert torch.allclose(y[2, 0, :4], torch.tensor(want, dtype=F64))


def test_short_convolution_is_causal_and_ends_on_the_current_token():
    x = torch.tensor([[1.0], [10.0], [100.0], [1000.0]], dtype=F64)
    taps = torch.tensor([[2.0, 3.0, 5.0]], dtype=F64)       # the last column is the current token's
    assert P.short_conv(x, taps).view(-1).tolist() == [5.0, 53.0, 532.0, 5320.0]


def test_delta_rule_by_hand():
    """One head, keys of two channels: the state after two tokens and the read-out that sees the token's own write."""
    D = 3
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "conv": 1}
    g = torch.Generator().manual_seed(4)
    r = lambda *s: torch.randn(*s, generator=g, dtype=F64)
    w = {"m.q": r(2, D), "m.k": r(2, D), "m.v": r(2, D), "m.q.conv": torch.ones(2, 1, dtype=F64),
         "m.k.conv": torch.ones(2, 1, dtype=F64), "m.v.conv": torch.ones(2, 1, dtype=F64), "m.b": r(1, D), "m.a": r(1, D),
         "m.A_log": r(1), "m.dt_bias": r(1), "m.g": r(2, D), "m.norm": torch.ones(2, dtype=F64), "m.o": torch.eye(D, 2, dtype=F64)}
    x = r(2, D)
    y = P.gated_delta(x, m, w, "m.", 1e-6)
    S = torch.zeros(2, 2, dtype=F64)
    outs = []
    for t in range(2):
        q, k, v = (P.silu(x[t] @ w["m." + n].T) for n in "qkv")
        q = q / torch.sqrt((q * q).sum() + 1e-6) * 2 ** -0.5
        k = k / torch.sqrt((k * k).sum() + 1e-6)
        beta = torch.sigmoid(x[t] @ w["m.b"].T)[0]
        decay = torch.exp(-torch.exp(w["m.A_log"][0]) * torch.log1p(torch.exp(x[t] @ w["m.a"].T + w["m.dt_bias"]))[0])
        S = decay * S
        S = S + torch.outer(k, beta * (v - S.T @ k))
        o = S.T @ q
        o = o / torch.sqrt((o * o).mean() + 1e-6) * P.silu(x[t] @ w["m.g"].T)
        outs.append(torch.cat([o, torch.zeros(1, dtype=F64)]))
    assert torch.allclose(y, torch.stack(outs))
    assert 0 < float(decay) < 1 and 0 < float(beta) < 1


def test_a_write_of_full_strength_replaces_what_the_key_held():
    """With beta = 1 and no decay, reading with the key just written returns the value just written."""
    S = torch.randn(4, 3, dtype=F64)
    k = torch.nn.functional.normalize(torch.randn(4, dtype=F64), dim=0)
    v = torch.randn(3, dtype=F64)
    S2 = S + torch.outer(k, 1.0 * (v - S.T @ k))
    assert torch.allclose(S2.T @ k, v)


def test_poly_norm_by_hand():
    z = torch.tensor([[1.0, -2.0, 3.0, 0.5]], dtype=F64)
    c = torch.tensor([0.5, -1.0, 2.0, 0.25], dtype=F64)
    n = lambda v: v / math.sqrt(float((v * v).mean()) + 1e-6)
    want = 0.5 * n(z[0]) - 1.0 * n(z[0] ** 2) + 2.0 * n(z[0] ** 3) + 0.25
    assert torch.allclose(P.poly_norm(z, c, 1e-6)[0], want)


def test_pair_rows_and_the_first_token():
    cfg = {"embedding": {"scale": 0.5, "bigram": {"buckets": 7, "mul_prev": 3, "mul_cur": 5}}}
    w = {"embed": torch.arange(10, dtype=F64)[:, None].repeat(1, 2), "bigram": 100.0 * torch.arange(8, dtype=F64)[:, None].repeat(1, 2)}
    x = P.embed([4, 9, 9, 0], cfg, w)
    rows = [7, (4 * 3 + 9 * 5) % 7, (9 * 3 + 9 * 5) % 7, (9 * 3 + 0) % 7]
    assert x[:, 0].tolist() == [0.5 * t + 100.0 * r for t, r in zip([4, 9, 9, 0], rows)]


def test_streams_with_identity_connections_are_the_plain_residual():
    g = torch.Generator().manual_seed(5)
    x = torch.randn(1, 4, 6, generator=g, dtype=F64)
    fn = lambda h: h * 2.0 + 1.0
    gain = torch.tensor(1.3, dtype=F64)
    plain = P.sublayer(x, fn, gain, 1e-6, {}, "hc1.")
    w = {"hc1.in": torch.ones(1, dtype=F64), "hc1.out": torch.ones(1, dtype=F64), "hc1.mix": torch.ones(1, 1, dtype=F64)}
    assert torch.allclose(P.sublayer(x, fn, gain, 1e-6, w, "hc1."), plain)
    assert torch.allclose(plain[0], x[0] + fn(P.scalar_norm(x[0], gain, 1e-6)))


def test_the_mix_matrix_is_indexed_from_to():
    x = torch.stack([torch.ones(1, 2, dtype=F64), 10 * torch.ones(1, 2, dtype=F64)])
    w = {"hc1.in": torch.tensor([1.0, 0.0], dtype=F64), "hc1.out": torch.tensor([0.0, 1.0], dtype=F64),
         "hc1.mix": torch.tensor([[0.0, 1.0], [0.0, 0.0]], dtype=F64)}       # stream 0 goes to stream 1
    seen = {}

    def fn(h):
        seen["h"] = h
        return 5.0 * torch.ones_like(h)
    y = P.sublayer(x, fn, torch.tensor(1.0, dtype=F64), 0.0, w, "hc1.")
    assert torch.allclose(seen["h"], torch.ones(1, 2, dtype=F64))            # reads stream 0 alone, normed
    assert y[0].abs().max() == 0 and torch.allclose(y[1], 6.0 * torch.ones(1, 2, dtype=F64))


def test_the_first_layer_with_mixed_values_keeps_its_own(tmp_path):
    """In a whole model the source layer's values stay unmixed: changing its mixing weight changes nothing."""
    path = write_fekolorn_model("A", str(tmp_path))
    cfg, w = P.load_model_dir(path)
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], 30).tolist()
    base = P.forward(toks, cfg, w)
    w2 = dict(w)
    w2["l1.mix.vmix"] = torch.tensor(0.9, dtype=F64)      # written by the random-weights mode only if present
    assert torch.equal(P.forward(toks, cfg, w2), base)
    w2["l2.mix.vmix"] = w["l2.mix.vmix"] + 0.3
    assert not torch.allclose(P.forward(toks, cfg, w2), base)
