"""The Pozelix design without a GPU: its configuration's keys and refusals, the model it is turned into (part kinds,
run order of a looped stretch, pages, tensor names), random model folders, the rescaled frequencies of the package
against the plain ones, and the plain implementation's own properties (what lies outside a window has no influence;
unit-norm heads forget the size of q and k; the gate closes a head; neighbouring pairs; a correction steers the choice
and not the weight; identity experts return their input; the stream re-enters every pass through the embedding)."""
import copy
import json
import math

import numpy as np
import pytest
import torch

import plain_pozelix as P
from pozelix_configs import POZELIX, POZELIX_A, POZELIX_B, POZELIX_D, POZELIX_E, write_pozelix_model

from llm_rs_b200.config import ConfigError, PozelixConfig, load_config, resolve_architecture
from llm_rs_b200.parts import DecoderModel

F64 = torch.float64


def test_config_reads_every_key_and_writes_them_back():
    cfg = PozelixConfig.from_dict(POZELIX_A)
    assert (cfg.vocab, cfg.width, cfg.norm_eps) == (211, 64, 1e-5)
    assert [l.type for l in cfg.layers] == ["latent_attention", "attention", "attention", "latent_attention"]
    assert (cfg.loop.start, cfg.loop.stop, cfg.loop.times) == (1, 3, 3)
    m = cfg.layers[0].mixer
    assert (m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.q_rank, m.scale, m.rot_base, m.rot_dims) == \
        (3, 16, 8, 24, 40, 24, 0.2, 1000.0, 8)
    assert (m.scaling.factor, m.scaling.original, m.scaling.fast, m.scaling.slow) == (4.0, 64, 8.0, 1.0)
    assert cfg.layers[3].mixer.scaling is None
    a = cfg.layers[1].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window, a.rot_base, a.rot_dims) == \
        (4, 2, 16, 32, 0.3, 20, 10000.0, 8)
    assert (cfg.layers[2].mixer.window, cfg.layers[2].mixer.rot_dims, cfg.layers[2].mlp) == (0, 0, None)
    f = cfg.layers[1].mlp
    assert (f.ff, f.experts, f.top, f.identity) == (40, 4, 2, 1) and cfg.layers[3].mlp.identity == 0
    assert cfg.layers[0].mlp.ff == 80
    again = PozelixConfig.from_dict(json.loads(json.dumps(cfg.to_dict())))
    assert again == cfg
    assert resolve_architecture(cfg.to_dict()).name == "Pozelix"
    assert PozelixConfig.from_dict(POZELIX_B).loop is None and "loop" not in PozelixConfig.from_dict(POZELIX_B).to_dict()


@pytest.mark.parametrize("change,message", [
    (lambda c: c.pop("width"), "width missing"),
    (lambda c: c.pop("norm"), "norm.eps missing"),
    (lambda c: c["layers"][0].update(type="conv"), "type must be one of"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank missing"),
    (lambda c: c["layers"][0]["mixer"].pop("q_rank"), "q_rank missing"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("fast"), "fast missing"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].update(factor=0.0), "must be positive"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "no multiple of 3 kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims 7 must be even"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18), "rot.dims 18 must be even and at most"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(scaling={"factor": 2.0}), "belongs to latent_attention"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale missing"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=6), "router.top 6 exceeds"),
    (lambda c: c["layers"][0]["mlp"].update(kind="conv"), "mlp.kind must be 'dense' or 'moe'"),
    (lambda c: c["layers"][0]["mixer"].update(heads=2.5), "heads must be an integer"),
    (lambda c: c["loop"].update(stop=5), "loop: layers 1 .. 4 of 4"),
    (lambda c: c["loop"].update(start=3), "loop: layers 3 .. 2 of 4"),
    (lambda c: c["loop"].update(times=0), "times"),
])
def test_config_refusals(change, message):
    raw = copy.deepcopy(POZELIX_A)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        PozelixConfig.from_dict(raw)


def test_the_model_it_is_turned_into():
    cfg = PozelixConfig.from_dict(POZELIX_A)
    spec = resolve_architecture(cfg.to_dict()).build_spec(cfg)
    assert [l.mixer.kind for l in spec.layers] == ["latent_attention", "scored_attention", "scored_attention",
                                                   "latent_attention"]
    assert [None if l.feed_forward is None else l.feed_forward.kind for l in spec.layers] == ["swiglu", "moe", None, "moe"]
    assert all(l.block.kind == "sandwich" for l in spec.layers) and spec.reentry.kind == "embedding_mix"
    # Layers 1 and 2 run three times: eight run-order entries, each with pages of its own; a pass re-enters at layer 1.
    assert [(s.layer, s.reenter) for s in spec.run_order] == [
        (0, False), (1, True), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    assert [(i, e) for i, e in P.run_order(POZELIX_A)] == [(s.layer, s.reenter) for s in spec.run_order]
    a = spec.layers[1].mixer.params
    assert (a["qk_norm"], a["gated"], a["mask"], a["mask_size"]) == ("head_unit", True, "window", 20)
    assert spec.layers[2].mixer.params["mask"] == "causal"
    l = spec.layers[0].mixer.params
    assert (l["rot_pairing"], l["q_rank"], l["gated"], l["window"]) == ("neighbours", 24, False, 0)
    f = spec.layers[1].feed_forward.params
    assert (f["router"], f["n_identity"], f["limit"]) == ("softmax_bias", 1, None)
    model = DecoderModel(spec)
    needs = model.cache_needs()
    assert len(needs) == 8
    assert needs[0][0].kind == "full" and needs[0][0].plane_widths == (40, 8) and needs[0][0].n_kv_heads == 1
    assert needs[1][0].kind == "window" and needs[1][0].window == 20 and needs[1][0].plane_widths == (16, 32)
    assert needs[2][0].kind == "full" and needs[3][0].kind == "window"
    assert all(n[1] is None for n in needs)       # no per-request state: attention only
    names = {s.name: tuple(s.shape) for s in model.weight_specs()}
    for name, shape in {"embed": (211, 64), "head": (211, 64), "final.norm": (64,), "loop.in": (64, 128),
                        "l0.norm1": (64,), "l0.norm1b": (64,), "l0.norm2": (64,), "l0.norm2b": (64,),
                        "l0.mix.dq": (24, 64), "l0.mix.dq.norm": (24,), "l0.mix.uq": (3 * 24, 24),
                        "l0.mix.dkv": (48, 64), "l0.mix.dkv.norm": (40,), "l0.mix.uk": (48, 40), "l0.mix.uv": (72, 40),
                        "l0.mix.o": (64, 72), "l0.mlp.gate": (80, 64), "l0.mlp.down": (64, 80),
                        "l1.mix.q": (64, 64), "l1.mix.k": (32, 64), "l1.mix.v": (64, 64), "l1.mix.g": (4, 64),
                        "l1.mix.o": (64, 128), "l1.mlp.router": (5, 64), "l1.mlp.correction": (5,),
                        "l1.mlp.e3.down": (64, 40), "l3.mlp.router": (3, 64), "l3.mlp.e2.gate": (24, 64)}.items():
        assert names.get(name) == shape, (name, names.get(name))
    assert not any(n in names for n in ("l2.norm2", "l2.norm2b", "l1.mlp.e4.gate", "l0.mix.q", "l0.mix.g"))
    # No loop: no re-entry and no tensor for it.
    cfg_b = PozelixConfig.from_dict(POZELIX_B)
    spec_b = resolve_architecture(cfg_b.to_dict()).build_spec(cfg_b)
    assert spec_b.reentry is None and not any(s.reenter for s in spec_b.run_order)
    assert "loop.in" not in {s.name for s in DecoderModel(spec_b).weight_specs()}
    # A loop of one layer that runs four times; a loop over all layers.
    order = lambda raw: [(s.layer, s.reenter) for s in
                         resolve_architecture(raw).build_spec(PozelixConfig.from_dict(raw)).run_order]
    assert order(POZELIX_E) == [(0, False), (1, True), (1, True), (1, True), (1, True), (2, False)]
    assert order(POZELIX_D) == [(0, True), (1, False), (2, False), (0, True), (1, False), (2, False)]


def test_random_folders_load_and_run_in_the_plain_implementation(tmp_path):
    for name in POZELIX:
        path = write_pozelix_model(name, str(tmp_path))
        entry, typed = load_config(path)
        assert entry.name == "Pozelix" and typed.to_dict()["layers"] == PozelixConfig.from_dict(POZELIX[name][0]).to_dict()["layers"]
        cfg, w = P.load_model_dir(path)
        assert set(w) == {s.name for s in DecoderModel(entry.build_spec(typed)).weight_specs()}
        res = []
        logits = P.forward(list(range(12)), cfg, w, res)
        assert logits.shape == (12, cfg["vocab"]) and bool(torch.isfinite(logits).all())
        assert len(res) == len(P.run_order(cfg))


@pytest.mark.parametrize("dims,base,scaling", [
    (16, 10000.0, None), (8, 1000.0, (4.0, 64, 8.0, 1.0)), (32, 10000.0, (8.0, 128, 16.0, 2.0)),
    (10, 100.0, (2.0, 16, 4.0, 0.5)), (6, 77.0, (1.5, 40, 3.0, 1.0)), (2, 5.0, (3.0, 8, 2.0, 1.0)),
    (64, 50000.0, (40.0, 4096, 32.0, 1.0)), (16, 10000.0, (16.0, 32, 32.0, 1.0)), (4, 10.0, (2.0, 100000, 1.0, 1.0))])
def test_rescaled_frequencies_against_plain(dims, base, scaling):
    """The package's frequencies against the plain ones; and by hand: pairs that turn faster than ``fast`` times in the
    original context keep their frequency, pairs slower than ``slow`` have it divided by the factor."""
    from llm_rs_b200.parts.latent_attention import rescaled_frequencies
    sc = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
    f, mag = rescaled_frequencies(dims, base, sc)
    pf, pmag = P.frequencies(dims, base, sc)
    assert torch.allclose(f, pf, rtol=1e-14, atol=0) and mag == pmag
    plain = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    if sc is None:
        assert torch.allclose(f, plain, rtol=1e-14) and mag == 1.0
        return
    assert abs(mag - (0.1 * math.log(sc["factor"]) + 1.0)) < 1e-15
    turns = plain * sc["original"] / (2 * math.pi)
    for i in range(dims // 2):
        lo = max(math.floor(dims * math.log(sc["original"] / (2 * math.pi * sc["fast"])) / (2 * math.log(base))), 0)
        hi = min(math.ceil(dims * math.log(sc["original"] / (2 * math.pi * sc["slow"])) / (2 * math.log(base))), dims - 1)
        if i <= lo:
            assert abs(float(f[i] / plain[i]) - 1.0) < 1e-12, (i, float(turns[i]))
        elif i >= hi and hi > lo:
            assert abs(float(f[i] / plain[i]) - 1.0 / sc["factor"]) < 1e-12
        else:
            assert 1.0 / sc["factor"] - 1e-12 <= float(f[i] / plain[i]) <= 1.0 + 1e-12


# ---- the plain implementation's own properties ------------------------------------------------------
def _random_mixer_weights(names_shapes, seed):
    g = torch.Generator().manual_seed(seed)
    return {n: torch.randn(shape, generator=g, dtype=F64) / math.sqrt(shape[-1]) for n, shape in names_shapes.items()}


def test_plain_window_sees_itself_and_the_tokens_before_it_only():
    m = {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 6, "scale": 0.4, "mask": {"size": 5}, "rot": {"base": 100.0, "dims": 4}}
    w = _random_mixer_weights({"m.q": (16, 12), "m.k": (8, 12), "m.v": (6, 12), "m.g": (2, 12), "m.o": (12, 12)}, 1)
    x = torch.randn(30, 12, generator=torch.Generator().manual_seed(2), dtype=F64)
    base = P.window_attention(x, m, w, "m.", 1e-6)
    other = x.clone()
    other[10] = 9.0 * torch.randn(12, generator=torch.Generator().manual_seed(3), dtype=F64)
    moved = (P.window_attention(other, m, w, "m.", 1e-6) - base).abs().amax(dim=1)
    assert bool((moved[:10] == 0).all()) and bool((moved[15:] == 0).all())      # 10 is seen by 10 .. 14
    assert bool((moved[10:15] > 1e-6).all())
    # A window of one key: every token sees itself only, so its row depends on nothing else.
    m1 = dict(m, mask={"size": 1})
    alone = torch.cat([P.window_attention(x[i:i + 1], dict(m1, rot=None), w, "m.", 1e-6) for i in range(4)])
    assert torch.allclose(P.window_attention(x[:4], dict(m1, rot=None), w, "m.", 1e-6), alone, atol=1e-12)


def test_plain_unit_norm_heads_forget_the_size_of_q_and_k_and_a_shut_gate_closes_a_head():
    m = {"heads": 2, "kv_heads": 2, "dim": 8, "vdim": 6, "scale": 0.4, "rot": {"base": 100.0, "dims": 8}}
    w = _random_mixer_weights({"m.q": (16, 12), "m.k": (16, 12), "m.v": (12, 12), "m.g": (2, 12), "m.o": (12, 12)}, 4)
    x = torch.randn(9, 12, generator=torch.Generator().manual_seed(5), dtype=F64)
    base = P.window_attention(x, m, w, "m.", 0.0)
    big = dict(w)
    big["m.q"], big["m.k"] = 7.0 * w["m.q"], 0.01 * w["m.k"]
    assert torch.allclose(P.window_attention(x, m, big, "m.", 0.0), base, atol=1e-10)
    # With head 1's gate row zeroed its gate is sigmoid(0) = 1/2 everywhere: that isolates the head's ungated output.
    shut = dict(w)
    shut["m.g"] = w["m.g"].clone()
    shut["m.g"][1] = 0.0
    half = P.window_attention(x, m, shut, "m.", 0.0)          # sigmoid(0) = 1/2 on head 1
    no_head = dict(w)
    no_head["m.o"] = w["m.o"].clone()
    no_head["m.o"][:, 6:] = 0.0
    only0 = P.window_attention(x, m, no_head, "m.", 0.0)
    gate1 = torch.sigmoid(x @ w["m.g"][1])
    # out = head0 + gate1 * head1' ; with the zeroed gate row: head0 + head1' / 2
    head1 = (half - only0) * 2.0
    assert torch.allclose(base, only0 + gate1[:, None] * head1, atol=1e-10)


def test_plain_pairings_and_magnitude():
    x = torch.zeros(1, 1, 8, dtype=F64)
    x[0, 0, 0] = 1.0
    pos = torch.tensor([3])
    near = P.rotate(x, pos, 4, 10.0, "neighbours")[0, 0]
    half = P.rotate(x, pos, 4, 10.0, "half")[0, 0]
    assert abs(float(near[0]) - math.cos(3.0)) < 1e-12 and abs(float(near[1]) - math.sin(3.0)) < 1e-12
    assert abs(float(half[0]) - math.cos(3.0)) < 1e-12 and abs(float(half[2]) - math.sin(3.0)) < 1e-12
    assert float(near[2:].abs().max()) == 0.0 and float(half[1]) == 0.0 and float(half[3:].abs().max()) == 0.0
    sc = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    scaled = P.rotate(x, pos, 4, 10.0, "neighbours", sc)[0, 0]
    assert abs(float(scaled[:2].norm()) - (0.1 * math.log(4.0) + 1.0)) < 1e-12      # cos and sin times the magnitude


def test_plain_correction_steers_the_choice_and_not_the_weight_and_identity_experts_return_their_input():
    f = {"kind": "moe", "expert": {"ff": 5}, "router": {"experts": 2, "top": 1, "identity": 1}}
    g = torch.Generator().manual_seed(6)
    w = {"f.router": torch.randn(3, 4, generator=g, dtype=F64), "f.correction": torch.zeros(3, dtype=F64)}
    for e in range(2):
        w.update({f"f.e{e}.gate": torch.randn(5, 4, generator=g, dtype=F64), f"f.e{e}.up": torch.randn(5, 4, generator=g, dtype=F64),
                  f"f.e{e}.down": torch.randn(4, 5, generator=g, dtype=F64)})
    h = torch.randn(6, 4, generator=g, dtype=F64)
    s = torch.softmax(h @ w["f.router"].T, dim=-1)
    w["f.correction"] = torch.tensor([0.0, 0.0, 2.0], dtype=F64)      # the identity expert wins everywhere
    chosen, weights = P.route(h, f, w, "f.")
    assert chosen.flatten().tolist() == [2] * 6 and torch.allclose(weights[:, 0], s[:, 2])
    assert torch.allclose(P.routed_experts(h, f, w, "f."), s[:, 2:3] * h)
    w["f.correction"] = torch.tensor([2.0, 0.0, 0.0], dtype=F64)
    assert torch.allclose(P.routed_experts(h, f, w, "f."), s[:, 0:1] * P.gated_unit(h, w, "f.e0."))


def test_plain_every_pass_of_a_loop_re_enters_through_the_embedding(tmp_path):
    cfg, w = P.load_model_dir(write_pozelix_model("E", str(tmp_path)))
    toks = list(range(3, 40))
    ref = P.forward(toks, cfg, w)
    once = json.loads(json.dumps(cfg))
    once["loop"]["times"] = 1
    assert float((P.forward(toks, once, w) - ref).abs().max()) > 1e-2
    blind = dict(w)
    blind["loop.in"] = w["loop.in"].clone()
    blind["loop.in"][:, cfg["width"]:] = 0.0
    assert float((P.forward(toks, cfg, blind) - ref).abs().max()) > 1e-2
    res = []
    P.forward(toks, cfg, w, res)
    assert len(res) == 6      # layer 0, four passes of layer 1, layer 2
