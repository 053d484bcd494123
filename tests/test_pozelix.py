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
