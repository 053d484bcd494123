"""Small Fekolorn configurations for the tests: they differ in every size and option (layer order, number of streams,
with and without the pair table, an embedding scale or none, grouped and single key heads, key and value widths that
differ, windows shorter and longer than a page and none, partial, full and no rotation, bias tables of few and many
rows whose reach is shorter or longer than the window, one, two and no layers with mixed values, convolutions of one to
five taps, layers without a feed-forward, sizes that are multiples of nothing useful)."""
import os

import torch


def _softmax(heads, kv_heads, dim, vdim, scale, window=0, bias=None, v_mix=False, rot=None, sink=True):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if bias:
        m["bias_rows"], m["bias_max"] = bias
    if v_mix:
        m["v_mix"] = True
    if rot:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    if not sink:
        m["sink"] = False
    return m


def _attention(*a, **k):
    return {"type": "attention", "mixer": _softmax(*a, **k)}


def _parallel(left, right, left_scale, right_scale):
    heads, kv_heads, dim, vdim, conv = right
    return {"type": "parallel", "mixer": {
        "left": left, "right": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
        "left_scale": left_scale, "right_scale": right_scale}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _layers(*pairs):
    return [{**mixer, "mlp": mlp} for mixer, mlp in pairs]


# Two streams; the recurrent side with grouped key heads and values narrower than keys; a window of 20 (longer than a
# page of 16) with a bias that reaches beyond it, then a window of 7 with a bias that ends inside it (every distance from
# 5 on in the last of six rows); three layers mix values (a source and two mixed), one of them inside a parallel mixer.
FEKOLORN_A = {
    "architecture": "Fekolorn", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "streams": 2,
    "embedding": {"scale": 0.7, "bigram": {"buckets": 101, "mul_prev": 13, "mul_cur": 5}},
    "layers": _layers(
        (_parallel(_softmax(4, 2, 16, 8, 0.3, rot=(10000.0, 8)), (4, 2, 16, 8, 4), 0.6, 1.2), _dense(80)),
        (_attention(4, 1, 16, 16, 0.25, window=20, bias=(8, 64), v_mix=True), _dense(48)),
        (_attention(2, 1, 24, 16, 0.2, window=7, bias=(6, 5), v_mix=True), None),
        (_parallel(_softmax(2, 1, 8, 16, 0.4, window=33, bias=(4, 40), v_mix=True, rot=(500.0, 8)), (2, 2, 8, 24, 2), 1.0,
                   0.5), _dense(64)))}

# Three streams; attention first: no window (every page stays) and a bias over hundreds of positions; no pair table and
# no embedding scale; the softmax side of the parallel mixer looks through a window while the recurrent side does not
# forget; an odd width; a layer without a feed-forward at the end.
FEKOLORN_B = {
    "architecture": "Fekolorn", "vocab": 157, "width": 72, "norm": {"eps": 1e-6}, "streams": 3,
    "layers": _layers(
        (_attention(3, 3, 8, 24, 0.35, bias=(10, 300)), _dense(50)),
        (_parallel(_softmax(6, 2, 12, 12, 0.28, window=24, rot=(77.0, 12)), (2, 2, 8, 24, 2), 0.9, 0.8), _dense(36)),
        (_attention(5, 1, 24, 8, 0.2, window=64, bias=(32, 48)), None))}

# Sizes at which the bfloat16 kernels take the tensor cores (multiples of 16 and 64); four streams; windows of 48 and
# 130; keys of 64 and 128 channels in the recurrence.
FEKOLORN_C = {
    "architecture": "Fekolorn", "vocab": 512, "width": 256, "norm": {"eps": 1e-6}, "streams": 4,
    "embedding": {"scale": 1.5, "bigram": {"buckets": 1024, "mul_prev": 1, "mul_cur": 3}},
    "layers": _layers(
        (_attention(4, 2, 64, 32, 0.11, window=48, bias=(18, 100), v_mix=True), _dense(256)),
        (_parallel(_softmax(6, 3, 96, 32, 0.1, rot=(1e6, 32)), (4, 2, 64, 64, 4), 0.75, 1.1), _dense(128)),
        (_attention(4, 2, 32, 32, 0.17, window=130, bias=(20, 130), v_mix=True), _dense(256)),
        (_parallel(_softmax(4, 4, 128, 128, 0.09, rot=(1e4, 128)), (2, 1, 128, 32, 3), 1.1, 0.7), _dense(64)))}

# ONE stream with learned connections; a convolution of one tap (no rows to carry); a softmax side without a sink and
# with a full rotation; a single layer with v_mix (a source nobody reads); three value heads over one key head; sizes
# that are multiples of nothing (width 100, heads of 12 x 20, a vocabulary of 61); a pair table of ONE bucket.
FEKOLORN_D = {
    "architecture": "Fekolorn", "vocab": 61, "width": 100, "norm": {"eps": 1e-6}, "streams": 1,
    "embedding": {"scale": 1.0, "bigram": {"buckets": 1, "mul_prev": 7, "mul_cur": 7}},
    "layers": _layers(
        (_parallel(_softmax(3, 3, 12, 20, 0.33, rot=(300.0, 12), sink=False), (3, 1, 12, 20, 1), 1.0, 1.0), _dense(36)),
        (_attention(2, 2, 20, 12, 0.25, window=50, bias=(3, 9), v_mix=True), _dense(28)),
        (_parallel(_softmax(1, 1, 40, 6, 0.2), (1, 1, 20, 12, 5), 0.5, 2.0), None))}

# No hyper-connection tensors at all (plain residual sums); a window of ONE position; a bias of two rows; windows
# only in the attention layers, five streams' worth of nothing; a convolution of five taps, longer than most portions.
FEKOLORN_E = {
    "architecture": "Fekolorn", "vocab": 130, "width": 48, "norm": {"eps": 1e-5},
    "embedding": {"scale": 2.0, "bigram": {"buckets": 37, "mul_prev": 2, "mul_cur": 0}},
    "layers": _layers(
        (_attention(2, 2, 16, 16, 0.3, window=1, bias=(2, 3)), _dense(64)),
        (_parallel(_softmax(4, 1, 16, 8, 0.3, rot=(1e5, 4)), (4, 4, 32, 16, 5), 0.7, 0.7), _dense(32)),
        (_attention(6, 3, 8, 8, 0.4, window=5, bias=(9, 4.5)), _dense(48)))}

# Five streams and windows only beside the recurrence: every page comes back as the windows pass.
FEKOLORN_F = {
    "architecture": "Fekolorn", "vocab": 97, "width": 40, "norm": {"eps": 1e-6}, "streams": 5,
    "embedding": {"bigram": {"buckets": 53, "mul_prev": 3, "mul_cur": 11}},
    "layers": _layers(
        (_parallel(_softmax(2, 2, 16, 16, 0.25, window=33, rot=(1e4, 16)), (2, 1, 16, 12, 3), 0.8, 0.8), _dense(40)),
        (_attention(4, 2, 8, 12, 0.35, window=9, bias=(12, 200), v_mix=True), _dense(24)),
        (_attention(2, 2, 16, 12, 0.25, window=40, v_mix=True), None))}

# name -> (config.json, seed, sigma of matrices, page size)
FEKOLORN = {"A": (FEKOLORN_A, 3, 0.15, 16), "B": (FEKOLORN_B, 4, 0.15, 8), "C": (FEKOLORN_C, 5, 0.06, 16),
            "D": (FEKOLORN_D, 6, 0.12, 16), "E": (FEKOLORN_E, 7, 0.15, 16), "F": (FEKOLORN_F, 8, 0.2, 32)}


def write_fekolorn_model(name: str, folder: str, dtype=torch.bfloat16) -> str:
    """Write a small Fekolorn folder with random weights; returns its path. Tensors whose random default would hide
    their mechanism are drawn larger: sinks and distance biases of the size of the scores, value-mixing weights between
    a quarter and three quarters, connection weights that differ from stream to stream, decays that forget within tens
    of tokens."""
    import json

    from llm_rs_b200.config import FekolornConfig, resolve_architecture
    from llm_rs_b200.parts import DecoderModel
    from llm_rs_b200.weights.random_init import random_tensors
    from llm_rs_b200.weights.safetensors_io import save_file
    raw, seed, sigma, _ = FEKOLORN[name]
    cfg = FekolornConfig.from_dict(raw)
    path = os.path.join(folder, f"fekolorn_{name}")
    model = DecoderModel(resolve_architecture(raw).build_spec(cfg))
    tensors = random_tensors(model.weight_specs(), seed, sigma, 0.3, dtype, "cpu")
    g = torch.Generator().manual_seed(1000 + seed)
    for key, t in tensors.items():
        if key.endswith(".sink") or key.endswith(".rel"):
            tensors[key] = torch.randn(t.shape, generator=g).to(dtype)
        elif key.endswith(".vmix"):
            tensors[key] = (0.25 + 0.5 * torch.rand(t.shape, generator=g)).to(dtype)
        elif key.endswith(".A_log") or key.endswith(".dt_bias"):
            tensors[key] = (torch.randn(t.shape, generator=g) - 1.0).to(dtype)
        elif key in ("embed", "bigram"):
            tensors[key] = torch.randn(t.shape, generator=g).to(dtype)
        elif ".hc" in key and key.endswith("in"):
            tensors[key] = (1.0 / t.numel() + 0.3 * torch.randn(t.shape, generator=g)).to(t.dtype)
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f, indent=2)
    save_file(tensors, os.path.join(path, "model.safetensors"))
    return path
