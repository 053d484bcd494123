"""Small Pozelix configurations for the tests: they differ in every size and option (layer order, grouped and single
key heads, key and value widths that differ, windows shorter and longer than a page, of one key and none at all, partial,
full and no rotation, latents of the queries and of the keys of unequal size, rotated parts of 2 to 32 entries, rescaled
frequencies or not, dense / routed / no feed-forward, identity experts or none, one expert or all per token, a looped
stretch at the start, in the middle, over all layers, of one layer, and no loop; sizes that are multiples of nothing)."""
import os

import torch


def _window(heads, kv_heads, dim, vdim, scale, window=0, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return {"type": "attention", "mixer": m}


def _latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, scaling=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                      "scale": scale, "rot": rot}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, top, identity=0):
    router = {"experts": experts, "top": top}
    if identity:
        router["identity"] = identity
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def _layers(*pairs):
    return [{**mixer, "mlp": mlp} for mixer, mlp in pairs]


# Latent first; a latent of 40 (no tensor-core kernel is built for it); frequencies rescaled by 4 for an original
# context of 64; a window of 20 over pages of 16; grouped key heads (4 over 2); rotation of 8 of 16 channels; an
# attention layer without a mask and without a feed-forward; layers 1 and 2 run three times.
POZELIX_A = {
    "architecture": "Pozelix", "vocab": 211, "width": 64, "norm": {"eps": 1e-5},
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": _layers(
        (_latent(3, 16, 8, 24, 40, 24, 0.2, 1000.0, (4.0, 64, 8.0, 1.0)), _dense(80)),
        (_window(4, 2, 16, 32, 0.3, window=20, rot=(10000.0, 8)), _moe(40, 4, 2, identity=1)),
        (_window(4, 4, 8, 8, 0.5), None),
        (_latent(2, 24, 4, 8, 32, 48, 0.15, 500.0), _moe(24, 3, 3)))}

# Attention first; one key head for five query heads; a window of 7 (shorter than a page of 8) and a window of ONE key;
# a rotated part of 2 entries; more identity experts than real ones with every output chosen; one expert of five in the
# last layer (a pick that rounding turns then moves that token's logits only, not every later one's); no loop.
POZELIX_B = {
    "architecture": "Pozelix", "vocab": 157, "width": 72, "norm": {"eps": 1e-6},
    "layers": _layers(
        (_window(5, 1, 24, 8, 0.25, window=7, rot=(500.0, 24)), _moe(30, 2, 5, identity=3)),
        (_latent(2, 8, 2, 40, 64, 8, 0.3, 10000.0), _dense(50)),
        (_window(2, 2, 8, 40, 0.4, window=1), _moe(56, 5, 1)))}

# Sizes at which the bfloat16 engine's kernels take the tensor cores (multiples of 16 and 64): latents of 128 and 64,
# heads of 64 and 128, windows of 48 and 130, eight experts; the first two layers run twice.
POZELIX_C = {
    "architecture": "Pozelix", "vocab": 512, "width": 256, "norm": {"eps": 1e-6},
    "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": _layers(
        (_latent(4, 64, 32, 64, 128, 96, 0.1, 10000.0, (8.0, 128, 16.0, 2.0)), _moe(128, 8, 3, identity=2)),
        (_window(8, 2, 64, 64, 0.125, window=48, rot=(1e6, 32)), _dense(256)),
        (_window(4, 4, 128, 128, 0.09, window=130, rot=(1e4, 128)), _moe(64, 8, 2)),
        (_latent(8, 32, 16, 32, 64, 64, 0.12, 50000.0), _dense(128)))}

# Latent layers only (every page stays); the loop covers all layers; one layer without a feed-forward; one identity
# expert beside two real ones with one chosen; a rotation whose every pair is rescaled.
POZELIX_D = {
    "architecture": "Pozelix", "vocab": 97, "width": 48, "norm": {"eps": 1e-6},
    "loop": {"start": 0, "stop": 3, "times": 2},
    "layers": _layers(
        (_latent(1, 18, 10, 10, 20, 12, 0.2, 100.0, (2.0, 16, 4.0, 0.5)), _moe(32, 2, 1, identity=1)),
        (_latent(3, 10, 6, 7, 48, 30, 0.3, 3000.0), None),
        (_latent(2, 32, 16, 40, 16, 64, 0.1, 10000.0, (16.0, 32, 32.0, 1.0)), _dense(30)))}

# Windows only: every page comes back as the windows pass, so a request runs far beyond the pool. A window of 33 over
# pages of 32, a window of 5; a loop of ONE layer that runs four times.
POZELIX_E = {
    "architecture": "Pozelix", "vocab": 130, "width": 64, "norm": {"eps": 1e-5},
    "loop": {"start": 1, "stop": 2, "times": 4},
    "layers": _layers(
        (_window(4, 4, 16, 16, 0.3, window=33, rot=(1e5, 16)), _dense(64)),
        (_window(6, 3, 16, 16, 0.3, window=5, rot=(300.0, 4)), _moe(32, 4, 2, identity=2)),
        (_window(2, 1, 32, 16, 0.2, window=64), _dense(48)))}

# Sizes that are multiples of nothing: a width of 100, heads of 12 x 20, a latent of 36 with a rotated part of 6, a
# window of 50, rotation of 2 channels, every expert chosen (5 of 5), a vocabulary of 61; a loop that runs once.
POZELIX_F = {
    "architecture": "Pozelix", "vocab": 61, "width": 100, "norm": {"eps": 1e-6},
    "loop": {"start": 2, "stop": 4, "times": 1},
    "layers": _layers(
        (_window(3, 3, 12, 20, 0.33, window=50, rot=(77.0, 2)), _moe(28, 5, 5)),
        (_latent(5, 12, 6, 20, 36, 20, 0.25, 77.0, (1.5, 40, 3.0, 1.0)), _dense(36)),
        (_window(8, 2, 80, 48, 0.1, window=64, rot=(1e4, 80)), None),
        (_latent(2, 20, 12, 12, 100, 50, 0.2, 1e4), _moe(20, 2, 1, identity=1)))}

# name -> (config.json, seed, sigma of matrices, page size)
POZELIX = {"A": (POZELIX_A, 3, 0.15, 16), "B": (POZELIX_B, 4, 0.15, 8), "C": (POZELIX_C, 5, 0.06, 16),
           "D": (POZELIX_D, 6, 0.2, 16), "E": (POZELIX_E, 7, 0.15, 32), "F": (POZELIX_F, 8, 0.12, 16)}


def write_pozelix_model(name: str, folder: str, dtype=torch.bfloat16) -> str:
    """Write a small Pozelix folder with random weights; returns its path. The routers' corrections are drawn of the
    size of the scores' differences, so that both the scores and the corrections decide the choice."""
    import json

    from llm_rs_b200.config import PozelixConfig, resolve_architecture
    from llm_rs_b200.parts import DecoderModel
    from llm_rs_b200.weights.random_init import random_tensors
    from llm_rs_b200.weights.safetensors_io import save_file
    raw, seed, sigma, _ = POZELIX[name]
    cfg = PozelixConfig.from_dict(raw)
    path = os.path.join(folder, f"pozelix_{name}")
    model = DecoderModel(resolve_architecture(raw).build_spec(cfg))
    tensors = random_tensors(model.weight_specs(), seed, sigma, 0.2, dtype, "cpu")
    for key in tensors:
        if key.endswith(".correction"):
            tensors[key] = (tensors[key].float() * 0.3).to(dtype)
        if key.endswith(".router"):
            tensors[key] = (tensors[key].float() * 4.0).to(dtype)
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f, indent=2)
    save_file(tensors, os.path.join(path, "model.safetensors"))
    return path
