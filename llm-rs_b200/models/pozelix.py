"""The Pozelix design as a ``ModelSpec``.

Every layer is a ``sandwich`` block (a norm ahead of each branch and one on its output) around one of two mixers:
``scored_attention`` with a sliding window, rotation by halves, unit-norm heads after the rotation and a sigmoid gate
per head, or ``latent_attention`` with queries through a latent of their own, rotation of neighbouring pairs and
rescaled frequencies, every earlier token visible unless the layer names a window, no gate. The feed-forward is the gated SiLU unit, dense or as routed
experts whose router scores all experts by a softmax, chooses by score plus a stored correction and may name identity
experts. A stretch of layers may run several times with the same weights: every pass has run-order entries (so pages)
of its own and starts by mixing the stream with the embedding output (``embedding_mix``).

What the design fixes is given to the parts here: which pairing and norm each mixer uses, the experts' plain SiLU
unit, the tensor names.
"""
from __future__ import annotations

from ..config import ArchitectureEntry, register_architecture
from ..config.pozelix import DenseMLP, LatentMixer, PozelixConfig, WindowMixer
from ..parts import LayerSpec, ModelSpec, PartSpec, RunStep

EMBEDDING, FINAL_NORM, HEAD, LOOP_IN = "embed", "final.norm", "head", "loop.in"
MIXER_SCOPE, FEED_FORWARD_SCOPE = "mix.", "mlp."
OUT_NORMS = ("norm1b", "norm2b")
DENSE_NAMES = {"gate": "gate", "up": "up", "down": "down"}
# No key of the configuration bounds a sequence; a layer that keeps every key bounds it by the pool.
MAX_POSITIONS = 1 << 30


def run_order(cfg: PozelixConfig):
    """The layers in the order they run; the first entry of every pass over the looped stretch re-enters."""
    n = len(cfg.layers)
    if cfg.loop is None:
        return tuple(RunStep(i) for i in range(n))
    a, b = cfg.loop.start, cfg.loop.stop
    order = [RunStep(i) for i in range(a)]
    for _ in range(cfg.loop.times):
        order += [RunStep(i, reenter=(i == a)) for i in range(a, b)]
    return tuple(order + [RunStep(i) for i in range(b, n)])


def build_spec(cfg: PozelixConfig) -> ModelSpec:
    D = cfg.width
    norm = lambda name: PartSpec("rmsnorm", {"dim": D, "eps": cfg.norm_eps, "name": name})
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if isinstance(m, WindowMixer):
            mixer = PartSpec("scored_attention", {
                "hidden_size": D, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim,
                "scale": m.scale, "mask": "window" if m.window else "causal", "mask_size": m.window,
                "qk_norm": "head_unit", "norm_eps": cfg.norm_eps, "rot_dims": m.rot_dims, "rot_base": m.rot_base,
                "gated": True})
        else:
            assert isinstance(m, LatentMixer)
            mixer = PartSpec("latent_attention", {
                "hidden_size": D, "n_heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim,
                "rank": m.kv_rank, "q_rank": m.q_rank, "scale": m.scale, "rot_base": m.rot_base,
                "rot_dims": m.rot_dims, "rot_pairing": "neighbours",
                "rot_scaling": None if m.scaling is None else m.scaling.to_dict(), "window": m.window,
                "norm_eps": cfg.norm_eps, "gated": False})
        f, ffn = layer.mlp, None
        if isinstance(f, DenseMLP):
            ffn = PartSpec("swiglu", {"hidden_size": D, "intermediate_size": f.ff, "names": DENSE_NAMES,
                                      "suffix": ""})
        elif f is not None:
            ffn = PartSpec("moe", {"hidden_size": D, "expert_size": f.ff, "n_experts": f.experts, "top": f.top,
                                   "router": "softmax_bias", "n_identity": f.identity, "limit": None, "alpha": 1.0,
                                   "up_shift": 0.0})
        layers.append(LayerSpec(
            prefix=f"l{i}.", block=PartSpec("sandwich", {"out_norms": OUT_NORMS}),
            mixer=mixer, feed_forward=ffn, mixer_norm=norm("norm1"),
            feed_forward_norm=norm("norm2") if ffn is not None else None,
            mixer_scope=MIXER_SCOPE, feed_forward_scope=FEED_FORWARD_SCOPE))
    return ModelSpec(
        hidden_size=D, vocab_size=cfg.vocab, layers=tuple(layers), run_order=run_order(cfg),
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": D, "name": EMBEDDING}),
        final_norm=PartSpec("rmsnorm", {"dim": D, "eps": cfg.norm_eps, "name": FINAL_NORM}),
        lm_head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": D, "name": HEAD}),
        reentry=PartSpec("embedding_mix", {"hidden_size": D, "name": LOOP_IN}) if cfg.loop is not None else None,
        max_positions=MAX_POSITIONS, eos_token_ids=())


register_architecture(ArchitectureEntry(
    name=PozelixConfig.architecture, model_type=PozelixConfig.model_type,
    config_cls=PozelixConfig, build_spec=build_spec), replace=True)
