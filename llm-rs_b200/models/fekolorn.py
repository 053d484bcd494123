"""The Fekolorn design as a ``ModelSpec``.

Every layer is a ``hyper`` block (several residual streams; a sublayer reads a weighted sum of them through a norm with
one number as weight and writes back through a learned mix) around one of two mixers: ``parallel`` (softmax attention
with a partial rotation, values of unit root mean square and a sink, beside a gated delta rule behind short
convolutions; a weighted sum of the two) or ``scored_attention`` with norms over the whole q and k rows, no rotation,
a learned bias per distance bucket, a sliding window, a sink, and values mixed with those of the first such layer. The
feed-forward is dense with the PolyNorm activation, or absent. The embedding has a scale and a hashed table of token
pairs.

The constants the design fixes are given to the parts here: the 1e-6 under the root of the recurrent side's unit
vectors, its query scale dim^-1/2, which norms each softmax mixer has.
"""
from __future__ import annotations

from ..config import ArchitectureEntry, register_architecture
from ..config.fekolorn import FekolornConfig, ParallelMixer, SoftmaxMixer
from ..parts import LayerSpec, ModelSpec, PartSpec, RunStep

EMBEDDING, PAIRS, FINAL_NORM, HEAD = "embed", "bigram", "final.norm", "head"
MIXER_SCOPE, FEED_FORWARD_SCOPE = "mix.", "mlp."
HYPER_SCOPES = ("hc1.", "hc2.")
UNIT_KEY_EPS = 1e-6
V_FIRST = "fekolorn.v_first"
# No key of the configuration bounds a sequence; a layer that keeps every key bounds it by the pool.
MAX_POSITIONS = 1 << 30


def _softmax(m: SoftmaxMixer, D: int, eps: float, own_norms: bool, v_mix: str) -> PartSpec:
    """``own_norms``: the mixer that stands alone norms its whole q and k rows; the one beside the delta rule norms its
    values per head instead."""
    return PartSpec("scored_attention", {
        "hidden_size": D, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
        "sink": m.sink, "mask": "window" if m.window else "causal", "mask_size": m.window,
        "qk_norm": "whole" if own_norms else "none", "v_norm": "none" if own_norms else "head_unit", "norm_eps": eps,
        "rot_dims": m.rot_dims, "rot_base": m.rot_base, "bias_rows": m.bias_rows, "bias_max": m.bias_max,
        "v_mix": v_mix, "v_mix_key": V_FIRST})


def build_spec(cfg: FekolornConfig) -> ModelSpec:
    D, eps = cfg.width, cfg.norm_eps
    streams = cfg.streams if cfg.hyper else 1
    norm = lambda name: PartSpec("rmsnorm", {"dim": D, "eps": eps, "name": name, "scalar": True})
    layers, order = [], []
    seen_v_mix = False
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer

        def v_mix_of(sm: SoftmaxMixer) -> str:
            nonlocal seen_v_mix
            if not sm.v_mix:
                return "none"
            kind = "mixed" if seen_v_mix else "source"
            seen_v_mix = True
            return kind
        if isinstance(m, ParallelMixer):
            r = m.right
            right = PartSpec("gated_delta", {"hidden_size": D, "n_heads": r.heads, "n_kv_heads": r.kv_heads, "dim": r.dim,
                                             "vdim": r.vdim, "conv": r.conv, "norm_eps": eps, "key_eps": UNIT_KEY_EPS,
                                             "q_scale": r.dim ** -0.5})
            mixer = PartSpec("parallel", {"left": _softmax(m.left, D, eps, False, v_mix_of(m.left)), "right": right,
                                          "left_scale": m.left_scale, "right_scale": m.right_scale})
        else:
            assert isinstance(m, SoftmaxMixer)
            mixer = _softmax(m, D, eps, True, v_mix_of(m))
        ffn = None
        if layer.mlp is not None:
            ffn = PartSpec("dense", {"hidden_size": D, "intermediate_size": layer.mlp.ff, "activation": "polynorm",
                                     "act_eps": eps})
        layers.append(LayerSpec(
            prefix=f"l{i}.", block=PartSpec("hyper", {"streams": streams, "names": HYPER_SCOPES, "learned": cfg.hyper}),
            mixer=mixer, feed_forward=ffn, mixer_norm=norm("norm1"),
            feed_forward_norm=norm("norm2") if ffn is not None else None,
            mixer_scope=MIXER_SCOPE, feed_forward_scope=FEED_FORWARD_SCOPE))
        order.append(RunStep(i))
    p = cfg.pairs
    return ModelSpec(
        hidden_size=D, vocab_size=cfg.vocab, layers=tuple(layers), run_order=tuple(order),
        embedding=PartSpec("pair_embedding", {
            "vocab_size": cfg.vocab, "hidden_size": D, "scale": cfg.embedding_scale, "streams": streams,
            "buckets": p.buckets if p else 0, "mul_prev": p.mul_prev if p else 0, "mul_cur": p.mul_cur if p else 0,
            "name": EMBEDDING, "pairs_name": PAIRS}),
        final_norm=PartSpec("rmsnorm", {"dim": D, "eps": eps, "name": FINAL_NORM, "scalar": True}),
        lm_head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": D, "name": HEAD}),
        max_positions=MAX_POSITIONS, eos_token_ids=())


register_architecture(ArchitectureEntry(
    name=FekolornConfig.architecture, model_type=FekolornConfig.model_type,
    config_cls=FekolornConfig, build_spec=build_spec), replace=True)
