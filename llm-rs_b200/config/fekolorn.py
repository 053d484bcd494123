"""Typed configuration of the Fekolorn design, read from its own config.json keys.

A Fekolorn model is a list of pre-norm layers over several residual streams (hyper-connections), each layer with one of
two mixers and a dense feed-forward (or none), behind an embedding with a scale and a hashed table of token pairs:

    {"architecture": "Fekolorn", "vocab": V, "width": D, "norm": {"eps": e}, "streams": S,
     "embedding": {"scale": s, "bigram": {"buckets": B, "mul_prev": a, "mul_cur": b}},
     "layers": [{"type": "parallel" | "attention", "mixer": {...}, "mlp": {"kind": "dense", "ff": F} | null}, ...]}

    attention mixer  heads, kv_heads, dim, vdim, scale, mask.size (optional: a sliding window), bias_max (optional: a
                     learned bias per distance bucket, reaching to that distance; the table's rows are the tensor's),
                     v_mix (optional: values mixed with those of the first such layer), rot.base / rot.dims (optional)
    parallel mixer   left: an attention mixer's keys; right: heads, kv_heads, dim, vdim, conv (taps); left_scale,
                     right_scale

Optional keys that are absent switch their mechanism off. Whether a softmax mixer has a sink, whether the layers carry
hyper-connection tensors and how many rows a bias table has is read from the folder's tensors when they are at hand;
without them (a configuration made in memory) the keys ``streams`` and ``bias_rows`` say so. Constants the design fixes
live with the parts (``models/fekolorn.py`` passes them as parameters).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .errors import ConfigError
from .rusadra import _get

MIXERS = ("parallel", "attention")


@dataclass(frozen=True)
class SoftmaxMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int = 0          # mask.size; 0 (no mask key): every earlier token is seen
    bias_max: float = 0.0    # 0 (no key): no distance bias
    bias_rows: int = 0
    v_mix: bool = False
    rot_base: float = 1.0
    rot_dims: int = 0        # 0 (no rot key): no rotation
    sink: bool = True

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                             "scale": self.scale}
        if self.window:
            d["mask"] = {"size": self.window}
        if self.bias_rows:
            d["bias_max"] = self.bias_max
            d["bias_rows"] = self.bias_rows
        if self.v_mix:
            d["v_mix"] = True
        if self.rot_dims:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        if not self.sink:
            d["sink"] = False
        return d


@dataclass(frozen=True)
class RecurrentMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}


@dataclass(frozen=True)
class ParallelMixer:
    left: SoftmaxMixer
    right: RecurrentMixer
    left_scale: float
    right_scale: float

    def to_dict(self) -> Dict[str, Any]:
        return {"left": self.left.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale,
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class DenseMLP:
    ff: int

    def to_dict(self) -> Dict[str, Any]:
        return {"kind": "dense", "ff": self.ff}


@dataclass(frozen=True)
class FekolornLayer:
    type: str
    mixer: Any                    # ParallelMixer or SoftmaxMixer
    mlp: Optional[DenseMLP]


@dataclass(frozen=True)
class PairTable:
    buckets: int
    mul_prev: int
    mul_cur: int

    def to_dict(self) -> Dict[str, Any]:
        return {"buckets": self.buckets, "mul_prev": self.mul_prev, "mul_cur": self.mul_cur}


def _softmax_mixer(m: Mapping, where: str, rel_rows: Optional[int], has_sink: Optional[bool]) -> SoftmaxMixer:
    heads, dim = _get(m, "heads", int, where, 1), _get(m, "dim", int, where, 1)
    kv_heads = _get(m, "kv_heads", int, where, 1, optional=True) or heads
    if heads % kv_heads:
        raise ConfigError(f"{where}: {heads} heads are no multiple of {kv_heads} kv_heads")
    rot_dims = _get(m, "rot.dims", int, where, 0, optional=True) or 0
    if rot_dims % 2 or rot_dims > dim:
        raise ConfigError(f"{where}: rot.dims {rot_dims} must be even and at most dim {dim}")
    bias_max = _get(m, "bias_max", float, where, optional=True) or 0.0
    rows = 0
    if bias_max:
        rows = rel_rows if rel_rows is not None else (_get(m, "bias_rows", int, where, 2, optional=True) or 0)
        if rows < 2 or bias_max <= rows // 2:
            raise ConfigError(f"{where}: a distance bias reaching to {bias_max} needs a table of at least 2 rows "
                              f"(got {rows}) and a reach beyond half of them")
    v_mix = m.get("v_mix", False)
    if not isinstance(v_mix, bool):
        raise ConfigError(f"{where}: v_mix must be true or false, got {v_mix!r}")
    return SoftmaxMixer(
        heads=heads, kv_heads=kv_heads, dim=dim, vdim=_get(m, "vdim", int, where, 1, optional=True) or dim,
        scale=_get(m, "scale", float, where), window=_get(m, "mask.size", int, where, 1, optional=True) or 0,
        bias_max=float(bias_max), bias_rows=rows, v_mix=v_mix,
        rot_base=(_get(m, "rot.base", float, where) if rot_dims else 1.0), rot_dims=rot_dims,
        sink=has_sink if has_sink is not None else bool(m.get("sink", True)))


@dataclass(frozen=True)
class FekolornConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[FekolornLayer, ...]
    streams: int = 1
    hyper: bool = True            # the layers carry hyper-connection tensors (else: one stream, plain residual sums)
    embedding_scale: float = 1.0
    pairs: Optional[PairTable] = None
    torch_dtype: str = "bfloat16"

    architecture = "Fekolorn"
    model_type = "fekolorn"
    wants_tensor_shapes = True      # ``load_config`` passes the folder's tensor shapes to ``from_dict``

    @classmethod
    def from_dict(cls, raw: Dict[str, Any], tensor_shapes: Optional[Mapping[str, Tuple[int, ...]]] = None):
        vocab = _get(raw, "vocab", int, "config", 1)
        width = _get(raw, "width", int, "config", 1)
        eps = _get(raw, "norm.eps", float, "config", 0.0)
        streams = _get(raw, "streams", int, "config", 1, optional=True)
        scale = _get(raw, "embedding.scale", float, "config", optional=True)
        pairs = None
        if isinstance(raw.get("embedding"), Mapping) and raw["embedding"].get("bigram") is not None:
            b = raw["embedding"]["bigram"]
            pairs = PairTable(_get(b, "buckets", int, "embedding.bigram", 1), _get(b, "mul_prev", int, "embedding.bigram", 0),
                              _get(b, "mul_cur", int, "embedding.bigram", 0))
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config: layers must be a non-empty list")
        shapes = tensor_shapes
        has = (lambda name: name in shapes) if shapes is not None else None
        rows_of = (lambda name: (shapes[name][0] if name in shapes and len(shapes[name]) == 2 else 0)) \
            if shapes is not None else (lambda name: None)
        layers = []
        for i, lr in enumerate(layers_raw):
            where = f"layers[{i}]"
            if not isinstance(lr, Mapping) or lr.get("type") not in MIXERS:
                raise ConfigError(f"{where}: type must be one of {MIXERS}, got "
                                  f"{lr.get('type') if isinstance(lr, Mapping) else lr!r}")
            m = lr.get("mixer")
            if not isinstance(m, Mapping):
                raise ConfigError(f"{where}: mixer missing from config")
            if lr["type"] == "attention":
                mixer = _softmax_mixer(m, where, rows_of(f"l{i}.mix.rel"), has(f"l{i}.mix.sink") if has else None)
            else:
                left, right = m.get("left"), m.get("right")
                if not isinstance(left, Mapping) or not isinstance(right, Mapping):
                    raise ConfigError(f"{where}: a parallel mixer needs left and right")
                rw = where + ".right"
                heads = _get(right, "heads", int, rw, 1)
                kv_heads = _get(right, "kv_heads", int, rw, 1, optional=True) or heads
                if heads % kv_heads:
                    raise ConfigError(f"{rw}: {heads} heads are no multiple of {kv_heads} kv_heads")
                dim = _get(right, "dim", int, rw, 1)
                mixer = ParallelMixer(
                    left=_softmax_mixer(left, where + ".left", rows_of(f"l{i}.mix.left.rel"),
                                        has(f"l{i}.mix.left.sink") if has else None),
                    right=RecurrentMixer(heads, kv_heads, dim, _get(right, "vdim", int, rw, 1, optional=True) or dim,
                                         _get(right, "conv", int, rw, 1)),
                    left_scale=_get(m, "left_scale", float, where, optional=True) if "left_scale" in m else 1.0,
                    right_scale=_get(m, "right_scale", float, where, optional=True) if "right_scale" in m else 1.0)
            mlp_raw, mlp = lr.get("mlp"), None
            if mlp_raw is not None:
                if not isinstance(mlp_raw, Mapping) or mlp_raw.get("kind") != "dense":
                    raise ConfigError(f"{where}: mlp.kind must be 'dense' (or mlp null)")
                mlp = DenseMLP(_get(mlp_raw, "ff", int, where, 1))
            layers.append(FekolornLayer(lr["type"], mixer, mlp))
        # Layers whose values are mixed must agree on the values' shape with the first of them.
        softmax = [l.mixer if isinstance(l.mixer, SoftmaxMixer) else l.mixer.left for l in layers]
        mixed = [m for m in softmax if m.v_mix]
        for m in mixed[1:]:
            if (m.kv_heads, m.vdim) != (mixed[0].kv_heads, mixed[0].vdim):
                raise ConfigError("config: layers with v_mix must have the first such layer's kv_heads and vdim")
        hyper = has("l0.hc1.in") if has else streams is not None
        return cls(vocab=vocab, width=width, norm_eps=eps, layers=tuple(layers), streams=streams or 1, hyper=bool(hyper),
                   embedding_scale=1.0 if scale is None else scale, pairs=pairs,
                   torch_dtype=str(raw.get("torch_dtype", "bfloat16")))

    def to_dict(self) -> Dict[str, Any]:
        emb: Dict[str, Any] = {"scale": self.embedding_scale}
        if self.pairs is not None:
            emb["bigram"] = self.pairs.to_dict()
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "embedding": emb,
             "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict()}
                        for l in self.layers]}
        if self.hyper:
            d["streams"] = self.streams
        return d
