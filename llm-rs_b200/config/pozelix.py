"""Typed configuration of the Pozelix design, read from its own config.json keys.

A Pozelix model is a list of layers, each with one of two mixers and a dense or mixture-of-experts feed-forward (or
none), every branch between two norms; a stretch of the layers may run several times in a row with the same weights:

    {"architecture": "Pozelix", "vocab": V, "width": D, "norm": {"eps": e},
     "loop": {"start": a, "stop": b, "times": n},                                   (optional)
     "layers": [{"type": "attention" | "latent_attention", "mixer": {...}, "mlp": {...} | null}, ...]}

    attention mixer:         heads, kv_heads, dim, vdim, scale, mask.size (optional: a sliding window),
                             rot.base, rot.dims (optional: no rotation without them)
    latent_attention mixer:  heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot.base, rot.dims,
                             rot.scaling {factor, original, fast, slow} (optional), mask.size (optional)
    mlp:                     kind "dense": ff
                             kind "moe":   expert.ff, router.experts, router.top, router.identity (optional)

Every size and constant that may differ between models comes from here; what the design fixes lives with the parts
(``models/pozelix.py`` passes it as parameters).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .errors import ConfigError
from .rusadra import _get

MIXERS = ("attention", "latent_attention")


@dataclass(frozen=True)
class RotScaling:
    factor: float
    original: float
    fast: float
    slow: float

    def to_dict(self) -> Dict[str, Any]:
        return {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}


@dataclass(frozen=True)
class WindowMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int          # mask.size: a token sees itself and the window - 1 before it; 0 (no mask key): all before it
    rot_base: float
    rot_dims: int        # 0: no rotation

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                             "scale": self.scale}
        if self.window:
            d["mask"] = {"size": self.window}
        if self.rot_dims:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        return d


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    scaling: Optional[RotScaling] = None
    window: int = 0      # mask.size, as in the other mixer; 0 (no mask key): every earlier token is seen

    def to_dict(self) -> Dict[str, Any]:
        rot: Dict[str, Any] = {"base": self.rot_base, "dims": self.rot_dims}
        if self.scaling is not None:
            rot["scaling"] = self.scaling.to_dict()
        d = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
             "kv_rank": self.kv_rank, "q_rank": self.q_rank, "scale": self.scale, "rot": rot}
        if self.window:
            d["mask"] = {"size": self.window}
        return d


@dataclass(frozen=True)
class DenseMLP:
    ff: int

    def to_dict(self) -> Dict[str, Any]:
        return {"kind": "dense", "ff": self.ff}


@dataclass(frozen=True)
class MoEMLP:
    ff: int
    experts: int         # experts with weights
    top: int
    identity: int = 0    # further router outputs whose expert returns its input

    def to_dict(self) -> Dict[str, Any]:
        router: Dict[str, Any] = {"experts": self.experts, "top": self.top}
        if self.identity:
            router["identity"] = self.identity
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": router}


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int

    def to_dict(self) -> Dict[str, Any]:
        return {"start": self.start, "stop": self.stop, "times": self.times}


@dataclass(frozen=True)
class PozelixLayer:
    type: str
    mixer: Any
    mlp: Any             # DenseMLP, MoEMLP or None


@dataclass(frozen=True)
class PozelixConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[PozelixLayer, ...]
    loop: Optional[Loop] = None
    torch_dtype: str = "bfloat16"

    architecture = "Pozelix"
    model_type = "pozelix"

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "PozelixConfig":
        vocab = _get(raw, "vocab", int, "config", 1)
        width = _get(raw, "width", int, "config", 1)
        eps = _get(raw, "norm.eps", float, "config", 0.0)
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config: layers must be a non-empty list")
        layers = []
        for i, lr in enumerate(layers_raw):
            where = f"layers[{i}]"
            if not isinstance(lr, Mapping) or lr.get("type") not in MIXERS:
                raise ConfigError(f"{where}: type must be one of {MIXERS}, got "
                                  f"{lr.get('type') if isinstance(lr, Mapping) else lr!r}")
            m = lr.get("mixer")
            if not isinstance(m, Mapping):
                raise ConfigError(f"{where}: mixer missing from config")
            heads, dim = _get(m, "heads", int, where, 1), _get(m, "dim", int, where, 1)
            vdim = _get(m, "vdim", int, where, 1, optional=True) or dim
            scale = _get(m, "scale", float, where)
            if lr["type"] == "attention":
                kv_heads = _get(m, "kv_heads", int, where, 1, optional=True) or heads
                if heads % kv_heads:
                    raise ConfigError(f"{where}: {heads} heads are no multiple of {kv_heads} kv_heads")
                rot_dims = _get(m, "rot.dims", int, where, 0, optional=True) or 0
                if rot_dims % 2 or rot_dims > dim:
                    raise ConfigError(f"{where}: rot.dims {rot_dims} must be even and at most dim {dim}")
                if isinstance(m.get("rot"), Mapping) and m["rot"].get("scaling") is not None:
                    raise ConfigError(f"{where}: rot.scaling belongs to latent_attention layers")
                mixer: Any = WindowMixer(
                    heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale,
                    window=_get(m, "mask.size", int, where, 1, optional=True) or 0,
                    rot_base=(_get(m, "rot.base", float, where) if rot_dims else 1.0), rot_dims=rot_dims)
            else:
                rot_dim = _get(m, "rot_dim", int, where, 2)
                rot_dims = _get(m, "rot.dims", int, where, 0, optional=True)
                rot_dims = rot_dim if rot_dims is None else rot_dims
                if rot_dims % 2 or rot_dims > rot_dim:
                    raise ConfigError(f"{where}: rot.dims {rot_dims} must be even and at most rot_dim {rot_dim}")
                scaling = None
                sc = m["rot"].get("scaling") if isinstance(m.get("rot"), Mapping) else None
                if sc is not None:
                    sw = where + ".rot.scaling"
                    if not isinstance(sc, Mapping):
                        raise ConfigError(f"{sw} must be an object")
                    scaling = RotScaling(factor=_get(sc, "factor", float, sw), original=_get(sc, "original", float, sw),
                                         fast=_get(sc, "fast", float, sw), slow=_get(sc, "slow", float, sw))
                    if scaling.factor <= 0 or scaling.original <= 0 or scaling.fast <= 0 or scaling.slow <= 0:
                        raise ConfigError(f"{sw}: factor, original, fast and slow must be positive")
                mixer = LatentMixer(
                    heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=_get(m, "kv_rank", int, where, 1),
                    q_rank=_get(m, "q_rank", int, where, 1), scale=scale,
                    rot_base=(_get(m, "rot.base", float, where) if rot_dims else 1.0), rot_dims=rot_dims,
                    scaling=scaling, window=_get(m, "mask.size", int, where, 1, optional=True) or 0)
            mlp_raw, mlp = lr.get("mlp"), None
            if mlp_raw is not None:
                if not isinstance(mlp_raw, Mapping) or mlp_raw.get("kind") not in ("dense", "moe"):
                    raise ConfigError(f"{where}: mlp.kind must be 'dense' or 'moe' (or mlp null)")
                if mlp_raw["kind"] == "dense":
                    mlp = DenseMLP(_get(mlp_raw, "ff", int, where, 1))
                else:
                    mlp = MoEMLP(ff=_get(mlp_raw, "expert.ff", int, where, 1),
                                 experts=_get(mlp_raw, "router.experts", int, where, 1),
                                 top=_get(mlp_raw, "router.top", int, where, 1),
                                 identity=_get(mlp_raw, "router.identity", int, where, 0, optional=True) or 0)
                    if mlp.top > mlp.experts + mlp.identity:
                        raise ConfigError(f"{where}: router.top {mlp.top} exceeds the router's "
                                          f"{mlp.experts + mlp.identity} outputs")
            layers.append(PozelixLayer(lr["type"], mixer, mlp))
        loop = None
        if raw.get("loop") is not None:
            lp = raw["loop"]
            if not isinstance(lp, Mapping):
                raise ConfigError("config: loop must be an object")
            loop = Loop(start=_get(lp, "start", int, "loop", 0), stop=_get(lp, "stop", int, "loop", 0),
                        times=_get(lp, "times", int, "loop", 1))
            if not loop.start < loop.stop <= len(layers):
                raise ConfigError(f"loop: layers {loop.start} .. {loop.stop - 1} of {len(layers)}")
        return cls(vocab=vocab, width=width, norm_eps=eps, layers=tuple(layers), loop=loop,
                   torch_dtype=str(raw.get("torch_dtype", "bfloat16")))

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                             "norm": {"eps": self.norm_eps},
                             "layers": [{"type": l.type, "mixer": l.mixer.to_dict(),
                                         "mlp": None if l.mlp is None else l.mlp.to_dict()} for l in self.layers]}
        if self.loop is not None:
            d["loop"] = self.loop.to_dict()
        return d
