"""RMSNorm, fused with the residual sum that precedes it."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import Norm, Runtime
from .registry import register
from .spec import WeightSpec


@register("norm", "rmsnorm")
class RMSNorm(Norm):
    """``y = x / sqrt(mean(x^2) + eps) * w`` with float32 statistics and a plain weight
    (llm-core/src/backends/attention.rs:55-68,98-104). ``dim`` and ``eps`` are parameters;
    ``name`` is the weight's name after the prefix. With ``offset`` the stored weight lies around zero and the
    factor is ``offset + w`` (added once at load, in float32). With ``scalar`` the stored weight is ONE number for all
    coordinates (a tensor without axes); it is spread over ``dim`` at load.

    ``add_normed(h, y)`` is the norm of a block that norms a branch's OUTPUT: ``h += norm(y)``;
    ``post_normed(h, y, ...)`` that of a block that norms after the residual sum."""

    def __init__(self, dim: int, eps: float, name: str = "weight", offset: float = 0.0, scalar: bool = False,
                 prefix: str = ""):
        self.dim, self.eps, self.prefix, self.name = dim, float(eps), prefix, name
        self.offset, self.scalar = float(offset), bool(scalar)
        self.gain: Optional[torch.Tensor] = None        # the one number of a scalar norm, float32 [1] on the device
        self.weight: Optional[torch.Tensor] = None
        self.act_dtype = None

    def weight_specs(self):
        return [WeightSpec(self.prefix + self.name, () if self.scalar else (self.dim,),
                           role="norm_offset" if self.offset else "norm")]

    def bind(self, tensors, runtime: Runtime):
        self.weight = tensors[self.prefix + self.name].to(torch.float32).contiguous()
        if self.offset:
            self.weight = self.weight + self.offset
        if self.scalar:
            self.gain = self.weight.reshape(1).contiguous()
            self.weight = self.gain.expand(self.dim).contiguous()
        self.act_dtype = runtime.act_dtype

    def forward(self, h, delta, rows=None):
        return ops.add_rmsnorm(h, delta, self.weight, self.eps, self.act_dtype, rows=rows)

    def add_normed(self, h, y):
        return ops.outnorm_add(h, y, self.weight, self.eps)

    def post_normed(self, h, y, layer_scale, alpha: float, out_dtype=None):
        """The norm of a block that norms AFTER the sum: ``h = norm(alpha * h + y * layer_scale)`` in place; returns
        the rows rounded to ``out_dtype`` (what the next branch reads), or None without one."""
        return ops.post_norm(h, y, layer_scale, self.weight, alpha, self.eps, out_dtype)

    def link(self):
        return (self.weight, self.eps) if self.act_dtype == torch.bfloat16 else None
