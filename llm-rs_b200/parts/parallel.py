"""Two mixers side by side that read the same input; their outputs are added with fixed weights."""
from __future__ import annotations

import os

import torch

from .. import ops
from .base import Mixer, Runtime
from .linear import Linear
from .registry import build, register
from .spec import PartSpec, StateNeed

# LLMRS_FUSE_PARALLEL=0: each side runs its own output projection and the two results are added by a kernel.
FUSE_PARALLEL = os.environ.get("LLMRS_FUSE_PARALLEL", "1") != "0"


@register("mixer", "parallel")
class ParallelMixer(Mixer):
    """``left_scale * left(x) + right_scale * right(x)`` for two mixers given as ``PartSpec``s; their tensors live under
    ``left_scope`` and ``right_scope`` after this mixer's prefix. At most one side may ask for pages (the entry's pages
    are that side's); the sides' per-request state is kept side by side under the sides' own names; a side that plans
    its step on the host keeps doing so.

    When both sides offer ``heads(x, ctx, cache, out, out_scale)`` (their concatenated heads before the output
    projection) and end in a plain product ``o_proj``, the two output projections are ONE product: each side writes
    its heads, already multiplied by its weight (in float32, before the one rounding to the activation type), into
    its columns of a common row, and the product with ``[W_o,left | W_o,right]`` gives the weighted sum. Otherwise each
    side's output is made in float32 and the two are added by a kernel."""

    def __init__(self, left: PartSpec, right: PartSpec, left_scale: float = 1.0, right_scale: float = 1.0,
                 left_scope: str = "left.", right_scope: str = "right.", prefix: str = ""):
        self.left = build("mixer", left, prefix=prefix + left_scope)
        self.right = build("mixer", right, prefix=prefix + right_scope)
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)
        if self.left.cache_need() is not None and self.right.cache_need() is not None:
            raise ValueError("both sides of a parallel mixer ask for pages; an entry of the run order has one set")
        ls, rs = self.left.state_need(), self.right.state_need()
        clash = set(ls.tensors if ls else ()) & set(rs.tensors if rs else ())
        if clash:
            raise ValueError(f"both sides of a parallel mixer keep state named {sorted(clash)}")
        self.graph_safe = getattr(self.left, "graph_safe", True) and getattr(self.right, "graph_safe", True)
        self.fused = None

    def sides(self):
        return [self.left, self.right]

    def weight_specs(self):
        return self.left.weight_specs() + self.right.weight_specs()

    def bind(self, tensors, runtime: Runtime):
        self.act_dtype = runtime.act_dtype
        for side in self.sides():
            side.bind(tensors, runtime)
        self.fused = None
        lo, ro = getattr(self.left, "o_proj", None), getattr(self.right, "o_proj", None)
        if (FUSE_PARALLEL and all(hasattr(side, "heads") for side in self.sides()) and isinstance(lo, Linear)
                and isinstance(ro, Linear) and lo.bias is None and ro.bias is None and lo.weight.dtype == ro.weight.dtype):
            self.widths = (lo.weight.size(1), ro.weight.size(1))
            self.fused = Linear(torch.cat([lo.weight, ro.weight], dim=1).contiguous(), None, runtime.act_dtype)

    def chain(self):
        return []

    def cache_need(self):
        return self.left.cache_need() or self.right.cache_need()

    def state_need(self):
        merged = {}
        for side in self.sides():
            need = side.state_need()
            if need is not None:
                merged.update(need.tensors)
        return StateNeed(merged) if merged else None

    def planners(self):
        """(plan key, mixer that plans) of the sides that plan their step on the host."""
        out = []
        for side in self.sides():
            out += side.planners() if hasattr(side, "planners") else (
                [(side.plan_key(), side)] if side.plan_key() is not None else [])
        return out

    def forward(self, x, ctx, cache, out_dtype=None):
        if self.fused is not None:
            wl, wr = self.widths
            row = torch.empty((ctx.n_tokens, wl + wr), dtype=self.act_dtype, device=x.device)
            self.left.heads(x, ctx, cache, out=row[:, :wl], out_scale=self.left_scale)
            self.right.heads(x, ctx, cache, out=row[:, wl:], out_scale=self.right_scale)
            return self.fused.forward(row, out_dtype=out_dtype)
        a = self.left.forward(x, ctx, cache, out_dtype=torch.float32)
        b = self.right.forward(x, ctx, cache, out_dtype=torch.float32)
        y = ops.scaled_sum(a, b, self.left_scale, self.right_scale)
        return y if out_dtype == torch.float32 else y.to(out_dtype or self.act_dtype)
