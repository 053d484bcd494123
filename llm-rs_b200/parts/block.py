"""Arrangements of a mixer and a feed-forward around the residual stream."""
from __future__ import annotations

import inspect
import os

import torch

from .. import ops
from .base import Block, Part, PreNormed, Runtime
from .registry import build, register
from .spec import LayerSpec, PartSpec, StateNeed, WeightSpec


# Steps of few tokens spread each norm over the products around it (see ``PreNormed``); LLMRS_LINK_NORMS=0
# keeps the norm kernels.
LINK_NORMS = os.environ.get("LLMRS_LINK_NORMS", "1") != "0"
# LLMRS_FUSE_SANDWICH=0: a block with norms on both sides of a branch runs every norm as a kernel of its own.
FUSE_SANDWICH = os.environ.get("LLMRS_FUSE_SANDWICH", "1") != "0"


@register("block", "prenorm")
class PreNormBlock(Block):
    """``h += mixer(norm1(h)); h += feed_forward(norm2(h))``
    (llm-core/src/graph/builder.rs:74-88,223-254,322-333: norm before each branch, no
    norm on a branch's output). Each sum into ``h`` is fused with the norm that follows
    it, so the feed-forward's output leaves the block not yet added. A part that sets
    ``fuses_residual`` is handed ``h`` and may add its output itself (it then returns None).
    In steps of few tokens a part that can do so also writes the input of the norm after it
    (``PreNormed``), and the part after that norm applies its factor: no norm kernel runs."""

    def __init__(self, layer: LayerSpec, prefix: str = ""):
        p = layer.prefix
        self.mixer_norm = build("norm", layer.mixer_norm, prefix=p)
        self.mixer = build("mixer", layer.mixer, prefix=p + layer.mixer_scope)
        self.feed_forward_norm = build("norm", layer.feed_forward_norm, prefix=p)
        self.feed_forward = build("feed_forward", layer.feed_forward, prefix=p + layer.feed_forward_scope)

    def parts(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def chain(self):
        return [lin for part in self.parts() for lin in part.chain()]

    def weight_specs(self):
        return [s for part in self.parts() for s in part.weight_specs()]

    def bind(self, tensors, runtime: Runtime):
        for part in self.parts():
            part.bind(tensors, runtime)

    links_norms = True

    def accepts_prenormed(self, n_tokens: int) -> bool:
        return LINK_NORMS and self.mixer_norm.link() is not None and self.mixer.takes_prenormed(n_tokens)

    def forward(self, h, pending, ctx, cache, next_norm=None):
        n = ctx.n_tokens
        # A PreNormed ``pending`` was made for this block's first norm by the block before (h holds the sum).
        x = pending if isinstance(pending, PreNormed) else self.mixer_norm.forward(h, pending)
        fused = getattr(self.mixer, "fuses_residual", False)
        link = self.feed_forward_norm.link() if LINK_NORMS and fused else None
        if link and self.mixer.emits_prenormed(n) and self.feed_forward.takes_prenormed(n):
            y = self.mixer.forward(x, ctx, cache, residual=h, next_norm=link)
        else:
            a = self.mixer.forward(x, ctx, cache, residual=h) if fused else self.mixer.forward(x, ctx, cache)
            y = self.feed_forward_norm.forward(h, a)
        fused = getattr(self.feed_forward, "fuses_residual", False)
        if next_norm is not None and fused and self.feed_forward.emits_prenormed(n):
            return h, self.feed_forward.forward(y, ctx, residual=h, next_norm=next_norm)
        if fused:
            return h, self.feed_forward.forward(y, ctx, residual=h)
        return h, self.feed_forward.forward(y, ctx)


class TokenShift(Part):
    """``y_t = x_t + (x_{t-1} - x_t) * mu``: what a mixer reads is mixed, channel by channel, with the previous
    token's row as it was before the mixing (zeros before a sequence's first token). The last row of a step is kept
    per request as fixed-size state, so a sequence may be cut anywhere. ``name`` is mu's tensor after the prefix."""
    STATE = "shift.previous"

    def __init__(self, dim: int, name: str = "shift", prefix: str = ""):
        self.dim, self.name = dim, prefix + name

    def weight_specs(self):
        return [WeightSpec(self.name, (self.dim,), role="bias")]

    def bind(self, tensors, runtime: Runtime):
        self.mu = tensors[self.name].to(torch.float32).contiguous()
        self.act_dtype = runtime.act_dtype

    def state_need(self) -> StateNeed:
        return StateNeed({self.STATE: (self.dim,)})

    def forward(self, h, ctx, cache):
        return ops.token_shift(h, self.mu, cache.state[self.STATE], ctx, self.act_dtype)


@register("block", "outnorm")
class OutNormBlock(Block):
    """``h += norm1(mixer(shift(h))); h += norm2(feed_forward(h))``: the branches read the residual stream itself
    (rounded to the activation type) and the norms sit on their OUTPUTS. ``token_shift`` (the name of its tensor,
    or "") puts a ``TokenShift`` before the mixer; a layer may have no feed-forward. The residual sums and the
    norms' statistics are float32."""

    def __init__(self, layer: LayerSpec, token_shift: str = "", prefix: str = ""):
        p = layer.prefix
        self.mixer_norm = build("norm", layer.mixer_norm, prefix=p)
        self.mixer = build("mixer", layer.mixer, prefix=p + layer.mixer_scope)
        self.shift = TokenShift(self.mixer_norm.dim, token_shift, prefix=p) if token_shift else None
        self.feed_forward = self.feed_forward_norm = None
        if layer.feed_forward is not None:
            self.feed_forward_norm = build("norm", layer.feed_forward_norm, prefix=p)
            self.feed_forward = build("feed_forward", layer.feed_forward, prefix=p + layer.feed_forward_scope)

    def parts(self):
        return [p for p in (self.shift, self.mixer, self.mixer_norm, self.feed_forward, self.feed_forward_norm)
                if p is not None]

    def chain(self):
        return []

    def weight_specs(self):
        return [s for part in self.parts() for s in part.weight_specs()]

    def bind(self, tensors, runtime: Runtime):
        self.act_dtype = runtime.act_dtype
        for part in self.parts():
            part.bind(tensors, runtime)

    def state_need(self):
        return self.shift.state_need() if self.shift is not None else None

    def forward(self, h, pending, ctx, cache):
        if pending is not None:      # a block before this one left its last branch unadded
            ops.residual_add(h, pending)
        x = self.shift.forward(h, ctx, cache) if self.shift is not None else ops.token_shift(
            h, None, None, ctx, self.act_dtype)
        self.mixer_norm.add_normed(h, self.mixer.forward(x, ctx, cache))
        if self.feed_forward is not None:
            x = h if getattr(self.feed_forward, "reads_residual", False) else ops.token_shift(
                h, None, None, ctx, self.act_dtype)
            self.feed_forward_norm.add_normed(h, self.feed_forward.forward(x, ctx))
        return h, None


@register("block", "postnorm")
class PostNormBlock(Block):
    """``h = norm1(alpha * h + ls1 * mixer(h)); h = norm2(alpha * h + ls2 * feed_forward(h))``: the norm comes after
    the residual sum, the branches read the stream itself (rounded to the activation type by the norm's own pass) and
    each branch's output may be scaled channel by channel before the sum (layer scale). ``alpha`` weighs the stream in
    the sum. ``layer_scale`` names the two scale vectors after the layer's prefix ((), or ("", "") : none); a layer
    may have no feed-forward, and then no second norm unless ``lone_norm`` keeps it (``h = norm2(alpha * h)``).
    Sums, statistics and the normed stream are float32."""

    def __init__(self, layer: LayerSpec, alpha: float = 1.0, layer_scale=(), lone_norm: bool = False, prefix: str = ""):
        p = layer.prefix
        self.alpha = float(alpha)
        self.mixer_norm = build("norm", layer.mixer_norm, prefix=p)
        self.mixer = build("mixer", layer.mixer, prefix=p + layer.mixer_scope)
        self.feed_forward = self.feed_forward_norm = None
        if layer.feed_forward is not None:
            self.feed_forward = build("feed_forward", layer.feed_forward, prefix=p + layer.feed_forward_scope)
        if layer.feed_forward is not None or lone_norm:
            self.feed_forward_norm = build("norm", layer.feed_forward_norm, prefix=p)
        names = tuple(layer_scale) + ("", "")
        self.scale_names = [p + n if n else "" for n in names[:2]]
        if self.feed_forward is None:
            self.scale_names[1] = ""
        self.dim = self.mixer_norm.dim
        self.scales = [None, None]

    def parts(self):
        return [p for p in (self.mixer, self.mixer_norm, self.feed_forward, self.feed_forward_norm) if p is not None]

    def chain(self):
        return []

    def weight_specs(self):
        specs = [s for part in self.parts() for s in part.weight_specs()]
        return specs + [WeightSpec(n, (self.dim,), role="norm") for n in self.scale_names if n]

    def bind(self, tensors, runtime: Runtime):
        self.act_dtype = runtime.act_dtype
        for part in self.parts():
            part.bind(tensors, runtime)
        self.scales = [tensors[n].to(torch.float32).contiguous() if n else None for n in self.scale_names]

    def forward(self, h, pending, ctx, cache):
        if pending is not None:      # a block of another kind left its last branch unadded
            ops.residual_add(h, pending)
            ctx.stream_copy = None
        # The norm that ends a block leaves the stream's rounded copy for the block after it (same step, same stream).
        left = getattr(ctx, "stream_copy", None)
        x = left[1] if left is not None and left[0] is h else ops.token_shift(h, None, None, ctx, self.act_dtype)
        y = self.mixer.forward(x, ctx, cache)
        x = self.mixer_norm.post_normed(h, y, self.scales[0], self.alpha, self.act_dtype)
        if self.feed_forward_norm is not None:
            y = self.feed_forward.forward(x, ctx) if self.feed_forward is not None else None
            x = self.feed_forward_norm.post_normed(h, y, self.scales[1], self.alpha, self.act_dtype)
        ctx.stream_copy = (h, x)
        return h, None


@register("block", "sandwich")
class SandwichBlock(Block):
    """``h += norm_b(mixer(norm_a(h))); h += norm_d(feed_forward(norm_c(h)))``: a norm ahead of every branch AND one on
    its output. ``layer.mixer_norm`` and ``layer.feed_forward_norm`` are the norms ahead of the branches; ``out_norms``
    names the weights of the two output norms after the layer's prefix (same size and eps). A layer may have no
    feed-forward. The norm on the mixer's output, the residual sum and the norm ahead of the feed-forward are one pass
    over the rows (``ops.outnorm_add_norm``). Sums and statistics are float32."""

    def __init__(self, layer: LayerSpec, out_norms=("norm1b", "norm2b"), prefix: str = ""):
        p = layer.prefix
        self.mixer_norm = build("norm", layer.mixer_norm, prefix=p)
        self.mixer = build("mixer", layer.mixer, prefix=p + layer.mixer_scope)
        dim, eps = self.mixer_norm.dim, self.mixer_norm.eps
        out_spec = lambda name: PartSpec("rmsnorm", {"dim": dim, "eps": eps, "name": name})
        self.mixer_out_norm = build("norm", out_spec(out_norms[0]), prefix=p)
        self.feed_forward = self.feed_forward_norm = self.feed_forward_out_norm = None
        if layer.feed_forward is not None:
            self.feed_forward_norm = build("norm", layer.feed_forward_norm, prefix=p)
            self.feed_forward = build("feed_forward", layer.feed_forward, prefix=p + layer.feed_forward_scope)
            self.feed_forward_out_norm = build("norm", out_spec(out_norms[1]), prefix=p)
        self.dim = dim

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.mixer_out_norm, self.feed_forward_norm,
                            self.feed_forward, self.feed_forward_out_norm) if p is not None]

    def chain(self):
        return []

    def weight_specs(self):
        return [s for part in self.parts() for s in part.weight_specs()]

    def bind(self, tensors, runtime: Runtime):
        self.act_dtype = runtime.act_dtype
        for part in self.parts():
            part.bind(tensors, runtime)

    def forward(self, h, pending, ctx, cache):
        x = self.mixer_norm.forward(h, pending)
        y = self.mixer.forward(x, ctx, cache)
        if self.feed_forward is None:
            self.mixer_out_norm.add_normed(h, y)
            return h, None
        nxt = self.feed_forward_norm
        if (FUSE_SANDWICH and self.dim <= ops.OUTNORM_ADD_NORM_MAX_WIDTH and nxt.eps == self.mixer_out_norm.eps
                and (y.dtype == self.act_dtype or y.dtype == torch.float32)):
            x = ops.outnorm_add_norm(h, y, self.mixer_out_norm.weight, nxt.weight, nxt.eps, self.act_dtype)
        else:
            self.mixer_out_norm.add_normed(h, y)
            x = nxt.forward(h, None)
        self.feed_forward_out_norm.add_normed(h, self.feed_forward.forward(x, ctx))
        return h, None


class HyperPending:
    """A branch output that a hyper-connected block has not written into the streams yet: ``y`` [tokens, width] with
    the ``mix`` [streams, streams] and ``out`` [streams] of its write."""
    __slots__ = ("y", "mix", "out")

    def __init__(self, y, mix, out):
        self.y, self.mix, self.out = y, mix, out

    def write(self):
        return (self.y, self.mix, self.out)


@register("block", "hyper")
class HyperBlock(Block):
    """Hyper-connections around a pre-norm layer: the residual stream is ``streams`` copies ``x_1 .. x_S`` per token (all
    equal to the embedding output at the start; ``h`` is float32 [tokens, streams * width], a token's streams side by
    side). Sublayer q (1: the mixer, 2: the feed-forward) with its tensors ``in`` [S], ``out`` [S] and ``mix`` [S, S]
    (indexed [from, to]):

        u = sum_s in[s] x_s;   y = sublayer(norm(u));   x_t <- sum_s mix[s, t] x_s + out[t] y   (all t from the old x)

    and the model reads the SUM of the streams at the end (``leave``). The write of one sublayer and the read and norm of
    the next are one pass over the token's streams (``ops.hyper_step``), across layers too: the feed-forward's output
    leaves the block unwritten (a ``HyperPending``); the last write of a model is folded into the sum of the streams of
    the wanted rows. The norms must be ``rmsnorm`` parts with one number as weight (``scalar``). ``names`` gives the
    scopes of the two sublayers' tensors after the layer's prefix. A layer may have no feed-forward. Everything but
    the normed rows is float32. ``learned`` False: no such tensors, in = out = 1 and mix the identity; with one stream
    that is the plain pre-norm layer ``x <- x + sublayer(norm(x))``."""

    def __init__(self, layer: LayerSpec, streams: int, names=("hc1.", "hc2."), learned: bool = True, prefix: str = ""):
        if not 1 <= streams <= ops.HYPER_MAX_STREAMS:
            raise ValueError(f"{streams} streams: the kernels take 1 to {ops.HYPER_MAX_STREAMS}")
        p = layer.prefix
        self.streams, self.learned = int(streams), bool(learned)
        self.mixer_norm = build("norm", layer.mixer_norm, prefix=p)
        self.mixer = build("mixer", layer.mixer, prefix=p + layer.mixer_scope)
        self.feed_forward = self.feed_forward_norm = None
        if layer.feed_forward is not None:
            self.feed_forward_norm = build("norm", layer.feed_forward_norm, prefix=p)
            self.feed_forward = build("feed_forward", layer.feed_forward, prefix=p + layer.feed_forward_scope)
        for norm in (self.mixer_norm, self.feed_forward_norm):
            if norm is not None and not getattr(norm, "scalar", False):
                raise ValueError("a hyper-connected block takes norms with one number as weight (rmsnorm, scalar=True)")
        self.scopes = [p + names[0]] + ([p + names[1]] if self.feed_forward is not None else [])
        self.dim = self.mixer_norm.dim
        self.hc = []

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward) if p is not None]

    def chain(self):
        return []

    def weight_specs(self):
        S = self.streams
        specs = [s for part in self.parts() for s in part.weight_specs()]
        for scope in self.scopes if self.learned else ():
            specs += [WeightSpec(scope + "in", (S,), role="norm"), WeightSpec(scope + "out", (S,), role="norm"),
                      WeightSpec(scope + "mix", (S, S), role="identity")]
        return specs

    def bind(self, tensors, runtime: Runtime):
        self.act_dtype = runtime.act_dtype
        for part in self.parts():
            part.bind(tensors, runtime)
        f32 = lambda name: tensors[name].to(torch.float32).contiguous()
        if self.learned:
            self.hc = [(f32(scope + "in"), f32(scope + "mix"), f32(scope + "out")) for scope in self.scopes]
        else:
            ones = torch.ones((self.streams,), dtype=torch.float32, device=runtime.device)
            eye = torch.eye(self.streams, dtype=torch.float32, device=runtime.device)
            self.hc = [(ones, eye, ones) for _ in self.scopes]

    def _sublayer_out(self, part, x, *args):
        """A sublayer's output, in float32 where the part can give it unrounded (its ``forward`` takes ``out_dtype``)."""
        if "out_dtype" in inspect.signature(part.forward).parameters:
            return part.forward(x, *args, out_dtype=torch.float32)
        return part.forward(x, *args)

    def forward(self, h, pending, ctx, cache):
        if pending is not None and not isinstance(pending, HyperPending):
            raise TypeError("a hyper-connected block follows a block that left a plain branch output unadded")
        in1, mix1, out1 = self.hc[0]
        norm1 = self.mixer_norm
        x = ops.hyper_step(h, write=pending.write() if pending is not None else None, read=(in1, norm1.gain),
                           eps=norm1.eps, act_dtype=self.act_dtype)
        y = self._sublayer_out(self.mixer, x, ctx, cache)
        if self.feed_forward is None:
            return h, HyperPending(y, mix1, out1)
        in2, mix2, out2 = self.hc[1]
        norm2 = self.feed_forward_norm
        x = ops.hyper_step(h, write=(y, mix1, out1), read=(in2, norm2.gain), eps=norm2.eps, act_dtype=self.act_dtype)
        return h, HyperPending(self._sublayer_out(self.feed_forward, x, ctx), mix2, out2)

    def leave(self, h, pending, rows):
        """What the model's last norm reads: the sum of the streams of the given rows, float32 [rows, width]."""
        if pending is not None and not isinstance(pending, HyperPending):
            raise TypeError("a hyper-connected block cannot take a plain branch output")
        return ops.hyper_leave(h, self.streams, write=pending.write() if pending is not None else None, rows=rows)
