"""Delta rules: recurrent mixers with a matrix state per head (the generalized one with a decay and a removal rate per
channel, and the gated one with a decay and a write strength per head behind short convolutions)."""
from __future__ import annotations

import math

import torch

from .. import ops
from .base import Mixer, Runtime
from .linear import Linear
from .registry import register
from .spec import StateNeed, WeightSpec


@register("mixer", "general_delta")
class GeneralDelta(Mixer):
    """Per head a state S [key channel, value channel] (float32, zero at a sequence's start, kept per request):

        S_t = diag(w_t) S_{t-1} - (a_t * u_t) (u_t^T S_{t-1}) + k_t v_t^T,      o_t = S_t^T r_t

    with r, k, v projections of the input (``n_heads`` x ``dim``), the unit key ``u = k / sqrt(sum(k^2) + key_eps)``,
    the decay ``w = exp(-decay_scale * sigmoid(W_w2 tanh(W_w1 x) + w0))`` and the removal rate
    ``a = sigmoid(W_a x + a_bias)``, both per head and key channel. Each head's o is divided by its root mean square
    (``norm_eps``), the heads are concatenated, multiplied by a plain weight and by ``sigmoid(W_g x)``, then the
    output projection. Decay, removal rate, unit key, state and the norm are float32; the projections run in the
    activation type. ``decay_scale`` defaults to exp(-1/2).

    r, k, v, g, a and the first decay projection read the same input and are one product. No pages: the mixer asks for
    fixed-size state only, so its cost per token does not grow with the sequence.

    ``names`` maps the roles r, k, v, g, a, a_bias, w1, w2, w0, norm, o to tensor names after the prefix.
    """
    ROLES = ("r", "k", "v", "g", "a", "a_bias", "w1", "w2", "w0", "norm", "o")
    STATE = "delta.state"

    def __init__(self, hidden_size: int, n_heads: int, dim: int, decay_rank: int, norm_eps: float = 1e-6,
                 key_eps: float = 1e-6, decay_scale: float = math.exp(-0.5), names=None, prefix: str = ""):
        if dim > 256:
            raise ValueError(f"heads of {dim} channels: the recurrence kernel takes at most 256")
        self.hidden_size, self.n_heads, self.dim, self.decay_rank = hidden_size, n_heads, dim, decay_rank
        self.norm_eps, self.key_eps, self.decay_scale = float(norm_eps), float(key_eps), float(decay_scale)
        self.prefix = prefix
        self.names = {"r": "r", "k": "k", "v": "v", "g": "g", "a": "a", "a_bias": "a.b", "w1": "w1", "w2": "w2",
                      "w0": "w0", "norm": "norm", "o": "o"}
        self.names.update(names or {})
        if set(self.names) != set(self.ROLES):
            raise ValueError(f"names may rename {self.ROLES}, got {sorted(set(self.names) - set(self.ROLES))}")
        self.width = n_heads * dim

    def _name(self, role: str) -> str:
        return self.prefix + self.names[role]

    def weight_specs(self):
        H, W, nm = self.hidden_size, self.width, self._name
        return [WeightSpec(nm(r), (W, H)) for r in ("r", "k", "v", "g", "a")] + [
            WeightSpec(nm("a_bias"), (W,), role="bias"), WeightSpec(nm("w1"), (self.decay_rank, H)),
            WeightSpec(nm("w2"), (W, self.decay_rank)), WeightSpec(nm("w0"), (W,), role="bias"),
            WeightSpec(nm("norm"), (W,), role="norm"), WeightSpec(nm("o"), (H, W))]

    def bind(self, tensors, runtime: Runtime):
        nm = self._name
        self.act_dtype = runtime.act_dtype
        ws = [tensors[nm(r)] for r in ("r", "k", "v", "g", "a", "w1")]
        dt = ws[0].dtype if all(w.dtype == ws[0].dtype for w in ws) else torch.float32
        self.in_proj = Linear(torch.cat([w.to(dt) for w in ws], dim=0).contiguous(), None, runtime.act_dtype)
        self.decay_proj = Linear(tensors[nm("w2")], None, runtime.act_dtype)
        self.o_proj = Linear(tensors[nm("o")], None, runtime.act_dtype)
        f32 = lambda role: tensors[nm(role)].to(torch.float32).contiguous()
        self.a_bias, self.decay_bias, self.norm_w = f32("a_bias"), f32("w0"), f32("norm")

    def state_need(self):
        return StateNeed({self.STATE: (self.n_heads, self.dim, self.dim)})

    def forward(self, x, ctx, cache):
        W = self.width
        proj = self.in_proj.forward(x)
        r, k, v, g, a = (proj[:, i * W:(i + 1) * W] for i in range(5))
        hidden = ops.tanh_slice(proj[:, 5 * W: 5 * W + self.decay_rank], self.act_dtype)
        decay_raw = self.decay_proj.forward(hidden, out_dtype=torch.float32)
        out = ops.delta_rule(r, k, v, g, a, decay_raw, self.decay_bias, self.a_bias, self.norm_w,
                             cache.state[self.STATE], ctx, self.n_heads, self.dim, self.decay_scale, self.key_eps,
                             self.norm_eps)
        return self.o_proj.forward(out)


@register("mixer", "gated_delta")
class GatedDelta(Mixer):
    """Per value head a state S [key channel, value channel] (float32, zero at a sequence's start, kept per request):

        S <- g_t S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t

    so the read-out sees the token's own write. q and k are projections of ``n_kv_heads`` x ``dim`` (value head h reads
    q/k head h // (n_heads / n_kv_heads)), v of ``n_heads`` x ``vdim``; each passes a short causal convolution over time
    per channel (``conv`` taps, the last one the current token's, no bias, zeros before the start) and SiLU; q and k are
    then unit vectors per head (``x / sqrt(sum(x^2) + key_eps)``) and q is multiplied by ``q_scale`` (default
    dim^-1/2). ``beta = sigmoid(W_b x)`` and ``g = exp(-exp(A_log) * softplus(W_a x + dt_bias))`` are one number per
    head. Each head's o is divided by its root mean square over vdim (``norm_eps``), multiplied by a plain weight of
    size vdim that the heads share and by ``silu(W_g x)``, then the output projection.

    The decay, the write strength, the unit norms, the state and the output norm are float32, and W_a, W_b are float32
    products; q, k, v and the gate come from one product in the activation type. Per-request state: S and the last
    ``conv`` - 1 rows that entered the convolutions; no pages. ``heads(...)`` gives the gated heads before the output
    projection, optionally scaled and written into a view, for a mixer that runs this one beside another.

    ``names`` maps the roles q, k, v, q_conv, k_conv, v_conv, b, a, A_log, dt_bias, g, norm, o to tensor names."""
    ROLES = ("q", "k", "v", "q_conv", "k_conv", "v_conv", "b", "a", "A_log", "dt_bias", "g", "norm", "o")
    STATE, CONV_STATE = "gated_delta.state", "gated_delta.conv"

    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, dim: int, vdim: int, conv: int,
                 norm_eps: float = 1e-6, key_eps: float = 1e-6, q_scale=None, names=None, prefix: str = ""):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} value heads are no multiple of {n_kv_heads} key heads")
        if dim > 256:
            raise ValueError(f"key heads of {dim} channels: the recurrence kernel takes at most 256")
        if conv < 1:
            raise ValueError(f"a convolution of {conv} taps")
        self.hidden_size, self.n_heads, self.n_kv_heads, self.dim, self.vdim = hidden_size, n_heads, n_kv_heads, dim, vdim
        self.conv, self.norm_eps, self.key_eps = int(conv), float(norm_eps), float(key_eps)
        self.q_scale = float(q_scale) if q_scale is not None else dim ** -0.5
        self.prefix = prefix
        self.names = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "b": "b",
                      "a": "a", "A_log": "A_log", "dt_bias": "dt_bias", "g": "g", "norm": "norm", "o": "o"}
        self.names.update(names or {})
        if set(self.names) != set(self.ROLES):
            raise ValueError(f"names may rename {self.ROLES}, got {sorted(set(self.names) - set(self.ROLES))}")
        self.k_width, self.v_width = n_kv_heads * dim, n_heads * vdim
        self.channels = 2 * self.k_width + self.v_width      # what passes the convolutions

    def _name(self, role: str) -> str:
        return self.prefix + self.names[role]

    def weight_specs(self):
        H, nm, K, V, nh, taps = self.hidden_size, self._name, self.k_width, self.v_width, self.n_heads, self.conv
        return [WeightSpec(nm("q"), (K, H)), WeightSpec(nm("k"), (K, H)), WeightSpec(nm("v"), (V, H)),
                WeightSpec(nm("q_conv"), (K, taps), role="conv"), WeightSpec(nm("k_conv"), (K, taps), role="conv"),
                WeightSpec(nm("v_conv"), (V, taps), role="conv"), WeightSpec(nm("b"), (nh, H)), WeightSpec(nm("a"), (nh, H)),
                WeightSpec(nm("A_log"), (nh,), role="bias"), WeightSpec(nm("dt_bias"), (nh,), role="bias"),
                WeightSpec(nm("g"), (V, H)), WeightSpec(nm("norm"), (self.vdim,), role="norm"),
                WeightSpec(nm("o"), (H, V))]

    def bind(self, tensors, runtime: Runtime):
        nm = self._name
        self.act_dtype = runtime.act_dtype
        ws = [tensors[nm(r)] for r in ("q", "k", "v", "g")]
        dt = ws[0].dtype if all(w.dtype == ws[0].dtype for w in ws) else torch.float32
        self.in_proj = Linear(torch.cat([w.to(dt) for w in ws], dim=0).contiguous(), None, runtime.act_dtype)
        self.o_proj = Linear(tensors[nm("o")], None, runtime.act_dtype)
        f32 = lambda role: tensors[nm(role)].to(torch.float32).contiguous()
        self.taps = torch.cat([f32("q_conv"), f32("k_conv"), f32("v_conv")], dim=0).contiguous()
        # The decay's and the write strength's projections are float32 products whatever the activation type: what
        # enters the recurrence is not rounded.
        stored = [tensors[nm("b")], tensors[nm("a")]]
        self.ba_w = torch.cat([f32("b"), f32("a")], dim=0).contiguous()
        self.ba_w_stored = torch.cat(stored, dim=0).contiguous() if stored[0].dtype == stored[1].dtype else self.ba_w
        self.a_log, self.dt_bias, self.norm_w = f32("A_log"), f32("dt_bias"), f32("norm")

    def chain(self):
        return []

    def state_need(self):
        return StateNeed({self.STATE: (self.n_heads, self.dim, self.vdim),
                          self.CONV_STATE: (self.conv - 1, self.channels)})

    def heads(self, x, ctx, cache, out=None, out_scale: float = 1.0):
        proj = self.in_proj.forward(x)
        ba = ops.product_f32(x, self.ba_w_stored, self.ba_w, None)
        return ops.gated_delta(proj[:, : self.channels], proj[:, self.channels: self.channels + self.v_width], self.taps,
                               ba, self.a_log, self.dt_bias, self.norm_w, cache.state[self.STATE],
                               cache.state[self.CONV_STATE], ctx, self.n_kv_heads, self.n_heads, self.dim, self.vdim,
                               self.key_eps, self.q_scale, self.norm_eps, out=out, out_scale=out_scale)

    def forward(self, x, ctx, cache, out_dtype=None):
        return self.o_proj.forward(self.heads(x, ctx, cache), out_dtype=out_dtype)
