"""Latent attention: all heads share one cached row per token."""
from __future__ import annotations

import math
import os
from typing import Mapping, Optional

import numpy as np
import torch

from .. import ops
from .base import Mixer, Plan, Runtime, StepInfo
from .linear import Linear
from .registry import register
from .spec import CacheNeed, WeightSpec


# Prompt portions in bfloat16 take the tensor-core kernel from this many tokens a step on; LLMRS_LATENT_MMA=0 keeps the
# CUDA-core kernel for everything.
_LATENT_MMA = os.environ.get("LLMRS_LATENT_MMA", "1") != "0"
PREFILL_MIN_TOKENS = 32


def rescaled_frequencies(dims: int, base: float, scaling: Optional[Mapping] = None):
    """(inverse frequencies float64 [dims/2], magnitude) of a rotation of ``dims`` entries: ``f_i = base^(-2i/dims)``.

    ``scaling`` (factor, original, fast, slow) stretches the slow pairs for contexts longer than the ``original`` one
    (YaRN: Peng, Quesnelle, Fan, Shippole, "YaRN: Efficient Context Window Extension of Large Language Models"). A
    pair that turns ``t`` times within the original context has index ``d(t) = dims * ln(original / (2 pi t)) / (2 ln
    base)``; pairs below ``lo = max(floor(d(fast)), 0)`` keep their frequency, pairs above ``hi = min(ceil(d(slow)),
    dims - 1)`` have it divided by ``factor``, and between them the two are blended by ``ramp_i = clamp((i - lo) /
    max(hi - lo, 0.001), 0, 1)``: ``f_i / factor * ramp_i + f_i * (1 - ramp_i)``. Cosines and sines are multiplied by
    the magnitude ``0.1 ln(factor) + 1``."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / max(dims, 1))
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])
    index = lambda turns: dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))
    lo = max(math.floor(index(float(scaling["fast"]))), 0)
    hi = min(math.ceil(index(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def portion_tiles(q_start, n_new, tile_tokens: int) -> np.ndarray:
    """int32 [n, 2]: (first token of the step, tokens) of tiles of at most ``tile_tokens`` consecutive tokens that do
    not cross a request."""
    firsts, counts = [], []
    for qs, n in zip(np.asarray(q_start).tolist(), np.asarray(n_new).tolist()):
        a = np.arange(0, n, tile_tokens, dtype=np.int32)
        firsts.append(qs + a)
        counts.append(np.minimum(tile_tokens, n - a))
    if not firsts:
        return np.zeros((0, 2), np.int32)
    return np.stack([np.concatenate(firsts), np.concatenate(counts)], axis=1).astype(np.int32)


@register("mixer", "latent_attention")
class LatentAttention(Mixer):
    """Attention whose keys and values are up-projections of a small cached latent.

    Per token the down-projection gives ``rank + rot_dim`` numbers: the first ``rank``, RMS-normed with a plain
    weight, are the latent c; the last ``rot_dim`` (rotated by position, not normed) are a key part shared by all
    heads. Only these are cached. A query head is [``dim`` unrotated | ``rot_dim`` rotated]; head h's unrotated key
    is ``W_uk,h c`` and its value ``W_uv,h c``. The score is ``(q_n . k_n + q_r . k_r) * scale`` over the causal keys
    (the last ``window`` of them when ``window`` > 0), ordinary softmax; head h's output is multiplied by
    ``sigmoid(W_g x)_h`` when ``gated``; then the output projection.

    Computed in the folded form: ``qa_h = W_uk,h^T q_n,h`` (a batched product), attention over the cached rows with
    values c, then ``W_uv,h`` on the result (a batched product): the cache is read once for all heads and no key or
    value is ever materialised. The rotation pairs entry i of the rotated part with entry i + rot_dims/2 for the first
    ``rot_dims`` entries (``rot_pairing`` "half"), or entry 2i with 2i + 1 ("neighbours"), angle ``position *
    rot_base^(-2i/rot_dims)``; ``rot_scaling`` rescales the frequencies (``rescaled_frequencies``).

    ``q_rank`` > 0: the queries go through a latent of their own, ``q = W_uq rmsnorm(W_dq x)`` with a plain norm
    weight; the down-projection shares the product of the gates and the key/value down-projection.

    A layer with ``shares_cache`` has no down-projection: its run-order entry reads another entry's pages
    (``RunStep.cache_of``) with its own up-projections, queries and window. ``cache_window`` is the window the pages
    are kept for (the widest window of the layers that read them; default: this layer's).

    ``names`` maps the roles q, dq, dq_norm, uq, dkv, dkv_norm, uk, uv, g, o to tensor names after the prefix.
    """
    ROLES = ("q", "dq", "dq_norm", "uq", "dkv", "dkv_norm", "uk", "uv", "g", "o")
    PAIRINGS = ("half", "neighbours")

    def __init__(self, hidden_size: int, n_heads: int, dim: int, rot_dim: int, vdim: int, rank: int, scale: float,
                 rot_base: float, rot_dims: Optional[int] = None, window: int = 0, cache_window: Optional[int] = None,
                 norm_eps: float = 1e-6, gated: bool = True, shares_cache: bool = False, q_rank: int = 0,
                 rot_pairing: str = "half", rot_scaling: Optional[Mapping] = None, names=None, prefix: str = ""):
        self.hidden_size, self.n_heads, self.dim, self.rot_dim, self.vdim = hidden_size, n_heads, dim, rot_dim, vdim
        self.rank, self.scale, self.rot_base = rank, float(scale), float(rot_base)
        self.rot_dims = rot_dim if rot_dims is None else int(rot_dims)
        if self.rot_dims % 2 or not 0 <= self.rot_dims <= rot_dim:
            raise ValueError(f"{self.rot_dims} rotated dimensions of a rotated part of {rot_dim}")
        if rot_pairing not in self.PAIRINGS:
            raise ValueError(f"unknown rot_pairing {rot_pairing!r}; known: {self.PAIRINGS}")
        self.q_rank, self.rot_pairing = int(q_rank), rot_pairing
        self.rot_scaling = dict(rot_scaling) if rot_scaling else None
        if rank > 512:
            raise ValueError(f"a latent of {rank}: the attention kernel takes at most 512")
        self.window = int(window)
        self.cache_window = self.window if cache_window is None else int(cache_window)
        if self.cache_window and (self.window == 0 or self.window > self.cache_window):
            raise ValueError(f"pages kept for the last {self.cache_window} keys cannot serve a window of "
                             f"{self.window or 'all'} keys")
        self.norm_eps, self.gated, self.shares_cache = float(norm_eps), bool(gated), bool(shares_cache)
        self.prefix = prefix
        self.names = {"q": "q", "dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm",
                      "uk": "uk", "uv": "uv", "g": "g", "o": "o"}
        self.names.update(names or {})
        if set(self.names) != set(self.ROLES):
            raise ValueError(f"names may rename {self.ROLES}, got {sorted(set(self.names) - set(self.ROLES))}")
        self.q_width = n_heads * (dim + rot_dim)
        self._tile = None

    def _name(self, role: str) -> str:
        return self.prefix + self.names[role]

    def weight_specs(self):
        H, nh, nm = self.hidden_size, self.n_heads, self._name
        specs = [WeightSpec(nm("uk"), (nh * self.dim, self.rank)),
                 WeightSpec(nm("uv"), (nh * self.vdim, self.rank)), WeightSpec(nm("o"), (H, nh * self.vdim))]
        if self.q_rank:
            specs += [WeightSpec(nm("dq"), (self.q_rank, H)), WeightSpec(nm("dq_norm"), (self.q_rank,), role="norm"),
                      WeightSpec(nm("uq"), (self.q_width, self.q_rank))]
        else:
            specs.append(WeightSpec(nm("q"), (self.q_width, H)))
        if self.gated:
            specs.append(WeightSpec(nm("g"), (nh, H)))
        if not self.shares_cache:
            specs += [WeightSpec(nm("dkv"), (self.rank + self.rot_dim, H)),
                      WeightSpec(nm("dkv_norm"), (self.rank,), role="norm")]
        return specs

    def bind(self, tensors, runtime: Runtime):
        nm, nh = self._name, self.n_heads
        self.act_dtype = runtime.act_dtype
        ws = [tensors[nm("dq") if self.q_rank else nm("q")]]
        self.q_up = self.q_norm_w = None
        if self.q_rank:
            self.q_up = Linear(tensors[nm("uq")], None, runtime.act_dtype)
            self.q_norm_w = tensors[nm("dq_norm")].to(torch.float32).contiguous()
        if self.gated:
            ws.append(tensors[nm("g")])
        if not self.shares_cache:
            ws.append(tensors[nm("dkv")])
        dt = ws[0].dtype if all(w.dtype == ws[0].dtype for w in ws) else torch.float32
        # One product for the queries, the gates and the down-projection: they read the same input.
        self.in_proj = Linear(torch.cat([w.to(dt) for w in ws], dim=0).contiguous(), None, runtime.act_dtype)
        self.o_proj = Linear(tensors[nm("o")], None, runtime.act_dtype)
        # W_uk,h transposed to [rank, dim]: the folded query is an ordinary product with it.
        self.w_uk_t = tensors[nm("uk")].view(nh, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[nm("uv")].view(nh, self.vdim, self.rank).contiguous()
        self.latent_norm_w = None if self.shares_cache else tensors[nm("dkv_norm")].to(torch.float32).contiguous()
        self.open_gate = torch.full((1, nh), 30.0, dtype=runtime.act_dtype, device=runtime.device)
        inv_freq, self.rot_magnitude = rescaled_frequencies(self.rot_dims, self.rot_base, self.rot_scaling)
        self.inv_freq = inv_freq.to(runtime.device)

    def cache_need(self):
        if self.shares_cache:
            return None
        return CacheNeed("window" if self.cache_window > 0 else "full", 1, self.rank, self.cache_window,
                         planes=(self.rank, self.rot_dim))

    # -- the step's plan: tiles of a prompt's tokens for the tensor-core kernel -------------------------------------
    def _tile_tokens(self) -> int:
        if self._tile is None:      # asked of the kernel library at first use: constructing a part needs no library
            self._tile = ops.latent_prefill_tile_tokens(self.n_heads)
        return self._tile

    def plan_key(self):
        return ("latent_attention_tiles", self._tile_tokens())

    def plan(self, step: StepInfo) -> Plan:
        """Steps that bring a prompt's portion are cut into tiles of tokens (none for steps of single tokens, which
        the CUDA-core kernel takes with its keys cut over blocks, and which may be replayed from a graph)."""
        if step.for_graph or step.n_tokens < PREFILL_MIN_TOKENS or int(np.max(step.n_new, initial=0)) <= 1:
            return Plan(arrays={"tiles": np.zeros((0, 2), np.int32)}, values={"n_tiles": 0})
        tiles = portion_tiles(step.q_start, step.n_new, self._tile_tokens())
        return Plan(arrays={"tiles": tiles}, values={"n_tiles": int(tiles.shape[0])})

    def _tiles(self, ctx):
        """(device tiles, how many) for this step; None when the step has no plan of them."""
        if hasattr(ctx, "plan"):
            view = ctx.plan(self.plan_key())
            return (view.arrays["tiles"], view.values["n_tiles"]) if view.values["n_tiles"] else None
        # Called outside the step function (a part alone): plan here, from the device's arrays.
        n_new = ctx.n_new.cpu().numpy()
        if ctx.n_tokens < PREFILL_MIN_TOKENS or int(n_new.max(initial=0)) <= 1:
            return None
        tiles = portion_tiles(ctx.q_start.cpu().numpy(), n_new, self._tile_tokens())
        return torch.from_numpy(tiles).to(ctx.n_new.device), int(tiles.shape[0])

    def forward(self, x, ctx, cache):
        nh, dn, dr, rank = self.n_heads, self.dim, self.rot_dim, self.rank
        if cache.owns == self.shares_cache:
            raise RuntimeError("a latent attention layer that shares a cache must run as an entry with cache_of "
                               "(and one that owns its cache must not)")
        T = ctx.n_tokens
        proj = self.in_proj.forward(x)
        if self.q_rank:      # queries through their own latent: norm (float32 statistics), then the up-projection
            q = self.q_up.forward(ops.rmsnorm_rows(proj[:, : self.q_rank], self.q_norm_w, self.norm_eps))
            at = self.q_rank
        else:
            q = proj[:, : self.q_width]
            at = self.q_width
        if self.gated:
            gate = proj[:, at: at + nh]
            at += nh
        else:       # sigmoid(+large) = 1: one constant row, read by every token (row stride 0)
            gate = self.open_gate.expand(T, nh)
        dkv = None if self.shares_cache else proj[:, at: at + rank + dr]
        pages = self._pages(cache)
        ops.latent_prepare(q, dkv, self.latent_norm_w, self.inv_freq, ctx, cache.block_table,
                           None if self.shares_cache else pages, cache.page_size, nh, dn, dr, self.rot_dims, rank,
                           self.norm_eps, neighbours=self.rot_pairing == "neighbours", magnitude=self.rot_magnitude)
        q3 = q.unflatten(1, (nh, dn + dr))
        qa = torch.empty((T, nh, rank), dtype=proj.dtype, device=proj.device)
        ops.gemm_batched(q3[:, :, :dn], self.w_uk_t, qa)
        lat = torch.empty((T, nh, rank), dtype=proj.dtype, device=proj.device)
        tiles = self._tiles(ctx) if _LATENT_MMA and proj.dtype == torch.bfloat16 else None
        if tiles is not None and ops.latent_attention_prefill(
                qa, q, gate, pages, cache.block_table, ctx, tiles[0], tiles[1], lat, nh, dn, dr, rank, cache.page_size,
                self.window, self.scale):
            out = torch.empty((T, nh, self.vdim), dtype=proj.dtype, device=proj.device)
            ops.gemm_batched(lat, self.w_uv, out)
            return self.o_proj.forward(out.view(T, nh * self.vdim))
        # Steps of few tokens cut the visible keys over several blocks. The span is what the step's shape implies (the
        # window, else what the block table can hold), not the requests' lengths: a captured step replays it.
        span = self.window if self.window > 0 else cache.block_table.size(1) * cache.page_size
        splits, split_keys = ops.latent_attention_splits(
            T, nh, span, ops.sm_count(proj.device),
            mma=T <= ops.LATENT_FEW_TOKENS and ops.latent_decode_takes_mma(proj.dtype, rank, dr, cache.page_size))
        ops.latent_attention(qa, q, gate, pages, cache.block_table, ctx, lat, nh, dn, dr, rank, cache.page_size,
                             self.window, self.scale, splits=splits, split_keys=split_keys)
        out = torch.empty((T, nh, self.vdim), dtype=proj.dtype, device=proj.device)
        ops.gemm_batched(lat, self.w_uv, out)
        return self.o_proj.forward(out.view(T, nh * self.vdim))

    @staticmethod
    def _pages(cache):
        """The entry's pages as one tensor [pages, page_size * (rank + rot_dim)]: plane 0 (the latents) and plane 1
        (the rotated key parts) of a page follow one another."""
        p0 = cache.planes[0]
        return p0.as_strided((p0.size(0), p0.stride(0)), (p0.stride(0), 1), p0.storage_offset())
