"""Grouped-query attention whose scores are capped or biased by distance, whose softmax has a sink, and whose mask may
be a window or chunked."""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import host, ops
from .attention import _ATTN_TC, PREFILL_TILE
from .base import Mixer, Plan, Runtime, StepInfo
from .linear import Linear
from .registry import register
from .spec import CacheNeed, WeightSpec

MASKS = {"causal": ops.MASK_CAUSAL, "window": ops.MASK_WINDOW, "chunk": ops.MASK_CHUNK}
# Keys per block of the decode kernel at least, doubled while a step has too many blocks: a block of the kernel that
# takes a key head's query heads together walks 128 keys a turn (a lane per key), the kernel of a warp per key 16.
DECODE_SPLIT_KEYS = {True: 128, False: 64}
DECODE_MAX_BLOCKS = 8192


@register("mixer", "scored_attention")
class ScoredAttention(Mixer):
    """``n_heads`` query heads over ``n_kv_heads`` key/value heads (query head h reads key head h // (n_heads /
    n_kv_heads)); keys of ``dim`` channels, values of ``vdim``. In order:

    q, k, v projections (no biases) -> RMS norm over the WHOLE q row and the whole k row, all heads at once, with
    plain weights of that size (``qk_norm`` "whole"; "none": no norm) -> rotation of the first ``rot_dims`` channels
    of every head, channel i paired with i + rot_dims/2, angle position * rot_base^(-2i/rot_dims) (q and k, not v)
    -> with ``qk_norm`` "head_unit": every head of q and k divided by its own root mean square, AFTER the rotation,
    without a weight -> new keys and values into the pages -> score = (q . k) * ``scale``, then ``softcap * tanh(score / softcap)``
    when ``softcap`` > 0 -> mask: causal, and with ``mask`` "window" the last ``mask_size`` keys, with "chunk" only
    keys of the query's own chunk of ``mask_size`` positions (chunks counted from position 0 of the sequence) ->
    softmax whose denominator also holds exp(sink_h), one learned number per query head (``sink``; it has no key
    and no value and is neither scaled nor capped) -> output projection.

    Options on the values and the score: ``v_norm`` "head_unit" divides every head's value by its own root mean square
    (no weight) before it is kept in the pages. ``v_mix`` "source" publishes the layer's values of the step's tokens
    under ``v_mix_key`` for later layers; "mixed" keeps ``(1 - m) v + m v_first`` in the pages instead of v, with
    ``v_first`` what the source layer published and ``m`` the layer's own learned number (role ``vmix``). ``bias_rows``
    > 0: a learned table [bias_rows, heads] (role ``rel``) adds ``rel[bucket(query - key), head]`` to the score after
    the scale (it is neither scaled nor capped, and the sink gets none), with ``bucket(n) = n`` below half the rows
    and ``min(rows - 1, half + floor(ln(n / half) / ln(bias_max / half) * (rows - half)))`` from there on; the table
    is laid out per distance once at load. ``heads(...)`` gives the concatenated heads before the output projection,
    optionally scaled and written into a view, for a mixer that runs this one beside another.

    Scores, weights, norms, positions and angles are float32 (angles are made in double). Pages: a group of kind
    "window" for the masks that bound how far back a query reads (a chunk never reaches further back than
    ``mask_size`` - 1 keys), else "full"; a token stores ``dim`` + ``vdim`` numbers per key head. Prompt portions run
    on the tensor cores in bfloat16 (``csrc/attention_scored.cu``: ``mma.sync``; long portions of heads of 128
    channels: the tcgen05 kernel of ``csrc/attention_tc.cu``, which takes the cap, the sink and the mask in its
    softmax; ``LLMRS_ATTN_TC=0`` keeps ``mma.sync``); requests that bring one token take the decode kernel in the
    same step. ``names`` maps the roles q, k, v, o, q_norm, k_norm, sink, g, rel, vmix."""
    ROLES = ("q", "k", "v", "o", "q_norm", "k_norm", "sink", "g", "rel", "vmix")

    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, dim: int, vdim: int, scale: float,
                 softcap: float = 0.0, sink: bool = False, mask: str = "causal", mask_size: int = 0,
                 qk_norm: str = "whole", norm_eps: float = 1e-6, rot_dims: int = 0, rot_base: float = 10000.0,
                 gated: bool = False, v_norm: str = "none", v_mix: str = "none", v_mix_key: str = "v_first",
                 bias_rows: int = 0, bias_max: float = 0.0, names=None, prefix: str = ""):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} query heads are no multiple of {n_kv_heads} key/value heads")
        if mask not in MASKS or (mask != "causal" and mask_size < 1):
            raise ValueError(f"mask {mask!r} of size {mask_size}; known masks: {sorted(MASKS)}")
        if qk_norm not in ("whole", "none", "head_unit"):
            raise ValueError(f"unknown qk_norm {qk_norm!r}; known: 'whole', 'none', 'head_unit'")
        if rot_dims % 2 or not 0 <= rot_dims <= dim:
            raise ValueError(f"rot_dims {rot_dims} must be even and at most dim {dim}")
        if not (1 <= dim <= 256 and 1 <= vdim <= 256):
            raise ValueError(f"head sizes {dim} / {vdim}: the attention kernels take 1 to 256")
        if v_norm not in ("none", "head_unit") or v_mix not in ("none", "source", "mixed"):
            raise ValueError(f"v_norm {v_norm!r} (known: 'none', 'head_unit'), v_mix {v_mix!r} (known: 'none', 'source', "
                             "'mixed')")
        if v_mix == "source" and v_norm != "none":
            raise ValueError("a layer whose values are normed per head cannot be the source of mixed values")
        if bias_rows and (bias_rows < 2 or bias_max <= bias_rows // 2):
            raise ValueError(f"a distance bias of {bias_rows} rows reaching to {bias_max}: at least 2 rows, and the "
                             "reach beyond half of them")
        self.hidden_size, self.n_heads, self.n_kv_heads, self.dim, self.vdim = hidden_size, n_heads, n_kv_heads, dim, vdim
        self.scale, self.softcap, self.has_sink = float(scale), float(softcap), bool(sink)
        self.mask, self.mask_size = mask, int(mask_size) if mask != "causal" else 0
        self.qk_norm, self.norm_eps = qk_norm, float(norm_eps)
        self.rot_dims, self.rot_base = int(rot_dims), float(rot_base)
        self.gated = bool(gated)
        self.v_norm, self.v_mix, self.v_mix_key = v_norm, v_mix, v_mix_key
        self.bias_rows, self.bias_max = int(bias_rows), float(bias_max)
        self.prefix = prefix
        self.names = {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "sink": "sink",
                      "g": "g", "rel": "rel", "vmix": "vmix"}
        self.names.update(names or {})
        if set(self.names) != set(self.ROLES):
            raise ValueError(f"names may rename {self.ROLES}, got {sorted(set(self.names) - set(self.ROLES))}")
        self.q_width, self.k_width, self.v_width = n_heads * dim, n_kv_heads * dim, n_kv_heads * vdim

    def _name(self, role: str) -> str:
        return self.prefix + self.names[role]

    def weight_specs(self):
        H, nm = self.hidden_size, self._name
        specs = [WeightSpec(nm("q"), (self.q_width, H)), WeightSpec(nm("k"), (self.k_width, H)),
                 WeightSpec(nm("v"), (self.v_width, H)), WeightSpec(nm("o"), (H, self.n_heads * self.vdim))]
        if self.qk_norm == "whole":
            specs += [WeightSpec(nm("q_norm"), (self.q_width,), role="norm"),
                      WeightSpec(nm("k_norm"), (self.k_width,), role="norm")]
        if self.has_sink:
            specs.append(WeightSpec(nm("sink"), (self.n_heads,), role="bias"))
        if self.gated:
            specs.append(WeightSpec(nm("g"), (self.n_heads, H)))
        if self.bias_rows:
            specs.append(WeightSpec(nm("rel"), (self.bias_rows, self.n_heads), role="bias"))
        if self.v_mix != "none":      # the source layer's number is stored too, and unused
            specs.append(WeightSpec(nm("vmix"), (), role="bias", optional=self.v_mix == "source",
                                    load=self.v_mix == "mixed"))
        return specs

    def bind(self, tensors, runtime: Runtime):
        nm = self._name
        self.act_dtype = runtime.act_dtype
        ws = [tensors[nm(r)] for r in "qkv"]
        if self.gated:
            # The gates' rows follow v's in the same product; zero rows fill up to a multiple of eight, so that a
            # product whose width fitted the tensor-core kernels still does.
            g = tensors[nm("g")]
            fill = -(self.q_width + self.k_width + self.v_width + self.n_heads) % 8
            ws += [g, g.new_zeros((fill, g.size(1)))] if fill else [g]
        dt = ws[0].dtype if all(w.dtype == ws[0].dtype for w in ws) else torch.float32
        wqkv = torch.cat([w.to(dt) for w in ws], dim=0).contiguous()
        self.qkv_proj = Linear(wqkv, None, runtime.act_dtype)
        # For entries that read another's pages: the queries (and the gates) alone.
        wq = wqkv[: self.q_width] if not self.gated else torch.cat(
            [wqkv[: self.q_width], wqkv[self.q_width + self.k_width + self.v_width:]], dim=0).contiguous()
        self.q_proj = Linear(wq, None, runtime.act_dtype)
        self.o_proj = Linear(tensors[nm("o")], None, runtime.act_dtype)
        f32 = lambda role: tensors[nm(role)].to(torch.float32).contiguous()
        self.q_norm_w = f32("q_norm") if self.qk_norm == "whole" else None
        self.k_norm_w = f32("k_norm") if self.qk_norm == "whole" else None
        self.sink = f32("sink") if self.has_sink else None
        i = torch.arange(self.rot_dims // 2, dtype=torch.float64)
        self.inv_freq = (self.rot_base ** (-2.0 * i / max(self.rot_dims, 1))).to(runtime.device)
        self.v_mix_w = f32("vmix").reshape(1) if self.v_mix == "mixed" else None
        self.bias = None
        if self.bias_rows:
            # One row per distance: a query never looks further back than its mask allows, and from ``bias_max`` on
            # every distance falls into the last bucket (the kernels take the last row for anything beyond the table).
            reach = min(runtime.max_positions, int(math.ceil(self.bias_max)) + 1)
            if self.mask_size:
                reach = min(reach, self.mask_size)
            buckets = torch.tensor([distance_bucket(n, self.bias_rows, self.bias_max) for n in range(max(reach, 1))],
                                   dtype=torch.long, device=runtime.device)
            self.bias = f32("rel").index_select(0, buckets).contiguous()

    def cache_need(self):
        kind = "full" if self.mask == "causal" else "window"
        return CacheNeed(kind, self.n_kv_heads, self.dim, self.mask_size, planes=(self.dim, self.vdim))

    # The plan of paged attention (tiles of prompt portions, the list of single tokens) is the one grouped-query
    # attention makes: layers of either kind share it within a step.
    def plan_key(self):
        return ("paged_attention", PREFILL_TILE)

    def plan(self, step: StepInfo) -> Plan:
        tiles, decode, max_kv, long_portions = host.plan_paged_attention(step.n_new, step.cached_len, PREFILL_TILE)
        if step.for_graph and decode.size and step.block_tables:
            max_kv = max(t.shape[1] for t in step.block_tables) * step.page_size
        return Plan(arrays={"prefill_tiles": tiles, "decode_reqs": decode},
                    values={"n_prefill_tiles": int(tiles.shape[0]), "n_decode": int(decode.size),
                            "max_decode_kv_len": int(max_kv), "long_portions": int(long_portions)})

    def heads(self, x, ctx, cache, out: Optional[torch.Tensor] = None, out_scale: float = 1.0) -> torch.Tensor:
        """The concatenated heads [tokens, n_heads * vdim] before the output projection, times ``out_scale``, written
        into ``out`` (a view with dense rows) when given."""
        table = cache.block_table
        if cache.owns:
            qkv = self.qkv_proj.forward(x)
            q = qkv[:, : self.q_width]
            k = qkv[:, self.q_width: self.q_width + self.k_width]
            at = self.q_width + self.k_width + self.v_width
            v = qkv[:, self.q_width + self.k_width: at]
            gate = qkv[:, at: at + self.n_heads] if self.gated else None
        else:
            qg = self.q_proj.forward(x)
            q, k, v = qg[:, : self.q_width], None, None
            gate = qg[:, self.q_width: self.q_width + self.n_heads] if self.gated else None
        v_first = None
        if v is not None and self.v_mix == "source":
            ctx.shared[self.v_mix_key] = v          # stays alive with the context: later layers of the step read it
        elif v is not None and self.v_mix == "mixed":
            v_first = ctx.shared[self.v_mix_key]
        pages = _pages(cache)
        ops.scored_prepare(q, k, v, self.q_norm_w, self.k_norm_w, self.inv_freq, ctx, table,
                           pages if cache.owns else None, self.n_heads, self.n_kv_heads, self.dim, self.vdim,
                           self.rot_dims, cache.page_size, self.norm_eps, unit_heads=self.qk_norm == "head_unit",
                           unit_values=self.v_norm == "head_unit", v_first=v_first,
                           v_mix=self.v_mix_w if v_first is not None else None)
        if out is None:
            out = torch.empty((ctx.n_tokens, self.n_heads * self.vdim), dtype=q.dtype, device=q.device)
        plan = ctx.plan(self.plan_key())
        n_tiles, n_decode, max_kv = (plan.values[key] for key in ("n_prefill_tiles", "n_decode", "max_decode_kv_len"))
        mask = MASKS[self.mask]
        args = (self.n_heads, self.n_kv_heads, self.dim, self.vdim, cache.page_size, self.scale, self.softcap,
                self.sink, mask, self.mask_size)
        scale = 1.0 if self.gated else out_scale      # with a gate the scale goes on after it
        if n_tiles:
            ops.scored_prefill(q, out, pages, plan.arrays["prefill_tiles"], n_tiles, ctx, table, *args,
                               prefer_tc=bool(plan.values["long_portions"]) and _ATTN_TC, bias=self.bias,
                               out_scale=scale)
        if n_decode:
            span = max(1, min(max_kv, self.mask_size) if self.mask_size else max_kv)   # keys a query can see at most
            group = ops.scored_decode_group(self.n_heads, self.n_kv_heads, self.dim, self.vdim, cache.page_size, q.dtype)
            split_keys = DECODE_SPLIT_KEYS[group > 0]
            blocks = n_decode * self.n_kv_heads * -(-(self.n_heads // self.n_kv_heads) // group) if group else \
                n_decode * self.n_heads
            while blocks * -(-span // split_keys) > DECODE_MAX_BLOCKS and split_keys < 4096:
                split_keys *= 2
            ops.scored_decode(q, out, pages, plan.arrays["decode_reqs"], n_decode, ctx, table, -(-span // split_keys),
                              split_keys, *args, bias=self.bias, out_scale=scale)
        if gate is not None:
            ops.head_gate(out, gate, self.n_heads, self.vdim)
            if out_scale != 1.0:
                out.mul_(out_scale)
        return out

    def forward(self, x, ctx, cache, out_dtype=None):
        return self.o_proj.forward(self.heads(x, ctx, cache), out_dtype=out_dtype)


def distance_bucket(n: int, rows: int, reach: float) -> int:
    """The row of a bias table of ``rows`` rows for a key ``n`` >= 0 positions behind its query: one row per distance
    below half the rows, then rows spaced by the logarithm of the distance up to ``reach``, the last row beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(reach / half) * (rows - half))))


def _pages(cache) -> torch.Tensor:
    """One entry's pages as the kernels address them: [pages, key heads, page_size * (dim + vdim)]. The planes are
    views into that tensor; the first one starts where it starts."""
    keys, values = cache.planes
    n_pages, n_heads, page_size, dk = keys.shape
    return keys.as_strided((n_pages, n_heads, page_size * (dk + values.size(3))),
                           (keys.stride(0), keys.stride(1), 1), keys.storage_offset())
