"""Token embedding and the output head."""
from __future__ import annotations

import torch

from .. import ops
from .base import Part, Runtime
from .linear import Linear
from .registry import register
from .spec import StateNeed, WeightSpec


@register("embedding", "token_embedding")
class TokenEmbedding(Part):
    """``h0[t] = table[id_t]``, no scale (llm-core/src/graph/builder.rs:8-14,
    llm-core/src/backends/candle.rs:1238-1261). The result is the float32 residual stream."""

    def __init__(self, vocab_size: int, hidden_size: int, name: str = "embedding.weight", prefix: str = ""):
        self.vocab_size, self.hidden_size, self.name = vocab_size, hidden_size, prefix + name

    def weight_specs(self):
        return [WeightSpec(self.name, (self.vocab_size, self.hidden_size), role="embedding")]

    def bind(self, tensors, runtime: Runtime):
        self.table = tensors[self.name]

    def forward(self, token_ids):
        return ops.embedding(self.table, token_ids)


@register("embedding", "pair_embedding")
class PairEmbedding(Part):
    """``h0[t] = table[id_t] * scale + pairs[(id_(t-1) * mul_prev + id_t * mul_cur) mod buckets]``: a token embedding
    with a scale plus a hashed embedding of the token PAIR; a sequence's first token takes row number ``buckets`` (the
    last row) of the pair table. The token before a step's first token of a request is per-request state (one number
    per slot, kept by the cache manager with the first run-order entry's state), so a sequence may be cut anywhere and
    decode steps replay from CUDA graphs. ``buckets`` 0: no pair table. The result is the float32 residual stream,
    written ``streams`` times side by side for a model whose blocks keep several streams."""
    STATE = "embedding.previous_token"
    needs_context = True

    def __init__(self, vocab_size: int, hidden_size: int, scale: float = 1.0, buckets: int = 0, mul_prev: int = 0,
                 mul_cur: int = 0, streams: int = 1, name: str = "embedding.weight", pairs_name: str = "pairs",
                 prefix: str = ""):
        if buckets < 0 or mul_prev < 0 or mul_cur < 0 or streams < 1:
            raise ValueError(f"pair embedding: buckets {buckets}, multipliers {mul_prev} / {mul_cur}, {streams} streams")
        if vocab_size > 1 << 24:
            raise ValueError(f"a vocabulary of {vocab_size} does not fit the previous token's float32 state")
        self.vocab_size, self.hidden_size, self.scale = vocab_size, hidden_size, float(scale)
        self.buckets, self.mul_prev, self.mul_cur, self.streams = int(buckets), int(mul_prev), int(mul_cur), int(streams)
        self.name, self.pairs_name = prefix + name, prefix + pairs_name

    def weight_specs(self):
        specs = [WeightSpec(self.name, (self.vocab_size, self.hidden_size), role="embedding")]
        if self.buckets:
            specs.append(WeightSpec(self.pairs_name, (self.buckets + 1, self.hidden_size), role="embedding"))
        return specs

    def bind(self, tensors, runtime: Runtime):
        self.table = tensors[self.name]
        self.pairs = tensors[self.pairs_name] if self.buckets else None
        if self.pairs is not None and self.pairs.dtype != self.table.dtype:
            self.table, self.pairs = self.table.to(torch.float32), self.pairs.to(torch.float32)

    def state_need(self):
        return StateNeed({self.STATE: (1,)}) if self.buckets else None

    def forward(self, ctx, state):
        return ops.bigram_embedding(self.table, self.pairs, ctx, state.get(self.STATE) if self.buckets else None,
                                    self.streams, self.scale, self.buckets, self.mul_prev, self.mul_cur)


@register("lm_head", "linear_head")
class LinearHead(Part):
    """``logits = x @ W^T`` in float32, no bias, no soft cap
    (llm-core/src/graph/builder.rs:408-437). ``tied_to`` names the embedding table that
    serves as W when the model ties them (llm-core/src/backends/weights.rs:144-157): one
    buffer, used by both. A tied model's folder may still store the head's matrix (a copy of the
    table); it is accepted and not read. ``scale`` other than 1 multiplies the float32 logits; ``softcap`` > 0:
    ``logits = softcap * tanh(logits / softcap)`` (after the scale)."""

    def __init__(self, vocab_size: int, hidden_size: int, name: str = "head.weight", tied_to: str = "",
                 softcap: float = 0.0, scale: float = 1.0, prefix: str = ""):
        self.vocab_size, self.hidden_size, self.softcap = vocab_size, hidden_size, float(softcap)
        self.scale = float(scale)
        self.name, self.tied_to = prefix + name, tied_to

    def weight_specs(self):
        if self.tied_to:
            return [WeightSpec(self.name, (self.vocab_size, self.hidden_size), optional=True, load=False)]
        return [WeightSpec(self.name, (self.vocab_size, self.hidden_size))]

    def bind(self, tensors, runtime: Runtime):
        self.proj = Linear(tensors[self.tied_to or self.name], None, runtime.act_dtype)

    def chain(self):
        return [self.proj]

    def forward(self, x):
        logits = self.proj.forward(x, out_dtype=torch.float32)
        if self.scale != 1.0:
            ops.scale_(logits, self.scale)
        return ops.softcap_(logits, self.softcap) if self.softcap > 0 else logits


@register("reentry", "embedding_mix")
class EmbeddingMix(Part):
    """``h <- W [h ; h0]`` with ``W`` of shape [hidden, 2 hidden] (the stream's half first) and ``h0`` the embedding
    output: what a looped stretch of layers does to the stream ahead of every pass. The product is split into its two
    halves, ``W_a h + W_b h0``; the second term is the same in every pass of a step and is made once (``prepare``).
    The rows enter the products in the activation type; the sum and the new stream are float32."""

    def __init__(self, hidden_size: int, name: str = "loop.in", prefix: str = ""):
        self.hidden_size, self.name = hidden_size, prefix + name

    def weight_specs(self):
        return [WeightSpec(self.name, (self.hidden_size, 2 * self.hidden_size))]

    def bind(self, tensors, runtime: Runtime):
        w, D = tensors[self.name], self.hidden_size
        self.act_dtype = runtime.act_dtype
        self.of_stream = Linear(w[:, :D].contiguous(), None, runtime.act_dtype)
        self.of_embedding = Linear(w[:, D:].contiguous(), None, runtime.act_dtype)
        self.of_stream.warms_next = self.of_embedding.warms_next = False

    def prepare(self, h0, ctx):
        """``W_b h0`` in float32 for the step's tokens."""
        return self.of_embedding.forward(ops.token_shift(h0, None, None, ctx, self.act_dtype), out_dtype=torch.float32)

    def forward(self, h, pending, entered, ctx):
        """The new stream (a tensor of its own: ``h`` and ``entered`` stay as they are). ``pending`` is a branch output
        that the block before has not added yet."""
        if pending is not None:
            ops.residual_add(h, pending)
        ctx.stream_copy = None
        new = entered.clone()
        x = ops.token_shift(h, None, None, ctx, self.act_dtype)
        if x.dtype == torch.bfloat16 and self.of_stream.uses_tc(x.size(0)):
            ops.gemm_bf16(x, self.of_stream.weight, out=new, epilogue="residual")      # new += W_a x in the epilogue
        else:
            ops.residual_add(new, self.of_stream.forward(x, out_dtype=torch.float32))
        return new
