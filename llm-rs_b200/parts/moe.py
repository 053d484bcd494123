"""Mixtures of experts."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import FeedForward, Runtime
from .registry import register
from .spec import WeightSpec


@register("feed_forward", "moe")
class MixtureOfExperts(FeedForward):
    """``experts`` small gated feed-forward layers of which every token uses ``top``; the output is the weighted sum
    of the chosen experts' outputs.

    Expert (no biases): ``g = min(W_gate x, limit)``, ``u = clamp(W_up x, -limit, limit)``,
    ``y = g * sigmoid(alpha * g) * (u + up_shift)``, output ``W_down y``; ``limit``, ``alpha`` and ``up_shift`` are
    parameters.

    Router ``"table"``: no learned router; an integer table [vocab, top] names each token id's experts (the entries
    of a row differ), each weighted 1/top. Router ``"linear"``: logits ``W_router x + b`` as a float32 product (x may be
    its rounding to the activation type), the ``top`` largest are chosen (the lower expert among equals) and weighted
    by the softmax over the chosen logits only. Router ``"softmax_bias"``: the same float32 logits without a bias, over
    ``experts + n_identity`` outputs; scores ``s = softmax(logits)`` over all of them; the ``top`` largest ``s +
    correction`` are chosen (``correction``: one stored number per output, which steers the choice only) and weighted
    by ``s`` itself, not renormalised. The last ``n_identity`` outputs are identity experts: no tensors, their output
    is the feed-forward's input times the weight. A router only fills (expert, weight) per assignment on the device; the
    grouping of rows by expert, the two grouped products and the weighted sum do not depend on which router ran.

    ``limit`` None leaves gate and up unclamped; with ``alpha`` 1 and ``up_shift`` 0 the unit is ``silu(g) * u``.

    ``shared_size`` > 0 adds an expert of that size and the same form that every token uses (one fused gate|up
    product, as the dense gated feed-forward); with ``shared_gated`` its output is multiplied by
    ``sigmoid(w_sg . x)``, one number per token, computed beside the router's logits.

    The rows are sorted by expert so that a tile of rows shares one expert's weights; the first product has the gated
    unit as its epilogue; bfloat16 products run on the tensor cores (``csrc/gemm_grouped.cu``). ``forward`` takes the
    float32 residual stream itself (``reads_residual``) and rounds its rows to the activation type. Tensor names: ``<prefix>e<i>.gate|up|down`` and
    ``<prefix>table`` unless ``names`` renames the roles."""

    reads_residual = True
    ROLES = ("expert", "gate", "up", "down", "table", "router", "router_bias", "shared", "shared_gate", "correction")
    ROUTERS = ("table", "linear", "softmax_bias")

    def __init__(self, hidden_size: int, expert_size: int, n_experts: int, top: int, vocab_size: int = 0,
                 router: str = "table", limit: Optional[float] = 1.0, alpha: float = 1.702, up_shift: float = 1.0,
                 shared_size: int = 0, shared_gated: bool = False, n_identity: int = 0, names=None, prefix: str = ""):
        if router not in self.ROUTERS:
            raise ValueError(f"unknown router {router!r}; known: {self.ROUTERS}")
        if n_identity and router != "softmax_bias":
            raise ValueError(f"identity experts come with the router 'softmax_bias', not {router!r}")
        if n_identity and shared_size:
            raise ValueError("identity experts beside a shared expert: not built")
        if not 1 <= top <= n_experts + n_identity:
            raise ValueError(f"top {top} of {n_experts + n_identity} experts")
        self.n_identity = int(n_identity)
        if router == "table" and vocab_size < 1:
            raise ValueError("the table router needs the vocabulary's size")
        self.hidden_size, self.expert_size, self.n_experts, self.top = hidden_size, expert_size, n_experts, top
        self.vocab_size, self.router = vocab_size, router
        self.limit = float("inf") if limit is None else float(limit)
        self.alpha, self.up_shift = float(alpha), float(up_shift)
        self.shared_size, self.shared_gated = int(shared_size), bool(shared_gated) and shared_size > 0
        self.prefix = prefix
        self.names = {"expert": "e{}.", "gate": "gate", "up": "up", "down": "down", "table": "table",
                      "router": "router", "router_bias": "router.b", "shared": "shared.", "shared_gate": "shared.sg",
                      "correction": "correction"}
        self.names.update(names or {})
        if set(self.names) != set(self.ROLES):
            raise ValueError(f"names may rename {self.ROLES}, got {sorted(set(self.names) - set(self.ROLES))}")

    def _name(self, e: int, role: str) -> str:
        return f"{self.prefix}{self.names['expert'].format(e)}{self.names[role]}"

    def weight_specs(self):
        H, F = self.hidden_size, self.expert_size
        specs = []
        for e in range(self.n_experts):
            specs += [WeightSpec(self._name(e, "gate"), (F, H)), WeightSpec(self._name(e, "up"), (F, H)),
                      WeightSpec(self._name(e, "down"), (H, F))]
        if self.router == "table":
            specs.append(WeightSpec(self.prefix + self.names["table"], (self.vocab_size, self.top),
                                    role="expert_table", limit=self.n_experts))
        elif self.router == "linear":
            specs += [WeightSpec(self.prefix + self.names["router"], (self.n_experts, H)),
                      WeightSpec(self.prefix + self.names["router_bias"], (self.n_experts,), role="bias")]
        else:
            n_all = self.n_experts + self.n_identity
            specs += [WeightSpec(self.prefix + self.names["router"], (n_all, H)),
                      WeightSpec(self.prefix + self.names["correction"], (n_all,), role="bias")]
        if self.shared_size:
            S, sp = self.shared_size, self.prefix + self.names["shared"]
            specs += [WeightSpec(sp + self.names["gate"], (S, H)), WeightSpec(sp + self.names["up"], (S, H)),
                      WeightSpec(sp + self.names["down"], (H, S))]
            if self.shared_gated:
                specs.append(WeightSpec(self.prefix + self.names["shared_gate"], (1, H)))
        return specs

    def bind(self, tensors, runtime: Runtime):
        self.act_dtype = runtime.act_dtype
        stack = lambda role: torch.stack([tensors[self._name(e, role)] for e in range(self.n_experts)]).contiguous()
        self.w_gate, self.w_up, self.w_down = stack("gate"), stack("up"), stack("down")
        if len({self.w_gate.dtype, self.w_up.dtype, self.w_down.dtype}) != 1:
            self.w_gate, self.w_up, self.w_down = (w.to(torch.float32) for w in (self.w_gate, self.w_up, self.w_down))
        self.table = self.router_w = self.router_w_stored = self.router_b = self.shared = None
        if self.router == "table":
            self.table = tensors[self.prefix + self.names["table"]].contiguous()
            bad = (self.table < 0) | (self.table >= self.n_experts)
            if bool(bad.any()):
                raise ValueError(f"{self.prefix}{self.names['table']} names experts outside 0..{self.n_experts - 1}")
        rows, bias = [], []
        if self.router == "linear":
            rows.append(tensors[self.prefix + self.names["router"]])
            bias.append(tensors[self.prefix + self.names["router_bias"]].to(torch.float32))
        self.correction = None
        if self.router == "softmax_bias":
            rows.append(tensors[self.prefix + self.names["router"]])
            bias.append(torch.zeros((rows[-1].size(0),), dtype=torch.float32, device=rows[-1].device))
            self.correction = tensors[self.prefix + self.names["correction"]].to(torch.float32).contiguous()
        if self.shared_gated:       # the shared expert's gate is one more row of the router's product
            rows.append(tensors[self.prefix + self.names["shared_gate"]])
            bias.append(torch.zeros((1,), dtype=torch.float32, device=rows[-1].device))
        if rows:
            self.router_w = torch.cat([r.to(torch.float32) for r in rows], dim=0).contiguous()
            self.router_b = torch.cat(bias, dim=0).contiguous()
            # The same rows as the folder stores them (see ``ops.product_f32``).
            same = all(r.dtype == rows[0].dtype for r in rows)
            self.router_w_stored = torch.cat(rows, dim=0).contiguous() if same else self.router_w
        if self.shared_size:
            from .mlp import SwiGLU
            sp = self.prefix + self.names["shared"]
            self.shared = SwiGLU(self.hidden_size, self.shared_size)
            self.shared.bind({self.shared._name(r): tensors[sp + self.names[r]] for r in ("gate", "up", "down")}, runtime)

    def forward(self, x, ctx):
        """x: the step's rows, float32 (the residual stream) or the activation type. Returns float32 [tokens, hidden]."""
        if self.act_dtype == torch.bfloat16 and x.dtype == torch.float32:
            x = ops.token_shift(x, None, None, None, torch.bfloat16)     # the rows as activations: the tensor cores' type
        logits = (ops.product_f32(x, self.router_w_stored, self.router_w, self.router_b)
                  if self.router_w is not None else None)
        if self.router == "table":
            expert_of, weight_of = ops.moe_route_table(ctx.token_ids, self.table, self.n_experts)
        elif self.router == "linear":
            expert_of, weight_of = ops.moe_route_top(logits, self.n_experts, self.top)
        else:
            expert_of, weight_of = ops.moe_route_biased(logits, self.correction, self.n_experts + self.n_identity,
                                                        self.n_experts, self.top)
        n_rows = expert_of.numel()
        tile_rows = ops.grouped_tile_rows(n_rows, self.n_experts)
        if self.n_identity:
            # Assignments to identity experts are sorted into one more group that runs no product; the weighted sum
            # takes the token's own row for them.
            row_of, src_token, tiles, n_tiles = ops.moe_sort(expert_of, self.top, self.n_experts + 1, tile_rows,
                                                             tiled_groups=self.n_experts)
        else:
            row_of, src_token, tiles, n_tiles = ops.moe_sort(expert_of, self.top, self.n_experts, tile_rows)
        act = torch.empty((n_rows, self.expert_size), dtype=self.act_dtype, device=x.device)
        ops.gemm_grouped(x, self.w_gate, act, tiles, n_tiles, src_token, w2=self.w_up, limit=self.limit,
                         alpha=self.alpha, shift=self.up_shift, tile_rows=tile_rows)
        rows = torch.empty((n_rows, self.hidden_size), dtype=torch.float32, device=x.device)
        ops.gemm_grouped(act, self.w_down, rows, tiles, n_tiles, None, tile_rows=tile_rows)
        if self.n_identity:
            return ops.moe_combine_identity(rows, row_of, weight_of, expert_of, x, self.top, self.n_experts)
        if self.shared is None:
            return ops.moe_combine(rows, row_of, weight_of, self.top)
        gate = logits[:, logits.size(1) - 1] if self.shared_gated else None
        return ops.moe_combine_shared(rows, row_of, weight_of, self.top, self.shared.forward(x, ctx), gate)
