"""A decoder model assembled from a ``ModelSpec``: embedding, blocks in run order, final
norm, output head. It knows parts and their interfaces, not architectures."""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .base import Runtime
from .registry import build
from .spec import CacheNeed, ModelSpec, StateNeed, WeightSpec


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        spec.validate()
        self.spec = spec
        self.embedding = build("embedding", spec.embedding)
        self.blocks = [build("block", layer.block, layer=layer) for layer in spec.layers]
        self.final_norm = build("norm", spec.final_norm)
        self.lm_head = build("lm_head", spec.lm_head)
        self.reentry = build("reentry", spec.reentry) if spec.reentry is not None else None

    def parts(self):
        extra = [self.reentry] if self.reentry is not None else []
        return [self.embedding, *extra, *self.blocks, self.final_norm, self.lm_head]

    def weight_specs(self) -> List[WeightSpec]:
        seen: Dict[str, WeightSpec] = {}
        for part in self.parts():
            for s in part.weight_specs():
                if s.name in seen and seen[s.name].shape != s.shape:
                    raise ValueError(f"two parts want {s.name} with shapes {seen[s.name].shape} and {s.shape}")
                seen.setdefault(s.name, s)
        return list(seen.values())

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        for part in self.parts():
            part.bind(tensors, runtime)
        # Every product learns which weights are streamed after its own (see ``Part.chain``).
        order = [lin for step in self.spec.run_order for lin in getattr(self.blocks[step.layer], "chain", list)()]
        order += getattr(self.lm_head, "chain", list)()
        for lin, after in zip(order, order[1:]):
            lin.next_weight = after.weight if lin.warms_next and after.weight.dtype == torch.bfloat16 else None

    def cache_needs(self) -> List[Tuple[Optional[CacheNeed], Optional[StateNeed]]]:
        """Per run-order entry: the pages and the state its mixer wants, plus the state its block wants for itself.
        An entry that reads another entry's cache wants no pages and no mixer state of its own (it sees the other
        entry's), but keeps its block's state."""
        needs = []
        # State that the embedding keeps per request (the token before a step's first) lives with the first entry's.
        of_embedding = getattr(self.embedding, "state_need", lambda: None)()
        for s, step in enumerate(self.spec.run_order):
            block = self.blocks[step.layer]
            own = getattr(block, "state_need", lambda: None)()       # state of the block itself (a token shift)
            if s == 0 and of_embedding is not None:
                own = StateNeed({**(own.tensors if own is not None else {}), **of_embedding.tensors})
            if step.cache_of is not None:
                needs.append((None, own))
            else:
                mixer = block.mixer
                state = mixer.state_need()
                if own is not None:
                    state = StateNeed({**(state.tensors if state is not None else {}), **own.tensors})
                needs.append((mixer.cache_need(), state))
        return needs

    def forward(self, ctx) -> Optional[torch.Tensor]:
        """Run the step's tokens through every run-order entry; float32 logits of the
        wanted rows ([wanted, vocab]), or None when nothing is wanted."""
        order = self.spec.run_order
        if getattr(self.embedding, "needs_context", False):      # an embedding that reads more of the step than the ids
            h = self.embedding.forward(ctx, ctx.layer_cache(0).state if order else {})
        else:
            h = self.embedding.forward(ctx.token_ids)
        pending = None
        # What the passes over a looped stretch take from the embedding output is the same in every pass: made once.
        entered = self.reentry.prepare(h, ctx) if self.reentry is not None else None
        for s, step in enumerate(order):
            block = self.blocks[step.layer]
            if step.reenter:
                h, pending = self.reentry.forward(h, pending, entered, ctx), None
            after = self.blocks[order[s + 1].layer] if s + 1 < len(order) and not order[s + 1].reenter else None
            if (getattr(block, "links_norms", False) and getattr(after, "links_norms", False)
                    and after.accepts_prenormed(ctx.n_tokens)):
                # The norm between the two blocks is spread over this block's last product and the next one's first.
                h, pending = block.forward(h, pending, ctx, ctx.layer_cache(s), next_norm=after.mixer_norm.link())
            else:
                h, pending = block.forward(h, pending, ctx, ctx.layer_cache(s))
        if ctx.n_want == 0:
            return None
        last = self.blocks[order[-1].layer] if order else None
        if hasattr(last, "leave"):
            # A block that keeps the stream in a form of its own (several streams) hands over what the last norm reads.
            x = self.final_norm.forward(last.leave(h, pending, ctx.want_rows), None)
        else:
            x = self.final_norm.forward(h, pending, rows=ctx.want_rows)
        return self.lm_head.forward(x)
