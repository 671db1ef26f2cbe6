"""A model built from a plan: embedding, the layers' blocks, final norm, output head.

``forward`` runs one step's packed tokens through the schedule and returns the
logits at the wanted rows only (the reference computes logits for every row of
a prompt and keeps the last, core/runtime.cpp:1093-1095, 3179-3183).
"""
from __future__ import annotations

import torch

from ..parts.base import BoundWeights, Runtime, StepContext, UnitCache
from ..parts.linear import settle
from ..parts.registry import build_part
from ..weights.manifest import TensorSpec
from .plan import ModelPlan


class Model:
    def __init__(self, plan: ModelPlan, runtime: Runtime):
        plan.validate()
        self.plan = plan
        self.runtime = runtime
        self.embedding = build_part("embedding", plan.embedding, runtime)
        self._positions: dict = {}
        self.blocks = []
        for layer in plan.layers:
            position = None
            if layer.position is not None:
                key = (layer.position.kind, tuple(sorted(layer.position.params.items())))
                if key not in self._positions:          # layers with the same encoding share one object
                    self._positions[key] = build_part("position", layer.position, runtime)
                position = self._positions[key]
            self.blocks.append(build_part("block", layer.block, runtime, layer=layer, position=position))
        self.final_norm = build_part("norm", plan.final_norm, runtime)
        self.head = build_part("head", plan.head, runtime)
        self.schedule = list(plan.schedule)

    # ---- weights
    def parts(self):
        return [self.embedding, *self.blocks, self.final_norm, self.head]

    def tensors(self) -> list[TensorSpec]:
        seen, out = set(), []
        for part in self.parts():
            for t in part.tensors():
                if t.name not in seen:
                    seen.add(t.name)
                    out.append(t)
        return out

    def bind(self, weights: dict) -> None:
        """Hand every part its tensors.  Tensors that a part only copies from (into a fused matrix) are taken out of
        ``weights`` as the binding goes, unless another part names them too."""
        uses: dict = {}
        for part in self.parts():
            for t in part.tensors():
                uses[t.name] = uses.get(t.name, 0) + 1
        bound = BoundWeights(weights, uses)
        for part in self.parts():
            part.bind(bound)

    def kernel_modules(self) -> list[str]:
        mods = []
        for part in self.parts() + list(self._positions.values()):
            for m in part.kernel_modules():
                if m not in mods:
                    mods.append(m)
        return mods

    # ---- cache needs, one entry per scheduled run
    def cache_units(self):
        """[(kv_spec or None, state_spec or None, cache_of or None)] in schedule order."""
        out = []
        for run in self.schedule:
            mixer = self.blocks[run.layer].mixer
            out.append((mixer.kv_spec(), mixer.state_spec(), run.cache_of))
        return out

    # ---- one step
    def forward(self, ctx: StepContext, unit_caches: list[UnitCache], want_rows: torch.Tensor) -> torch.Tensor:
        for position in self._positions.values():       # the step's tables first: no layer's kernels find them half made
            position.prepare(ctx)
        h = self.embedding.forward(ctx.token_ids)
        delta = None
        for i, run in enumerate(self.schedule):
            h, delta = self.blocks[run.layer].forward(h, delta, ctx, unit_caches[i])
        if want_rows.numel() == 0:
            return torch.empty((0, self.plan.vocab_size), dtype=torch.float32, device=h.device)
        x = self.final_norm.forward(h, settle(h, delta, self.final_norm), rows=want_rows)
        return self.head.forward(x)
