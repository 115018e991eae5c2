"""The generic decoder: built from a ``ModelSpec``, it owns the parts, runs
the schedule over a step's rows and returns logits for the wanted rows.

Order of a forward pass (infernum-llama/src/graph_builder.rs:442-536):
embedding -> scheduled layers -> final norm on the wanted rows only -> head.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..errors import ConfigError
from ..ops import core
from ..parts import (EMBEDDINGS, HEADS, NORMS, Block, ModelSpec, PagedCacheSpec, ResidualStream,
                     Runtime, StateSpec, WeightSpec, build_layer)


@dataclass(frozen=True)
class CacheNeed:
    """What one scheduled run of a layer needs from the cache manager."""

    position: int  # index in the schedule
    paged: Optional[PagedCacheSpec]
    state: Optional[StateSpec]
    cache_of: Optional[int]  # reads the cache of this earlier schedule position


class Model:
    def __init__(self, spec: ModelSpec, rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.embedding = EMBEDDINGS.get(spec.embedding.kind)(spec.embedding.params, rt)
        self.layers: List[Block] = [build_layer(ls, rt) for ls in spec.layers]
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm.params, rt)
        self.head = HEADS.get(spec.lm_head.kind)(spec.lm_head.params, rt)
        self.schedule = tuple(spec.schedule)
        for pos, item in enumerate(self.schedule):
            if not 0 <= item.layer < len(self.layers):
                raise ConfigError(f"schedule[{pos}] names layer {item.layer}, there are "
                                  f"{len(self.layers)}")
            if item.cache_of is not None and not 0 <= item.cache_of < pos:
                raise ConfigError(f"schedule[{pos}].cache_of must name an earlier position")
            if item.cache_of is not None and self.schedule[item.cache_of].cache_of is not None:
                raise ConfigError(f"schedule[{pos}].cache_of must name a run that owns its cache")
        self.bound = False

    # ---- declarations -------------------------------------------------------
    def _all_parts(self):
        return [self.embedding, *self.layers, self.final_norm, self.head]

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs: Dict[str, WeightSpec] = {}
        for part in self._all_parts():
            for name, ws in part.weight_specs().items():
                if name in specs and specs[name].shape != ws.shape:
                    raise ConfigError(f"tensor {name!r} is declared twice with different shapes")
                specs[name] = ws
        return specs

    def bind(self, weights: Dict[str, torch.Tensor]) -> None:
        for part in self._all_parts():
            part.bind(weights)
        self.bound = True

    @property
    def replayable(self) -> bool:
        """Whether every part can run from a recorded CUDA graph."""
        return all(part.all_replayable() for part in self._all_parts())

    def cache_needs(self) -> List[CacheNeed]:
        needs = []
        for pos, item in enumerate(self.schedule):
            mixer = self.layers[item.layer].mixer
            paged = mixer.cache_spec() if mixer is not None else None
            state = mixer.state_spec() if mixer is not None else None
            needs.append(CacheNeed(pos, paged, state, item.cache_of))
        return needs

    def step_weight_bytes(self) -> int:
        """Bytes of weights that one step reads: every scheduled layer once, the
        final norm and the head; of the embedding only the rows looked up."""
        total = self.final_norm.weight_bytes() + self.head.weight_bytes()
        for item in self.schedule:
            total += self.layers[item.layer].weight_bytes()
        return total

    # ---- the forward pass of one step ---------------------------------------
    def forward(self, ctx, caches) -> Optional[torch.Tensor]:
        """Runs the step's rows through the schedule.  ``caches[i]`` is the
        ``LayerCache`` of schedule position i.  Returns float32 logits
        [wanted rows, vocab], or None when no row is wanted."""
        if not self.bound:
            raise ConfigError("the model has no weights bound")
        with core.step_stream(self.rt.device):
            # nothing of this step starts before what describes it (positions, tables) is complete
            core.step_fence(self.rt.device)
            stream = ResidualStream(self.embedding.forward(ctx.token_ids))
            for item, cache in zip(self.schedule, caches):
                self.layers[item.layer].forward(stream, ctx, cache)
            if ctx.logit_rows is None or ctx.logit_rows.numel() == 0:
                return None
            normed = self.final_norm.forward(stream, row_idx=ctx.logit_rows)
            return self.head.forward(normed)
