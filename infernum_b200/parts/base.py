"""Interfaces of the parts a decoder is put together from, and their registries.

A model is described by data (``ModelSpec``): a list of layers, each naming a
block arrangement, a mixer, a feed-forward and norms by *kind* with their
parameters, and a schedule that says in which order layers run and whose cache
each run uses.  The kinds are looked up in the registries below, so a new
mixer, feed-forward, norm, position encoding or block is added by registering
a class; nothing else in the package changes.  No part knows which model it is
in: it only sees its own parameters, its weights, the rows of the step and the
cache view it is handed.

The reference composes its decoder from the same pieces inside one graph
builder (infernum-llama/src/graph_builder.rs:399-549 for prefill, :756-921 for
paged decode); here they are separate objects chosen per layer.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from ..errors import ConfigError


# --------------------------------------------------------------------------
# Descriptions (plain data)
# --------------------------------------------------------------------------
@dataclass(frozen=True)
class WeightSpec:
    """One tensor a part wants from the checkpoint.

    ``kind``: "float" tensors are kept in bfloat16 (float32 when the file
    stores them in 32-bit, or when the engine runs in float32); "int" tensors
    become int32 tables.  ``init`` drives the random-weights mode: "normal"
    draws N(0, std), "norm" draws 1 + U(-0.1, 0.1), "zeros" and "ones" are
    constant.
    """

    shape: Tuple[int, ...]
    kind: str = "float"
    init: str = "normal"
    std: float = 0.02
    # another tensor name to take when this one is absent from the checkpoint
    fallback: Optional[str] = None


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer: which block arrangement and which parts fill it."""

    block: str
    parts: Dict[str, PartSpec]
    name: str = ""


@dataclass(frozen=True)
class ScheduleItem:
    """One run of a layer.  ``cache_of`` names an earlier schedule position
    whose cache this run reads instead of owning one."""

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleItem, ...]
    final_norm: PartSpec
    lm_head: PartSpec
    max_position: int
    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    # checkpoint tensors that may be present without being used
    ignorable: Tuple[str, ...] = ()


@dataclass(frozen=True)
class PagedCacheSpec:
    """What a mixer needs from the paged cache: keys and values of
    ``kv_heads`` x ``head_dim`` per token; ``window`` > 0 means only the last
    ``window`` tokens are ever read, so older pages can be given back."""

    kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size per-request state of a mixer (one tensor of this shape per
    request slot, zeroed when the slot is taken)."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class Runtime:
    """What every part needs to know about the engine it runs in."""

    device: torch.device
    dtype: torch.dtype  # activation / weight dtype: torch.bfloat16 or torch.float32
    err: Optional[torch.Tensor] = None  # device error word shared by the kernels
    options: Dict[str, Any] = field(default_factory=dict)

    @property
    def is_fp32(self) -> bool:
        return self.dtype == torch.float32

    def error_word(self) -> torch.Tensor:
        """The device error word, made on first use: every kernel of a step is
        given this one word, and the engine reads it after the step."""
        if self.err is None:
            from ..ops import core

            self.err = core.new_error_word(self.device)
        return self.err


# --------------------------------------------------------------------------
# Part interfaces
# --------------------------------------------------------------------------
class Part:
    """Base of all parts.  ``params`` are the part's own sizes and constants."""

    kind: str = ""
    # Recurring steps are recorded as CUDA graphs and replayed with new
    # contents in the step's device tensors.  A part whose ``forward`` cannot
    # run that way (it branches on values it reads back from the device, or on
    # host-side fields that differ between steps of one shape) sets this to
    # False, and an engine with such a part runs every step eagerly.
    replayable: bool = True

    def __init__(self, params: Dict[str, Any], rt: Runtime):
        self.params = dict(params)
        self.rt = rt

    def all_replayable(self) -> bool:
        return bool(self.replayable)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        """Checkpoint tensor name -> what it must look like."""
        return {}

    def bind(self, weights: Dict[str, torch.Tensor]) -> None:
        """Take the loaded tensors (on the device, already in their kept dtype)."""

    def weight_bytes(self) -> int:
        """Bytes of weights one step reads from this part (for rooflines)."""
        return 0


class Norm(Part):
    """``forward(stream)`` folds the stream's pending delta into its residual
    and returns the normed rows in the activation dtype."""

    def forward(self, stream: "ResidualStream", row_idx: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError

    def apply(self, x: torch.Tensor) -> torch.Tensor:
        """Norm of a plain float32 tensor of rows (no residual bookkeeping)."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Position information for a mixer.  ``apply(q, k, positions)`` changes
    ``q`` [N, heads, hd] and ``k`` [N, kv_heads, hd] in place.  A mixer may use
    a fused route for encodings it knows (rotary) and this method otherwise."""

    def apply(self, q: torch.Tensor, k: Optional[torch.Tensor], positions: torch.Tensor) -> None:
        raise NotImplementedError


class Mixer(Part):
    """Token mixing (attention, or anything that moves information between
    positions).  ``forward(x, ctx, cache)``: ``x`` is [N, hidden] in the
    activation dtype, ``ctx`` the step's ``StepContext``, ``cache`` the
    ``LayerCache`` this run reads and writes.  Returns [N, hidden]."""

    def cache_spec(self) -> Optional[PagedCacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def forward(self, x: torch.Tensor, ctx: Any, cache: Any) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    """Per-token transformation.  ``forward(x, ctx)`` -> [N, hidden]."""

    def forward(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """The arrangement of a layer's parts around the residual stream."""

    def __init__(self, params: Dict[str, Any], rt: Runtime, parts: Dict[str, Part]):
        super().__init__(params, rt)
        self.parts = parts

    @property
    def mixer(self) -> Optional[Mixer]:
        m = self.parts.get("mixer")
        return m if isinstance(m, Mixer) else None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs: Dict[str, WeightSpec] = {}
        for part in self.parts.values():
            specs.update(part.weight_specs())
        return specs

    def bind(self, weights: Dict[str, torch.Tensor]) -> None:
        for part in self.parts.values():
            part.bind(weights)

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in self.parts.values())

    def all_replayable(self) -> bool:
        return bool(self.replayable) and all(p.all_replayable() for p in self.parts.values())

    def forward(self, stream: "ResidualStream", ctx: Any, cache: Any) -> None:
        raise NotImplementedError


class ResidualStream:
    """The hidden state between parts: a float32 residual [N, hidden] and, at
    most, one pending delta in the activation dtype that the next norm (or
    ``flush``) adds to it.  Keeping the sum in 32-bit and fusing the add into
    the norm kernel saves one pass over the rows per sub-layer."""

    def __init__(self, residual: torch.Tensor):
        self.residual = residual
        self.pending: Optional[torch.Tensor] = None

    def push(self, delta: torch.Tensor) -> None:
        if self.pending is not None:
            self.flush()
        self.pending = delta

    def flush(self) -> None:
        if self.pending is not None:
            from ..ops import core

            core.residual_add(self.residual, self.pending)
            self.pending = None


# --------------------------------------------------------------------------
# Registries
# --------------------------------------------------------------------------
class Registry:
    def __init__(self, what: str):
        self.what = what
        self._items: Dict[str, Callable[..., Part]] = {}

    def register(self, kind: str, factory: Optional[Callable[..., Part]] = None):
        def deco(f):
            self._items[kind] = f
            try:
                f.kind = kind
            except (AttributeError, TypeError):
                pass
            return f

        return deco(factory) if factory is not None else deco

    def get(self, kind: str) -> Callable[..., Part]:
        try:
            return self._items[kind]
        except KeyError:
            raise ConfigError(
                f"unknown {self.what} kind {kind!r}; registered: {sorted(self._items)}"
            ) from None

    def kinds(self) -> List[str]:
        return sorted(self._items)


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("output head")

_ROLE_REGISTRY = {
    "mixer": MIXERS,
    "ffn": FEED_FORWARDS,
    "feed_forward": FEED_FORWARDS,
}


def registry_for_role(role: str, spec: PartSpec) -> Registry:
    """Which registry a named part of a layer comes from: by role name, norms
    by the ``norm`` prefix."""
    if role in _ROLE_REGISTRY:
        return _ROLE_REGISTRY[role]
    if role.startswith("norm") or role.endswith("norm"):
        return NORMS
    raise ConfigError(f"layer part {role!r}: cannot tell which registry it comes from")


def build_part(role: str, spec: PartSpec, rt: Runtime) -> Part:
    return registry_for_role(role, spec).get(spec.kind)(spec.params, rt)


def build_layer(spec: LayerSpec, rt: Runtime) -> Block:
    parts = {role: build_part(role, ps, rt) for role, ps in spec.parts.items()}
    return BLOCKS.get(spec.block)({"name": spec.name}, rt, parts)


def register_mixer(kind: str, factory=None):
    return MIXERS.register(kind, factory)


def register_feed_forward(kind: str, factory=None):
    return FEED_FORWARDS.register(kind, factory)


def register_norm(kind: str, factory=None):
    return NORMS.register(kind, factory)


def register_position_encoding(kind: str, factory=None):
    return POSITION_ENCODINGS.register(kind, factory)


def register_block(kind: str, factory=None):
    return BLOCKS.register(kind, factory)
