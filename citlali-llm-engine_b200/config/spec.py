"""Architecture-neutral description of a decoder: what an architecture's config is turned into.

A :class:`ModelSpec` is data.  It lists the distinct layers (each a choice of
block arrangement, mixer, feed-forward and norms, every one with its own sizes
and constants), the order in which they run, and the tensors around the stack.
The engine builds a model from it through the part registries; no part reads an
architecture's config directly.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: ``kind`` names a registered part class, ``params`` are its
    sizes and constants, ``prefix`` is where its tensors live in the checkpoint."""
    kind: str
    params: Dict[str, Any]
    prefix: str


@dataclass(frozen=True)
class LayerSpec:
    """One layer with weights of its own: an arrangement (``block``) of a mixer, a
    feed-forward and their norms."""
    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    block_params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class ScheduleStep:
    """One entry of the run order.  ``layer`` indexes :attr:`ModelSpec.layers` and may
    repeat.  ``cache_of`` names an earlier schedule step whose cache this step reads
    instead of keeping one of its own."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding_name: str
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleStep, ...]
    final_norm: PartSpec
    head_name: str
    tie_head_to_embedding: Optional[bool]   # None: tied iff the head tensor is absent
    stop_token_ids: Tuple[int, ...] = ()

    def validate(self):
        from ..errors import require
        require(len(self.schedule) > 0, "model spec has an empty schedule")
        for i, step in enumerate(self.schedule):
            require(0 <= step.layer < len(self.layers),
                    f"schedule step {i} names layer {step.layer}, model has {len(self.layers)}")
            if step.cache_of is not None:
                require(0 <= step.cache_of < i,
                        f"schedule step {i} reads the cache of step {step.cache_of}, which does not run before it")
                require(self.schedule[step.cache_of].cache_of is None,
                        f"schedule step {i} reads the cache of step {step.cache_of}, which has none of its own")
