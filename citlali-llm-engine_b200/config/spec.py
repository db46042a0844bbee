"""Architecture-neutral description of a decoder: what an architecture's config is turned into.

A :class:`ModelSpec` is data.  It lists the distinct layers (each a choice of
block arrangement, mixer, feed-forward and norms, every one with its own sizes
and constants), the order in which they run, and the tensors around the stack.
The engine builds a model from it through the part registries; no part reads an
architecture's config directly.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: ``kind`` names a registered part class, ``params`` are its
    sizes and constants, ``prefix`` is where its tensors live in the checkpoint."""
    kind: str
    params: Dict[str, Any]
    prefix: str


@dataclass(frozen=True)
class LayerSpec:
    """One layer with weights of its own: an arrangement (``block``) and the parts it arranges, by name,
    in the order given.  Which names a block kind needs, and which registry each is looked up in, is the
    block's business: the pre-norm block takes ``mixer_norm``, ``mixer``, ``feed_forward_norm`` and
    ``feed_forward`` (either pair may be absent); a block with four norms, or with one norm shared by a
    mixer and a feed-forward that run side by side, names its parts as it likes."""
    block: str
    parts: Mapping[str, PartSpec]
    block_params: Dict[str, Any] = field(default_factory=dict)

    def part(self, name: str) -> PartSpec:
        from ..errors import require
        require(name in self.parts, f"a '{self.block}' layer needs a part named '{name}'; it has: "
                                    f"{', '.join(self.parts) or '(none)'}")
        return self.parts[name]


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
    embedding_scale: Optional[float] = None  # the embedding rows are multiplied by it (None: a plain row copy)
    logit_scale: Optional[float] = None      # the logits are multiplied by it (None: as the output matrix gives them)

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
