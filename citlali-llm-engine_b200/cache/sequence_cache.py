"""The cache of a model: a slot per live sequence, keys and values per cached layer in pages,
and fixed-size per-sequence state beside them.

The reference keeps one sequence: two buffers [max_context, kv_heads, head_dim] per layer and
the position as a host argument (include/citlali/model/qwen_model.h:29-30,
src/model/qwen_model.cpp:177-178, :239).  Here:

* A *slot* stands for one sequence of a batch.  It has a length (tokens cached so far), a row
  in every group's page table, and a row in every state region.  Slots are given back when
  their sequence ends and handed out again; state regions are zeroed on acquire, and keys and
  values past a slot's length are never read.
* Cached layers (steps of the model's schedule) with equal needs form a *group* with storage
  of its own: ``[layer, page, kv_head, page_size, head_dim]`` for keys and for values, a page
  pool and a page table.  A group whose mixer attends to a window of keys gives a sequence's
  pages back once no later token can see them.
* A *state region* is ``[layer, slot, ...]`` of fixed size per sequence, for mixers that carry
  state instead of keys; this architecture has none, the storage exists for those that do.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..errors import CitlaliError, require
from .allocators import PageAllocator, SlotAllocator

PAGE_SIZE = 64


@dataclass(frozen=True)
class KVRequirement:
    """What an attention-like mixer needs cached per token: keys and values of ``num_kv_heads``
    heads of ``head_dim``; ``window`` keys back at most (None: all of them)."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateRequirement:
    """What a mixer with state of its own needs per sequence: a tensor of fixed shape."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class KVGroup:
    requirement: KVRequirement
    steps: List[int]
    pages: PageAllocator
    table_host: torch.Tensor          # [slots, max_pages] int32, the host's record
    table: torch.Tensor               # the same on the device
    keys: torch.Tensor                # [layers, pages, kv_heads, page_size, head_dim]
    values: torch.Tensor
    held: Dict[int, Dict[int, int]] = field(default_factory=dict)   # slot -> {page index -> page}


@dataclass
class StateGroup:
    requirement: StateRequirement
    steps: List[int]
    storage: torch.Tensor             # [layers, slots, *shape]


@dataclass
class KVView:
    """What a mixer sees of the cache: its layer's keys and values and the group's page table."""
    keys: torch.Tensor                # [pages, kv_heads, page_size, head_dim]
    values: torch.Tensor
    page_table: torch.Tensor          # [slots, max_pages] int32
    page_size: int
    requirement: KVRequirement


@dataclass
class StateView:
    storage: torch.Tensor             # [slots, *shape]
    requirement: StateRequirement


class SequenceCache:
    def __init__(self, requirements: Sequence[object], num_slots: int, capacity_tokens: int,
                 max_sequence_tokens: int, dtype: torch.dtype, device, page_size: int = PAGE_SIZE):
        """``requirements[i]`` is what schedule step ``i`` keeps: a KVRequirement, a
        StateRequirement or None.  ``capacity_tokens`` bounds the tokens all live sequences hold
        together, each sequence's count rounded up to whole pages."""
        require(page_size > 0 and capacity_tokens > 0 and max_sequence_tokens > 0, "cache sizes must be positive")
        self.page_size = page_size
        self.device = torch.device(device)
        self.dtype = dtype
        self.num_pages = (capacity_tokens + page_size - 1) // page_size
        self.max_sequence_tokens = max_sequence_tokens
        self.max_pages_per_slot = (max_sequence_tokens + page_size - 1) // page_size
        self.slots = SlotAllocator(num_slots)
        self.lengths = [0] * num_slots
        self.kv_groups: List[KVGroup] = []
        self.state_groups: List[StateGroup] = []
        self._where: Dict[int, Tuple[str, int, int]] = {}     # step -> (kind, group, layer in group)
        by_kv: Dict[KVRequirement, List[int]] = {}
        by_state: Dict[StateRequirement, List[int]] = {}
        for step, req in enumerate(requirements):
            if req is None:
                continue
            if isinstance(req, KVRequirement):
                by_kv.setdefault(req, []).append(step)
            elif isinstance(req, StateRequirement):
                by_state.setdefault(req, []).append(step)
            else:
                raise CitlaliError(f"schedule step {step} asks for a cache of unknown kind {type(req).__name__}")
        self._pin = self.device.type == "cuda"
        self._has_window = any(req.window is not None for req in by_kv)
        for req, steps in by_kv.items():
            shape = (len(steps), self.num_pages, req.num_kv_heads, page_size, req.head_dim)
            table_host = torch.zeros((num_slots, self.max_pages_per_slot), dtype=torch.int32)
            group = KVGroup(req, steps, PageAllocator(self.num_pages), table_host,
                            torch.zeros_like(table_host, device=self.device),
                            torch.zeros(shape, dtype=dtype, device=self.device),
                            torch.zeros(shape, dtype=dtype, device=self.device))
            for j, s in enumerate(steps):
                self._where[s] = ("kv", len(self.kv_groups), j)
            self.kv_groups.append(group)
        for req, steps in by_state.items():
            storage = torch.zeros((len(steps), num_slots) + tuple(req.shape), dtype=req.dtype, device=self.device)
            for j, s in enumerate(steps):
                self._where[s] = ("state", len(self.state_groups), j)
            self.state_groups.append(StateGroup(req, steps, storage))

    # ---- slots -----------------------------------------------------------------------
    def acquire(self) -> int:
        slot = self.slots.acquire()
        self.lengths[slot] = 0
        for g in self.kv_groups:
            g.held[slot] = {}
        for g in self.state_groups:
            g.storage[:, slot].zero_()
        return slot

    def release(self, slot: int) -> None:
        self.slots.release(slot)
        for g in self.kv_groups:
            g.pages.free(list(g.held.pop(slot).values()))
        self.lengths[slot] = 0

    def length(self, slot: int) -> int:
        require(self.slots.is_held(slot), f"slot {slot} is not held")
        return self.lengths[slot]

    # ---- growing a sequence -----------------------------------------------------------
    def reserve(self, slot: int, new_length: int) -> None:
        """Make room for positions below ``new_length`` in every group.  Either all groups get
        their pages or none does."""
        require(self.slots.is_held(slot), f"slot {slot} is not held")
        require(new_length <= self.max_sequence_tokens,
                f"a sequence of {new_length} tokens exceeds the cache's limit of {self.max_sequence_tokens} per sequence")
        have = self.lengths[slot]
        if have > 0 and (new_length - 1) // self.page_size == (have - 1) // self.page_size:
            return          # the page that holds the last token also holds the new ones
        need_index = (new_length + self.page_size - 1) // self.page_size
        plans = []
        for g in self.kv_groups:
            have = g.held[slot]
            first_visible = 0
            if g.requirement.window is not None:
                # positions the tokens still to come can see start here
                first_visible = max(0, self.lengths[slot] - g.requirement.window + 1) // self.page_size
            missing = [i for i in range(first_visible, need_index) if i not in have]
            plans.append((g, missing))
        for g, missing in plans:
            if len(missing) > g.pages.free_count:
                raise CitlaliError(f"the cache is full: slot {slot} needs {len(missing)} more pages of "
                                   f"{self.page_size} tokens and {g.pages.free_count} of {g.pages.num_pages} are free")
        for g, missing in plans:
            if not missing:
                continue
            for i, page in zip(missing, g.pages.allocate(len(missing))):
                g.held[slot][i] = page
                g.table_host[slot, i] = page
            lo, hi = missing[0], missing[-1] + 1
            # The host runs ahead of the device, and a slot given back may be taken again before an
            # earlier step has run: every update travels in a pinned buffer of its own (the pinned
            # allocator hands a buffer out again only after the copy from it is done), so a copy
            # still queued never sees a later step's entries.
            stage = g.table_host[slot, lo:hi].clone()
            if self._pin:
                stage = stage.pin_memory()
            g.table[slot, lo:hi].copy_(stage, non_blocking=True)

    def commit(self, slot: int, new_length: int) -> None:
        """The step that wrote positions below ``new_length`` has been issued."""
        require(self.slots.is_held(slot), f"slot {slot} is not held")
        self.lengths[slot] = new_length
        if not self._has_window:
            return
        for g in self.kv_groups:
            w = g.requirement.window
            if w is None:
                continue
            first_visible = max(0, new_length - w + 1) // self.page_size
            gone = [i for i in g.held[slot] if i < first_visible]
            if gone:
                g.pages.free([g.held[slot].pop(i) for i in gone])

    def rewind(self, slot: int, new_length: int) -> None:
        """Forget a sequence's tokens from ``new_length`` on (they will be computed again or replaced).
        Pages stay with the slot.  Not for caches with a window group, whose early pages are already gone."""
        require(self.slots.is_held(slot), f"slot {slot} is not held")
        require(0 <= new_length <= self.lengths[slot],
                f"slot {slot} holds {self.lengths[slot]} tokens and cannot be rewound to {new_length}")
        require(not self._has_window, "a cache with a windowed group cannot be rewound")
        self.lengths[slot] = new_length

    # ---- what layers see ---------------------------------------------------------------
    def view(self, step: int):
        require(step in self._where, f"schedule step {step} keeps no cache")
        kind, gi, j = self._where[step]
        if kind == "kv":
            g = self.kv_groups[gi]
            return KVView(g.keys[j], g.values[j], g.table, self.page_size, g.requirement)
        g = self.state_groups[gi]
        return StateView(g.storage[j], g.requirement)

    def has_view(self, step: int) -> bool:
        return step in self._where

    def bytes(self) -> int:
        total = 0
        for g in self.kv_groups:
            total += 2 * g.keys.numel() * g.keys.element_size()
        for g in self.state_groups:
            total += g.storage.numel() * g.storage.element_size()
        return total

    def pages_held(self) -> int:
        return sum(g.pages.held_count for g in self.kv_groups)
