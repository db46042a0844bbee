"""The step function's host side: from a list of entries to the packed rows of one step.

An entry is one sequence's next tokens.  The sequences of a step either all start (their
slots are empty) or all go on; their lengths differ freely.  Rows are packed without padding:
sequence after sequence, each in position order.  Everything the kernels need to know about
the rows goes to the device in one copy from pinned memory.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Sequence

import torch

from ..errors import require
from ..parts.base import StepBatch


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)   # places among `tokens` whose logits are asked for


def pack_step(entries: List[StepEntry], past: List[int], vocab_size: int, device) -> StepBatch:
    """``past[i]`` is the number of tokens entry i's slot already holds."""
    require(len(entries) > 0, "a step needs at least one entry")
    seen = set()
    rows = 0
    for e in entries:
        require(e.slot not in seen, f"slot {e.slot} appears twice in one step")
        seen.add(e.slot)
        require(len(e.tokens) > 0, f"the entry of slot {e.slot} brings no tokens")
        for w in e.want:
            require(0 <= w < len(e.tokens),
                    f"slot {e.slot}: logits asked at place {w} of {len(e.tokens)} tokens")
        rows += len(e.tokens)
    B = len(entries)
    wanted = sum(len(e.want) for e in entries)
    # layout of the one int32 buffer: tokens | row_slot | row_pos | seq_start | seq_slot | seq_past | want_rows
    sizes = [rows, rows, rows, B + 1, B, B, wanted]
    offsets = [0]
    for s in sizes:
        offsets.append(offsets[-1] + ((s + 3) // 4) * 4)      # 16-byte aligned pieces
    pin = torch.device(device).type == "cuda"
    host = torch.zeros(max(offsets[-1], 4), dtype=torch.int32, pin_memory=pin)
    tokens, row_slot, row_pos, seq_start, seq_slot, seq_past, want_rows = (
        host[offsets[i]:offsets[i] + sizes[i]] for i in range(7))
    r = 0
    w = 0
    for b, e in enumerate(entries):
        n = len(e.tokens)
        ids = torch.as_tensor(list(e.tokens), dtype=torch.int64)
        if int(ids.min()) < 0 or int(ids.max()) >= vocab_size:        # as the reference checks (qwen_model.cpp:240-241)
            bad = int(ids[(ids < 0) | (ids >= vocab_size)][0])
            require(False, f"token id {bad} out of vocab range [0, {vocab_size})")
        tokens[r:r + n] = ids.to(torch.int32)
        row_slot[r:r + n] = e.slot
        row_pos[r:r + n] = torch.arange(past[b], past[b] + n, dtype=torch.int32)
        seq_start[b] = r
        seq_slot[b] = e.slot
        seq_past[b] = past[b]
        for place in e.want:
            want_rows[w] = r + place
            w += 1
        r += n
    seq_start[B] = r
    dev = host.to(device, non_blocking=True)
    parts = [dev[offsets[i]:offsets[i] + sizes[i]] for i in range(7)]
    return StepBatch(*parts, slots=[e.slot for e in entries], past=list(past),
                     n_new=[len(e.tokens) for e in entries])
