"""Decoding through CUDA graphs.

One decode step launches a few hundred small kernels; at batch 1 their launch cost on the
host would exceed the time the GPU needs.  The step for a given number of sequences is
therefore captured once and replayed.  Everything that changes from step to step lives in
device buffers of fixed address: the tokens, each row's slot and position, the sampling
parameters, the page tables.  The host fills a pinned mirror, issues one copy, and replays.

A model can be replayed only if none of its parts looks at the host-side lists of a step
(slots, lengths): every part answers for itself, once bound, with ``graph_safe`` (an attention
part says yes only for the dtype and head size whose single-token kernel reads positions on the
device); for other models the session keeps stepping without graphs.

The host runs ahead of the device: ``launch`` returns before the replay has run.  A pinned mirror
must therefore not be rewritten while a copy from it may still be pending; the mirrors form a ring,
and each waits for the event recorded behind its last copy before it is written again.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import ops
from ..errors import require
from ..parts.base import StepBatch


def model_is_graph_safe(model) -> bool:
    """Every part of every layer, as bound, steps from device memory alone."""
    for block in model.layers:
        if getattr(block, "graph_safe", True) is False:        # an arrangement may veto for code of its own
            return False
        for part in block.parts():
            if not getattr(part, "graph_safe", False):
                return False
    return True


class _PinnedRing:
    """A few pinned host buffers of one shape used in turn.  ``next()`` hands out the buffer whose last
    copy is longest ago, after waiting for that copy; ``sent(stream)`` marks the copy just issued."""

    def __init__(self, shape, dtype, depth: int = 4):
        self.buffers = [torch.zeros(shape, dtype=dtype, pin_memory=True) for _ in range(depth)]
        self.events = [None] * depth
        self.at = -1

    def next(self) -> torch.Tensor:
        self.at = (self.at + 1) % len(self.buffers)
        ev = self.events[self.at]
        if ev is not None:
            ev.synchronize()
        return self.buffers[self.at]

    def sent(self) -> None:
        ev = self.events[self.at]
        if ev is None:
            ev = self.events[self.at] = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())


class DecodeGraphRunner:
    def __init__(self, model, cache, max_batch: int):
        self.model = model
        self.cache = cache
        self.max_batch = max_batch
        dev = model.ctx.device
        B = max_batch
        # int32 layout: tokens | row_slot | row_pos | seq_start | seq_slot | seq_past | want_rows
        self._sizes = [B, B, B, B + 1, B, B, B]
        self._offsets = [0]
        for s in self._sizes:
            self._offsets.append(self._offsets[-1] + (s + 3) // 4 * 4)
        self.ints_ring = _PinnedRing((self._offsets[-1],), torch.int32)
        self.ints = torch.zeros(self._offsets[-1], dtype=torch.int32, device=dev)
        self.floats_ring = _PinnedRing((2, B), torch.float32)                           # temperature, uniform
        self.floats = torch.zeros((2, B), dtype=torch.float32, device=dev)
        self.out_tokens = torch.zeros(B, dtype=torch.int32, device=dev)
        self.out_host = torch.zeros(B, dtype=torch.int32, pin_memory=True)
        self.graphs: Dict[Tuple[int, bool], torch.cuda.CUDAGraph] = {}
        self.logits: Dict[Tuple[int, bool], torch.Tensor] = {}
        self.kernels_per_replay: Dict[Tuple[int, bool], int] = {}
        self._pool = None
        # constant parts, in every mirror and on the device: one row per sequence
        for host in self.ints_ring.buffers:
            self._piece(host, 3, B + 1).copy_(torch.arange(B + 1, dtype=torch.int32))
            self._piece(host, 6, B).copy_(torch.arange(B, dtype=torch.int32))
        self.ints.copy_(self.ints_ring.buffers[0])

    def _piece(self, buf, i, n):
        return buf[self._offsets[i]:self._offsets[i] + n]

    def _batch(self, n: int) -> StepBatch:
        d = self.ints
        return StepBatch(self._piece(d, 0, n), self._piece(d, 1, n), self._piece(d, 2, n), self._piece(d, 3, n + 1),
                         self._piece(d, 4, n), self._piece(d, 5, n), self._piece(d, 6, n),
                         slots=[0] * n, past=[0] * n, n_new=[1] * n)

    def _body(self, n: int, greedy: bool):
        logits = self.model.forward(self._batch(n), self.cache)
        if greedy:
            ops.argmax_rows(logits, self.out_tokens[:n])
        else:
            ops.sample_rows(logits, self.floats[0], self.floats[1], self.out_tokens[:n])
        return logits

    def _run(self, n: int, greedy: bool) -> None:
        """Run the step whose inputs are in place: replay its graph, or, the first time a batch size is met, run it
        with plain launches (which also sizes scratch buffers and sets kernel attributes) and capture the graph for
        the steps to come.  A step is never run twice: a mixer's state of its own would be advanced twice."""
        key = (n, greedy)
        g = self.graphs.get(key)
        if g is not None:
            g.replay()
            return
        first = self._body(n, greedy)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        with torch.cuda.graph(g, pool=self._pool):
            self.logits[key] = self._body(n, greedy)
        self.kernels_per_replay[key] = ops.launch_count() - before
        self.logits[key].copy_(first)             # this step's logits, where later steps' logits will be found
        if self._pool is None:
            self._pool = g.pool()
        self.graphs[key] = g

    def fill(self, slots: Sequence[int], tokens: Optional[Sequence[int]], positions: Sequence[int],
             temperature: float, uniforms: Sequence[float]) -> None:
        """Write the step's inputs into the pinned mirror and issue the copies.  ``tokens`` None:
        keep the device's token buffer (fed from the last step's output on the device)."""
        n = len(slots)
        host = self.ints_ring.next()
        h, o = host.numpy(), self._offsets               # the same pinned memory, written without tensor ops
        if tokens is not None:
            h[o[0]:o[0] + n] = tokens
        h[o[1]:o[1] + n] = slots
        h[o[2]:o[2] + n] = positions
        h[o[4]:o[4] + n] = slots
        h[o[5]:o[5] + n] = positions
        lo = 0 if tokens is not None else o[1]
        hi = o[6]
        self.ints[lo:hi].copy_(host[lo:hi], non_blocking=True)
        self.ints_ring.sent()
        if temperature > 0.0:
            fh = self.floats_ring.next()
            fh[0, :n] = float(temperature)
            fh[1, :n] = torch.as_tensor(list(uniforms), dtype=torch.float32)
            self.floats.copy_(fh, non_blocking=True)
            self.floats_ring.sent()

    def launch(self, slots: Sequence[int], tokens: Optional[Sequence[int]], temperature: float,
               uniforms: Sequence[float]) -> int:
        """Reserve cache room, copy the inputs, replay the graph, advance the lengths.  Returns the
        number of kernels the replay launched.  Nothing is synchronised: steps may be issued back to
        back, each step's inputs travel in a pinned buffer no later step touches until its copy is done."""
        n = len(slots)
        require(0 < n <= self.max_batch, f"{n} sequences exceed the runner's {self.max_batch}")
        positions = [self.cache.length(s) for s in slots]
        greedy = temperature <= 0.0
        for s, p in zip(slots, positions):
            self.cache.reserve(s, p + 1)
        self.fill(slots, tokens, positions, temperature, uniforms)
        self._run(n, greedy)
        for s, p in zip(slots, positions):
            self.cache.commit(s, p + 1)
        return self.kernels_per_replay[(n, greedy)]

    def feed_back(self, n: int) -> None:
        """Make the tokens just sampled the next step's input, on the device."""
        self._piece(self.ints, 0, n).copy_(self.out_tokens[:n], non_blocking=True)

    def read_tokens(self, n: int) -> List[int]:
        self.out_host[:n].copy_(self.out_tokens[:n], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self.out_host[:n].tolist()
