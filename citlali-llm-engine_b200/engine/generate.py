"""The generation loop: batches of unequal prompts, stop tokens, sequences that end earlier,
and as many batches one after another as the requests need.

For one sequence the decisions are the reference's (generate_from_prompt_text,
src/runtime/session.cpp:61-104): the stop test comes before anything else and a stop token
is neither emitted nor fed back (:79-82); otherwise the token is emitted and counted
(:84-90); the loop ends at max_new_tokens, or when the sequence fills its context (:94-97).
Unlike the reference no forward pass is spent on a token that will not be used.  The loop
knows nothing of devices: it drives a *stepper* (acquire / release / prefill / decode) and
is tested on the CPU with a fake one.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from ..errors import require
from ..sampling.rng import uniform


class StopReason(enum.Enum):       # include/citlali/runtime/session.h:23-27
    EOS = "eos"
    MAX_NEW_TOKENS = "max_new_tokens"
    CONTEXT_LIMIT = "context_limit"


@dataclass
class GenerationOptions:           # include/citlali/runtime/session.h:16-20, plus sampling
    max_new_tokens: int = 256
    max_context: int = 2048
    temperature: float = 0.0       # 0: greedy, the reference's only mode
    seed: int = 0
    stop_ids: Optional[Sequence[int]] = None    # None: the model's eos ids from config.json
    max_batch: Optional[int] = None             # None: as many as the session has slots


@dataclass
class GenerationResult:            # include/citlali/runtime/session.h:30-34, token ids for text
    tokens: List[int] = field(default_factory=list)
    generated_tokens: int = 0
    stop_reason: StopReason = StopReason.MAX_NEW_TOKENS


def run_generation(stepper, prompts: Sequence[Sequence[int]], options: GenerationOptions,
                   stop_ids: Sequence[int], max_batch: int,
                   on_token: Optional[Callable[[int, int], None]] = None) -> List[GenerationResult]:
    """``stepper`` provides ``acquire() -> slot``, ``release(slot)``,
    ``prefill(slots, prompts, temperature, uniforms) -> tokens`` and
    ``decode(slots, tokens, temperature, uniforms) -> tokens`` (one sampled token per sequence)."""
    require(len(prompts) > 0, "no prompts were given")
    require(max_batch > 0, "max_batch must be positive")
    require(options.max_new_tokens >= 0, "max_new_tokens must not be negative")
    for i, p in enumerate(prompts):
        require(len(p) > 0, f"prompt {i} produced no tokens")
        require(len(p) < options.max_context,
                f"prompt {i} has {len(p)} tokens, which leaves no room in a context of {options.max_context}")
    stops = set(int(s) for s in stop_ids)
    results = [GenerationResult() for _ in prompts]
    for first in range(0, len(prompts), max_batch):
        _run_batch(stepper, prompts, list(range(first, min(first + max_batch, len(prompts)))),
                   options, stops, results, on_token)
    return results


def _run_batch(stepper, prompts, requests, options, stops, results, on_token):
    if options.max_new_tokens == 0:
        return
    temperature = float(options.temperature)

    def draws(active):
        if temperature <= 0.0:
            return []
        return [uniform(options.seed, r, results[r].generated_tokens) for r, _ in active]

    active = []
    held = set()

    def release(slot):
        held.discard(slot)
        stepper.release(slot)

    try:
        for r in requests:
            slot = stepper.acquire()
            held.add(slot)
            active.append((r, slot))
        sampled = stepper.prefill([s for _, s in active], [prompts[r] for r, _ in active],
                                  temperature, draws(active))
        while True:
            survivors, feed = [], []
            for (r, slot), token in zip(active, sampled):
                res = results[r]
                done = None
                if token in stops:
                    done = StopReason.EOS
                else:
                    res.tokens.append(int(token))
                    res.generated_tokens += 1
                    if on_token is not None:
                        on_token(r, int(token))
                    if res.generated_tokens >= options.max_new_tokens:
                        done = StopReason.MAX_NEW_TOKENS
                    elif len(prompts[r]) + res.generated_tokens >= options.max_context:
                        done = StopReason.CONTEXT_LIMIT
                if done is None:
                    survivors.append((r, slot))
                    feed.append(int(token))
                else:
                    res.stop_reason = done
                    release(slot)
            active = survivors
            if not active:
                break
            sampled = stepper.decode([s for _, s in active], feed, temperature, draws(active))
    finally:
        for slot in sorted(held):
            stepper.release(slot)
