"""InferenceSession: a model, its cache and the calls a user makes.

The reference's session (include/citlali/runtime/session.h:36-59) loads a GGUF file and
generates text for one sequence.  This one loads a model folder (config.json and
safetensors), takes and returns token ids, and serves batches; ``load_model``'s
``max_context`` and the generation options keep the reference's names, defaults and meaning
(session.h:16-20, :38-41).
"""
from __future__ import annotations

import time
from typing import Callable, Dict, List, Optional, Sequence

import torch

from .. import ops
from ..cache import PAGE_SIZE, SequenceCache
from ..config.registry import config_from_model_dir
from ..errors import CitlaliError, require
from ..parts.base import BuildContext
from ..sampling.sampler import Sampler
from ..weights.loader import WeightHandle, WeightLoader
from ..weights.random_init import random_tensor
from .graph import DecodeGraphRunner, model_is_graph_safe
from .generate import GenerationOptions, GenerationResult, run_generation
from .model import DecoderModel
from .step import StepEntry, pack_step

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        require(name in (torch.bfloat16, torch.float32), f"dtype must be bfloat16 or float32, not {name}")
        return name
    require(str(name) in _DTYPES, f"dtype must be bfloat16 or float32, not '{name}'")
    return _DTYPES[str(name)]


def _cuda_device(device) -> torch.device:
    dev = torch.device(device)
    require(dev.type == "cuda", f"models run on a CUDA device only, not on '{dev}'")
    require(torch.cuda.is_available(), "no CUDA device is available; there is no CPU path")
    return dev


class InferenceSession:
    def __init__(self):
        self.model: Optional[DecoderModel] = None
        self.cache: Optional[SequenceCache] = None
        self.config = None
        self.sampler: Optional[Sampler] = None
        self.max_context = 0
        self.stats: Dict[str, float] = {}
        self.runner = None
        self.use_graphs = True     # set False before loading to step without CUDA graphs
        self.page_size = PAGE_SIZE  # tokens a cache page holds; set before loading (the tensor-core attention kernels take 64)

    # ---- loading ---------------------------------------------------------------------
    def load_model(self, model_path: str, max_context: int = 2048, dtype="bfloat16", device="cuda:0",
                   max_batch: int = 8, max_tokens: Optional[int] = None, progress=None) -> "InferenceSession":
        """``max_context``: the most tokens one sequence may hold, capped by the model's own limit
        (src/model/qwen_model.cpp:51).  ``max_batch``: sequence slots.  ``max_tokens``: the most
        tokens all live sequences hold together, each rounded up to whole cache pages (default:
        every slot full)."""
        config = config_from_model_dir(model_path)
        dev = _cuda_device(device)
        loader = WeightLoader(model_path)
        try:
            spec = config.to_model_spec()
            ctx = self._context(dev, dtype)
            model = DecoderModel(spec, ctx)
            weights = loader.load_all(model.tensor_specs(), device="cpu", progress=progress)
            model.bind(weights)
        finally:
            loader.close()
        return self._finish(config, model, max_context, max_batch, max_tokens)

    def load_random(self, config, seed: int, max_context: int = 2048, dtype="bfloat16", device="cuda:0",
                    max_batch: int = 8, max_tokens: Optional[int] = None, gain_spread: float = 0.0,
                    stored_dtype=None) -> "InferenceSession":
        """Random weights made on the device, tensor by tensor, for measurements and for tests at
        sizes a folder would be too large for: nothing is written.  ``stored_dtype`` (default:
        ``dtype``) is the precision the values are rounded to before the model takes them, as if
        they had been stored so: two sessions with the same seed and ``stored_dtype`` hold the same
        values whatever they compute in."""
        dev = _cuda_device(device)
        spec = config.to_model_spec()
        ctx = self._context(dev, dtype)
        model = DecoderModel(spec, ctx)
        stored = parse_dtype(stored_dtype if stored_dtype is not None else dtype)
        handles: Dict[str, WeightHandle] = {}
        for s in model.tensor_specs():
            if s.optional and spec.tie_head_to_embedding is not False:
                continue
            # made when a part asks, and not kept: the model's own buffers are the only copy that stays
            make = (lambda s=s: random_tensor(s, seed, stored, dev, gain_spread=gain_spread))
            handles[s.name] = WeightHandle(s.name, torch.int32 if s.role == "table" else stored, tuple(s.shape),
                                           produce=make)
        model.bind(handles)
        return self._finish(config, model, max_context, max_batch, max_tokens)

    def _context(self, dev, dtype) -> BuildContext:
        flag = torch.zeros(4, dtype=torch.int32, device=dev)
        return BuildContext(device=dev, dtype=parse_dtype(dtype), error_flag=flag)

    def _finish(self, config, model, max_context, max_batch, max_tokens):
        require(max_context > 0 and max_batch > 0, "max_context and max_batch must be positive")
        self.config = config
        self.model = model
        self.max_context = min(int(max_context), model.spec.max_positions)
        capacity = int(max_tokens) if max_tokens is not None else None
        page = int(self.page_size)
        if capacity is None:
            capacity = max_batch * ((self.max_context + page - 1) // page) * page
        self.cache = SequenceCache(model.cache_requirements(), max_batch, capacity, self.max_context,
                                   model.ctx.dtype, model.ctx.device, page_size=page)
        self.sampler = Sampler(model.ctx.device, max_rows=max_batch)
        self.max_batch = max_batch
        self.runner = DecodeGraphRunner(model, self.cache, max_batch) if (
            self.use_graphs and model_is_graph_safe(model)) else None
        return self

    # ---- slots and steps -----------------------------------------------------------------
    def acquire(self) -> int:
        return self.cache.acquire()

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run the given tokens of every entry as one batch from the cache; return float32 logits
        ``[wanted, vocab]`` on the device, in the order of the entries and of their ``want``.
        Every entry appends its tokens to its slot, whatever the slot holds: sequences that start,
        sequences that go on by one token and sequences that go on by several may share a step, and
        their lengths may differ.  A step in which every entry brings one token runs the single-token
        kernels; any other step runs the ones for runs of tokens."""
        require(self.model is not None, "no model is loaded")
        entries = list(entries)
        require(len(entries) > 0, "a step needs at least one entry")
        past = []
        for e in entries:
            require(self.cache.slots.is_held(e.slot), f"slot {e.slot} was not acquired")
            p = self.cache.length(e.slot)
            require(p + len(e.tokens) <= self.max_context,
                    f"slot {e.slot}: {p} cached + {len(e.tokens)} new tokens exceed max_context {self.max_context}")
            past.append(p)
        batch = pack_step(entries, past, self.model.spec.vocab_size, self.model.ctx.device)
        for e, p in zip(entries, past):
            self.cache.reserve(e.slot, p + len(e.tokens))
        logits = self.model.forward(batch, self.cache)
        for e, p in zip(entries, past):
            self.cache.commit(e.slot, p + len(e.tokens))
        return logits

    def assume_cached(self, slot: int, tokens: int) -> None:
        """Declare that ``slot`` holds ``tokens`` tokens without computing them: room is reserved
        and the length is set, the keys and values are whatever the cache's memory holds.  For
        measurements at a given context length only."""
        require(tokens <= self.max_context, f"{tokens} tokens exceed max_context {self.max_context}")
        self.cache.reserve(slot, tokens)
        self.cache.commit(slot, tokens)

    def check_device_errors(self) -> None:
        """Read the word kernels raise when they meet a fault they can detect (a token id outside
        the embedding table, a wait that ran out).  Synchronises."""
        flag = self.model.ctx.error_flag
        if flag is not None:
            v = flag.tolist()
            if any(v):
                flag.zero_()
                ops.zero_counters()
                raise CitlaliError(f"a kernel reported a fault: flag words {v}")

    # ---- generation ------------------------------------------------------------------------
    def prefill(self, slots, prompts, temperature, uniforms) -> List[int]:
        t0 = time.perf_counter()
        logits = self.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        tokens = self.sampler.sample(logits, temperature, uniforms)
        self.stats["prefill_s"] = self.stats.get("prefill_s", 0.0) + time.perf_counter() - t0
        self.stats["prefill_tokens"] = self.stats.get("prefill_tokens", 0) + sum(len(p) for p in prompts)
        return tokens

    def decode(self, slots, tokens, temperature, uniforms) -> List[int]:
        t0 = time.perf_counter()
        if self.runner is not None and len(slots) <= self.runner.max_batch:
            vocab = self.model.spec.vocab_size
            for s, t in zip(slots, tokens):
                require(self.cache.slots.is_held(s), f"slot {s} was not acquired")
                require(0 <= int(t) < vocab, f"token id {t} out of vocab range [0, {vocab})")
                require(self.cache.length(s) + 1 <= self.max_context,
                        f"slot {s}: one more token exceeds max_context {self.max_context}")
            self.runner.launch(slots, tokens, temperature, uniforms)
            out = self.runner.read_tokens(len(slots))
        else:
            logits = self.step([StepEntry(s, [t], [0]) for s, t in zip(slots, tokens)])
            out = self.sampler.sample(logits, temperature, uniforms)
        self.stats["decode_s"] = self.stats.get("decode_s", 0.0) + time.perf_counter() - t0
        self.stats["decode_tokens"] = self.stats.get("decode_tokens", 0) + len(slots)
        return out

    def generate(self, prompts: Sequence[Sequence[int]], options: Optional[GenerationOptions] = None,
                 on_token: Optional[Callable[[int, int], None]] = None) -> List[GenerationResult]:
        """Generate for every prompt (lists of token ids).  Prompts run in batches of at most
        ``options.max_batch`` (default: the session's slots), one batch after another; within a
        batch all prompts are prefilled in one step, then every live sequence gets one token per
        step, and a sequence that ends gives its slot back at once."""
        require(self.model is not None, "no model is loaded")
        options = options or GenerationOptions()
        context = min(options.max_context, self.max_context)
        opts = GenerationOptions(options.max_new_tokens, context, options.temperature, options.seed,
                                 options.stop_ids, options.max_batch)
        stops = options.stop_ids if options.stop_ids is not None else self.model.spec.stop_token_ids
        batch = min(options.max_batch or self.max_batch, self.max_batch)
        self.stats = {}
        results = run_generation(self, prompts, opts, stops, batch, on_token)
        self.check_device_errors()
        return results

    # The reference's session serves one sequence at a time under these names (include/citlali/runtime/session.h:40-45),
    # with text in and out; here the same calls take and give token ids.
    def generate_once_result(self, prompt: Sequence[int], options: Optional[GenerationOptions] = None,
                             on_token: Optional[Callable[[int], None]] = None) -> GenerationResult:
        """One sequence: its generated tokens, their number and why it stopped."""
        each = (lambda index, token: on_token(token)) if on_token is not None else None
        return self.generate([prompt], options, each)[0]

    def generate_once(self, prompt: Sequence[int], options: Optional[GenerationOptions] = None,
                      on_token: Optional[Callable[[int], None]] = None) -> List[int]:
        """One sequence: its generated tokens."""
        return self.generate_once_result(prompt, options, on_token).tokens
