"""A decoder built from a ModelSpec: embedding, the schedule of layers, final norm, head.

The forward pass follows QwenModel::forward_token (src/model/qwen_model.cpp:239-419) for a
batch of rows instead of one token: embedding rows, each scheduled layer on all rows, and
only for the rows whose logits are wanted the final norm and the output matrix (the
reference skips both for prompt tokens that are not the last, :378-380).  Which layers
exist, what they are made of, and in which order they run is the spec's data.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from ..config.spec import ModelSpec
from ..errors import require
from ..parts.base import BuildContext, StepBatch, build_part, part_class
from ..parts.linear import DenseLinear
from ..weights.loader import TensorSpec, WeightHandle


def _numel(shape) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n


def _build_layers(spec: ModelSpec):
    return [part_class("block", l.block)(l) for l in spec.layers]


def expected_tensors(spec: ModelSpec) -> List[TensorSpec]:
    """Every checkpoint tensor the model reads, in a fixed order.  No device is touched."""
    specs = [TensorSpec(spec.embedding_name, (spec.vocab_size, spec.hidden_size), "matrix")]
    for block in _build_layers(spec):
        specs.extend(block.tensor_specs())
    specs.extend(build_part("norm", spec.final_norm).tensor_specs())
    # tied: the head is the embedding and a stored head is ignored; undecided: used if present
    specs.append(TensorSpec(spec.head_name, (spec.vocab_size, spec.hidden_size), "matrix",
                            optional=spec.tie_head_to_embedding is not False))
    seen = set()
    for s in specs:
        require(s.name not in seen, f"two parts of the model claim the tensor '{s.name}'")
        seen.add(s.name)
    return specs


def cache_requirements_of(spec: ModelSpec, layers=None) -> List[object]:
    """Per schedule step: what it keeps (a KVRequirement, a StateRequirement, or None for a step that keeps
    nothing or reads another step's cache).  No device is touched."""
    layers = layers if layers is not None else _build_layers(spec)
    return [None if step.cache_of is not None else layers[step.layer].cache_requirement() for step in spec.schedule]


class DecoderModel:
    def __init__(self, spec: ModelSpec, ctx: BuildContext):
        spec.validate()
        self.spec = spec
        self.ctx = ctx
        self.layers = _build_layers(spec)
        self.final_norm = build_part("norm", spec.final_norm)
        self.head = DenseLinear([spec.head_name], [spec.vocab_size], spec.hidden_size)
        self.embedding: Optional[torch.Tensor] = None
        self.tied = None

    def tensor_specs(self) -> List[TensorSpec]:
        return expected_tensors(self.spec)

    def cache_requirements(self) -> List[object]:
        return cache_requirements_of(self.spec, self.layers)

    def bind(self, weights: Dict[str, WeightHandle]) -> None:
        ctx, spec = self.ctx, self.spec
        emb = weights[spec.embedding_name]
        require(tuple(emb.shape) == (spec.vocab_size, spec.hidden_size),
                f"unexpected tensor shape for {spec.embedding_name}: got {list(emb.shape)}, "
                f"expected {[spec.vocab_size, spec.hidden_size]}")
        self.embedding = torch.empty((spec.vocab_size, spec.hidden_size), dtype=ctx.dtype, device=ctx.device)
        emb.copy_into(self.embedding)
        for block in self.layers:
            block.bind(weights, ctx)
        self.final_norm.bind(weights, ctx)
        tie = spec.tie_head_to_embedding
        if tie is None:
            tie = spec.head_name not in weights      # absent head: reuse the embedding (qwen_model.cpp:71-75)
        self.tied = bool(tie)
        if self.tied:
            self.head.bind_shared(self.embedding, ctx)
        else:
            require(spec.head_name in weights, f"missing required tensor: {spec.head_name}")
            self.head.bind(weights, ctx)

    def weight_bytes_read_per_step(self) -> int:
        """Bytes of weights one step reads when each matrix it uses is read once: every tensor the layers
        declare as a matrix (``tensor_specs()``, so lists of matrices inside a part count too), once per
        schedule step that runs the layer, plus the output matrix.  The embedding's rows and the norm
        gains are left out: they are thousands of times smaller."""
        size = torch.tensor([], dtype=self.ctx.dtype).element_size()
        per_layer = [sum(_numel(t.shape) for t in block.tensor_specs() if t.role == "matrix") * size
                     for block in self.layers]
        return self.head.nbytes + sum(per_layer[step.layer] for step in self.spec.schedule)

    def forward(self, batch: StepBatch, cache) -> torch.Tensor:
        """Logits ``[wanted, vocab]`` float32 for ``batch.want_rows``, in that order."""
        ctx, spec = self.ctx, self.spec
        x = torch.empty((batch.rows, spec.hidden_size), dtype=torch.float32, device=ctx.device)
        ops.embed_rows(self.embedding, batch.tokens, x, ctx.error_flag,
                       1.0 if spec.embedding_scale is None else float(spec.embedding_scale))
        batch.norm_carry = None
        for i, step in enumerate(spec.schedule):
            source = i if step.cache_of is None else step.cache_of
            view = cache.view(source) if cache.has_view(source) else None
            # what the layer before left for this layer's first norm, if it left anything (parts/block.py)
            batch.norm_carry_in, batch.norm_carry = batch.norm_carry, None
            self.layers[step.layer].forward(x, batch, view, write_cache=step.cache_of is None)
        batch.norm_carry_in = batch.norm_carry = None
        wanted = int(batch.want_rows.numel())
        if wanted == 0:
            return torch.empty((0, spec.vocab_size), dtype=torch.float32, device=ctx.device)
        h = self.final_norm.forward(x, row_index=batch.want_rows)
        logits = self.head.forward(h, out_dtype=torch.float32)
        if spec.logit_scale is not None:
            ops.scale_(logits, float(spec.logit_scale))
        return logits
