"""What a part is, and the registries parts are chosen from.

A layer is put together from parts: a *mixer* (mixes information between positions;
attention here), a *feed-forward* (acts on each position alone), *norms*, a *position
encoding* inside the mixer, and a *block* that arranges them around the residual stream.
A configuration names each part by ``kind`` and gives its sizes and constants as
``params``; a part never looks at the model it is in.

Interfaces (all tensors are on the model's device; ``x`` is the float32 residual stream
``[rows, hidden]``; ``h`` is a normed copy in the compute dtype):

* every part: ``__init__(params, prefix)`` (no device work), ``tensor_specs()`` -> the
  checkpoint tensors it needs, ``bind(weights, ctx)`` -> take them from a ``{name: WeightHandle}``
  map onto the device.
* norm: ``forward(x, row_index=None) -> h`` (``row_index`` int32 picks and orders rows).
* mixer: ``cache_requirement()`` -> KVRequirement | StateRequirement | None;
  ``forward(h, batch, cache_view, residual, write_cache)`` adds its output into ``residual``
  in place.  ``batch`` is a :class:`StepBatch`: the rows of one sequence are consecutive and in
  position order, ``batch.row_slot`` / ``batch.row_pos`` say whose they are and where.
* feed-forward: ``forward(h, batch, residual)`` adds its output into ``residual`` in place.
* position encoding: ``__init__(params, head_dim)``; see :mod:`.rotary`.
* block: ``__init__(layer_spec)`` builds the parts it knows by name from ``layer_spec.parts``
  (:func:`build_part`); ``parts()``, ``tensor_specs()``, ``cache_requirement()``, ``bind``;
  ``forward(x, batch, cache_view, write_cache)`` updates ``x`` in place.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..errors import require

_REGISTRIES: Dict[str, Dict[str, type]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {},
}


def register_part(role: str, kind: str, cls: type, replace: bool = False) -> None:
    require(role in _REGISTRIES, f"unknown part role '{role}'; roles: {', '.join(_REGISTRIES)}")
    require(replace or kind not in _REGISTRIES[role], f"{role} kind '{kind}' is already registered")
    _REGISTRIES[role][kind] = cls


def unregister_part(role: str, kind: str) -> None:
    _REGISTRIES[role].pop(kind, None)


def part_class(role: str, kind: str) -> type:
    require(role in _REGISTRIES, f"unknown part role '{role}'")
    table = _REGISTRIES[role]
    require(kind in table, f"unknown {role} kind '{kind}'; registered: {', '.join(sorted(table)) or '(none)'}")
    return table[kind]


def registered_parts(role: str) -> List[str]:
    return sorted(_REGISTRIES[role])


def build_part(role: str, spec):
    """The part a :class:`PartSpec` describes, from the registry of ``role``."""
    return part_class(role, spec.kind)(spec.params, spec.prefix)


@dataclass
class BuildContext:
    """Where and how a model is built: device, compute dtype (bfloat16: the serving kernels and
    precisions; float32: everything in true 32-bit) and the device word kernels raise on a
    fault they detect themselves."""
    device: torch.device
    dtype: torch.dtype
    error_flag: Optional[torch.Tensor] = None

    @property
    def is_float32(self) -> bool:
        return self.dtype == torch.float32


@dataclass
class NormedRows:
    """Rows that stand for ``rms_norm(x)`` without having been normalised: ``rows`` is bfloat16(x), ``sumsq[r, g]``
    the sum of squares of x[r]'s g-th group of 32 features.  A product whose weights carry the norm's gain reads
    ``rows`` and multiplies its result rows by ``rsqrt(sum(sumsq[r]) / dim + eps)``: the same numbers as the product
    of the normalised rows, with the norm's kernel saved."""
    rows: torch.Tensor
    sumsq: torch.Tensor
    dim: int
    eps: float = 0.0

    def with_eps(self, eps: float) -> "NormedRows":
        return NormedRows(self.rows, self.sumsq, self.dim, float(eps))

    @property
    def scale(self):
        return (self.sumsq, self.dim, self.eps)


@dataclass
class StepBatch:
    """One step's rows.  Sequence ``b`` owns rows ``seq_start[b] .. seq_start[b+1]-1``, which are
    its new tokens in order, at positions ``past[b] .. past[b]+n_new[b]-1`` of slot ``slots[b]``."""
    tokens: torch.Tensor          # [rows] int32
    row_slot: torch.Tensor        # [rows] int32
    row_pos: torch.Tensor         # [rows] int32
    seq_start: torch.Tensor       # [sequences + 1] int32
    seq_slot: torch.Tensor        # [sequences] int32
    seq_past: torch.Tensor        # [sequences] int32
    want_rows: torch.Tensor       # [wanted] int32, rows whose logits are asked for
    slots: List[int]
    past: List[int]
    n_new: List[int]
    # A block that ends with a product which emitted what the next norm needs of the residual rows leaves it here
    # (``norm_carry``); the model hands it to the next layer as ``norm_carry_in`` and clears it, so a layer that does
    # not know of it breaks the chain instead of passing on something stale.
    norm_carry: Optional["NormedRows"] = None
    norm_carry_in: Optional["NormedRows"] = None

    @property
    def rows(self) -> int:
        return int(self.tokens.shape[0])

    @property
    def sequences(self) -> int:
        return len(self.slots)

    @property
    def is_decode(self) -> bool:
        """Every sequence brings exactly one token."""
        return all(n == 1 for n in self.n_new)

    @property
    def max_keys(self) -> int:
        return max(p + n for p, n in zip(self.past, self.n_new))

    @property
    def max_new(self) -> int:
        return max(self.n_new)


def bind_gain(weights, name: str, size: int, ctx: BuildContext) -> torch.Tensor:
    """A norm's gain on the device: float32 on the 32-bit path and when it is stored in 32-bit (a tensor
    stored so stays so), else bfloat16 (a float16 gain is rounded once)."""
    h = weights[name]
    require(tuple(h.shape) == (size,), f"unexpected tensor shape for {name}: got {list(h.shape)}, expected {[size]}")
    dtype = torch.float32 if (ctx.is_float32 or h.dtype == torch.float32) else torch.bfloat16
    return h.tensor.to(device=ctx.device, dtype=dtype).contiguous()
