"""Choosing tokens from logits on the device.

temperature == 0: the reference's greedy rule (sample_greedy_from_logits,
src/model/qwen_model.cpp:448-465: index order, non-finite skipped, lowest index wins ties),
without the reference's copy of all logits to the host.  temperature > 0:
p = softmax(logits / temperature) in 32-bit and the first index whose inclusive CDF exceeds
the row's uniform number.  The reference samples with nothing else (README.md:472).
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from .. import ops
from ..errors import require


class Sampler:
    def __init__(self, device, max_rows: int = 64):
        self.device = torch.device(device)
        self._grow(max_rows)

    def _grow(self, rows: int):
        self.max_rows = rows
        pin = self.device.type == "cuda"
        self._pin = pin
        self._params = torch.zeros((2, rows), dtype=torch.float32, device=self.device)
        self._tokens = torch.zeros(rows, dtype=torch.int32, device=self.device)
        self._tokens_host = torch.zeros(rows, dtype=torch.int32, pin_memory=pin)

    def sample_device(self, logits: torch.Tensor, temperature: float, uniforms: Sequence[float]) -> torch.Tensor:
        """Token ids (int32, on the device) for each row of ``logits``."""
        rows = logits.shape[0]
        if rows > self.max_rows:
            self._grow(max(rows, 2 * self.max_rows))
        tokens = self._tokens[:rows]
        if temperature <= 0.0:
            ops.argmax_rows(logits, tokens)
            return tokens
        require(len(uniforms) == rows, "one uniform number per sampled row is needed")
        # a pinned buffer of its own for every call: the caller need not wait for this copy before it samples again
        host = torch.empty((2, rows), dtype=torch.float32)
        host[0] = float(temperature)
        host[1] = torch.as_tensor(list(uniforms), dtype=torch.float32)
        if self._pin:
            host = host.pin_memory()
        self._params[:, :rows].copy_(host, non_blocking=True)
        ops.sample_rows(logits, self._params[0], self._params[1], tokens)
        return tokens

    def sample(self, logits: torch.Tensor, temperature: float, uniforms: Sequence[float]) -> List[int]:
        """Token ids on the host (one device-to-host copy and one synchronisation)."""
        rows = logits.shape[0]
        tokens = self.sample_device(logits, temperature, uniforms)
        self._tokens_host[:rows].copy_(tokens, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self._tokens_host[:rows].tolist()
