"""Next-token selection (batchspec/backends/utils/sampling.py:61-115):
temperature 0 is argmax; otherwise sample from softmax(logits / T), restricted to
the top_k most probable tokens if top_k > 0 and to the smallest set of mass
top_p if top_p > 0, both when both are set.

The reference draws from the library's samplers with the global generator, so a
request's token depends on the order of the batch.  Here every draw is a hash of
(seed, request id, index of the token in the request's output): the same request
gets the same tokens however it is batched or cut.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from ..kernels import ops


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_k: int = -1
    top_p: float = 0.0


class Sampler:
    def __init__(self, device, seed: int = 0, defaults: Optional[SamplingParams] = None):
        self.device = torch.device(device)
        self.seed = int(seed)
        self.defaults = defaults or SamplingParams()

    def greedy(self, logits: torch.Tensor) -> torch.Tensor:
        return ops.argmax(logits)

    def sample(self, logits: torch.Tensor, temperature: Sequence[float], top_k: Sequence[int],
               top_p: Sequence[float], stream_ids: Sequence[int], counters: Sequence[int]) -> torch.Tensor:
        """One token per row of ``logits`` (float32 [rows, vocab]); int32 on the device."""
        rows = logits.shape[0]
        if rows == 0:
            return torch.empty((0,), dtype=torch.int32, device=self.device)
        if all(t <= 0 for t in temperature):
            return ops.argmax(logits)
        f = np.empty((2, rows), dtype=np.float32)
        f[0], f[1] = temperature, top_p
        i = np.empty((2, rows), dtype=np.int64)
        i[0], i[1] = stream_ids, counters
        fd = torch.from_numpy(f).to(self.device, non_blocking=True)
        idv = torch.from_numpy(i).to(self.device, non_blocking=True)
        kd = torch.tensor(list(top_k), dtype=torch.int32).to(self.device, non_blocking=True)
        return ops.sample(logits, fd[0], kd, fd[1], idv[0], idv[1], self.seed)
