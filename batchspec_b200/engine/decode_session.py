"""A decode loop whose token ids never leave the device: every step feeds each
request the token that the previous step chose (greedy), so the only host work
per step is the page bookkeeping and one small metadata upload.  Used by the
benchmark's device-timed decode; ``Engine.generate`` is the path with host tokens
in and out."""
from __future__ import annotations

from typing import List, Sequence

import torch

from ..kernels import ops
from .step import StepEntry


class DecodeSession:
    def __init__(self, engine, req_ids: Sequence, first_tokens: Sequence[int]):
        self.engine = engine
        self.req_ids = list(req_ids)
        self.tokens = torch.tensor(list(first_tokens), dtype=torch.int32, device=engine.device)
        self.entries = [StepEntry(r, (0,), (0,)) for r in self.req_ids]
        self.history: List[torch.Tensor] = [self.tokens.clone()]
        self.launches = 0

    @torch.inference_mode()
    def step(self) -> None:
        before = ops.launch_count()
        logits = self.engine.runner.step(self.entries, device_tokens=self.tokens)
        self.tokens = ops.argmax(logits)
        self.history.append(self.tokens)
        self.launches += ops.launch_count() - before

    def generated(self) -> List[List[int]]:
        """Token ids per request, on the host (one device->host copy)."""
        return torch.stack(self.history, dim=1).cpu().tolist()

    def close(self) -> None:
        self.history = []
