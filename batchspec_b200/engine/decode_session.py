"""A decode loop whose token ids never leave the device: every step feeds each
request the token that the previous step chose (greedy), so the only host work
per step is the page bookkeeping and one small metadata upload.  Runs through
the captured decode graph when the engine has one for this batch size, else
through the plain step function.  Used by the benchmark's device-timed decode;
``Engine.generate`` is the path with host tokens in and out."""
from __future__ import annotations

from typing import List, Sequence

import torch

from ..kernels import ops
from .step import StepEntry


class DecodeSession:
    def __init__(self, engine, req_ids: Sequence, first_tokens: Sequence[int], keep_history: bool = False):
        self.engine = engine
        self.req_ids = list(req_ids)
        self.B = len(self.req_ids)
        self.first = list(first_tokens)
        self.tokens = torch.tensor(self.first, dtype=torch.int32, device=engine.device)
        self.entries = [StepEntry(r, (0,), (0,)) for r in self.req_ids]
        self.keep_history = keep_history
        self.history: List[torch.Tensor] = [self.tokens.clone()] if keep_history else []
        self.launches = 0
        self.steps = 0
        self.graph = engine.decode_graph(self.B)
        self._zeros_f = [0.0] * self.B
        self._zeros_i = [0] * self.B

    @torch.inference_mode()
    def step(self) -> None:
        before = ops.launch_count()
        eng = self.engine
        if self.graph is not None:
            for rid in self.req_ids:
                eng.cache.reserve(rid, 1)
            self.tokens = self.graph.run(self.req_ids, self.first if self.steps == 0 else None, self._zeros_f,
                                         self._zeros_i, self._zeros_f, self._zeros_i, self._zeros_i)
            for rid in self.req_ids:
                eng.cache.commit(rid, 1)
        else:
            logits = eng.runner.step(self.entries, device_tokens=self.tokens)
            self.tokens = ops.argmax(logits)
        if self.keep_history:
            self.history.append(self.tokens.clone())
        self.steps += 1
        self.launches += ops.launch_count() - before

    def generated(self) -> List[List[int]]:
        """Token ids per request, on the host (one device->host copy)."""
        ops.status_to_host_async()
        out = torch.stack(self.history, dim=1).cpu().tolist()
        ops.raise_if_gave_up()
        return out

    def close(self) -> None:
        """Ends the session; raises if a kernel of one of its steps gave up a bounded wait."""
        self.history = []
        ops.check_status()
