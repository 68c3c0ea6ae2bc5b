"""Device-side sampling of one token per logits row.

One kernel launch handles a batch whose rows mix greedy and sampled requests
(``ops.functional.sample_rows``); only the token ids cross to the host.  The
reference pulls the whole logits row to the host for a debug print on every
token (src/core/engine.cpp:91-110) before launching its kernels.
"""

from __future__ import annotations

from typing import List, Sequence

import torch

from ..ops import functional as F
from .params import SamplingParams, uniform


class Sampler:
    """Buffers come in two sets, used in turn: a second launch may be queued (for the step
    after) before the first one's tokens have been fetched."""

    def __init__(self, device, vocab_size: int, max_rows: int):
        self.device = device
        self.vocab_size = vocab_size
        self.max_rows = max_rows
        self._host = [torch.zeros(3, max_rows, dtype=torch.float32).pin_memory() for _ in range(2)]
        self._dev = [torch.zeros(3, max_rows, dtype=torch.float32, device=device) for _ in range(2)]
        self._probs = None
        self._out = [torch.zeros(max_rows, dtype=torch.int32, device=device) for _ in range(2)]
        self._out_host = [torch.zeros(max_rows, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._fetched = [torch.cuda.Event(), torch.cuda.Event()]
        self._rows = [0, 0]
        self._turn = 0

    def launch(self, logits: torch.Tensor, params: Sequence[SamplingParams], streams: Sequence[int],
               indices: Sequence[int]) -> int:
        """Queue the sampling of ``logits [R, V]`` (float32; row ``r`` is token number ``indices[r]``
        of stream ``streams[r]``) and the copy of the token ids to the host.  Returns the handle
        for :meth:`device_tokens` and :meth:`fetch`."""
        R = logits.shape[0]
        if R > self.max_rows:
            raise ValueError(f"Sampler: {R} rows exceed the {self.max_rows} it was built for")
        k = self._turn
        self._turn ^= 1
        self._rows[k] = R
        if R == 0:
            return k
        out = self._out[k][:R]
        if all(p.is_greedy for p in params):
            F.sample_rows(logits, out=out)
        else:
            h = self._host[k]
            for r, (p, s, i) in enumerate(zip(params, streams, indices)):
                h[0, r] = 0.0 if p.is_greedy else p.temperature
                h[1, r] = p.top_p
                h[2, r] = 0.0 if p.is_greedy else uniform(p.seed, s, i)
            dev = self._dev[k]
            dev.copy_(h, non_blocking=True)
            if self._probs is None or self._probs.shape[0] < R:
                self._probs = torch.empty(max(R, min(self.max_rows, 8)), self.vocab_size, dtype=torch.float32,
                                          device=self.device)
            F.sample_rows(logits, dev[0, :R], dev[1, :R], dev[2, :R], self._probs[:R], out)
        self._out_host[k][:R].copy_(out, non_blocking=True)
        self._fetched[k].record()
        return k

    def device_tokens(self, handle: int) -> torch.Tensor:
        """The token ids of a launch, int32 on the device (valid in stream order)."""
        return self._out[handle][:self._rows[handle]]

    def fetch(self, handle: int) -> List[int]:
        """Wait for a launch's token ids and return them."""
        R = self._rows[handle]
        if R == 0:
            return []
        self._fetched[handle].synchronize()
        return self._out_host[handle][:R].tolist()

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], streams: Sequence[int],
               indices: Sequence[int]) -> List[int]:
        """:meth:`launch` and :meth:`fetch` in one call."""
        return self.fetch(self.launch(logits, params, streams, indices))
