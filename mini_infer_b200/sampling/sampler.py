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
    def __init__(self, device, vocab_size: int, max_rows: int):
        self.device = device
        self.vocab_size = vocab_size
        self.max_rows = max_rows
        self._host = torch.zeros(3, max_rows, dtype=torch.float32).pin_memory()
        self._dev = torch.zeros(3, max_rows, dtype=torch.float32, device=device)
        self._probs = None
        self._out = torch.zeros(max_rows, dtype=torch.int32, device=device)
        self._out_host = torch.zeros(max_rows, dtype=torch.int32).pin_memory()

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], streams: Sequence[int],
               indices: Sequence[int]) -> List[int]:
        """``logits [R, V]`` float32; row ``r`` is token number ``indices[r]`` of stream ``streams[r]``."""
        R = logits.shape[0]
        if R == 0:
            return []
        if R > self.max_rows:
            raise ValueError(f"Sampler: {R} rows exceed the {self.max_rows} it was built for")
        out = self._out[:R]
        if all(p.is_greedy for p in params):
            F.sample_rows(logits, out=out)
        else:
            h = self._host
            for r, (p, s, i) in enumerate(zip(params, streams, indices)):
                h[0, r] = 0.0 if p.is_greedy else p.temperature
                h[1, r] = p.top_p
                h[2, r] = 0.0 if p.is_greedy else uniform(p.seed, s, i)
            self._dev.copy_(h, non_blocking=True)
            if self._probs is None or self._probs.shape[0] < R:
                self._probs = torch.empty(max(R, min(self.max_rows, 8)), self.vocab_size, dtype=torch.float32,
                                          device=self.device)
            F.sample_rows(logits, self._dev[0, :R], self._dev[1, :R], self._dev[2, :R], self._probs[:R], out)
        self._out_host[:R].copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self._out_host[:R].tolist()
