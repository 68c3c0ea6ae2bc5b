"""Per-request sampling parameters and the counter-based uniforms behind them.

Names and defaults follow the reference's ``SamplingParams{greedy=true,
top_p=0.9, temperature=1.0, seed=42}`` (src/scheduler/request.h:37-48) and its
``SamplingMode::{Greedy, TopP}`` (src/core/engine.h:18-21).  The reference
advances one global seed per call (src/core/engine.cpp:120-121) and its
scheduler samples greedily whatever the request says
(src/scheduler/scheduler.cpp:233, :310-312).  Here the uniform that decides
token ``n`` of a request is a pure function of (seed, stream, n), where the
stream is the request's number in its ``generate`` call, so what a request
generates does not depend on its batch, on step boundaries or on preemption.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Sequence, Tuple

_M0, _M1 = 0xD2511F53, 0xCD9E8D57
_W0, _W1 = 0x9E3779B9, 0xBB67AE85
_MASK = 0xFFFFFFFF


@dataclass
class SamplingParams:
    greedy: bool = True
    temperature: float = 1.0
    top_p: float = 0.9
    seed: int = 42
    max_new_tokens: int = 100
    stop_token_ids: Tuple[int, ...] = ()

    def __post_init__(self):
        if self.max_new_tokens < 1:
            raise ValueError("SamplingParams: max_new_tokens must be at least 1")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("SamplingParams: top_p must lie in (0, 1]")
        if self.temperature < 0.0:
            raise ValueError("SamplingParams: temperature must not be negative")
        self.stop_token_ids = tuple(int(t) for t in self.stop_token_ids)

    @property
    def is_greedy(self) -> bool:
        return self.greedy or self.temperature <= 0.0


def philox4x32(counter: Sequence[int], key: Sequence[int], rounds: int = 10) -> Tuple[int, int, int, int]:
    """Philox-4x32 with the usual ten rounds (Salmon, Moraes, Dror, Shaw, SC'11)."""
    c0, c1, c2, c3 = (int(x) & _MASK for x in counter)
    k0, k1 = (int(x) & _MASK for x in key)
    for _ in range(rounds):
        p0, p1 = _M0 * c0, _M1 * c2
        c0, c1, c2, c3 = ((p1 >> 32) ^ c1 ^ k0) & _MASK, p1 & _MASK, ((p0 >> 32) ^ c3 ^ k1) & _MASK, p0 & _MASK
        k0, k1 = (k0 + _W0) & _MASK, (k1 + _W1) & _MASK
    return c0, c1, c2, c3


def uniform(seed: int, stream: int, index: int) -> float:
    """Uniform in [0, 1) with 24 random bits for token ``index`` of ``stream`` under ``seed``."""
    r = philox4x32((index, index >> 32, stream, stream >> 32), (seed, seed >> 32))
    return (r[0] >> 8) * (1.0 / 16777216.0)
