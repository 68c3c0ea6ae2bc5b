"""A generation request as the scheduler sees it.

Reference: ``Request`` with states Pending -> Prefilling -> Decoding -> Finished,
``RequestMetrics`` (arrival, first token, decode time, finish reason) and
constructor checks (src/scheduler/request.h:24-143, src/scheduler/request.cpp:18-32).
Here a request is the list of all its tokens (prompt, then what it generated)
and a count of how many of them are in the cache; "prefill" and "decode" are
just "more than one token left to feed" and "exactly one".
"""

from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Hashable, List, Optional

from ..sampling.params import SamplingParams


class RequestState(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


@dataclass
class RequestMetrics:
    arrival: float = 0.0
    first_token: Optional[float] = None
    finished: Optional[float] = None
    steps: int = 0
    preemptions: int = 0

    @property
    def ttft(self) -> Optional[float]:
        return None if self.first_token is None else self.first_token - self.arrival


class Request:
    def __init__(self, rid: Hashable, prompt: List[int], params: SamplingParams, stream: int = 0):
        if len(prompt) == 0:
            raise ValueError("Request: the prompt is empty")   # src/scheduler/request.cpp:18-32
        self.rid = rid
        self.prompt = [int(t) for t in prompt]
        self.params = params
        self.stream = int(stream)
        self.generated: List[int] = []
        self.num_computed = 0            # tokens whose keys and values are in the cache
        self.state = RequestState.WAITING
        self.finish_reason: Optional[str] = None
        self.metrics = RequestMetrics(arrival=time.perf_counter())
        self.admit_order = -1

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.generated

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.generated)

    @property
    def remaining(self) -> int:
        """Tokens not yet fed; the request yields a new token when this reaches zero."""
        return self.num_tokens - self.num_computed

    def next_tokens(self, n: int) -> List[int]:
        lo = self.num_computed
        if lo + n <= len(self.prompt):
            return self.prompt[lo:lo + n]
        return self.tokens[lo:lo + n]

    def finish(self, reason: str) -> None:
        self.state = RequestState.FINISHED
        self.finish_reason = reason
        self.metrics.finished = time.perf_counter()
