"""Generation through the whole engine: model, cache, scheduler, sampler.

Reference: ``Engine::generate_paged`` (src/core/engine.cpp:233-330) prefills one
prompt and decodes token by token for one request; ``generate_batched_paged``
(:348-486) does the same for a fixed batch.  Here every call goes through the
continuous-batching scheduler, whatever the number of prompts.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, Hashable, Iterator, List, Optional, Sequence, Tuple, Union

import torch

from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .defaults import DEFAULT_PAGE_SIZE
from .loading import load_model
from .model import Model
from .request import Request
from .scheduler import IterationStats, Scheduler, SchedulerConfig
from ..cache.pages import OutOfPages
from .step import ModelRunner, StepEntry
from ..parts.tuning import TUNING


@dataclass
class GenerationOutput:
    prompt_token_ids: List[int]
    token_ids: List[int]
    finish_reason: Optional[str]
    ttft: Optional[float] = None
    seconds: float = 0.0
    preemptions: int = 0


class GPUExecutor:
    """What the scheduler drives: the model runner and the sampler.

    When the scheduler says that the next step will decode one token for exactly the requests
    sampled now (unless a stop token ends one), that step is launched *ahead*: it takes its token
    ids from the sampler's device buffer, so the device goes on while the host fetches the tokens
    and plans.  If the next call asks for that very step, it is adopted; anything else (a request
    ended, was added or preempted) drops it, and the step decided instead overwrites what it wrote.
    """

    lookahead_capable = True

    def __init__(self, runner: ModelRunner, sampler: Sampler):
        self.runner = runner
        self.sampler = sampler
        self.cache = runner.cache
        self._ahead = None          # (request ids, sampler handle, token ids the step was fed | None, note)
        self.steps_adopted = 0
        self.steps_dropped = 0
        # A debugging and testing hook: ``observer.after_forward(request ids, tokens of each, logits or
        # None) -> note`` is called right after every forward pass (before anything can overwrite what the
        # pass left behind), and ``observer.settled(note, kept)`` once it is known whether the step counts
        # (a step launched ahead may be dropped).
        self.observer = None

    def _drop_ahead(self) -> None:
        if self._ahead is not None:
            self.runner.drop_ahead(self._ahead[0])
            if self.observer is not None:
                self.observer.settled(self._ahead[3], False)
            self._ahead = None
            self.steps_dropped += 1

    def add_request(self, rid: Hashable) -> None:
        self._drop_ahead()
        self.runner.add_request(rid)

    def release(self, rid: Hashable) -> None:
        self._drop_ahead()
        self.runner.release(rid)

    def run(self, entries: Sequence[StepEntry], sample_for: Sequence[Request],
            lookahead: bool = False) -> Dict[Hashable, int]:
        rids = [r.rid for r in sample_for]
        ahead = self._ahead
        if ahead is not None and ahead[0] == rids and len(entries) == len(rids) and all(
                e.rid == rid and list(e.tokens) == [tok] and list(e.want) == [0]
                for e, rid, tok in zip(entries, rids, ahead[2])):
            self._ahead = None
            self.runner.adopt_ahead(rids)
            self.steps_adopted += 1
            handle = ahead[1]
            if self.observer is not None:
                self.observer.settled(ahead[3], True)
        else:
            self._drop_ahead()
            res = self.runner.step(entries)
            if self.observer is not None:
                self.observer.settled(self.observer.after_forward([e.rid for e in entries],
                                                                  [len(e.tokens) for e in entries], res.logits), True)
            if not sample_for:
                return {}
            assert [rid for rid, _ in res.index] == rids
            handle = self.sampler.launch(res.logits, [r.params for r in sample_for],
                                         [r.stream for r in sample_for], [len(r.generated) for r in sample_for])
        if lookahead and self.runner.can_step_ahead(rids):
            try:
                logits = self.runner.step_ahead(rids, self.sampler.device_tokens(handle))
            except OutOfPages:
                pass                # the scheduler decides what makes room
            else:
                nxt = self.sampler.launch(logits, [r.params for r in sample_for], [r.stream for r in sample_for],
                                          [len(r.generated) + 1 for r in sample_for])
                note = self.observer.after_forward(rids, [1] * len(rids), logits) if self.observer is not None else None
                self._ahead = (rids, nxt, None, note)
        toks = self.sampler.fetch(handle)
        if self._ahead is not None:
            self._ahead = (rids, self._ahead[1], toks, self._ahead[3])
        return {r.rid: t for r, t in zip(sample_for, toks)}


class LLM:
    """A loaded model ready to generate.

    ``max_seq_len`` is the context limit of a request (the reference's ``--max-seq-len``,
    src/core/main.cc:47, :75); ``num_pages`` defaults to what ``max_running`` requests of
    that length need, capped by ``memory_fraction`` of the free device memory.
    """

    def __init__(self, model: Union[str, Model], dtype: str = "bfloat16", device: str = "cuda:0",
                 max_seq_len: int = 2048, page_size: Optional[int] = None, num_pages: Optional[int] = None,
                 max_running: int = 64, max_tokens_per_step: int = 2048, prefill_chunk: int = 0,
                 memory_fraction: float = 0.85, runtime=None, cuda_graphs: bool = True):
        if isinstance(model, str):
            self.model, self.rt, self.config_json = load_model(model, dtype, device)
        else:
            self.model, self.rt, self.config_json = model, runtime, None
            if runtime is None:
                raise ValueError("LLM: a built model needs its runtime")
        page_size = page_size or DEFAULT_PAGE_SIZE
        max_seq_len = int(max_seq_len)
        pages_per_req = -(-max_seq_len // page_size)
        if num_pages is None:
            num_pages = max_running * pages_per_req
            item = 4 if self.rt.precision.name == "float32" else 2
            per_page = sum(g.num_layers * g.need.bytes_per_page(page_size, item) * float(g.need.pages_fraction)
                           for g in self.model.kv_groups)
            free, _ = torch.cuda.mem_get_info(self.rt.device)
            if per_page:
                num_pages = max(pages_per_req, min(num_pages, int(free * memory_fraction) // per_page))
        max_tokens_per_step = max(max_tokens_per_step, max_running)
        self.runner = ModelRunner(self.model, self.rt, page_size=page_size, num_pages=num_pages,
                                  max_requests=max_running, max_tokens_per_step=max_tokens_per_step,
                                  max_context=max_seq_len, cuda_graphs=cuda_graphs,
                                  graph_chunk_tokens=min(prefill_chunk or max_tokens_per_step, max_tokens_per_step)
                                  if TUNING.prefill_chunk_graph_min_tokens > 0 and
                                  min(prefill_chunk or max_tokens_per_step, max_tokens_per_step)
                                  >= TUNING.prefill_chunk_graph_min_tokens else 0)
        self.sampler = Sampler(self.rt.device, self.model.spec.vocab_size, max_running)
        self.executor = GPUExecutor(self.runner, self.sampler)
        self.sched_cfg = SchedulerConfig(max_tokens_per_step=max_tokens_per_step, max_running=max_running,
                                         prefill_chunk=prefill_chunk, max_context=max_seq_len)
        self.last_history: List[IterationStats] = []
        self._calls = 0

    def _submit(self, prompts, params):
        if params is None:
            params = SamplingParams()
        plist = list(params) if isinstance(params, (list, tuple)) else [params] * len(prompts)
        if len(plist) != len(prompts):
            raise ValueError("LLM.generate: one SamplingParams per prompt (or one for all)")
        V = self.model.spec.vocab_size
        for p in prompts:
            for t in p:
                if not 0 <= int(t) < V:
                    raise ValueError(f"LLM.generate: token id {t} outside [0, {V})")
        sched = Scheduler(self.executor, self.sched_cfg)
        self._calls += 1
        reqs = [Request((self._calls, i), list(p), sp, stream=i) for i, (p, sp) in enumerate(zip(prompts, plist))]
        for r in reqs:
            sched.submit(r)
        return sched, reqs

    def warm_up(self, batch_sizes: Optional[Sequence[int]] = None) -> int:
        """Capture the decode passes ahead of the first request: one step of ``B`` one-token requests for every
        captured batch size up to ``max_running`` (or for ``batch_sizes``), in the smallest context bucket.
        A capture costs tens of milliseconds, which the first requests of a serving process would otherwise
        wait for whenever their batch reaches a new size.  Returns the number of passes captured.  The
        requests it uses are released again; nothing of them stays in the cache."""
        runner = self.runner
        if not runner.cuda_graphs:
            return 0
        limit = min(runner.max_requests, runner.max_tokens)
        if batch_sizes is None:
            sizes = sorted({runner._graph_batch(b) for b in range(1, limit + 1)})
        else:
            sizes = sorted({runner._graph_batch(int(b)) for b in batch_sizes if 1 <= int(b) <= limit})
        sizes = sizes[:max(0, runner.max_context - 1)]       # the first request takes part in every step
        before = len(runner._graphs)
        rids = [("warm-up", i) for i in range(max(sizes, default=0))]
        done: List = []
        try:
            for rid in rids:
                runner.add_request(rid)
                done.append(rid)
            if rids:
                runner.step([StepEntry(rid, [0], []) for rid in rids])          # a first token each
            for b in sizes:
                runner.step([StepEntry(rid, [0], [0]) for rid in rids[:b]])     # the captured decode step
        except OutOfPages:
            pass                                              # a pool too small for this many requests: as far as it went
        finally:
            for rid in done:
                runner.release(rid)
        return len(runner._graphs) - before

    def generate(self, prompts: Sequence[Sequence[int]],
                 params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> List[GenerationOutput]:
        """Token ids in, token ids out; request ``i`` samples from random stream ``i``."""
        t0 = time.perf_counter()
        sched, reqs = self._submit(prompts, params)
        sched.run_until_done()
        self.last_history = sched.history
        return [self._output(r, t0) for r in reqs]

    @staticmethod
    def _output(r: Request, t0: float) -> GenerationOutput:
        return GenerationOutput(r.prompt, list(r.generated), r.finish_reason, r.metrics.ttft,
                                (r.metrics.finished or time.perf_counter()) - t0, r.metrics.preemptions)

    def generate_iter(self, prompts: Sequence[Sequence[int]],
                      params: Union[SamplingParams, Sequence[SamplingParams], None] = None
                      ) -> Iterator[Tuple[int, int]]:
        """As :meth:`generate`, but yields ``(request index, token id)`` as soon as the scheduler's step
        that sampled the token has ended (the reference streams the lines its binary prints,
        sdk/mini_infer_sdk/backends/local.py:218-254).  The outputs are in ``self.last_outputs`` when the
        iterator is exhausted; a consumer that stops early ends the requests and frees their pages."""
        t0 = time.perf_counter()
        sched, reqs = self._submit(prompts, params)
        seen = [0] * len(reqs)
        try:
            while not sched.done():
                before = (len(sched.running), len(sched.waiting), len(sched.finished))
                st = sched.step()
                for i, r in enumerate(reqs):
                    while seen[i] < len(r.generated):
                        yield i, r.generated[seen[i]]
                        seen[i] += 1
                if st.num_tokens == 0 and st.preempted == 0 and \
                        (len(sched.running), len(sched.waiting), len(sched.finished)) == before:
                    raise RuntimeError("Scheduler: no progress is possible (no tokens scheduled, nothing finished)")
        finally:
            for r in list(sched.running):
                sched._finish(r, "cancelled")
            sched.waiting.clear()
            self.last_history = sched.history
            self.last_outputs = [self._output(r, t0) for r in reqs]
