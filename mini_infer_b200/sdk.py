"""Python entry point in the manner of the reference's ``mini_infer_sdk`` (offline mode).

Same names and meanings: ``MiniInfer(model_path=...)`` with ``generate``,
``stream``, ``tokenize``, ``detokenize`` (sdk/mini_infer_sdk/engine.py:30-118);
``InferenceConfig`` and ``SamplingConfig`` with the same fields and defaults
(sdk/mini_infer_sdk/config.py:8-30); ``GenerationResult`` with the same
attributes (sdk/mini_infer_sdk/result.py:6-52).  The reference's local backend
starts the C++ binary once per call and parses its output
(sdk/mini_infer_sdk/backends/local.py:204-254); here the engine lives in the
calling process and the model stays loaded between calls.  ``endpoint=`` (the
HTTP backend), ``draft_path=`` (speculative decoding), ``chat`` and ``batch``
helpers that need the server are not part of this engine.

Token ids work everywhere a prompt does (``generate([1, 2, 3])``), because
random-weight models have no tokenizer; ``generate_ids`` runs many prompts as
one continuous batch.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from enum import Enum
from typing import Iterator, List, Optional, Sequence, Union


class SamplingMode(str, Enum):
    GREEDY = "greedy"
    TOP_P = "top_p"


@dataclass
class SamplingConfig:
    mode: SamplingMode = SamplingMode.GREEDY
    temperature: float = 1.0
    top_p: float = 0.9
    seed: int = 42


@dataclass
class InferenceConfig:
    max_new_tokens: int = 256
    max_seq_len: int = 2048
    device: int = 0
    paged: bool = True
    gamma: int = 4
    sampling: SamplingConfig = field(default_factory=SamplingConfig)
    draft_path: Optional[str] = None
    python_path: str = "python3"
    # additions of this engine
    dtype: str = "bfloat16"
    max_running: int = 64
    max_tokens_per_step: int = 2048
    prefill_chunk: int = 0
    page_size: Optional[int] = None
    num_pages: Optional[int] = None


class GenerationResult:
    """Attributes as in sdk/mini_infer_sdk/result.py:6-52."""

    def __init__(self, text: str, tokens: Optional[List[int]] = None, prompt_tokens: int = 0,
                 generated_tokens: Optional[int] = None, elapsed_sec: float = 0.0,
                 accept_rate: Optional[float] = None, tokens_per_sec: Optional[float] = None,
                 wall_sec: Optional[float] = None, finish_reason: Optional[str] = None):
        self.text = text
        self.tokens = tokens or []
        self.prompt_tokens = prompt_tokens
        if generated_tokens is not None:
            self.generated_tokens = generated_tokens
        else:
            self.generated_tokens = (len(self.tokens) - prompt_tokens) if tokens else 0
        self.elapsed_sec = elapsed_sec
        self.wall_sec = wall_sec if wall_sec is not None else elapsed_sec
        self.tokens_per_sec = tokens_per_sec if tokens_per_sec is not None else (
            self.generated_tokens / elapsed_sec if elapsed_sec > 0 else 0.0)
        self.accept_rate = accept_rate
        self.finish_reason = finish_reason

    @property
    def generated_ids(self) -> List[int]:
        return self.tokens[self.prompt_tokens:]

    def __repr__(self):
        return f"GenerationResult(generated={self.generated_tokens}, tps={self.tokens_per_sec:.1f})"


Prompt = Union[str, Sequence[int]]


class MiniInfer:
    def __init__(self, model_path: Optional[str] = None, draft_path: Optional[str] = None,
                 binary: Optional[str] = None, python_path: Optional[str] = None,
                 endpoint: Optional[str] = None, config: Optional[InferenceConfig] = None):
        if endpoint:
            raise NotImplementedError("MiniInfer: online mode (endpoint=) needs the HTTP server, "
                                      "which is not part of this engine")
        if draft_path:
            raise NotImplementedError("MiniInfer: speculative decoding (draft_path=) is not part of this engine")
        if not model_path:
            raise ValueError("Provide model_path (offline).")
        self.config = config or InferenceConfig()
        self.model_path = model_path
        from .engine.llm import LLM
        from .tokenizer import load_tokenizer
        c = self.config
        self.llm = LLM(model_path, dtype=c.dtype, device=f"cuda:{c.device}", max_seq_len=c.max_seq_len,
                       page_size=c.page_size, num_pages=c.num_pages, max_running=c.max_running,
                       max_tokens_per_step=c.max_tokens_per_step, prefill_chunk=c.prefill_chunk)
        self.tokenizer = load_tokenizer(model_path)

    # -- properties ---------------------------------------------------------- #
    @property
    def is_remote(self) -> bool:
        return False

    @property
    def model_name(self) -> str:
        import os
        return os.path.basename(os.path.normpath(self.model_path))

    # -- helpers ------------------------------------------------------------- #
    def tokenize(self, text: str) -> List[int]:
        if self.tokenizer is None:
            raise RuntimeError("MiniInfer: this model folder has no tokenizer.json; pass token ids")
        return self.tokenizer.encode(text)

    def detokenize(self, ids: List[int]) -> str:
        if self.tokenizer is None:
            return " ".join(str(i) for i in ids)
        return self.tokenizer.decode(ids)

    def _params(self, cfg: InferenceConfig, stop: Sequence[int]):
        from .sampling.params import SamplingParams
        s = cfg.sampling
        return SamplingParams(greedy=(SamplingMode(s.mode) == SamplingMode.GREEDY), temperature=s.temperature,
                              top_p=s.top_p, seed=s.seed, max_new_tokens=cfg.max_new_tokens,
                              stop_token_ids=tuple(stop))

    def _encode(self, prompt: Prompt):
        if isinstance(prompt, str):
            from .tokenizer import chatml
            tok = self.tokenizer
            if tok is None:
                raise RuntimeError("MiniInfer: this model folder has no tokenizer.json; pass token ids")
            if tok.has_chat_tokens:
                ids = tok.encode(chatml(prompt))
                stop = [tok.im_end_id] + ([tok.eos_token_id] if tok.eos_token_id >= 0 else [])
            else:
                ids = tok.encode(prompt)
                stop = [tok.eos_token_id] if tok.eos_token_id >= 0 else []
            return ids, stop
        stop = []
        if self.tokenizer is not None and self.tokenizer.eos_token_id >= 0:
            stop = [self.tokenizer.eos_token_id]
        return [int(t) for t in prompt], stop

    # -- core API ------------------------------------------------------------ #
    def generate(self, prompt: Prompt, config: Optional[InferenceConfig] = None) -> GenerationResult:
        return self.generate_ids([prompt], config)[0]

    def generate_ids(self, prompts: Sequence[Prompt], config: Optional[InferenceConfig] = None
                     ) -> List[GenerationResult]:
        """Many prompts as one continuous batch (request ``i`` uses random stream ``i``)."""
        cfg = config or self.config
        enc = [self._encode(p) for p in prompts]
        t0 = time.perf_counter()
        outs = self.llm.generate([e[0] for e in enc], [self._params(cfg, e[1]) for e in enc])
        wall = time.perf_counter() - t0
        res = []
        for (ids, _), o in zip(enc, outs):
            res.append(GenerationResult(text=self.detokenize(o.token_ids), tokens=list(ids) + o.token_ids,
                                        prompt_tokens=len(ids), generated_tokens=len(o.token_ids),
                                        elapsed_sec=o.seconds, wall_sec=wall, finish_reason=o.finish_reason))
        return res

    def stream(self, prompt: Prompt, config: Optional[InferenceConfig] = None) -> Iterator[str]:
        """Yield the text of each generated token once generation is done (the engine has no
        incremental host loop of its own; the reference streams lines of the binary's output,
        sdk/mini_infer_sdk/backends/local.py:218-254)."""
        r = self.generate(prompt, config)
        for t in r.generated_ids:
            yield self.detokenize([t])

    def __repr__(self):
        return f"MiniInfer(local, model={self.model_name})"
