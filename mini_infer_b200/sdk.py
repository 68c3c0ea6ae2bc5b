"""Python entry point in the manner of the reference's ``mini_infer_sdk`` (offline mode).

Same names and meanings: ``MiniInfer(model_path=...)`` with ``generate``,
``stream``, ``tokenize``, ``detokenize`` (sdk/mini_infer_sdk/engine.py:30-118);
``InferenceConfig`` and ``SamplingConfig`` with the same fields and defaults
(sdk/mini_infer_sdk/config.py:8-30); ``GenerationResult`` with the same
attributes (sdk/mini_infer_sdk/result.py:6-52).

Two backends.  By default the engine lives in the calling process and the model
stays loaded between calls.  With ``binary=`` (the path of this repository's
``bin/mini_infer``) every call starts that program and reads its output, which is
how the reference's local backend works (sdk/mini_infer_sdk/backends/local.py:204-254):
the result is parsed from the lines between ``--- generated ---`` and ``--- end ---``
and the ``[mini-infer] N tokens in Xs`` line, and ``stream`` yields the program's
output as it arrives.  ``stream`` of the in-process backend yields each token's
text as soon as the scheduler's step that sampled it has ended.

``chat(system_prompt)`` gives a conversation that keeps its history and sends the whole of it as one raw
prompt each turn, and ``batch()`` a helper that runs many prompts and reports totals
(sdk/mini_infer_sdk/engine.py:100-112, chat.py, batch.py).  Here the batch is ONE continuous batch of the
scheduler, not a loop of single calls, and its ``stream`` yields every result when its request ends.

Not part of this engine: ``endpoint=`` (the HTTP backend) and ``draft_path=`` (speculative decoding).

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


@dataclass
class GenerationResult:
    """What a call returns; attribute names as the reference's result object has them
    (sdk/mini_infer_sdk/result.py:6-52).  ``tokens`` holds the prompt's ids followed by the generated ones;
    ``elapsed_sec`` is the engine's time for the request and ``wall_sec`` the caller's wait."""

    text: str
    tokens: List[int] = field(default_factory=list)
    prompt_tokens: int = 0
    generated_tokens: int = -1
    elapsed_sec: float = 0.0
    accept_rate: Optional[float] = None
    tokens_per_sec: float = -1.0
    wall_sec: float = -1.0
    finish_reason: Optional[str] = None

    def __post_init__(self):
        self.tokens = list(self.tokens or [])
        if self.generated_tokens < 0:
            self.generated_tokens = max(0, len(self.tokens) - self.prompt_tokens)
        if self.wall_sec < 0:
            self.wall_sec = self.elapsed_sec
        if self.tokens_per_sec < 0:
            self.tokens_per_sec = self.generated_tokens / self.elapsed_sec if self.elapsed_sec > 0 else 0.0

    @property
    def generated_ids(self) -> List[int]:
        return self.tokens[self.prompt_tokens:]

    def __repr__(self):
        return f"GenerationResult(generated={self.generated_tokens}, tps={self.tokens_per_sec:.1f})"


Prompt = Union[str, Sequence[int]]


@dataclass
class ChatMessage:
    role: str
    content: str


class ChatSession:
    """A conversation with its history (sdk/mini_infer_sdk/chat.py:17-72): ``send`` returns the assistant's
    message, ``stream`` yields its text as it is produced; both append the turn to ``history``.  Every turn
    sends the whole history as one raw prompt (``tokenizer.chat_prompt``), so it needs a tokenizer."""

    def __init__(self, engine: "MiniInfer", system_prompt: Optional[str] = None,
                 config: Optional[InferenceConfig] = None):
        self._engine = engine
        self._config = config or engine.config
        self.history: List[ChatMessage] = []
        if system_prompt:
            self.history.append(ChatMessage("system", system_prompt))

    def _prompt_ids(self):
        return self._engine._encode_conversation([{"role": m.role, "content": m.content} for m in self.history])

    def send(self, message: str) -> ChatMessage:
        self.history.append(ChatMessage("user", message))
        try:
            ids, stop = self._prompt_ids()
            result = self._engine._generate_encoded([(ids, stop)], self._config)[0]
        except BaseException:
            self.history.pop()
            raise
        self.last_result = result
        self.history.append(ChatMessage("assistant", result.text))
        return self.history[-1]

    def stream(self, message: str) -> Iterator[str]:
        self.history.append(ChatMessage("user", message))
        pieces: List[str] = []
        try:
            ids, stop = self._prompt_ids()
            for piece in self._engine._stream_encoded(ids, stop, self._config):
                pieces.append(piece)
                yield piece
        finally:
            # a consumer that walks away keeps what it has seen as the assistant's turn
            self.history.append(ChatMessage("assistant", "".join(pieces)))

    def clear(self) -> None:
        self.history.clear()

    def last_message(self) -> Optional[ChatMessage]:
        return self.history[-1] if self.history else None

    def __repr__(self):
        return f"ChatSession(turns={sum(1 for m in self.history if m.role == 'user')})"


@dataclass
class BatchResult:
    prompt: Prompt
    result: GenerationResult
    index: int


@dataclass
class BatchStats:
    total_prompts: int
    total_generated_tokens: int
    total_elapsed: float
    tokens_per_sec: float
    results: List[BatchResult] = field(default_factory=list)


class BatchInfer:
    """Many prompts at once (sdk/mini_infer_sdk/batch.py:33-136 loops over single calls, in threads if asked).
    With the engine in this process the prompts are one continuous batch of the scheduler, so ``workers`` has
    nothing to add there; with the subprocess backend it is the number of programs run side by side."""

    def __init__(self, engine: "MiniInfer", config: Optional[InferenceConfig] = None):
        self._engine = engine
        self._config = config or engine.config

    def process(self, prompts: Sequence[Prompt], workers: int = 1) -> BatchStats:
        t0 = time.perf_counter()
        eng = self._engine
        if eng.llm is None and workers > 1:
            from concurrent.futures import ThreadPoolExecutor
            with ThreadPoolExecutor(max_workers=workers) as pool:
                results = list(pool.map(lambda p: eng.generate(p, self._config), prompts))
        else:
            results = eng.generate_ids(list(prompts), self._config)
        elapsed = time.perf_counter() - t0
        total = sum(r.generated_tokens for r in results)
        return BatchStats(len(results), total, elapsed, total / elapsed if elapsed > 0 else 0.0,
                          [BatchResult(p, r, i) for i, (p, r) in enumerate(zip(prompts, results))])

    def stream(self, prompts: Sequence[Prompt]) -> Iterator[BatchResult]:
        """Yield every prompt's result as soon as its request has ended (in that order, not the prompts')."""
        eng, cfg = self._engine, self._config
        if eng.llm is None:
            for i, p in enumerate(prompts):
                yield BatchResult(p, eng.generate(p, cfg), i)
            return
        enc = [eng._encode(p) for p in prompts]
        t0 = time.perf_counter()
        tokens = eng.llm.generate_iter([e[0] for e in enc], [eng._params(cfg, e[1]) for e in enc])
        gen: List[List[int]] = [[] for _ in enc]
        try:
            for i, token in tokens:
                gen[i].append(token)
                stopped = token in enc[i][1]
                if stopped or len(gen[i]) >= cfg.max_new_tokens:
                    ids = enc[i][0]
                    yield BatchResult(prompts[i], GenerationResult(
                        text=eng.detokenize(gen[i]), tokens=list(ids) + gen[i], prompt_tokens=len(ids),
                        generated_tokens=len(gen[i]), elapsed_sec=time.perf_counter() - t0,
                        finish_reason="stop" if stopped else "length"), i)
        finally:
            tokens.close()


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
        self.binary = binary
        self.llm = None
        from .tokenizer import load_tokenizer
        self.tokenizer = load_tokenizer(model_path)
        if binary is None:
            from .engine.llm import LLM
            c = self.config
            self.llm = LLM(model_path, dtype=c.dtype, device=f"cuda:{c.device}", max_seq_len=c.max_seq_len,
                           page_size=c.page_size, num_pages=c.num_pages, max_running=c.max_running,
                           max_tokens_per_step=c.max_tokens_per_step, prefill_chunk=c.prefill_chunk)

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

    def _encode_conversation(self, messages):
        """The ids of a whole conversation up to the assistant's next turn, and the ids that end that turn."""
        from .tokenizer import chat_prompt
        tok = self.tokenizer
        if tok is None:
            raise RuntimeError("MiniInfer: a chat needs text, and this model folder has no tokenizer.json")
        ids = tok.encode(chat_prompt(messages, tok.has_chat_tokens))
        stop = [tok.im_end_id] if tok.has_chat_tokens else []
        if tok.eos_token_id >= 0:
            stop.append(tok.eos_token_id)
        return ids, stop

    # -- core API ------------------------------------------------------------ #
    def generate(self, prompt: Prompt, config: Optional[InferenceConfig] = None) -> GenerationResult:
        return self.generate_ids([prompt], config)[0]

    def warm_up(self) -> int:
        """Capture the decode passes of every batch size ahead of the first request (in-process backend only;
        see ``LLM.warm_up``).  Returns how many were captured."""
        return self.llm.warm_up() if self.llm is not None else 0

    def chat(self, system_prompt: Optional[str] = None, config: Optional[InferenceConfig] = None) -> ChatSession:
        return ChatSession(self, system_prompt=system_prompt, config=config)

    def batch(self, config: Optional[InferenceConfig] = None) -> BatchInfer:
        return BatchInfer(self, config=config or self.config)

    def generate_ids(self, prompts: Sequence[Prompt], config: Optional[InferenceConfig] = None
                     ) -> List[GenerationResult]:
        """Many prompts as one continuous batch (request ``i`` uses random stream ``i``); with the
        subprocess backend one program run per prompt."""
        return self._generate_encoded([self._encode(p) for p in prompts], config or self.config)

    def _generate_encoded(self, enc, cfg: InferenceConfig) -> List[GenerationResult]:
        if self.llm is None:
            return [self._run_binary(ids, stop, cfg) for ids, stop in enc]
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
        """Yield the text of the generated tokens as they are produced: from the in-process engine after
        every scheduler step, from the subprocess backend as the program prints it."""
        ids, stop = self._encode(prompt)
        yield from self._stream_encoded(ids, stop, config or self.config)

    def _stream_encoded(self, ids, stop, cfg: InferenceConfig) -> Iterator[str]:
        if self.llm is None:
            yield from self._stream_binary(ids, cfg)
            return
        gen: List[int] = []
        shown = ""
        tokens = self.llm.generate_iter([ids], self._params(cfg, stop))
        try:
            for _, token in tokens:
                gen.append(token)
                if self.tokenizer is None:
                    yield str(token)
                    continue
                text = self.tokenizer.decode(gen)
                if text.endswith("\ufffd"):
                    continue                           # half of a character: wait for the rest
                yield text[len(shown):]
                shown = text
        finally:
            tokens.close()                             # a consumer that walks away ends the request at once

    # -- subprocess backend --------------------------------------------------- #
    def _command(self, ids: Sequence[int], cfg: InferenceConfig) -> List[str]:
        import sys
        s = cfg.sampling
        cmd = [sys.executable, self.binary, "generate", "--model", self.model_path, "--prompt-ids",
               ",".join(str(i) for i in ids), "--max-new-tokens", str(cfg.max_new_tokens), "--max-seq-len",
               str(cfg.max_seq_len), "--device", str(cfg.device), "--temperature", str(s.temperature), "--top-p",
               str(s.top_p), "--seed", str(s.seed), "--dtype", cfg.dtype, "--json"]
        if SamplingMode(s.mode) == SamplingMode.GREEDY:
            cmd.append("--greedy")
        if cfg.paged:
            cmd.append("--paged")
        return cmd

    def _run_binary(self, ids: Sequence[int], stop: Sequence[int], cfg: InferenceConfig) -> GenerationResult:
        """One run of the command-line program; the result is read from what it prints (the markers, the
        ``[mini-infer] N tokens in Xs (Y tok/s)`` line and the JSON line with the token ids)."""
        import json
        import re
        import subprocess
        t0 = time.perf_counter()
        p = subprocess.run(self._command(ids, cfg), capture_output=True, text=True,
                           timeout=cfg.max_new_tokens * 2 + 600)
        wall = time.perf_counter() - t0
        if p.returncode != 0:
            raise RuntimeError(f"mini_infer failed (rc={p.returncode}):\n{p.stderr[-2000:]}")
        lines = p.stdout.splitlines()
        try:
            a, b = lines.index("--- generated ---"), lines.index("--- end ---")
        except ValueError:
            raise RuntimeError("mini_infer printed no generated text:\n" + p.stdout[-2000:]) from None
        text = "\n".join(lines[a + 1:b]).strip()
        secs, tps, gen, reason = wall, None, None, None
        for line in lines[b + 1:]:
            m = re.match(r"\[mini-infer\] (\d+) tokens in ([\d.]+)s \(([\d.]+) tok/s\)", line)
            if m:
                secs, tps = float(m.group(2)), float(m.group(3))
            elif line.startswith("{"):
                j = json.loads(line)
                gen, reason = [int(t) for t in j["token_ids"]], j.get("finish_reason")
        if gen is None:
            gen = self.tokenize(text) if self.tokenizer is not None else [int(t) for t in text.split()]
        return GenerationResult(text=text, tokens=list(ids) + gen, prompt_tokens=len(ids), generated_tokens=len(gen),
                                elapsed_sec=secs, tokens_per_sec=tps if tps is not None else -1.0, wall_sec=wall,
                                finish_reason=reason)

    def _stream_binary(self, ids: Sequence[int], cfg: InferenceConfig) -> Iterator[str]:
        import subprocess
        proc = subprocess.Popen(self._command(ids, cfg), stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
                                bufsize=1)
        inside = False
        try:
            for line in proc.stdout:
                if line.strip() == "--- generated ---":
                    inside = True
                elif line.strip() == "--- end ---":
                    break
                elif inside:
                    yield line
        finally:
            proc.terminate()
            proc.wait()

    def __repr__(self):
        kind = "local" if self.llm is not None else "local, subprocess"
        return f"MiniInfer({kind}, model={self.model_name})"
