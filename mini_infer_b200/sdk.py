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

Not part of this engine: ``endpoint=`` (the HTTP backend), ``draft_path=``
(speculative decoding), and the ``chat`` and ``batch`` helpers, which in the
reference are conveniences over the same two backends
(sdk/mini_infer_sdk/engine.py:100-112, chat.py, batch.py): they belong to the
serving layer that this engine leaves out.

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

    # -- core API ------------------------------------------------------------ #
    def generate(self, prompt: Prompt, config: Optional[InferenceConfig] = None) -> GenerationResult:
        return self.generate_ids([prompt], config)[0]

    def generate_ids(self, prompts: Sequence[Prompt], config: Optional[InferenceConfig] = None
                     ) -> List[GenerationResult]:
        """Many prompts as one continuous batch (request ``i`` uses random stream ``i``); with the
        subprocess backend one program run per prompt."""
        cfg = config or self.config
        enc = [self._encode(p) for p in prompts]
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
        cfg = config or self.config
        ids, stop = self._encode(prompt)
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
