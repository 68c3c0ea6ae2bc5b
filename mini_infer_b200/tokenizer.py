"""Optional text <-> token ids through the ``tokenizers`` package.

The reference's C++ ``Tokenizer`` shells out to a Python helper for every call
(src/core/tokenizer.cpp:34-129, scripts/tokenize_helper.py:20-75); this engine is
hosted in Python and loads ``tokenizer.json`` directly.  A model folder without
``tokenizer.json`` (every random-weight folder) simply has no tokenizer: prompts
are then given, and results printed, as token ids.
"""

from __future__ import annotations

import os
from typing import List, Optional


class Tokenizer:
    def __init__(self, path: str):
        try:
            from tokenizers import Tokenizer as _Tok
        except ImportError as e:  # pragma: no cover
            raise RuntimeError("the 'tokenizers' package is needed to read tokenizer.json") from e
        self._tok = _Tok.from_file(path)
        # special ids, probed as scripts/tokenize_helper.py:20-31 does
        self.eos_token_id = self._id("eos_token")
        self.bos_token_id = self._id("bos_token")
        self.im_start_id = self._id("<|im_start|>")
        self.im_end_id = self._id("<|im_end|>")

    def _id(self, s: str) -> int:
        v = self._tok.token_to_id(s)
        return -1 if v is None else int(v)

    def encode(self, text: str) -> List[int]:
        return list(self._tok.encode(text).ids)

    def decode(self, ids: List[int]) -> str:
        return self._tok.decode([max(0, int(i)) for i in ids])

    @property
    def has_chat_tokens(self) -> bool:
        return self.im_start_id >= 0 and self.im_end_id >= 0


def load_tokenizer(model_dir: str) -> Optional[Tokenizer]:
    path = os.path.join(model_dir, "tokenizer.json")
    return Tokenizer(path) if os.path.exists(path) else None


def chatml(prompt: str) -> str:
    """The single-turn wrap of src/core/main.cc:133-135."""
    return "<|im_start|>user\n" + prompt + "<|im_end|>\n<|im_start|>assistant\n"


def chat_prompt(messages, chat_tokens: bool) -> str:
    """A conversation (``[{"role": ..., "content": ...}]``) as one raw prompt that ends where the assistant's
    next turn begins: ChatML turns when the vocabulary has the turn markers, plain ``Role: text`` lines
    otherwise (the two forms of sdk/mini_infer_sdk/backends/local.py:50-69)."""
    if chat_tokens:
        turns = [f"<|im_start|>{m['role']}\n{m['content']}<|im_end|>" for m in messages]
        return "\n".join(turns + ["<|im_start|>assistant\n"])
    names = {"system": "System", "assistant": "Assistant"}
    lines = [f"{names.get(m['role'], 'User')}: {m['content']}" for m in messages]
    return "\n".join(lines + ["Assistant: "])
