"""``mini_infer [generate] --model DIR --prompt TEXT ...`` - the reference's command line.

Flags, defaults and the printed contract follow src/core/main.cc:43-106 and
:209-215: ``--model``, ``--prompt``, ``--max-new-tokens`` (100), ``--max-seq-len``
(2048), ``--device`` (0), ``--temperature`` (1.0), ``--top-p`` (0.9), ``--greedy``,
``--paged``, ``--raw``, ``--python``, ``--seed`` (42); the default sampling mode is
top-p, as there; the result is printed between ``--- generated ---`` and
``--- end ---`` and followed by ``[mini-infer] N tokens in X.XXs (Y.YY tok/s)``,
which the reference's SDK parses (sdk/mini_infer_sdk/backends/local.py:170-190).
``--paged`` is accepted and changes nothing (the cache is always paged);
``--spec-draft``/``--gamma`` are refused (speculative decoding is not built);
``serve`` and ``client`` are refused (no server).  Added: ``--prompt-ids`` and
``--prompt-ids-file`` for models without a tokenizer, ``--dtype``, ``--page-size``,
``--num-pages``, ``--max-tokens-per-step``, ``--prefill-chunk``, ``--json``, and
the subcommand ``random-weights`` that writes a model folder from a
``config.json`` and a seed.
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List, Optional


def _parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="mini_infer", description="mini-infer for B200: offline generation")
    p.add_argument("--model", required=True, help="folder with config.json, safetensors and optionally tokenizer.json")
    p.add_argument("--prompt", default="你好，请介绍一下你自己。")
    p.add_argument("--prompt-ids", default=None, help="comma-separated token ids instead of --prompt")
    p.add_argument("--prompt-ids-file", default=None, help="file of whitespace/comma-separated token ids")
    p.add_argument("--max-new-tokens", type=int, default=100)
    p.add_argument("--max-seq-len", type=int, default=2048)
    p.add_argument("--device", type=int, default=0)
    p.add_argument("--temperature", type=float, default=1.0)
    p.add_argument("--top-p", type=float, default=0.9)
    p.add_argument("--greedy", action="store_true")
    p.add_argument("--paged", action="store_true", help="accepted for compatibility; the cache is always paged")
    p.add_argument("--raw", action="store_true", help="do not wrap the prompt in ChatML")
    p.add_argument("--python", default="python3", help="accepted for compatibility; the tokenizer runs in-process")
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--spec-draft", default=None, help=argparse.SUPPRESS)
    p.add_argument("--gamma", type=int, default=4, help=argparse.SUPPRESS)
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    p.add_argument("--page-size", type=int, default=None)
    p.add_argument("--num-pages", type=int, default=None)
    p.add_argument("--max-tokens-per-step", type=int, default=2048)
    p.add_argument("--prefill-chunk", type=int, default=0)
    p.add_argument("--json", action="store_true", help="also print one JSON line with ids and timings")
    return p


def _parse_ids(text: str) -> List[int]:
    return [int(x) for x in text.replace(",", " ").split()]


def run_generate(argv: List[str]) -> int:
    args = _parser().parse_args(argv)
    if args.spec_draft:
        print("mini_infer: speculative decoding (--spec-draft) is not part of this engine", file=sys.stderr)
        return 2
    from .engine.llm import LLM
    from .sampling.params import SamplingParams
    from .tokenizer import chatml, load_tokenizer

    print(f"[mini-infer] loading model from {args.model} ...")
    tok = load_tokenizer(args.model)
    stop_ids: List[int] = []
    if args.prompt_ids or args.prompt_ids_file:
        text = args.prompt_ids if args.prompt_ids else open(args.prompt_ids_file).read()
        prompt_ids = _parse_ids(text)
        if tok is not None and tok.eos_token_id >= 0:
            stop_ids.append(tok.eos_token_id)
    else:
        if tok is None:
            print("mini_infer: the model folder has no tokenizer.json; give --prompt-ids", file=sys.stderr)
            return 2
        # src/core/main.cc:131-143
        if not args.raw and tok.has_chat_tokens:
            prompt_ids = tok.encode(chatml(args.prompt))
            stop_ids = [tok.im_end_id] + ([tok.eos_token_id] if tok.eos_token_id >= 0 else [])
        else:
            prompt_ids = tok.encode(args.prompt)
            stop_ids = ([tok.eos_token_id] if tok.eos_token_id >= 0 else []) + \
                       ([tok.im_end_id] if tok.has_chat_tokens else [])
    if len(prompt_ids) > args.max_seq_len:
        # src/core/main.cc:145-149
        print(f"[mini-infer] Error: prompt length ({len(prompt_ids)}) exceeds max_seq_len ({args.max_seq_len})",
              file=sys.stderr)
        return 1
    llm = LLM(args.model, dtype=args.dtype, device=f"cuda:{args.device}", max_seq_len=args.max_seq_len,
              page_size=args.page_size, num_pages=args.num_pages, max_running=1,
              max_tokens_per_step=args.max_tokens_per_step, prefill_chunk=args.prefill_chunk)
    sp = SamplingParams(greedy=args.greedy, temperature=args.temperature, top_p=args.top_p, seed=args.seed,
                        max_new_tokens=args.max_new_tokens, stop_token_ids=tuple(stop_ids))
    # The text appears between the two marker lines as it is generated (a reader of the pipe can show it
    # line by line, as the reference's SDK does): each token's text is printed when its step has ended.
    t0 = time.perf_counter()
    print("\n--- generated ---", flush=True)
    gen: List[int] = []
    shown = ""
    for _, token in llm.generate_iter([prompt_ids], sp):
        gen.append(token)
        text = tok.decode(gen) if tok is not None else " ".join(str(t) for t in gen)
        if tok is not None and text.endswith("\ufffd"):
            continue                                   # half of a character: wait for the rest
        sys.stdout.write(text[len(shown):])
        sys.stdout.flush()
        shown = text
    out = llm.last_outputs[0]
    secs = time.perf_counter() - t0
    text = tok.decode(gen) if tok is not None else " ".join(str(t) for t in gen)
    print(f"{text[len(shown):]}\n--- end ---")
    print(f"[mini-infer] {len(gen)} tokens in {secs:.2f}s ({len(gen) / max(secs, 1e-9):.2f} tok/s)")
    if args.json:
        print(json.dumps({"prompt_tokens": len(prompt_ids), "token_ids": gen, "finish_reason": out.finish_reason,
                          "seconds": secs, "ttft": out.ttft}))
    return 0


def run_random_weights(argv: List[str]) -> int:
    p = argparse.ArgumentParser(prog="mini_infer random-weights",
                                description="write a model folder (config.json, model.safetensors) with seeded "
                                            "random weights")
    p.add_argument("--config", required=True, help="a config.json")
    p.add_argument("--seed", type=int, required=True)
    p.add_argument("--out", required=True)
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "float16"])
    args = p.parse_args(argv)
    import torch
    from .config.model_config import read_config_json
    from .weights.random_init import write_model_folder
    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}[args.dtype]
    write_model_folder(args.out, read_config_json(args.config), args.seed, dt)
    print(f"[mini-infer] wrote {args.out}")
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] in ("serve", "client"):
        print(f"mini_infer: '{argv[0]}' is not part of this engine (offline generation only)", file=sys.stderr)
        return 2
    if argv and argv[0] == "random-weights":
        return run_random_weights(argv[1:])
    if argv and argv[0] == "generate":     # src/core/main.cc:222-231: "generate" or the legacy bare form
        argv = argv[1:]
    return run_generate(argv)


if __name__ == "__main__":
    sys.exit(main())
