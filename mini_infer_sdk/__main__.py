"""``python -m mini_infer_sdk generate --model DIR --prompt TEXT`` (sdk/mini_infer_sdk/__main__.py:80-119).

Flags as there: ``--model``, ``--prompt``/``--p``, ``--max-tokens`` (128), ``--temperature``,
``--top-p``, ``--seed``, ``--greedy``, ``--python``; added ``--prompt-ids`` and ``--dtype``.
``chat`` is the reference's read-a-line, answer-a-line loop over ``MiniInfer.chat`` (``__main__.py:40-55``);
``serve`` needs the HTTP server and is refused; ``--endpoint`` likewise.
"""

import argparse
import sys

from . import InferenceConfig, MiniInfer, SamplingConfig, SamplingMode


def chat_loop(args) -> int:
    if args.endpoint:
        raise SystemExit("mini_infer_sdk: online mode (--endpoint) is not part of this engine")
    if not args.model:
        raise SystemExit("provide --model (offline)")
    mode = SamplingMode.GREEDY if args.greedy else SamplingMode.TOP_P
    cfg = InferenceConfig(max_new_tokens=args.max_tokens, dtype=args.dtype, max_running=1,
                          sampling=SamplingConfig(mode=mode, temperature=args.temperature, top_p=args.top_p,
                                                  seed=args.seed))
    engine = MiniInfer(model_path=args.model, config=cfg)
    chat = engine.chat(system_prompt=args.system)
    print(f"chat with {engine.model_name} ({args.dtype}); an empty line or 'exit' ends it")
    while True:
        try:
            user = input("user> ").strip()
        except (EOFError, KeyboardInterrupt):
            print()
            break
        if not user or user.lower() in ("exit", "quit"):
            break
        print("assistant> ", end="", flush=True)
        for piece in chat.stream(user):
            print(piece, end="", flush=True)
        print()
    return 0


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="mini_infer_sdk", description="mini-infer Python CLI (offline)")
    sub = p.add_subparsers(dest="command", required=True)
    g = sub.add_parser("generate", help="Single-prompt generation")
    g.add_argument("--prompt", "--p", dest="prompt", default=None)
    g.add_argument("--prompt-ids", default=None, help="comma-separated token ids instead of --prompt")
    g.add_argument("--model", required=False)
    g.add_argument("--endpoint", "--remote", dest="endpoint", default=None)
    g.add_argument("--draft", default=None)
    g.add_argument("--python", default="python3")
    g.add_argument("--max-tokens", type=int, default=128)
    g.add_argument("--temperature", type=float, default=1.0)
    g.add_argument("--top-p", type=float, default=0.9)
    g.add_argument("--seed", type=int, default=42)
    g.add_argument("--greedy", action="store_true")
    g.add_argument("--dtype", default="bfloat16")
    c = sub.add_parser("chat", help="Interactive conversation (needs the folder's tokenizer.json)")
    c.add_argument("--model", required=False)
    c.add_argument("--endpoint", "--remote", dest="endpoint", default=None)
    c.add_argument("--system", default=None, help="system prompt")
    c.add_argument("--max-tokens", type=int, default=256)
    c.add_argument("--temperature", type=float, default=1.0)
    c.add_argument("--top-p", type=float, default=0.9)
    c.add_argument("--seed", type=int, default=42)
    c.add_argument("--greedy", action="store_true")
    c.add_argument("--dtype", default="bfloat16")
    sub.add_parser("serve", help="needs the HTTP server: not part of this engine")
    args = p.parse_args(argv)
    if args.command == "serve":
        raise SystemExit("mini_infer_sdk: 'serve' needs the server, which is not part of this engine")
    if args.command == "chat":
        return chat_loop(args)
    if args.endpoint:
        raise SystemExit("mini_infer_sdk: online mode (--endpoint) is not part of this engine")
    if not args.model:
        raise SystemExit("provide --model (offline)")
    if args.prompt is None and args.prompt_ids is None:
        raise SystemExit("provide --prompt or --prompt-ids")
    mode = SamplingMode.GREEDY if args.greedy else SamplingMode.TOP_P
    cfg = InferenceConfig(max_new_tokens=args.max_tokens, dtype=args.dtype, max_running=1,
                          sampling=SamplingConfig(mode=mode, temperature=args.temperature, top_p=args.top_p,
                                                  seed=args.seed))
    engine = MiniInfer(model_path=args.model, config=cfg)
    prompt = args.prompt if args.prompt_ids is None else [int(x) for x in args.prompt_ids.replace(",", " ").split()]
    result = engine.generate(prompt, config=cfg)
    print(result.text)
    print(f"\n[mini-infer] {result.generated_tokens} tokens, {result.tokens_per_sec:.1f} tok/s", file=sys.stderr)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
