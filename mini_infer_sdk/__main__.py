"""``python -m mini_infer_sdk generate --model DIR --prompt TEXT`` (sdk/mini_infer_sdk/__main__.py:80-119).

Flags as there: ``--model``, ``--prompt``/``--p``, ``--max-tokens`` (128), ``--temperature``,
``--top-p``, ``--seed``, ``--greedy``, ``--python``; added ``--prompt-ids`` and ``--dtype``.
``chat`` and ``serve`` need the server and are refused; ``--endpoint`` likewise.
"""

import argparse
import sys

from . import InferenceConfig, MiniInfer, SamplingConfig, SamplingMode


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
    for name in ("chat", "serve"):
        sub.add_parser(name, help="needs the HTTP server: not part of this engine")
    args = p.parse_args(argv)
    if args.command != "generate":
        raise SystemExit(f"mini_infer_sdk: '{args.command}' needs the server, which is not part of this engine")
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
