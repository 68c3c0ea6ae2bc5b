#!/usr/bin/env python3
"""Engine against the plain model at real layer sizes (run by hand on a GPU; pytest does not collect it).

    python tests/full_size_check.py --config a27b --dtype float32 [--layers 24]
    python tests/full_size_check.py --config 57b  --dtype bfloat16 --layers 4

Workload of the first form (the benchmark description's fifth configuration): random weights of
Qwen1.5-MoE-A2.7B layer sizes, eight requests with random prompts of 1 to 1,500 tokens, prefilled in
portions of 512 beside decoding requests through the scheduler, then 64 greedy tokens each.  The
engine's logits at every sampled position are kept; afterwards the plain model (tests/plain_model.py,
on the same GPU, sharing nothing but the weight values) runs every request's prompt plus generated
tokens once, and each kept row is compared with the plain row for the same position (attention is
causal, so the plain row does not depend on later tokens).  Prints the largest error relative to the
largest logit, and how many of the engine's greedy tokens equal the plain model's arg-max.

Expert routing is discontinuous: where two router probabilities differ by less than the engine's
rounding, the engine may choose the other expert, and the logits then differ visibly although no
kernel is wrong.  The script therefore records the experts the engine chose for every token and
layer and prints a second figure, the error against the plain model made to follow that choice,
together with the number of tokens whose choice differed and the largest amount by which a chosen
expert's plain-model probability fell short of the K-th largest.

The plain model holds a second copy of the weights, so both fit one 180 GB GPU only up to about
70 GB of weights: use ``--layers`` to cut the 57B configuration down for the comparison.
"""

import argparse
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

CONFIGS = {
    "a27b": {
        "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
        "vocab_size": 151936, "hidden_size": 2048, "intermediate_size": 5632, "num_hidden_layers": 24,
        "num_attention_heads": 16, "num_key_value_heads": 16, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
        "max_position_embeddings": 8192, "tie_word_embeddings": False, "hidden_act": "silu",
        "num_experts": 60, "num_experts_per_tok": 4, "moe_intermediate_size": 1408,
        "shared_expert_intermediate_size": 5632, "norm_topk_prob": False, "decoder_sparse_step": 1,
        "mlp_only_layers": [], "use_sliding_window": False},
    "57b": {
        "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
        "vocab_size": 151936, "hidden_size": 3584, "intermediate_size": 18944, "num_hidden_layers": 28,
        "num_attention_heads": 28, "num_key_value_heads": 4, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
        "max_position_embeddings": 8192, "tie_word_embeddings": False, "hidden_act": "silu",
        "num_experts": 64, "num_experts_per_tok": 8, "moe_intermediate_size": 2560,
        "shared_expert_intermediate_size": 20480, "norm_topk_prob": False, "decoder_sparse_step": 1,
        "mlp_only_layers": [], "use_sliding_window": False},
}


class DictSource:
    """A tensor source over tensors that already sit on the device."""

    def __init__(self, tensors):
        self.t = tensors

    def names(self):
        return list(self.t)

    def shape(self, n):
        return tuple(self.t[n].shape)

    def dtype(self, n):
        return self.t[n].dtype

    def read(self, n):
        return self.t[n]

    def describe(self):
        return "tensors in memory"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="a27b", choices=sorted(CONFIGS))
    ap.add_argument("--dtype", default="float32", choices=["float32", "bfloat16"])
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--requests", type=int, default=8)
    ap.add_argument("--max-prompt", type=int, default=1500)
    ap.add_argument("--new-tokens", type=int, default=64)
    ap.add_argument("--chunk", type=int, default=512)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args()

    import torch
    import plain_model
    from mini_infer_b200.config import build_model_spec
    from mini_infer_b200.engine.llm import LLM
    from mini_infer_b200.engine.loading import _runtime
    from mini_infer_b200.engine.model import Model
    from mini_infer_b200.engine.step import StepEntry
    from mini_infer_b200.sampling import SamplingParams
    from mini_infer_b200.weights import RandomSource

    cfg = dict(CONFIGS[args.config])
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    rt = _runtime(args.dtype, "cuda:0")
    model = Model(build_model_spec(cfg))
    t0 = time.time()
    # the checkpoint's values: bfloat16 numbers, as a real checkpoint would hold them
    src = RandomSource(model.tensor_decls(), args.seed, torch.bfloat16, "cuda:0")
    plain_dtype = torch.float32
    weights = {n: src.read(n).to(plain_dtype) for n in src.names()}          # the plain model's copy
    model.load(DictSource(weights), rt)
    torch.cuda.synchronize()
    print(f"weights ready in {time.time() - t0:.0f}s; device memory in use "
          f"{torch.cuda.memory_allocated() / 2**30:.1f} GiB", flush=True)

    g = torch.Generator().manual_seed(args.seed)
    lens = [1] + torch.randint(2, args.max_prompt + 1, (args.requests - 1,), generator=g).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    ctx = args.max_prompt + args.new_tokens + 16
    llm = LLM(model, runtime=rt, max_seq_len=ctx, max_running=args.requests, max_tokens_per_step=args.chunk,
              prefill_chunk=args.chunk, num_pages=args.requests * (ctx // 16 + 1))
    # keep the logits the sampler saw, by wrapping the executor's run
    kept = {}
    routing = {}
    sparse = {i: l.feed_forward for i, l in enumerate(model.layers) if hasattr(l.feed_forward, "keep_routing")}
    for part in sparse.values():
        part.keep_routing = True          # (this also keeps decode steps out of CUDA graphs)
    inner_step = llm.runner.step

    def recording_step(entries):
        res = inner_step(entries)
        t = 0
        for e in entries:
            start = llm.runner.num_tokens(e.rid) - len(e.tokens)
            for li, part in sparse.items():
                idx = part.last_routing[0][t:t + len(e.tokens)]
                routing.setdefault(e.rid, {}).setdefault(li, {})[start] = idx.clone()
            t += len(e.tokens)
        if res.logits is not None:
            rows = res.logits.float()
            for r, (rid, place) in enumerate(res.index):
                e = next(e for e in entries if e.rid == rid)
                pos = llm.runner.num_tokens(rid) - len(e.tokens) + place
                kept.setdefault(rid, {})[pos] = rows[r].clone()
        return res
    llm.runner.step = recording_step
    t0 = time.time()
    outs = llm.generate(prompts, SamplingParams(greedy=True, max_new_tokens=args.new_tokens))
    torch.cuda.synchronize()
    steps = llm.last_history
    print(f"engine: {len(steps)} steps in {time.time() - t0:.1f}s; "
          f"{sum(1 for s in steps if s.prefill_tokens and s.decode_tokens)} of them mixed portions with decodes",
          flush=True)
    llm.runner.step = inner_step

    worst, worst_f, agree, total, differ, short = 0.0, 0.0, 0, 0, 0, 0.0
    K = cfg["num_experts_per_tok"]
    rids = sorted(kept, key=lambda r: r[1])
    for rid, prompt, out in zip(rids, prompts, outs):
        full = prompt + out.token_ids
        n_fed = len(full) - 1                                   # the last generated token was never fed
        rec = {}
        ref = plain_model.forward(cfg, weights, full[:n_fed], dtype=plain_dtype, by_expert=True, record=rec)
        forced = {li: torch.cat([per[s] for s in sorted(per)]).long() for li, per in routing[rid].items()}
        rec_f = {}
        ref_f = plain_model.forward(cfg, weights, full[:n_fed], dtype=plain_dtype, by_expert=True,
                                    forced_routing=forced, record=rec_f)
        for li, eng in forced.items():
            differ += int((torch.sort(eng, 1).values != torch.sort(rec["routing"][li][0], 1).values).any(1).sum())
            probs = rec_f["routing"][li][1]
            kth = torch.sort(probs, dim=1, descending=True).values[:, K - 1]
            short = max(short, float((kth[:, None] - probs.gather(1, eng)).max()))
        scale = float(ref.abs().max())
        for pos, row in sorted(kept[rid].items()):
            worst = max(worst, float((row - ref[pos]).abs().max()) / scale)
            worst_f = max(worst_f, float((row - ref_f[pos]).abs().max()) / scale)
            agree += int(int(ref[pos].argmax()) == full[pos + 1])
            total += 1
        print(f"request with {len(prompt):5d} prompt tokens: {len(kept[rid])} positions compared, largest error so far "
              f"{worst:.3e} ({worst_f:.3e} with the engine's routing) of the largest logit", flush=True)
    print(f"RESULT config={args.config} dtype={args.dtype} layers={cfg['num_hidden_layers']} positions={total} "
          f"max_rel_err={worst:.3e} max_rel_err_with_engine_routing={worst_f:.3e} greedy_agree={agree}/{total} "
          f"token_layers_routed_differently={differ} largest_probability_shortfall={short:.2e}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
