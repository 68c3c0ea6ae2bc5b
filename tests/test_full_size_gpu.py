"""The engine against the plain model at real layer sizes.

Two layers with the layer sizes of Qwen1.5-MoE-A2.7B (hidden 2048, 16 heads of 128, 60 experts of 1408
with top-4 routing, a shared expert of 5632, vocabulary 151936), random weights: here the bfloat16 path
runs the kernels that serving runs (tcgen05 grouped products and prefill attention, the split-KV decode
attention, the decode-sized expert products, CUDA-graph replays) inside the engine, under every cutting of
the work, and the float32 path shows what bfloat16 rounding would hide.  The plain model runs on the same
GPU from a float32 copy of the same values and shares nothing else with the engine.

Expert routing is discontinuous, so the comparison follows the engine's choice of experts wherever the
plain model's own probabilities say that the choice was a near-tie (``engine_harness.reference_logits``
fails otherwise); the number of (token, layer) pairs routed differently is bounded as well.
"""

import pytest
import torch

import tiny
import traces
from engine_harness import (DictSource, GenerationObserver, compare_generation, run_and_compare)

pytestmark = pytest.mark.gpu

A27B_TWO_LAYERS = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "vocab_size": 151936, "hidden_size": 2048, "intermediate_size": 5632, "num_hidden_layers": 2,
    "num_attention_heads": 16, "num_key_value_heads": 16, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "max_position_embeddings": 8192, "tie_word_embeddings": False, "hidden_act": "silu",
    "num_experts": 60, "num_experts_per_tok": 4, "moe_intermediate_size": 1408,
    "shared_expert_intermediate_size": 5632, "norm_topk_prob": False, "decoder_sparse_step": 1,
    "mlp_only_layers": [], "use_sliding_window": False, "sliding_window": 32768, "max_window_layers": 2,
}
TOL = {"float32": 2e-5, "bfloat16": 2e-2}
# the largest share of (token, layer) pairs that may be routed differently from the plain model (each one is
# checked to be a near-tie): rounding of the float32 path flips next to none, bfloat16 a few per cent
FLIPPED = {"float32": 0.002, "bfloat16": 0.12}
LENGTHS = {"a": 700, "b": 1, "c": 130, "d": 333}


@pytest.fixture(scope="module")
def checkpoint():
    """The checkpoint's values (bfloat16 numbers, as a real checkpoint holds them) as float32 on the GPU."""
    from mini_infer_b200.config import build_model_spec
    from mini_infer_b200.engine.model import declared_tensors
    from mini_infer_b200.weights import RandomSource
    cfg = dict(A27B_TWO_LAYERS)
    src = RandomSource(declared_tensors(build_model_spec(cfg)), 17, torch.bfloat16, "cuda:0")
    weights = {n: src.read(n).float() for n in src.names()}
    g = torch.Generator().manual_seed(17)
    reqs = {rid: torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for rid, n in LENGTHS.items()}
    yield {"cfg": cfg, "weights": weights, "reqs": reqs}
    weights.clear()
    torch.cuda.empty_cache()


_ENGINES = {}


def _engine(dtype, checkpoint):
    if dtype not in _ENGINES:
        from mini_infer_b200.config import build_model_spec
        from mini_infer_b200.engine.loading import _runtime
        from mini_infer_b200.engine.model import Model
        rt = _runtime(dtype, "cuda:0")
        model = Model(build_model_spec(checkpoint["cfg"]))
        model.load(DictSource(checkpoint["weights"]), rt)
        _ENGINES[dtype] = {"model": model, "rt": rt, "dtype": dtype}
    return _ENGINES[dtype]


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def engine(request, checkpoint):
    return _engine(request.param, checkpoint)


@pytest.fixture(scope="module", autouse=True)
def _free_engines():
    yield
    _ENGINES.clear()
    torch.cuda.empty_cache()


def _runner(engine, num_pages, page_size=16, max_tokens=1024):
    from mini_infer_b200.engine.step import ModelRunner
    return ModelRunner(engine["model"], engine["rt"], page_size=page_size, num_pages=num_pages, max_requests=4,
                       max_tokens_per_step=max_tokens, max_context=1024)


def _check(engine, checkpoint, runner, steps):
    stats = {}
    dtype = engine["dtype"]
    worst, got = run_and_compare(runner, steps, checkpoint["cfg"], checkpoint["weights"], checkpoint["reqs"], dtype,
                                 TOL[dtype], by_expert=True, stats=stats)
    assert len(got) == sum(LENGTHS.values())
    assert stats["flipped"] <= FLIPPED[dtype] * stats["pairs"], stats
    print(f"\n[full size, {dtype}] largest error {worst:.2e} of the largest logit; "
          f"{stats['flipped']} of {stats['pairs']} (token, layer) pairs routed differently")
    return worst


def test_whole(engine, checkpoint):
    _check(engine, checkpoint, _runner(engine, 96), traces.whole(checkpoint["reqs"]))


def test_tail_decoded_one_by_one(engine, checkpoint):
    runner = _runner(engine, 96)
    _check(engine, checkpoint, runner, traces.tail_decoded(checkpoint["reqs"], 32))
    assert runner.graph_replays >= 32 * 3


def test_portions_of_changing_size(engine, checkpoint):
    _check(engine, checkpoint, _runner(engine, 96),
           traces.portions(checkpoint["reqs"], (7, 2, 129, 3, 64, 250, 2, 33)))


def test_mixed_with_pages_used_again(engine, checkpoint):
    steps = traces.mixed(checkpoint["reqs"], max_live=3, seed=2, decode_tail=20, max_portion=160)
    peak = traces.live_token_peak(steps, 64)
    assert peak < sum(-(-n // 64) * 64 for n in LENGTHS.values())
    runner = _runner(engine, peak // 16)
    _check(engine, checkpoint, runner, steps)
    assert runner.cache.used_pages() == [0]
    assert runner.graph_replays == sum(1 for st in steps if all(len(t) == 1 for _, t, _ in st["entries"]))


def test_float32_cuttings_agree_bit_for_bit(checkpoint):
    """At real sizes too, the float32 path gives the same bits whole, in portions and mixed with others."""
    engine = _engine("float32", checkpoint)
    from engine_harness import run_trace
    reqs = checkpoint["reqs"]
    a = run_trace(_runner(engine, 96), traces.whole(reqs))
    b = run_trace(_runner(engine, 96), traces.portions(reqs, (7, 2, 129, 3, 64, 250, 2, 33)))
    c = run_trace(_runner(engine, 96), traces.mixed(reqs, max_live=3, seed=2, decode_tail=20, max_portion=160))
    for key in a:
        assert torch.equal(a[key], b[key]) and torch.equal(a[key], c[key]), key


def test_scheduler_workload(engine, checkpoint):
    """Eight requests with prompts of 1 to 1,500 tokens, prefilled in portions of 512 beside decoding
    requests, 64 greedy tokens each, through ``LLM.generate`` as serving runs it; every row of logits that
    a token was sampled from is compared."""
    from mini_infer_b200.engine.llm import LLM
    from mini_infer_b200.sampling import SamplingParams
    cfg, dtype = checkpoint["cfg"], engine["dtype"]
    g = torch.Generator().manual_seed(5)
    lens = [1, 1500] + torch.randint(2, 1500, (6,), generator=g).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    new_tokens, ctx = 64, 1500 + 64 + 16
    llm = LLM(engine["model"], runtime=engine["rt"], max_seq_len=ctx, max_running=8, max_tokens_per_step=512,
              prefill_chunk=512, num_pages=8 * (ctx // 16 + 1))
    obs = GenerationObserver(llm.runner, [len(p) for p in prompts])
    llm.executor.observer = obs
    try:
        outs = llm.generate(prompts, SamplingParams(greedy=True, max_new_tokens=new_tokens))
    finally:
        obs.close()
    assert all(len(o.token_ids) == new_tokens for o in outs)
    assert any(s.prefill_tokens and s.decode_tokens for s in llm.last_history)
    assert llm.runner.graph_replays > 0 and llm.executor.steps_adopted > 0
    stats = {}
    worst = compare_generation(obs, llm._calls, prompts, outs, cfg, checkpoint["weights"], dtype, TOL[dtype],
                               by_expert=True, stats=stats)
    assert stats["flipped"] <= FLIPPED[dtype] * stats["pairs"], stats
    print(f"\n[full size, {dtype}, scheduler workload] largest error {worst:.2e} of the largest logit over "
          f"{8 * new_tokens} sampled rows; {stats['flipped']} of {stats['pairs']} (token, layer) pairs routed "
          f"differently")
