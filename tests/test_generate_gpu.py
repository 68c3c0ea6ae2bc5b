"""Generation through the entry points: greedy and sampled tokens equal the plain model's,
alone, batched, cut into portions, and under preemption; the command line keeps its contract."""

import json
import os
import subprocess
import sys

import pytest
import torch

import plain_model as pm
import tiny

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name in ("A", "B", "C"):
        f = str(tmp_path_factory.mktemp(f"gen_{name}"))
        tiny.make_folder(f, tiny.CONFIGS[name], seed=31, dtype=torch.float32)
        out[name] = (f, tiny.CONFIGS[name], tiny.read_weights(f))
    return out


def clear_prompt(cfg, w, n, seed, new_tokens, temperature=0.0, top_p=1.0, stream=0, sseed=42, margin=1e-4):
    """A prompt whose plain generation meets no near-tie in routing or in the arg-max."""
    for s in range(seed, seed + 400):
        toks = tiny.pick_tokens(cfg, w, n, s)
        gen = pm.generate(cfg, w, toks, new_tokens, temperature, top_p, sseed, stream)
        full = toks + gen
        if tiny.min_routing_gap(cfg, w, full) < 1e-4:
            continue
        logits = pm.forward(cfg, w, full)[len(toks) - 1:-1]
        top2 = torch.topk(logits, 2, dim=-1).values
        if temperature == 0.0 and float((top2[:, 0] - top2[:, 1]).min()) < margin:
            continue
        return toks, gen
    raise RuntimeError("no clear prompt found")


def test_greedy_three_prompts_like_the_benchmark_workload(folders):
    """Configuration A: prompts of 5, 11 and 17 random tokens, 8 greedy tokens each."""
    from mini_infer_b200.engine.llm import LLM
    from mini_infer_b200.sampling import SamplingParams
    folder, cfg, w = folders["A"]
    cases = [clear_prompt(cfg, w, n, 100 * n, 8) for n in (5, 11, 17)]
    llm = LLM(folder, dtype="float32", max_seq_len=128, max_running=4, max_tokens_per_step=64)
    outs = llm.generate([c[0] for c in cases], SamplingParams(greedy=True, max_new_tokens=8))
    for o, (toks, gen) in zip(outs, cases):
        assert o.token_ids == gen and o.finish_reason == "length"
    # one at a time gives the same
    for toks, gen in cases:
        assert llm.generate([toks], SamplingParams(greedy=True, max_new_tokens=8))[0].token_ids == gen
    assert llm.runner.cache.used_pages() == [0]


def test_temperature_four_requests_in_portions_like_the_benchmark_workload(folders):
    """Configuration B: prompts of 1, 9, 23 and 40 tokens, prefilled in portions of 8 beside
    decoding requests, 12 tokens at temperature 0.8 under a fixed seed."""
    from mini_infer_b200.engine.llm import LLM
    from mini_infer_b200.sampling import SamplingParams
    folder, cfg, w = folders["B"]
    cases = [clear_prompt(cfg, w, n, 77 * n, 12, temperature=0.8, top_p=1.0, stream=i, sseed=1234)
             for i, n in enumerate((1, 9, 23, 40))]
    llm = LLM(folder, dtype="float32", max_seq_len=256, max_running=4, max_tokens_per_step=16, prefill_chunk=8)
    sp = SamplingParams(greedy=False, temperature=0.8, top_p=1.0, seed=1234, max_new_tokens=12)
    outs = llm.generate([c[0] for c in cases], sp)
    for o, (toks, gen) in zip(outs, cases):
        assert o.token_ids == gen
    steps = llm.last_history
    assert any(s.prefill_tokens and s.decode_tokens for s in steps)          # portions beside decodes
    assert all(s.num_tokens <= 16 for s in steps)


def test_top_p_and_stop_token(folders):
    from mini_infer_b200.engine.llm import LLM
    from mini_infer_b200.sampling import SamplingParams
    folder, cfg, w = folders["C"]
    toks, gen = clear_prompt(cfg, w, 30, 5, 10, temperature=1.2, top_p=0.7, stream=0, sseed=9)
    llm = LLM(folder, dtype="float32", max_seq_len=128, max_running=2)
    o = llm.generate([toks], SamplingParams(greedy=False, temperature=1.2, top_p=0.7, seed=9, max_new_tokens=10))[0]
    assert o.token_ids == gen
    stop = gen[4]
    first = gen.index(stop)
    o = llm.generate([toks], SamplingParams(greedy=False, temperature=1.2, top_p=0.7, seed=9, max_new_tokens=10,
                                            stop_token_ids=(stop,)))[0]
    assert o.token_ids == gen[:first + 1] and o.finish_reason == "stop"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_launched_ahead_change_nothing(folders, dtype):
    """The executor launches the next decode step before the host has the tokens of this one; with
    that switched off the tokens are the same, bit for bit, for greedy and sampled requests, and a
    stop token drops the step launched beside it."""
    from mini_infer_b200.engine.llm import LLM
    from mini_infer_b200.sampling import SamplingParams
    folder, cfg, w = folders["A"]
    prompts = [tiny.pick_tokens(cfg, w, n, 3 * n) for n in (6, 19, 11)]
    params = [SamplingParams(greedy=True, max_new_tokens=14),
              SamplingParams(greedy=False, temperature=0.9, top_p=0.8, seed=5, max_new_tokens=9),
              SamplingParams(greedy=False, temperature=1.3, top_p=1.0, seed=6, max_new_tokens=17)]
    llm = LLM(folder, dtype=dtype, max_seq_len=128, max_running=4, page_size=4)
    ahead = llm.generate(prompts, params)
    assert llm.executor.steps_adopted >= 10
    llm.executor.lookahead_capable = False
    adopted = llm.executor.steps_adopted
    plain = llm.generate(prompts, params)
    assert llm.executor.steps_adopted == adopted
    assert [o.token_ids for o in ahead] == [o.token_ids for o in plain]
    llm.executor.lookahead_capable = True
    stop = ahead[0].token_ids[5]
    first = ahead[0].token_ids.index(stop)
    params[0] = SamplingParams(greedy=True, max_new_tokens=14, stop_token_ids=(stop,))
    dropped = llm.executor.steps_dropped
    outs = llm.generate(prompts, params)
    assert outs[0].token_ids == ahead[0].token_ids[:first + 1] and outs[0].finish_reason == "stop"
    assert [o.token_ids for o in outs[1:]] == [o.token_ids for o in ahead[1:]]
    assert llm.executor.steps_dropped > dropped
    assert llm.runner.cache.used_pages() == [0]
    llm.runner.cache.check_invariants()


@pytest.mark.parametrize("name,dtype", [("D", "float32"), ("D", "bfloat16"), ("E", "bfloat16")])
def test_generation_as_the_product_runs_it_against_the_plain_model(tmp_path, name, dtype):
    """``LLM.generate`` with everything on that serving uses (prompts in portions beside decoding requests,
    decode steps as CUDA-graph replays, the next step launched before this one's tokens are on the host):
    the logits every token was sampled from are kept and compared with the plain model's, under the
    engine's routing where a near-tie allows either choice."""
    from engine_harness import GenerationObserver, compare_generation
    from mini_infer_b200.engine.llm import LLM
    from mini_infer_b200.sampling import SamplingParams
    cfg = tiny.CONFIGS[name]
    folder = tiny.make_folder(str(tmp_path), cfg, seed=53, dtype=torch.bfloat16)
    w = tiny.read_weights(folder)
    prompts = [tiny.pick_tokens(cfg, w, n, 7 * n) for n in (40, 75, 130, 9)]
    new_tokens = 24
    llm = LLM(folder, dtype=dtype, max_seq_len=512, max_running=4, max_tokens_per_step=96, prefill_chunk=64)
    obs = GenerationObserver(llm.runner, [len(p) for p in prompts])
    llm.executor.observer = obs
    outs = llm.generate(prompts, SamplingParams(greedy=True, max_new_tokens=new_tokens))
    assert llm.executor.steps_adopted > 0 and llm.runner.graph_replays > 0
    assert any(s.prefill_tokens and s.decode_tokens for s in llm.last_history)
    assert all(len(o.token_ids) == new_tokens for o in outs)
    compare_generation(obs, llm._calls, prompts, outs, cfg, w, dtype, 2e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generation_of_eleven_requests_on_batches_filled_up_to_a_captured_size(tmp_path, dtype, monkeypatch):
    """Eleven requests with different numbers of new tokens: the decode steps of 11, 10 and 9 requests are
    replays of the pass captured for 12 (filled up with rows of no request), launched ahead of the host's
    tokens as in serving; every row of logits a token was sampled from against the plain model."""
    from engine_harness import GenerationObserver, compare_generation
    from mini_infer_b200.engine.llm import LLM
    from mini_infer_b200.sampling import SamplingParams
    # a coarse ladder of captured sizes for the test: every size to 8, multiples of 4 above
    from mini_infer_b200.parts.tuning import Tuning
    monkeypatch.setattr(Tuning, "decode_graph_batch", lambda self, n: n if n <= 8 else -(-n // 4) * 4)
    cfg = tiny.CONFIGS["D"]
    folder = tiny.make_folder(str(tmp_path), cfg, seed=59, dtype=torch.bfloat16)
    w = tiny.read_weights(folder)
    prompts = [tiny.pick_tokens(cfg, w, n, 5 * n) for n in (12, 31, 7, 22, 40, 9, 17, 28, 5, 35, 14)]
    news = [10, 14, 10, 12, 14, 10, 14, 12, 14, 14, 14]
    llm = LLM(folder, dtype=dtype, max_seq_len=128, max_running=12, max_tokens_per_step=256)
    obs = GenerationObserver(llm.runner, [len(p) for p in prompts])
    llm.executor.observer = obs
    outs = llm.generate(prompts, [SamplingParams(greedy=True, max_new_tokens=n) for n in news])
    assert [len(o.token_ids) for o in outs] == news
    assert llm.executor.steps_adopted > 0 and 12 in {key[0] for key in llm.runner._graphs}
    assert not {9, 10, 11} & {key[0] for key in llm.runner._graphs}
    compare_generation(obs, llm._calls, prompts, outs, cfg, w, dtype, 2e-5 if dtype == "float32" else 2e-2)
    assert llm.runner.cache.used_pages() == [0]
    llm.runner.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_prompt_portions_are_graph_replays_too(tmp_path, dtype, monkeypatch):
    """With chunked prefill every full portion of a long prompt has the same shape; its pass is captured once
    and replayed with whatever context lies before it.  A prompt of 5 full portions and a rest, then decoding:
    the logits of every sampled token against the plain model."""
    from engine_harness import GenerationObserver, compare_generation
    from mini_infer_b200.engine.llm import LLM
    from mini_infer_b200.parts.tuning import TUNING
    from mini_infer_b200.sampling import SamplingParams
    monkeypatch.setattr(TUNING, "prefill_chunk_graph_min_tokens", 64)
    cfg = tiny.CONFIGS["E"]
    folder = tiny.make_folder(str(tmp_path), cfg, seed=59, dtype=torch.bfloat16)
    w = tiny.read_weights(folder)
    prompts = [tiny.pick_tokens(cfg, w, 5 * 64 + 37, 11)]
    llm = LLM(folder, dtype=dtype, max_seq_len=512, max_running=2, max_tokens_per_step=64, prefill_chunk=64)
    assert llm.runner.graph_chunk_tokens == 64
    obs = GenerationObserver(llm.runner, [len(p) for p in prompts])
    llm.executor.observer = obs
    outs = llm.generate(prompts, SamplingParams(greedy=True, max_new_tokens=6))
    chunk_keys = [k for k in llm.runner._graphs if k[3] is not None]
    assert chunk_keys == [(1, 512, chunk_keys[0][2], (64, False))]           # one captured pass, replayed 5 times
    assert llm.runner.graph_replays >= 5 + 4
    compare_generation(obs, llm._calls, prompts, outs, cfg, w, dtype, 2e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("dtype,new_tokens,margin", [("float32", 20, 1e-4), ("bfloat16", 6, 0.02)])
def test_preemption_recomputes_the_same_tokens(folders, dtype, new_tokens, margin):
    """So few pages that decoding requests are preempted and recomputed; tokens must not change.
    In bfloat16 the prompts are chosen with wide arg-max margins, so that rounding cannot flip a token."""
    from mini_infer_b200.engine.llm import LLM
    from mini_infer_b200.sampling import SamplingParams
    folder, cfg, w = folders["A"]
    cases = [clear_prompt(cfg, w, n, 40 * n, new_tokens, margin=margin) for n in (14, 9, 12)]
    sp = SamplingParams(greedy=True, max_new_tokens=new_tokens)
    roomy = LLM(folder, dtype=dtype, max_seq_len=64, max_running=4, page_size=4, num_pages=64)
    assert [o.token_ids for o in roomy.generate([c[0] for c in cases], sp)] == [c[1] for c in cases]
    pages = sum(-(-(len(c[0]) + new_tokens) // 4) for c in cases)
    tight = LLM(folder, dtype=dtype, max_seq_len=64, max_running=4, page_size=4, num_pages=pages - 4)
    outs = tight.generate([c[0] for c in cases], sp)
    assert sum(o.preemptions for o in outs) >= 1
    assert [o.token_ids for o in outs] == [c[1] for c in cases]
    assert tight.runner.cache.used_pages() == [0]


def test_sdk_entry_point(folders):
    from mini_infer_sdk import InferenceConfig, MiniInfer, SamplingConfig, SamplingMode
    folder, cfg, w = folders["A"]
    toks, gen = clear_prompt(cfg, w, 12, 900, 6)
    eng = MiniInfer(model_path=folder, config=InferenceConfig(max_new_tokens=6, max_seq_len=64, dtype="float32",
                                                              max_running=2))
    r = eng.generate(toks)
    assert r.generated_ids == gen and r.prompt_tokens == 12 and r.generated_tokens == 6
    assert r.tokens == toks + gen and r.finish_reason == "length" and r.tokens_per_sec > 0
    assert r.text == " ".join(str(t) for t in gen)                          # no tokenizer in a random-weight folder
    rs = eng.generate_ids([toks, toks[:5]], InferenceConfig(max_new_tokens=3, sampling=SamplingConfig(
        mode=SamplingMode.TOP_P, temperature=0.9, top_p=0.8, seed=3)))
    assert rs[0].generated_ids == pm.generate(cfg, w, toks, 3, 0.9, 0.8, 3, 0)
    assert rs[1].generated_ids == pm.generate(cfg, w, toks[:5], 3, 0.9, 0.8, 3, 1)
    with pytest.raises(NotImplementedError):
        MiniInfer(endpoint="http://localhost:8000")


def test_sdk_streams_tokens_as_the_scheduler_produces_them(folders):
    """``stream`` yields after every scheduler step (the scheduler has run exactly as many decode steps as
    tokens have been yielded), not once generation is over; stopping early ends the request and frees it."""
    from mini_infer_sdk import InferenceConfig, MiniInfer
    folder, cfg, w = folders["A"]
    toks, gen = clear_prompt(cfg, w, 12, 900, 6)
    eng = MiniInfer(model_path=folder, config=InferenceConfig(max_new_tokens=6, max_seq_len=64, dtype="float32",
                                                              max_running=2))
    seen, replays = [], []
    for piece in eng.stream(toks):
        seen.append(int(piece))
        replays.append(eng.llm.runner.graph_replays)
    assert seen == gen
    assert replays == sorted(replays) and replays[0] < replays[-1]      # steps ran between the yields
    it = eng.stream(toks)
    assert int(next(it)) == gen[0]
    it.close()                                                            # the consumer walks away
    assert eng.llm.runner.cache.used_pages() == [0] and eng.llm.last_outputs[0].finish_reason == "cancelled"
    assert eng.generate(toks).generated_ids == gen                        # and the engine is as before


def _folder_with_tokenizer(tmp_path, cfg):
    """A random-weight folder with a word-level ``tokenizer.json`` made for the test: one word per id
    (``t0``, ``t1`` ...), the two ChatML markers as special tokens, whitespace splitting."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    folder = tiny.make_folder(str(tmp_path), cfg, seed=61, dtype=torch.float32)
    V = cfg["vocab_size"]
    vocab = {"<unk>": 0, "<|im_start|>": 1, "<|im_end|>": 2, "user": 3, "assistant": 4, "system": 5}
    for i in range(len(vocab), V):
        vocab[f"t{i}"] = i
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    tok.add_special_tokens(["<|im_start|>", "<|im_end|>"])
    tok.save(os.path.join(folder, "tokenizer.json"))
    return folder, tiny.read_weights(folder)


def test_sdk_text_prompts_chat_and_batch(tmp_path):
    """Text goes through the folder's tokenizer: a single prompt is wrapped as one ChatML turn, a chat sends
    its whole history as one raw prompt each turn and stops at the end-of-turn marker, and a batch is one
    continuous batch whose results equal the single calls'.  Every token against the plain model."""
    from mini_infer_sdk import InferenceConfig, MiniInfer
    from mini_infer_b200.tokenizer import chat_prompt, chatml
    cfg = tiny.CONFIGS["A"]
    folder, w = _folder_with_tokenizer(tmp_path, cfg)
    eng = MiniInfer(model_path=folder, config=InferenceConfig(max_new_tokens=5, max_seq_len=256, dtype="float32",
                                                              max_running=4))
    tok = eng.tokenizer
    assert tok.has_chat_tokens and tok.im_start_id == 1 and tok.im_end_id == 2
    stop = [tok.im_end_id]

    def expect(ids):
        return pm.generate(cfg, w, ids, 5, stop_ids=stop)

    # one text prompt: a single ChatML turn
    ids = tok.encode(chatml("t9 t17 t40"))
    assert ids == [1, 3, 9, 17, 40, 2, 1, 4]
    r = eng.generate("t9 t17 t40")
    assert r.tokens[:r.prompt_tokens] == ids and r.generated_ids == expect(ids)
    assert r.text == tok.decode(r.generated_ids)
    # a conversation: the history grows and every turn sends all of it
    chat = eng.chat(system_prompt="t7 t8")
    first = chat.send("t20 t21 t22")
    msgs = [{"role": "system", "content": "t7 t8"}, {"role": "user", "content": "t20 t21 t22"}]
    ids1 = tok.encode(chat_prompt(msgs, True))
    assert ids1 == [1, 5, 7, 8, 2, 1, 3, 20, 21, 22, 2, 1, 4]
    assert chat.last_result.generated_ids == expect(ids1) and first.role == "assistant"
    assert first.content == tok.decode(expect(ids1))
    pieces = list(chat.stream("t30"))
    msgs += [{"role": "assistant", "content": first.content}, {"role": "user", "content": "t30"}]
    ids2 = tok.encode(chat_prompt(msgs, True))
    assert "".join(pieces) == tok.decode(expect(ids2)) == chat.last_message().content
    assert [m.role for m in chat.history] == ["system", "user", "assistant", "user", "assistant"]
    assert repr(chat) == "ChatSession(turns=2)"
    chat.clear()
    assert chat.history == [] and chat.last_message() is None
    # without the markers the conversation is plain lines
    assert chat_prompt(msgs[:2], False) == "System: t7 t8\nUser: t20 t21 t22\nAssistant: "
    # a batch: one continuous batch, results in the prompts' order; its stream yields as requests end
    prompts = ["t9 t17 t40", [11, 12, 13, 14, 15, 16, 17], "t50 t51"]
    stats = eng.batch().process(prompts)
    singles = [eng.generate(p) for p in prompts]
    assert [b.result.generated_ids for b in stats.results] == [r.generated_ids for r in singles]
    assert [b.index for b in stats.results] == [0, 1, 2] and stats.total_prompts == 3
    assert stats.total_generated_tokens == sum(r.generated_tokens for r in singles) and stats.tokens_per_sec > 0
    streamed = list(eng.batch().stream(prompts))
    assert sorted(b.index for b in streamed) == [0, 1, 2]
    for b in streamed:
        assert b.result.generated_ids == singles[b.index].generated_ids
        assert b.result.finish_reason == singles[b.index].finish_reason
    assert eng.llm.runner.cache.used_pages() == [0]
    # a folder without a tokenizer cannot chat
    plain_folder = tiny.make_folder(str(tmp_path / "no_tok"), cfg, seed=61, dtype=torch.float32)
    bare = MiniInfer(model_path=plain_folder, config=InferenceConfig(max_new_tokens=2, max_seq_len=64, dtype="float32",
                                                                     max_running=1))
    with pytest.raises(RuntimeError, match="tokenizer"):
        bare.chat().send("hello")
    assert bare.chat().history == []


def test_sdk_subprocess_backend(folders):
    """``binary=``: every call runs the command-line program and reads its printed contract, as the
    reference's local backend does."""
    from mini_infer_sdk import InferenceConfig, MiniInfer
    folder, cfg, w = folders["A"]
    toks, gen = clear_prompt(cfg, w, 12, 900, 6)
    eng = MiniInfer(model_path=folder, binary=os.path.join(ROOT, "bin", "mini_infer"),
                    config=InferenceConfig(max_new_tokens=6, max_seq_len=64, dtype="float32"))
    assert eng.llm is None and "subprocess" in repr(eng)
    r = eng.generate(toks)
    assert r.generated_ids == gen and r.prompt_tokens == 12 and r.finish_reason == "length"
    assert r.text == " ".join(str(t) for t in gen) and r.tokens_per_sec > 0 and r.wall_sec >= r.elapsed_sec
    assert [int(t) for t in "".join(eng.stream(toks)).split()] == gen


def test_command_line_contract(folders):
    folder, cfg, w = folders["A"]
    toks, gen = clear_prompt(cfg, w, 9, 333, 5)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "mini_infer"), "generate", "--model", folder, "--prompt-ids",
           ",".join(map(str, toks)), "--max-new-tokens", "5", "--greedy", "--paged", "--dtype", "float32",
           "--max-seq-len", "64", "--json"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = p.stdout.splitlines()
    i = lines.index("--- generated ---")
    assert lines[i + 1] == " ".join(map(str, gen)) and lines[i + 2] == "--- end ---"
    assert lines[i + 3].startswith("[mini-infer] 5 tokens in ") and lines[i + 3].endswith("tok/s)")
    assert json.loads(lines[i + 4])["token_ids"] == gen
    bad = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "mini_infer"), "serve", "--model", folder],
                         capture_output=True, text=True)
    assert bad.returncode == 2 and "not part of this engine" in bad.stderr


def test_command_line_with_text_and_the_chat_command(tmp_path):
    """``--prompt TEXT`` wraps the text as one ChatML turn unless ``--raw``, and stops at the end-of-turn
    marker; ``python -m mini_infer_sdk chat`` reads a line and answers it."""
    cfg = tiny.CONFIGS["A"]
    folder, w = _folder_with_tokenizer(tmp_path, cfg)
    base = [sys.executable, os.path.join(ROOT, "bin", "mini_infer"), "generate", "--model", folder, "--prompt",
            "t9 t17 t40", "--max-new-tokens", "5", "--greedy", "--dtype", "float32", "--max-seq-len", "64", "--json"]
    wrapped = [1, 3, 9, 17, 40, 2, 1, 4]
    for extra, ids in (([], wrapped), (["--raw"], [9, 17, 40])):
        p = subprocess.run(base + extra, capture_output=True, text=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        lines = p.stdout.splitlines()
        got = json.loads(lines[lines.index("--- end ---") + 2])["token_ids"]
        assert got == pm.generate(cfg, w, ids, 5, stop_ids=[2]), extra
    env = dict(os.environ, PYTHONPATH=ROOT)
    chat = subprocess.run([sys.executable, "-m", "mini_infer_sdk", "chat", "--model", folder, "--greedy",
                           "--max-tokens", "4", "--dtype", "float32", "--system", "t7"],
                          input="t20 t21\nexit\n", capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert chat.returncode == 0, chat.stderr[-2000:]
    ids = [1, 5, 7, 2, 1, 3, 20, 21, 2, 1, 4]
    words = " ".join(f"t{t}" for t in pm.generate(cfg, w, ids, 4, stop_ids=[2]) if t > 5)
    assert f"assistant> {words}" in chat.stdout


def test_warm_up_captures_the_decode_passes_ahead(folders):
    """``LLM.warm_up`` captures one pass per captured batch size; generation afterwards replays them, captures
    nothing more in the same context bucket, and gives the tokens it gives without a warm-up."""
    from mini_infer_b200.engine.llm import LLM
    from mini_infer_b200.sampling import SamplingParams
    folder, cfg, w = folders["A"]
    cases = [clear_prompt(cfg, w, n, 100 * n, 6) for n in (5, 11, 17)]
    sp = SamplingParams(greedy=True, max_new_tokens=6)
    llm = LLM(folder, dtype="float32", max_seq_len=128, max_running=20, max_tokens_per_step=64)
    captured = llm.warm_up()
    assert captured == 16 + 2 == len(llm.runner._graphs)                   # 1..16, 18, 20
    assert llm.runner.cache.used_pages() == [0] and llm.warm_up() == 0
    llm.runner.cache.check_invariants()
    outs = llm.generate([c[0] for c in cases], sp)
    assert [o.token_ids for o in outs] == [c[1] for c in cases]
    assert len(llm.runner._graphs) == captured and llm.runner.graph_replays > captured
    small = LLM(folder, dtype="float32", max_seq_len=128, max_running=4, max_tokens_per_step=64, num_pages=3)
    assert small.warm_up() == 0 and small.runner.cache.used_pages() == [0]     # too few pages: nothing happens
    assert small.warm_up([1, 2]) == 2
