"""Long decoding, the first tokens of a sequence, and a far key that must be found."""

import pytest
import torch

import plain_model as pm
import tiny
import traces
from engine_harness import compare, make_runner, run_and_compare, run_trace

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,dtype", [("D", "float32"), ("D", "bfloat16"), ("C", "bfloat16")])
def test_long_decoding(tmp_path, name, dtype):
    """A short prompt, then hundreds of tokens decoded one by one: crosses many pages and, for D,
    several splits of the decode kernel; for C, windows that slide over freed pages."""
    cfg = tiny.CONFIGS[name]
    folder = tiny.make_folder(str(tmp_path), cfg, seed=23, dtype=torch.bfloat16)
    w = tiny.read_weights(folder)
    n = 700 if name == "D" else 330
    toks = tiny.pick_tokens(cfg, w, n, 4)
    runner = make_runner(folder, dtype, page_size=16, num_pages=48, max_requests=2, max_tokens=64, max_context=768)
    steps = traces.tail_decoded({"x": toks}, tail=n - 3)
    _, got = run_and_compare(runner, steps, cfg, w, {"x": toks}, dtype, 2e-5 if dtype == "float32" else 3e-2)
    assert len(got) == n


@pytest.mark.parametrize("name,dtype,prompt,decoded", [("D", "float32", 1000, 60), ("D", "bfloat16", 990, 1100),
                                                       ("E", "bfloat16", 2030, 40)])
def test_decoding_with_graphs_across_context_buckets(tmp_path, name, dtype, prompt, decoded):
    """Decode steps are replays of passes captured per context bucket (1024, 2048, 4096 ...), each launched
    for the longest context of its bucket: a request that decodes across 1,024 and 2,048 tokens changes graph
    on the way, and every row must still be the plain model's."""
    cfg = tiny.CONFIGS[name]
    folder = tiny.make_folder(str(tmp_path), cfg, seed=41, dtype=torch.bfloat16)
    w = tiny.read_weights(folder)
    n = prompt + decoded
    toks = tiny.pick_tokens(cfg, w, n, 6)
    runner = make_runner(folder, dtype, page_size=16, num_pages=-(-n // 16) + 2, max_requests=2, max_tokens=2048,
                         max_context=2304)
    steps = traces.tail_decoded({"x": toks}, tail=decoded)
    for st in steps[1:]:
        st["entries"] = [(rid, t, want) for rid, t, want in st["entries"]]
    run_and_compare(runner, steps, cfg, w, {"x": toks}, dtype, 2e-5 if dtype == "float32" else 3e-2)
    assert runner.graph_replays == decoded
    buckets = sorted({key[1] for key in runner._graphs})
    assert len(buckets) >= 2, buckets


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(tmp_path, dtype):
    """Positions 0, 1, 2 ... one by one from an empty cache, for every configuration."""
    for name in ("A", "B", "C"):
        cfg = tiny.CONFIGS[name]
        folder = tiny.make_folder(str(tmp_path / name), cfg, seed=29, dtype=torch.bfloat16)
        w = tiny.read_weights(folder)
        toks = tiny.pick_tokens(cfg, w, 6, 8)
        tol = 2e-5 if dtype == "float32" else 2e-2
        runner = make_runner(folder, dtype, page_size=2, num_pages=8, max_requests=1, max_tokens=8, max_context=16)
        run_and_compare(runner, traces.tail_decoded({"x": toks}, tail=5), cfg, w, {"x": toks}, dtype, tol)
        run_and_compare(runner, traces.whole({"y": toks[:1]}), cfg, w, {"y": toks[:1]}, dtype, tol)


def test_window_group_gives_pages_back_while_decoding(tmp_path):
    cfg = tiny.CONFIG_C
    folder = tiny.make_folder(str(tmp_path), cfg, seed=3, dtype=torch.bfloat16)
    runner = make_runner(folder, "float32", page_size=4, num_pages=40, max_requests=1, max_tokens=32, max_context=160)
    w = tiny.read_weights(folder)
    toks = tiny.pick_tokens(cfg, w, 150, 2)
    run_and_compare(runner, traces.portions({"x": toks}, (9, 1, 1, 4, 1, 1, 1, 13)), cfg, w, {"x": toks},
                    "float32", 2e-5)
    win = [i for i, g in enumerate(runner.model.kv_groups) if g.window > 0][0]
    full = 1 - win
    assert runner.cache.pools[win].high_water <= (24 + 13) // 4 + 2          # window 24, portion 13, pages of 4
    assert runner.cache.pools[full].high_water == -(-150 // 4)


@pytest.mark.parametrize("name", ["D", "E"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_batches_filled_up_to_a_captured_size(tmp_path, dtype, name, monkeypatch):
    """Decode steps of 11, 9 and 5 requests: above 8 requests the step is filled up with rows of no request
    to the next captured batch size (12 here), so 11 and 9 requests replay the same pass.  The rows of the
    requests must be the plain model's, the filling rows must write nothing (pages, other requests' keys),
    and in float32 the logits are bit for bit those of the same trace launched eagerly without any filling."""
    # a coarse ladder of captured sizes for the test: every size to 8, multiples of 4 above
    from mini_infer_b200.parts.tuning import Tuning
    monkeypatch.setattr(Tuning, "decode_graph_batch", lambda self, n: n if n <= 8 else -(-n // 4) * 4)
    cfg = tiny.CONFIGS[name]                 # E: a window of 80 keys, a cache group of its own
    folder = tiny.make_folder(str(tmp_path), cfg, seed=47, dtype=torch.bfloat16)
    w = tiny.read_weights(folder)
    g = torch.Generator().manual_seed(9)
    more = 100 if name == "E" else 0         # past the window: pages are given back while the batch decodes
    lens = [n + more for n in (40, 33, 21, 30, 26, 35, 24, 22, 38, 20, 28)]
    tail = {f"r{i}": t for i, t in enumerate([12, 12, 6, 12, 6, 12, 3, 3, 12, 6, 6])}
    reqs = {f"r{i}": torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for i, n in enumerate(lens)}
    steps = traces.decoded_together(reqs, tail)
    sizes = [len(st["entries"]) for st in steps[len(reqs):]]
    assert sizes[0] == 11 and 9 in sizes and sizes[-1] == 5
    kw = dict(page_size=16, num_pages=128, max_requests=12, max_tokens=256, max_context=256)
    runner = make_runner(folder, dtype, **kw)
    _, got = run_and_compare(runner, steps, cfg, w, reqs, dtype, 2e-5 if dtype == "float32" else 3e-2)
    assert runner.graph_replays == len(sizes)
    assert sorted({key[0] for key in runner._graphs}) == [5, 12]
    assert not any(runner.cache.used_pages())
    if dtype == "float32":
        eager = run_trace(make_runner(folder, dtype, cuda_graphs=False, **kw), steps)
        assert set(eager) == set(got)
        for key in got:
            assert torch.equal(got[key], eager[key]), key


@pytest.mark.parametrize("name,page_size", [("D", 16), ("E", 16), ("E", 32), ("D", 4)])
def test_prompt_portions_behind_decoding_requests_take_two_attention_kernels(tmp_path, name, page_size, monkeypatch):
    """Six requests decode while a seventh and an eighth arrive in portions: in such a step the decoding
    requests stand first and are served by the split-KV decode attention, the portions by a prefill kernel
    (tcgen05, or mma.sync where the page size is not one the tcgen05 kernel takes), both over the same
    rows.  Every row against the plain model; in the steps with fewer than four decoding requests the
    prefill kernel serves all."""
    from mini_infer_b200.ops import functional as F
    cfg = tiny.CONFIGS[name]
    folder = tiny.make_folder(str(tmp_path), cfg, seed=67, dtype=torch.bfloat16)
    w = tiny.read_weights(folder)
    g = torch.Generator().manual_seed(11)
    lens = {"a": 150, "b": 41, "c": 97, "d": 64, "e": 33, "f": 120, "late": 170, "later": 75}
    reqs = {rid: torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for rid, n in lens.items()}
    steps, fed = [], {}
    for rid in "abcdef":
        n = lens[rid] - 14
        steps.append({"entries": [(rid, reqs[rid][:n], [n - 1])], "end": []})
        fed[rid] = n
    portions = {"late": [60, 2, 70, 38], "later": [40, 35]}
    fed.update(late=0, later=0)
    for i in range(14):
        entries = [(rid, [reqs[rid][fed[rid]]], [0]) for rid in "abcdef" if not (rid in "ab" and i >= 11)]
        for rid in ("late", "later"):
            if portions[rid] and (rid == "late" or i >= 5):
                k = portions[rid].pop(0)
                entries.append((rid, reqs[rid][fed[rid]:fed[rid] + k], [0, k - 1]))
        for rid, toks, _ in entries:
            fed[rid] += len(toks)
        steps.append({"entries": entries, "end": [rid for rid, _, _ in entries if fed[rid] == lens[rid]]})
    # the two requests that paused: their last three tokens, two requests to a step
    for i in range(3):
        steps.append({"entries": [(rid, [reqs[rid][fed[rid]]], [0]) for rid in "ab"], "end": []})
        for rid in "ab":
            fed[rid] += 1
    steps[-1]["end"] = ["a", "b"]
    assert all(fed[rid] == lens[rid] for rid in lens), fed
    calls = {"decode": 0, "prefill": 0}
    for face, key in (("decode_attention", "decode"), ("prefill_attention_tc", "prefill"), ("prefill_attention", "prefill")):
        def counted(*a, _fn=getattr(F, face), _key=key, **k):
            calls[_key] += 1
            return _fn(*a, **k)
        monkeypatch.setattr(F, face, counted)
    runner = make_runner(folder, "bfloat16", page_size=page_size, num_pages=1100 // page_size, max_requests=8,
                         max_tokens=256, max_context=256, cuda_graphs=False)
    run_and_compare(runner, steps, cfg, w, reqs, "bfloat16", 3e-2)
    layers = cfg["num_hidden_layers"]
    mixed = sum(1 for st in steps if any(len(t) > 1 for _, t, _ in st["entries"]) and
                sum(1 for _, t, _ in st["entries"] if len(t) == 1) >= 4)
    assert mixed == 6
    if F.decode_attention_supported(cfg["hidden_size"] // cfg["num_attention_heads"]):
        decode_only = sum(1 for st in steps if all(len(t) == 1 for _, t, _ in st["entries"]))
        assert calls["decode"] == (mixed + decode_only) * layers
        assert calls["prefill"] == (len(steps) - decode_only) * layers
    assert not any(runner.cache.used_pages())


@pytest.mark.parametrize("name,seed", [("D", 1), ("E", 2)])
def test_random_trace_of_24_live_requests_replayed_and_launched_eagerly(tmp_path, name, seed):
    """Forty requests, up to 24 live at a time, portions beside decoded tokens, requests sitting steps out:
    the decode steps (1 to 24 requests, above 16 filled up to an even size) replayed from captured passes
    give what the same trace gives launched kernel by kernel: bit for bit in float32, and in bfloat16 too
    (the same kernels in the same order); the bfloat16 rows against the plain model as well."""
    cfg = tiny.CONFIGS[name]
    folder = tiny.make_folder(str(tmp_path), cfg, seed=71, dtype=torch.bfloat16)
    w = tiny.read_weights(folder)
    g = torch.Generator().manual_seed(100 + seed)
    lens = torch.randint(20, 150, (40,), generator=g).tolist()
    reqs = {f"q{i}": torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for i, n in enumerate(lens)}
    steps = traces.mixed(reqs, max_live=24, seed=seed, decode_tail=18, max_portion=40)
    sizes = {len(st["entries"]) for st in steps if all(len(t) == 1 for _, t, _ in st["entries"])}
    assert max(sizes) > 16 and any(n % 2 for n in sizes if n > 16)
    kw = dict(page_size=16, num_pages=400, max_requests=24, max_tokens=1024, max_context=256)
    for dtype in ("float32", "bfloat16"):
        replayed = make_runner(folder, dtype, cuda_graphs=True, **kw)
        a = run_trace(replayed, steps)
        b = run_trace(make_runner(folder, dtype, cuda_graphs=False, **kw), steps)
        assert replayed.graph_replays > 0 and not any(key[0] % 2 for key in replayed._graphs if key[0] > 16)
        assert set(a) == set(b) and len(a) == sum(lens)
        for key in a:
            assert torch.equal(a[key], b[key]), (dtype, key)
    run_and_compare(make_runner(folder, "bfloat16", **kw), steps, cfg, w, reqs, "bfloat16", 3e-2)
