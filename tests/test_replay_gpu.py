"""The engine against the plain model under every way of cutting the work.

For each tiny configuration, in float32 and in bfloat16: each request alone and
whole; most of it in one step and the last 32 tokens one by one; portions of
changing size down to two tokens; and mixed batches of up to four live requests
with a page pool so small that pages are used again.  Every logit row the
engine returns is compared with the plain model's row for the same position.
"""

import os

import pytest
import torch

import plain_model
import tiny
import traces
from engine_harness import compare, make_runner, run_and_compare, run_trace

pytestmark = pytest.mark.gpu

# Largest allowed error, as a fraction of the request's largest reference logit.
TOL = {"float32": 2e-5, "bfloat16": 2e-2}
LENGTHS = {"A": [5, 41, 70, 17, 33, 64, 49, 9], "B": [1, 9, 23, 40, 77, 48, 65, 16],
           "C": [3, 90, 25, 57, 48, 31, 72, 12], "D": [37, 300, 129, 64], "E": [150, 41, 333, 96, 200]}


_CASES = {}


def _case(name, tmp_path_factory):
    """The model folder, weights and requests of one tiny configuration (made once per test session)."""
    if name not in _CASES:
        cfg = tiny.CONFIGS[name]
        folder = str(tmp_path_factory.mktemp(f"model_{name}"))
        tiny.make_folder(folder, cfg, seed=11 + ord(name), dtype=torch.bfloat16)
        weights = tiny.read_weights(folder)
        reqs = {f"r{i}": tiny.pick_tokens(cfg, weights, n, seed=1000 * (i + 1)) for i, n in enumerate(LENGTHS[name])}
        _CASES[name] = {"name": name, "cfg": cfg, "folder": folder, "reqs": reqs, "weights": weights}
    return _CASES[name]


@pytest.fixture(scope="module", params=["A", "B", "C", "D", "E"])
def case(request, tmp_path_factory):
    return _case(request.param, tmp_path_factory)


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def dtype(request):
    return request.param


def _runner(case, dtype, num_pages=64, page_size=16, cuda_graphs=True):
    return make_runner(case["folder"], dtype, page_size=page_size, num_pages=num_pages, max_requests=4,
                       max_tokens=512, max_context=512, cuda_graphs=cuda_graphs)


class KernelCalls:
    """Counts the calls of some kernels' Python faces while a trace runs (the parts look them up in
    ``ops.functional`` at every call, so replacing the attribute is seen)."""

    NAMES = ("grouped_gemm_tc", "prefill_attention_tc", "decode_attention", "grouped_gemm_skinny_pairs")

    def __init__(self, monkeypatch):
        from mini_infer_b200.ops import functional as F
        self.count = {n: 0 for n in self.NAMES}
        for n in self.NAMES:
            monkeypatch.setattr(F, n, self._wrap(n, getattr(F, n)))

    def _wrap(self, name, fn):
        def counted(*a, **k):
            self.count[name] += 1
            return fn(*a, **k)
        return counted


def _check(case, dtype, runner, steps):
    return run_and_compare(runner, steps, case["cfg"], case["weights"], case["reqs"], dtype, TOL[dtype])


def _tensor_core_case(case, dtype):
    return case["name"] == "E" and dtype == "bfloat16"


def test_whole(case, dtype, monkeypatch):
    calls = KernelCalls(monkeypatch)
    _, got = _check(case, dtype, _runner(case, dtype), traces.whole(case["reqs"]))
    assert len(got) == sum(len(t) for t in case["reqs"].values())
    if _tensor_core_case(case, dtype):
        assert calls.count["grouped_gemm_tc"] > 0 and calls.count["prefill_attention_tc"] > 0


@pytest.mark.parametrize("graphs", [True, False], ids=["graphs", "eager"])
def test_tail_decoded_one_by_one(case, dtype, graphs, monkeypatch):
    """With CUDA graphs (the way generation decodes) every one-token step is a replay of a captured
    pass; the recorded routing is read from the tensors the captured pass owns."""
    calls = KernelCalls(monkeypatch)
    runner = _runner(case, dtype, cuda_graphs=graphs)
    steps = traces.tail_decoded(case["reqs"], 32)
    _check(case, dtype, runner, steps)
    one_token = sum(1 for st in steps if all(len(t) == 1 for _, t, _ in st["entries"]))
    assert one_token >= sum(min(32, len(t) - 1) for t in case["reqs"].values())
    assert runner.graph_replays == (one_token if graphs else 0)
    if case["name"] in ("D", "E") and dtype == "bfloat16":
        assert calls.count["decode_attention"] > 0          # head size 64: the split-KV kernel


def test_portions_of_changing_size(case, dtype, monkeypatch):
    calls = KernelCalls(monkeypatch)
    sizes = (7, 2, 13, 3, 2, 5, 17, 2, 31, 4) if case["name"] != "E" else (40, 2, 75, 3, 18, 61, 2, 129)
    _check(case, dtype, _runner(case, dtype), traces.portions(case["reqs"], sizes))
    if _tensor_core_case(case, dtype):
        assert calls.count["grouped_gemm_tc"] > 0 and calls.count["prefill_attention_tc"] > 0


def _mixed(case, dtype, page_size, monkeypatch):
    calls = KernelCalls(monkeypatch)
    # the tensor-core configuration gets portions large enough for the tcgen05 grouped product
    steps = traces.mixed(case["reqs"], max_live=4, seed=3, max_portion=60 if case["name"] == "E" else 11)
    peak = traces.live_token_peak(steps, 64)
    total = sum(-(-len(t) // 64) * 64 for t in case["reqs"].values())
    assert peak < total, "the trace must not fit the pool without reuse"
    runner = _runner(case, dtype, num_pages=peak // page_size, page_size=page_size)
    _, got = _check(case, dtype, runner, steps)
    assert len(got) == sum(len(t) for t in case["reqs"].values())
    assert runner.cache.used_pages() == [0] * len(runner.cache.pools)
    assert all(p.high_water <= p.num_pages for p in runner.cache.pools)
    all_decode = sum(1 for st in steps if all(len(t) == 1 for _, t, _ in st["entries"]))
    assert runner.graph_replays == all_decode          # the all-decode steps of the trace were replays
    if _tensor_core_case(case, dtype):
        assert calls.count["grouped_gemm_tc"] > 0
        # the tcgen05 attention takes pages of 8 to 64 tokens; pages of 4 go to the mma.sync kernel
        assert (calls.count["prefill_attention_tc"] > 0) == (page_size >= 8)


@pytest.mark.parametrize("page_size", [16, 4])
def test_mixed_with_pages_used_again(case, dtype, page_size, monkeypatch):
    _mixed(case, dtype, page_size, monkeypatch)


def test_mixed_with_pages_of_64_tokens(dtype, tmp_path_factory, monkeypatch):
    """The largest page the tcgen05 attention takes (one TMA box per page fills a whole key tile), with the
    configuration whose sizes the tensor-core kernels take."""
    _mixed(_case("E", tmp_path_factory), dtype, 64, monkeypatch)


def test_cuttings_agree_with_each_other(case):
    """In float32 the logits at a position are the same BITS however the work was cut into steps, whatever
    else was in the batch and whichever pages were used: every kernel of that path adds in an order that
    depends on the token's own request only."""
    a = run_trace(_runner(case, "float32"), traces.whole(case["reqs"]))
    b = run_trace(_runner(case, "float32"), traces.portions(case["reqs"]))
    c = run_trace(_runner(case, "float32"), traces.mixed(case["reqs"], seed=5))
    d = run_trace(_runner(case, "float32", cuda_graphs=False), traces.tail_decoded(case["reqs"], 32))
    for key in a:
        assert torch.equal(a[key], b[key]), ("portions", key, float((a[key] - b[key]).abs().max()))
        assert torch.equal(a[key], c[key]), ("mixed", key, float((a[key] - c[key]).abs().max()))
        assert torch.equal(a[key], d[key]), ("tail decoded", key, float((a[key] - d[key]).abs().max()))
