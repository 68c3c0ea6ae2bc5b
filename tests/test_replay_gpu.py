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
           "C": [3, 90, 25, 57, 48, 31, 72, 12], "D": [37, 300, 129, 64]}


@pytest.fixture(scope="module", params=["A", "B", "C", "D"])
def case(request, tmp_path_factory):
    name = request.param
    cfg = tiny.CONFIGS[name]
    folder = str(tmp_path_factory.mktemp(f"model_{name}"))
    tiny.make_folder(folder, cfg, seed=11 + ord(name), dtype=torch.bfloat16)
    weights = tiny.read_weights(folder)
    reqs = {f"r{i}": tiny.pick_tokens(cfg, weights, n, seed=1000 * (i + 1)) for i, n in enumerate(LENGTHS[name])}
    return {"name": name, "cfg": cfg, "folder": folder, "reqs": reqs, "weights": weights}


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def dtype(request):
    return request.param


def _runner(case, dtype, num_pages=64, page_size=16):
    return make_runner(case["folder"], dtype, page_size=page_size, num_pages=num_pages, max_requests=4,
                       max_tokens=512, max_context=512)


def _check(case, dtype, runner, steps):
    return run_and_compare(runner, steps, case["cfg"], case["weights"], case["reqs"], dtype, TOL[dtype])


def test_whole(case, dtype):
    _, got = _check(case, dtype, _runner(case, dtype), traces.whole(case["reqs"]))
    assert len(got) == sum(len(t) for t in case["reqs"].values())


def test_tail_decoded_one_by_one(case, dtype):
    _check(case, dtype, _runner(case, dtype), traces.tail_decoded(case["reqs"], 32))


def test_portions_of_changing_size(case, dtype):
    _check(case, dtype, _runner(case, dtype), traces.portions(case["reqs"]))


@pytest.mark.parametrize("page_size", [16, 4])
def test_mixed_with_pages_used_again(case, dtype, page_size):
    steps = traces.mixed(case["reqs"], max_live=4, seed=3)
    peak = traces.live_token_peak(steps, 64)
    total = sum(-(-len(t) // 64) * 64 for t in case["reqs"].values())
    assert peak < total, "the trace must not fit the pool without reuse"
    runner = _runner(case, dtype, num_pages=peak // page_size, page_size=page_size)
    _, got = _check(case, dtype, runner, steps)
    assert len(got) == sum(len(t) for t in case["reqs"].values())
    assert runner.cache.used_pages() == [0] * len(runner.cache.pools)
    assert all(p.high_water <= p.num_pages for p in runner.cache.pools)


def test_cuttings_agree_with_each_other(case):
    """In float32 the four cuttings give the same logits up to rounding, far inside the tolerance."""
    a = run_trace(_runner(case, "float32"), traces.whole(case["reqs"]))
    b = run_trace(_runner(case, "float32"), traces.portions(case["reqs"]))
    c = run_trace(_runner(case, "float32"), traces.mixed(case["reqs"], seed=5))
    for key in a:
        scale = float(a[key].abs().max())
        assert float((a[key] - b[key]).abs().max()) <= 5e-6 * scale, key
        assert float((a[key] - c[key]).abs().max()) <= 5e-6 * scale, key
