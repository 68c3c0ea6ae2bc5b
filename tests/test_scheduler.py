"""The scheduler's decisions with a scripted executor (CPU): admission, token budget,
portions, decode first, finishing, exact max_new_tokens, and what happens when pages run out."""

import pytest

from mini_infer_b200.cache import CacheManager, KVGroupSpec, OutOfPages
from mini_infer_b200.engine.request import Request
from mini_infer_b200.engine.scheduler import Scheduler, SchedulerConfig
from mini_infer_b200.sampling import SamplingParams


class ScriptedExecutor:
    """A real cache manager, a fake model: the next token is a function of the tokens so far,
    so a recomputed request must generate what it generated before."""

    def __init__(self, num_pages=16, page_size=4, slots=4, vocab=50):
        self.cache = CacheManager([KVGroupSpec(1, 8, 0, (0,))], [num_pages], page_size, slots)
        self.vocab = vocab
        self.batches = []
        self.history = {}

    def add_request(self, rid):
        self.cache.add_request(rid)
        self.history[rid] = []

    def release(self, rid):
        self.cache.release(rid)
        del self.history[rid]

    def run(self, entries, sample_for):
        self.batches.append([(e.rid, len(e.tokens), list(e.want)) for e in entries])
        for e in entries:
            start = self.cache.reserve(e.rid, len(e.tokens))
            assert start == len(self.history[e.rid])
            self.history[e.rid].extend(e.tokens)
        for e in entries:
            self.cache.commit(e.rid)
        self.cache.check_invariants()
        return {r.rid: (sum(self.history[r.rid]) * 7 + len(self.history[r.rid])) % self.vocab for r in sample_for}


def expected_tokens(prompt, n, vocab=50):
    toks, out = list(prompt), []
    for _ in range(n):
        t = (sum(toks) * 7 + len(toks)) % vocab
        out.append(t)
        toks.append(t)
    return out


def run(ex, cfg, reqs):
    s = Scheduler(ex, cfg)
    for r in reqs:
        s.submit(r)
    done = s.run_until_done(max_steps=1000)
    assert s.done()
    return s, {r.rid: r for r in done}


def test_single_request_exact_length():
    ex = ScriptedExecutor()
    r = Request("a", [1, 2, 3], SamplingParams(max_new_tokens=1))
    s, done = run(ex, SchedulerConfig(max_tokens_per_step=64, max_context=64), [r])
    assert done["a"].generated == expected_tokens([1, 2, 3], 1) and done["a"].finish_reason == "length"
    assert ex.batches == [[("a", 3, [2])]]                      # one token, not two (reference quirk)
    assert ex.cache.free_pages() == [16]


def test_prompt_is_cut_under_the_token_budget_and_decodes_go_first():
    ex = ScriptedExecutor(num_pages=32)
    a = Request("a", list(range(1, 4)), SamplingParams(max_new_tokens=6))
    b = Request("b", list(range(1, 21)), SamplingParams(max_new_tokens=2))
    s, done = run(ex, SchedulerConfig(max_tokens_per_step=8, max_context=64), [a, b])
    assert ex.batches[0] == [("a", 3, [2]), ("b", 5, [])]       # budget 8: a whole, 5 of b
    assert ex.batches[1] == [("a", 1, [0]), ("b", 7, [])]       # decode token first, then the portion
    assert ex.batches[2] == [("a", 1, [0]), ("b", 7, [])]
    assert ex.batches[3] == [("a", 1, [0]), ("b", 1, [0])]      # b's last prompt token yields its first token
    assert done["a"].generated == expected_tokens(range(1, 4), 6)
    assert done["b"].generated == expected_tokens(range(1, 21), 2)
    assert all(sum(n for _, n, _ in batch) <= 8 for batch in ex.batches)


def test_prefill_chunk_and_fifo_admission():
    ex = ScriptedExecutor(num_pages=64, slots=2)
    reqs = [Request(i, [i + 1] * 10, SamplingParams(max_new_tokens=2)) for i in range(3)]
    s, done = run(ex, SchedulerConfig(max_tokens_per_step=32, max_running=2, prefill_chunk=4, max_context=64), reqs)
    assert ex.batches[0] == [(0, 4, []), (1, 4, [])]            # two slots: request 2 waits
    first_seen = {}
    for i, batch in enumerate(ex.batches):
        for rid, _, _ in batch:
            first_seen.setdefault(rid, i)
    assert first_seen[0] <= first_seen[1] < first_seen[2]
    assert all(n <= 4 for batch in ex.batches for _, n, want in batch)
    for i in range(3):
        assert done[i].generated == expected_tokens([i + 1] * 10, 2)


def test_stop_token_and_context_limit():
    ex = ScriptedExecutor(num_pages=32)
    first = expected_tokens([5, 6], 3)
    a = Request("a", [5, 6], SamplingParams(max_new_tokens=10, stop_token_ids=(first[2],)))
    b = Request("b", [9] * 6, SamplingParams(max_new_tokens=50))
    c = Request("c", [1] * 8, SamplingParams(max_new_tokens=5))
    s, done = run(ex, SchedulerConfig(max_tokens_per_step=16, max_context=8), [a, b, c])
    assert done["a"].finish_reason == "stop" and done["a"].generated == first
    assert done["b"].finish_reason == "max_context" and len(done["b"].generated) == 2
    assert done["c"].finish_reason == "prompt_too_long" and done["c"].generated == []
    assert ex.cache.free_pages() == [32]


def test_pages_run_out_during_decode_newest_is_preempted_and_recomputed():
    # 6 pages of 4 tokens; two requests of 8 prompt tokens fill 4 pages, decoding needs more
    ex = ScriptedExecutor(num_pages=6, page_size=4)
    a = Request("a", [1] * 8, SamplingParams(max_new_tokens=10))
    b = Request("b", [2] * 8, SamplingParams(max_new_tokens=10))
    s, done = run(ex, SchedulerConfig(max_tokens_per_step=32, max_context=64), [a, b])
    assert s.num_preemptions >= 1
    assert done["b"].metrics.preemptions >= 1 and done["a"].metrics.preemptions == 0   # the newest yields
    assert done["a"].generated == expected_tokens([1] * 8, 10)
    assert done["b"].generated == expected_tokens([2] * 8, 10)   # recomputation changed nothing
    assert done["a"].finish_reason == done["b"].finish_reason == "length"
    assert ex.cache.free_pages() == [6]
    # after preemption the request re-enters as a prompt of (prompt + generated so far)
    refeeds = [n for batch in ex.batches for rid, n, _ in batch if rid == "b" and n > 8]
    assert refeeds, "the preempted request must be fed prompt plus generated tokens again"


def test_a_request_that_cannot_fit_alone_fails_with_kv_capacity():
    ex = ScriptedExecutor(num_pages=2, page_size=4)
    a = Request("a", [1] * 20, SamplingParams(max_new_tokens=4))      # prompt needs 5 pages
    b = Request("b", [1] * 6, SamplingParams(max_new_tokens=10))      # outgrows 2 pages while decoding
    c = Request("c", [3] * 3, SamplingParams(max_new_tokens=2))
    s, done = run(ex, SchedulerConfig(max_tokens_per_step=32, max_context=64), [a, b, c])
    assert done["a"].finish_reason == "kv_capacity" and done["a"].generated == []
    assert done["b"].finish_reason == "kv_capacity" and len(done["b"].generated) == 3
    assert done["c"].finish_reason == "length" and done["c"].generated == expected_tokens([3] * 3, 2)
    assert ex.cache.free_pages() == [2]


def test_many_requests_small_pool_all_finish_right():
    ex = ScriptedExecutor(num_pages=10, page_size=4, slots=4)
    reqs = [Request(i, [(i * 3 + j) % 50 for j in range(3 + 2 * i)], SamplingParams(max_new_tokens=5 + i))
            for i in range(7)]
    s, done = run(ex, SchedulerConfig(max_tokens_per_step=12, max_running=4, max_context=40), reqs)
    for r in reqs:
        assert done[r.rid].finish_reason == "length"
        assert done[r.rid].generated == expected_tokens(r.prompt, 5 + r.rid)
    assert ex.cache.free_pages() == [10] and ex.cache.slots.num_free == 4
    assert all(sum(n for _, n, _ in b) <= 12 and len(b) <= 4 for b in ex.batches)
    assert s.history[-1].running == 0 and s.history[-1].waiting == 0


def test_empty_prompt_is_refused():
    with pytest.raises(ValueError, match="empty"):
        Request("x", [], SamplingParams())
    with pytest.raises(ValueError):
        SamplingParams(max_new_tokens=0)


class AheadExecutor(ScriptedExecutor):
    """The scripted executor with the look-ahead protocol of the real one: when told so, it
    'launches' the next decode step before returning (reserving its pages ahead) and adopts or drops
    it at the next call."""

    lookahead_capable = True

    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self.ahead = None
        self.adopted = self.dropped = self.hints = 0

    def _drop(self):
        if self.ahead is not None:
            for rid in self.ahead[0]:
                if self.cache.has_ahead(rid):
                    self.cache.cancel(rid)
            self.ahead = None
            self.dropped += 1

    def add_request(self, rid):
        self._drop()
        super().add_request(rid)

    def release(self, rid):
        self._drop()
        super().release(rid)

    def _token(self, rid):
        return (sum(self.history[rid]) * 7 + len(self.history[rid])) % self.vocab

    def run(self, entries, sample_for, lookahead=False):
        rids = [r.rid for r in sample_for]
        self.hints += bool(lookahead)
        if self.ahead is not None and self.ahead[0] == rids and len(entries) == len(rids) and all(
                e.rid == rid and list(e.tokens) == [t] and list(e.want) == [0]
                for e, rid, t in zip(entries, rids, self.ahead[1])):
            self.batches.append([(e.rid, 1, [0]) for e in entries])
            for e in entries:
                self.cache.adopt_ahead(e.rid)
                self.cache.commit(e.rid)
                self.history[e.rid].extend(e.tokens)
            self.ahead = None
            self.adopted += 1
            out = {rid: self._token(rid) for rid in rids}
        else:
            self._drop()
            out = super().run(entries, sample_for)
        if lookahead:
            try:
                done = []
                for rid in rids:
                    self.cache.reserve_ahead(rid, 1)
                    done.append(rid)
                self.ahead = (rids, [out[rid] for rid in rids])
            except OutOfPages:
                for rid in done:
                    self.cache.cancel(rid)
        self.cache.check_invariants()
        return out


def test_steps_launched_ahead_are_adopted_until_a_request_ends():
    ex = AheadExecutor(num_pages=32)
    a = Request("a", [1, 2, 3], SamplingParams(max_new_tokens=9))
    b = Request("b", [4, 5], SamplingParams(max_new_tokens=5))
    s, done = run(ex, SchedulerConfig(max_tokens_per_step=64, max_context=64), [a, b])
    assert done["a"].generated == expected_tokens([1, 2, 3], 9)
    assert done["b"].generated == expected_tokens([4, 5], 5)
    # steps 1..4 hint (both go on), so steps 2..5 are adopted; step 5 is b's last and its end is known,
    # so step 6 (a alone) is decided the ordinary way; it and steps 7, 8 hint, steps 7..9 are adopted
    assert ex.adopted == 4 + 3 and ex.dropped == 0 and ex.hints == 4 + 3
    assert ex.cache.free_pages() == [32]


def test_a_stop_token_drops_the_step_launched_ahead():
    ex = AheadExecutor(num_pages=32)
    stop = expected_tokens([1, 2, 3], 3)[2]
    a = Request("a", [1, 2, 3], SamplingParams(max_new_tokens=20, stop_token_ids=(stop,)))
    b = Request("b", [4, 5], SamplingParams(max_new_tokens=6))
    s, done = run(ex, SchedulerConfig(max_tokens_per_step=64, max_context=64), [a, b])
    assert done["a"].finish_reason == "stop" and done["a"].generated == expected_tokens([1, 2, 3], 3)
    assert done["b"].generated == expected_tokens([4, 5], 6)
    assert ex.dropped == 1                           # the step launched beside a's stop token
    assert ex.cache.free_pages() == [32]


def test_look_ahead_with_a_pool_that_runs_out_still_finishes_right():
    ex = AheadExecutor(num_pages=6, page_size=4, slots=4)
    reqs = [Request(i, list(range(1, 6 + i)), SamplingParams(max_new_tokens=7)) for i in range(3)]
    s, done = run(ex, SchedulerConfig(max_tokens_per_step=64, max_context=64), reqs)
    for i in range(3):
        assert done[i].generated == expected_tokens(range(1, 6 + i), 7)
    assert s.num_preemptions >= 1
    assert ex.cache.free_pages() == [6]


def test_captured_batch_sizes_form_a_ladder():
    """Every size to 16 has a captured pass of its own; above, sizes are rounded up in steps of 2, 4 and 8,
    never down, never by more than a step."""
    from mini_infer_b200.parts.tuning import Tuning
    t = Tuning()
    sizes = [t.decode_graph_batch(n) for n in range(1, 200)]
    assert sizes[:16] == list(range(1, 17))
    assert all(n <= s < n + 8 for n, s in zip(range(1, 200), sizes)) and sizes == sorted(sizes)
    assert t.decode_graph_batch(17) == 18 and t.decode_graph_batch(33) == 36 and t.decode_graph_batch(65) == 72
    assert len(set(sizes[:128])) == 16 + 8 + 8 + 8
