"""Drive the engine's step function over a trace and compare with the plain model.

Expert routing is discontinuous: when the K-th and (K+1)-th router probabilities
of a token differ by less than the engine's rounding, either choice is right and
the logits differ visibly.  The harness therefore records which experts the
engine chose for every (request, position, layer), checks that every choice is
legitimate (the chosen experts' plain-model probabilities are within ``gap_tol``
of the plain model's K-th largest), and compares the logits with the plain model
run with that same choice.  For a token without a near-tie this is the plain
model unchanged.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

import plain_model

GAP_TOL = {"float32": 2e-6, "bfloat16": 4e-3}


def make_runner(folder: str, dtype: str, *, page_size: int = 16, num_pages: int = 64, max_requests: int = 8,
                max_tokens: int = 512, max_context: int = 512, cuda_graphs: bool = True):
    from mini_infer_b200.engine.loading import load_model
    from mini_infer_b200.engine.step import ModelRunner
    model, rt, cfg = load_model(folder, dtype, "cuda:0")
    return ModelRunner(model, rt, page_size=page_size, num_pages=num_pages, max_requests=max_requests,
                       max_tokens_per_step=max_tokens, max_context=max_context, cuda_graphs=cuda_graphs)


def _sparse_parts(runner):
    """{layer index: sparse feed-forward part} for layers that route."""
    out = {}
    for i, layer in enumerate(runner.model.layers):
        if hasattr(layer.feed_forward, "keep_routing"):
            out[i] = layer.feed_forward
    return out


def run_trace(runner, steps: List[dict], routing: Optional[dict] = None) -> Dict[Tuple[str, int], torch.Tensor]:
    """Returns ``{(rid, absolute position): logits row (CPU float32)}``.  With ``routing`` (a dict),
    fills ``routing[rid][layer][position] = chosen experts`` for every token fed."""
    from mini_infer_b200.engine.step import StepEntry
    out: Dict[Tuple[str, int], torch.Tensor] = {}
    fed: Dict[str, int] = {}
    sparse = _sparse_parts(runner) if routing is not None else {}
    for part in sparse.values():
        part.keep_routing = True
    for st in steps:
        entries = []
        for rid, toks, want in st["entries"]:
            if not runner.has_request(rid):
                runner.add_request(rid)
                fed[rid] = 0
            entries.append(StepEntry(rid, toks, want))
        res = runner.step(entries)
        starts = {e.rid: fed[e.rid] for e in entries}
        if res.logits is not None:
            rows = res.logits.float().cpu()
            for r, (rid, place) in enumerate(res.index):
                out[(rid, starts[rid] + place)] = rows[r]
        if routing is not None:
            for li, part in sparse.items():
                idx = part.last_routing[0].cpu()
                t = 0
                for e in entries:
                    per = routing.setdefault(e.rid, {}).setdefault(li, {})
                    for j in range(len(e.tokens)):
                        per[starts[e.rid] + j] = idx[t].tolist()
                        t += 1
        for e in entries:
            fed[e.rid] += len(e.tokens)
        for rid in st["end"]:
            runner.release(rid)
            fed.pop(rid, None)
        runner.cache.check_invariants()
    for part in sparse.values():
        part.keep_routing = False
    return out


def reference_logits(cfg: dict, weights, tokens: List[int], routing_of_request: Optional[dict], gap_tol: float,
                     what: str = "", by_expert: bool = False, stats: Optional[dict] = None) -> torch.Tensor:
    """Plain logits for ``tokens`` (float32 on the CPU; the plain model runs where ``weights`` lie); if the
    engine's recorded routing differs somewhere, check that the difference is a near-tie and return the
    plain logits under the engine's choice.  ``stats`` counts ``pairs`` (token, layer) and how many were
    ``flipped``; ``by_expert`` takes the plain model's expert-by-expert loop, for real sizes."""
    rec: dict = {}
    ref = plain_model.forward(cfg, weights, tokens, record=rec, by_expert=by_expert)
    if not routing_of_request:
        return ref.float().cpu()
    S, K = len(tokens), cfg["num_experts_per_tok"]
    forced, differs = {}, 0
    for li, per in routing_of_request.items():
        idx_plain, probs = rec["routing"][li]
        eng = torch.tensor([per[p] for p in range(S)], dtype=torch.long, device=idx_plain.device)
        forced[li] = eng
        differs += int((torch.sort(eng, dim=1).values != torch.sort(idx_plain, dim=1).values).any(dim=1).sum())
    if stats is not None:
        stats["pairs"] = stats.get("pairs", 0) + S * len(forced)
        stats["flipped"] = stats.get("flipped", 0) + differs
    if not differs:
        return ref.float().cpu()
    # legitimacy must be judged on the forced run: an earlier flip changes later probabilities
    rec2: dict = {}
    ref2 = plain_model.forward(cfg, weights, tokens, forced_routing=forced, record=rec2, by_expert=by_expert)
    for li, eng in forced.items():
        _, probs = rec2["routing"][li]
        kth = torch.sort(probs, dim=1, descending=True).values[:, K - 1]
        chosen = probs.gather(1, eng)
        short = (kth[:, None] - chosen).max()
        assert float(short) <= gap_tol, (f"{what}: layer {li} routes to an expert whose probability is "
                                         f"{float(short):.2e} below the K-th largest (tolerance {gap_tol:.1e})")
    return ref2.float().cpu()


def compare(got: Dict[Tuple[str, int], torch.Tensor], ref: Dict[str, torch.Tensor], rel_tol: float) -> float:
    """Largest error relative to the largest reference logit of the request; fails with the first
    (request, position) beyond ``rel_tol``."""
    worst = 0.0
    by_req: Dict[str, List[int]] = {}
    for (rid, pos) in got:
        by_req.setdefault(rid, []).append(pos)
    for rid, poss in by_req.items():
        scale = float(ref[rid].abs().max())
        for pos in sorted(poss):
            err = float((got[(rid, pos)] - ref[rid][pos]).abs().max()) / scale
            worst = max(worst, err)
            assert err <= rel_tol, (f"request {rid} position {pos}: error {err:.3e} of the largest logit "
                                    f"exceeds {rel_tol:.1e} (first failing place)")
    return worst


def run_and_compare(runner, steps, cfg, weights, reqs: Dict[str, List[int]], dtype: str, rel_tol: float,
                    by_expert: bool = False, stats: Optional[dict] = None) -> float:
    """Run a trace that feeds every request whole (in any cutting) and compare all returned rows."""
    routing: dict = {}
    got = run_trace(runner, steps, routing)
    ref = {rid: reference_logits(cfg, weights, toks, routing.get(rid), GAP_TOL[dtype], rid, by_expert, stats)
           for rid, toks in reqs.items()}
    return compare(got, ref, rel_tol), got


class DictSource:
    """A tensor source over tensors that are in memory already (same interface as a checkpoint folder)."""

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


class GenerationObserver:
    """An observer of ``GPUExecutor``: keeps, for every step that counted, the logits it was sampled from
    and the experts every layer chose for every token it fed.  ``prompt_len[i]`` is the prompt length of
    request ``i`` of the ``generate`` call (its id is ``(call number, i)``)."""

    def __init__(self, runner, prompt_len):
        self.prompt_len = prompt_len
        self.sparse = _sparse_parts(runner)
        for part in self.sparse.values():
            part.keep_routing = True
        self.fed, self.logits, self.routing = {}, {}, {}

    def after_forward(self, rids, counts, logits):
        return (list(rids), list(counts), None if logits is None else logits.clone(),
                {li: part.last_routing[0].clone() for li, part in self.sparse.items()})

    def settled(self, note, kept):
        if not kept:
            return
        rids, counts, logits, routing = note
        routing = {li: idx.cpu() for li, idx in routing.items()}
        t = 0
        for rid, n in zip(rids, counts):
            start = self.fed.get(rid, 0)
            for li, idx in routing.items():
                per = self.routing.setdefault(rid, {}).setdefault(li, {})
                for j in range(n):
                    per[start + j] = idx[t + j].tolist()
            t += n
            self.fed[rid] = start + n
        if logits is not None:
            rows = logits.float().cpu()
            # one row for every entry whose prompt has been fed to its end, in the order of the entries
            r = 0
            for rid in rids:
                if self.fed[rid] >= self.prompt_len[rid[1]]:
                    self.logits[(rid, self.fed[rid] - 1)] = rows[r]
                    r += 1
            assert r == rows.shape[0]

    def close(self):
        for part in self.sparse.values():
            part.keep_routing = False


def compare_generation(obs: "GenerationObserver", call: int, prompts, outs, cfg, weights, dtype: str, rel_tol: float,
                       by_expert: bool = False, stats: Optional[dict] = None) -> float:
    """Every row of logits that ``LLM.generate`` sampled from against the plain model's row for the same
    position (under the engine's routing where a near-tie allows either), and every sampled token
    against the arg-max of the engine's own row.  Returns the largest relative error."""
    worst = 0.0
    for i, (p, o) in enumerate(zip(prompts, outs)):
        rid = (call, i)
        fed = list(p) + list(o.token_ids[:-1])
        ref = reference_logits(cfg, weights, fed, obs.routing[rid], GAP_TOL[dtype], f"request {i}", by_expert, stats)
        scale = float(ref.abs().max())
        for k, tok in enumerate(o.token_ids):
            pos = len(p) - 1 + k
            got = obs.logits[(rid, pos)]
            err = float((got - ref[pos]).abs().max()) / scale
            worst = max(worst, err)
            assert err <= rel_tol, f"request {i}, generated token {k}: logits differ by {err:.2e} of the largest"
            assert tok == int(torch.argmax(got)), f"request {i}, generated token {k} is not the arg-max of its row"
    return worst
