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
                     what: str = "") -> torch.Tensor:
    """Plain logits for ``tokens``; if the engine's recorded routing differs somewhere, check that
    the difference is a near-tie and return the plain logits under the engine's choice."""
    rec: dict = {}
    ref = plain_model.forward(cfg, weights, tokens, record=rec)
    if not routing_of_request:
        return ref
    S, K = len(tokens), cfg["num_experts_per_tok"]
    forced, differs = {}, False
    for li, per in routing_of_request.items():
        idx_plain, probs = rec["routing"][li]
        eng = torch.tensor([per[p] for p in range(S)], dtype=torch.long)
        forced[li] = eng
        if not torch.equal(torch.sort(eng, dim=1).values, torch.sort(idx_plain, dim=1).values):
            differs = True
    if not differs:
        return ref
    # legitimacy must be judged on the forced run: an earlier flip changes later probabilities
    rec2: dict = {}
    ref2 = plain_model.forward(cfg, weights, tokens, forced_routing=forced, record=rec2)
    for li, eng in forced.items():
        _, probs = rec2["routing"][li]
        kth = torch.sort(probs, dim=1, descending=True).values[:, K - 1]
        chosen = probs.gather(1, eng)
        short = (kth[:, None] - chosen).max()
        assert float(short) <= gap_tol, (f"{what}: layer {li} routes to an expert whose probability is "
                                         f"{float(short):.2e} below the K-th largest (tolerance {gap_tol:.1e})")
    return ref2


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


def run_and_compare(runner, steps, cfg, weights, reqs: Dict[str, List[int]], dtype: str, rel_tol: float) -> float:
    """Run a trace that feeds every request whole (in any cutting) and compare all returned rows."""
    routing: dict = {}
    got = run_trace(runner, steps, routing)
    ref = {rid: reference_logits(cfg, weights, toks, routing.get(rid), GAP_TOL[dtype], rid)
           for rid, toks in reqs.items()}
    return compare(got, ref, rel_tol), got
