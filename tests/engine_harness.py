"""Drive the engine's step function over a trace and collect logits per (request, position)."""

from __future__ import annotations

from typing import Dict, List, Tuple

import torch


def make_runner(folder: str, dtype: str, *, page_size: int = 16, num_pages: int = 64, max_requests: int = 8,
                max_tokens: int = 512, max_context: int = 512):
    from mini_infer_b200.engine.loading import load_model
    from mini_infer_b200.engine.step import ModelRunner
    model, rt, cfg = load_model(folder, dtype, "cuda:0")
    return ModelRunner(model, rt, page_size=page_size, num_pages=num_pages, max_requests=max_requests,
                       max_tokens_per_step=max_tokens, max_context=max_context)


def run_trace(runner, steps: List[dict]) -> Dict[Tuple[str, int], torch.Tensor]:
    """Returns ``{(rid, absolute position): logits row (CPU float32)}``."""
    from mini_infer_b200.engine.step import StepEntry
    out: Dict[Tuple[str, int], torch.Tensor] = {}
    fed: Dict[str, int] = {}
    for st in steps:
        entries = []
        for rid, toks, want in st["entries"]:
            if not runner.has_request(rid):
                runner.add_request(rid)
                fed[rid] = 0
            entries.append(StepEntry(rid, toks, want))
        res = runner.step(entries)
        if res.logits is not None:
            rows = res.logits.float().cpu()
            starts = {e.rid: fed[e.rid] for e in entries}
            for r, (rid, place) in enumerate(res.index):
                out[(rid, starts[rid] + place)] = rows[r]
        for e in entries:
            fed[e.rid] += len(e.tokens)
        for rid in st["end"]:
            runner.release(rid)
            fed.pop(rid, None)
        runner.cache.check_invariants()
    return out


def compare(got: Dict[Tuple[str, int], torch.Tensor], ref: Dict[str, torch.Tensor], rel_tol: float):
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
