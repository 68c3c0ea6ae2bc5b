"""bin/trace_run as a user runs it: a subprocess fed JSON lines, files of logits out."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_model as pm
import tiny
import traces
from engine_harness import GAP_TOL, reference_logits

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def replay(folder, dtype, steps, out_dir, max_tokens):
    lines = []
    for i, st in enumerate(steps):
        lines.append(json.dumps({"step": i, "entries": [{"id": rid, "tokens": toks, "want": want}
                                                        for rid, toks, want in st["entries"]], "end": st["end"]}))
    p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out_dir,
                        "--max-tokens", str(max_tokens), "--dump-routing"], input="\n".join(lines) + "\n", capture_output=True,
                       text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-3000:]
    assert p.stdout.split() == [x for i in range(len(steps)) for x in ("done", str(i))]
    return p


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16"), ("C", "float32")])
def test_trace_run_mixed(tmp_path, name, dtype):
    cfg = tiny.CONFIGS[name]
    folder = tiny.make_folder(str(tmp_path / "model"), cfg, seed=17, dtype=torch.bfloat16)
    w = tiny.read_weights(folder)
    reqs = {f"q{i}": tiny.pick_tokens(cfg, w, n, 50 + i) for i, n in enumerate([40, 66, 12, 35, 90, 20])}
    steps = traces.mixed(reqs, max_live=4, seed=9)
    for st in steps[::3]:                                   # some steps want nothing, some only the last place
        st["entries"] = [(rid, toks, []) for rid, toks, _ in st["entries"]]
    for st in steps[1::3]:
        st["entries"] = [(rid, toks, [len(toks) - 1]) for rid, toks, _ in st["entries"]]
    out = str(tmp_path / "out")
    replay(folder, dtype, steps, out, traces.live_token_peak(steps, 64))
    # the experts the engine chose, per request, layer and position (see engine_harness)
    routing, fed = {}, {rid: 0 for rid in reqs}
    for i, st in enumerate(steps):
        with open(os.path.join(out, f"{i}.routing.json")) as f:
            chosen = json.load(f)
        t = 0
        for rid, toks, _ in st["entries"]:
            for j in range(len(toks)):
                for li, rows in chosen.items():
                    routing.setdefault(rid, {}).setdefault(int(li), {})[fed[rid] + j] = rows[t + j]
            t += len(toks)
            fed[rid] += len(toks)
    ref = {rid: reference_logits(cfg, w, toks, routing.get(rid), GAP_TOL[dtype], rid) for rid, toks in reqs.items()}
    fed = {rid: 0 for rid in reqs}
    tol = 2e-5 if dtype == "float32" else 2e-2
    V = cfg["vocab_size"]
    for i, st in enumerate(steps):
        wanted = [(rid, fed[rid] + k) for rid, toks, want in st["entries"] for k in want]
        path = os.path.join(out, f"{i}.f32")
        if not wanted:
            assert not os.path.exists(path)
        else:
            arr = np.fromfile(path, dtype="<f4")
            assert arr.size == len(wanted) * V
            arr = torch.from_numpy(arr.reshape(len(wanted), V).copy())
            for row, (rid, pos) in zip(arr, wanted):
                assert float((row - ref[rid][pos]).abs().max()) <= tol * float(ref[rid].abs().max()), (i, rid, pos)
        for rid, toks, _ in st["entries"]:
            fed[rid] += len(toks)


def test_trace_run_dumps_the_residual_stream_after_every_layer(tmp_path):
    """``--dump-intermediates``: the hidden rows after each layer, against the plain model's record, for a
    prompt cut into two portions and a decoded token (float32, so that every layer must agree closely)."""
    cfg = tiny.CONFIGS["B"]
    folder = tiny.make_folder(str(tmp_path / "model"), cfg, seed=19, dtype=torch.bfloat16)
    w = tiny.read_weights(folder)
    toks = tiny.pick_tokens(cfg, w, 30, 3, min_gap=1e-4)
    cuts = [(0, 17), (17, 29), (29, 30)]
    lines = [json.dumps({"step": i, "entries": [{"id": "x", "tokens": toks[a:b], "want": [b - a - 1]}], "end": []})
             for i, (a, b) in enumerate(cuts)]
    out = str(tmp_path / "out")
    p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", out,
                        "--max-tokens", "64", "--dump-intermediates"], input="\n".join(lines) + "\n",
                       capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-3000:]
    rec = {}
    pm.forward(cfg, w, toks, record=rec)
    H = cfg["hidden_size"]
    for i, (a, b) in enumerate(cuts):
        for layer in range(cfg["num_hidden_layers"]):
            got = np.fromfile(os.path.join(out, f"{i}.layer{layer}.f32"), dtype="<f4").reshape(b - a, H)
            ref = rec["hidden"][layer][a:b]
            err = float((torch.from_numpy(got.copy()) - ref).abs().max())
            assert err <= 2e-5 * float(ref.abs().max()), (i, layer, err)
