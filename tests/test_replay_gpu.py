"""Engine against the plain implementation under every way of cutting the work.

The same requests are replayed (a) each alone and whole, (b) with the last 32 tokens one
by one, (c) in batches of unequal lengths whose shorter requests end earlier, one batch
after another with a cache that holds just one batch, so that slots and pages are used
again — in 32-bit and in bfloat16, for six tiny configurations (E and F decode through the one-kernel path in bfloat16).
"""
import json
import os
import subprocess
import sys

import pytest
import torch

import tiny
import traces
from plain import llama_plain as P

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 9, 13, 40, 70, 100], "B": [1, 7, 40, 100, 130, 200], "C": [3, 33, 64, 65, 128, 20],
           "D": [150, 2, 64, 31, 90, 17], "E": [70, 129, 3, 200, 64, 33], "F": [40, 1, 130, 65, 7, 90]}
DECODE = {"A": [2, 0, 9, 33, 5, 40], "B": [0, 6, 33, 1, 64, 70], "C": [2, 32, 1, 64, 3, 19],
          "D": [40, 1, 0, 30, 33, 16], "E": [33, 70, 2, 64, 0, 32], "F": [39, 0, 66, 1, 6, 30]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (cfg, init) in tiny.TINIES.items():
        folder = tmp_path_factory.mktemp(f"tiny_{name}")
        tiny.make_folder(cfg, init, folder)
        pcfg, weights = P.read_model_folder(folder)
        reqs = {f"r{i}": tiny.random_prompt(cfg["vocab_size"], n, 100 * i + n) for i, n in enumerate(LENGTHS[name])}
        ref = {}
        for rid, toks in reqs.items():
            logits = P.model_logits(pcfg, weights, toks, torch.float64)
            for p in range(len(toks)):
                ref[(rid, p)] = logits[p]
        out[name] = dict(folder=str(folder), cfg=cfg, requests=reqs, ref=ref)
    return out


def check(got: dict, ref: dict, tol: float, what: str):
    assert set(got) == set(ref), f"{what}: wrong set of (request, position) rows"
    scale = max(float(v.abs().max()) for v in ref.values())
    worst, where = 0.0, None
    for key, row in got.items():
        err = float((row.double() - ref[key]).abs().max()) / scale
        if not (err <= worst):          # catches NaN too
            worst, where = err, key
    assert worst <= tol, f"{what}: worst error {worst:.3e} of the largest logit at {where} (allowed {tol:.1e})"
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_cuts_agree_with_plain(models, name, dtype, tmp_path):
    m = models[name]
    V = m["cfg"]["vocab_size"]
    reqs = m["requests"]
    decode = {rid: d for rid, d in zip(reqs, DECODE[name])}
    cuts = {
        "whole": traces.whole(reqs),
        "tail": traces.tail_one_by_one(reqs, 32),
        "ragged": traces.ragged_batches(reqs, 3, decode),
        "ragged_pairs": traces.ragged_batches(dict(reversed(list(reqs.items()))), 2, decode),
    }
    results = {}
    for cut, steps in cuts.items():
        out = tmp_path / cut
        traces.run_in_process(m["folder"], dtype, steps, str(out))
        results[cut] = traces.collect(steps, str(out), V)
        check(results[cut], m["ref"], tiny.TOL[dtype], f"{name}/{dtype}/{cut}")
    # the cuts among themselves: the same tokens at the same positions, beyond rounding
    base = results["whole"]
    scale = max(float(v.abs().max()) for v in base.values())
    for cut in ("tail", "ragged", "ragged_pairs"):
        for key, row in results[cut].items():
            err = float((row - base[key]).abs().max()) / scale
            assert err <= tiny.TOL[dtype], f"{name}/{dtype}: {cut} differs from whole at {key} by {err:.3e}"


def test_trace_run_executable(models, tmp_path):
    """The program itself: JSON lines in, files and ``done`` lines out."""
    m = models["B"]
    reqs = dict(list(m["requests"].items())[:4])
    steps = traces.ragged_batches(reqs, 2, {"r1": 3, "r2": 20, "r3": 5})
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", m["folder"], "--dtype", "float32",
         "--out", str(out), "--max-tokens", str(traces.tokens_needed(steps))],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [x for s in steps for x in ("done", str(s["step"]))]
    got = traces.collect(steps, str(out), m["cfg"]["vocab_size"])
    ref = {k: v for k, v in m["ref"].items() if k[0] in reqs}
    check(got, ref, tiny.TOL["float32"], "trace_run")
