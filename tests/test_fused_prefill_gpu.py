"""Prompt steps with the norms, the rotation and the cache write folded into the products (engine/fused_prefill.py)
against the same steps part by part and against the plain implementation."""
import pytest
import torch

import tiny
from plain import llama_plain as P
from spissa_b200 import Engine
from spissa_b200.csrc import lib as K

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name in ("E", "F"):
        cfg, init = tiny.TINIES[name]
        f = tmp_path_factory.mktemp(f"fusedpre_{name}")
        tiny.make_folder(cfg, init, f)
        out[name] = (str(f),) + P.read_model_folder(f)
    return out


# above 128 tokens a step the tile kernel's epilogues run, from 17 to 64 those of the kernel that streams the weights
@pytest.mark.parametrize("lens,first", [([300, 250, 40], [160, 90, 20]), ([30, 25, 9], [20, 15, 5]), ([40, 25], [20, 3])])
@pytest.mark.parametrize("name", ["E", "F"])
def test_fused_prompt_steps_match_plain_and_the_parts(folders, name, lens, first):
    folder, pcfg, w = folders[name]
    V, L = pcfg["vocab_size"], pcfg["num_hidden_layers"]
    # the prompts arrive in two steps: the second reads the first's keys
    seqs = [tiny.random_prompt(V, n, 5 * n) for n in lens]
    refs = [P.model_logits(pcfg, w, s, torch.float64) for s in seqs]
    scale = max(float(r.abs().max()) for r in refs)
    rows = {}
    launches = {}
    for fused in (True, False):
        engine = Engine.from_folder(folder, dtype="bfloat16", max_tokens=64 * 12, fuse_prefill=fused)
        engine.model.host_steps = False                 # the same kernels from Python: the launches can be counted
        slots = [engine.acquire() for _ in seqs]
        l0 = K.launches
        a = engine.step([(s, q[:n], list(range(n))) for s, q, n in zip(slots, seqs, first)]).cpu()
        launches[fused] = K.launches - l0
        b = engine.step([(s, q[n:], list(range(len(q) - n))) for s, q, n in zip(slots, seqs, first)]).cpu()
        got, ia, ib = [], 0, 0
        for q, n in zip(seqs, first):
            got.append(torch.cat([a[ia:ia + n], b[ib:ib + len(q) - n]]))
            ia += n
            ib += len(q) - n
        rows[fused] = got
        runs = engine.model._fused_prefill.runs if engine.model._fused_prefill else 0
        assert runs == (2 if fused else 0)
        worst = max(float((g.double() - r).abs().max()) / scale for g, r in zip(got, refs))
        print(f"{name} fused={fused}: worst error {worst:.2e} of the largest logit")
        assert worst <= tiny.TOL["bfloat16"]
        engine.cache.check()
    for g, p in zip(rows[True], rows[False]):
        assert float((g - p).abs().max()) / scale <= tiny.TOL["bfloat16"]
    # per layer: norm, rotate-and-store and norm are gone; one launch prepares the first norm, one the angle table
    assert launches[True] == launches[False] - 3 * L + 2, launches


def test_short_prompts_run_from_cpp_and_other_models_part_by_part(folders):
    folder, pcfg, w = folders["E"]
    engine = Engine.from_folder(folder, dtype="bfloat16", max_tokens=64 * 8)
    s = engine.acquire()
    engine.step([(s, tiny.random_prompt(777, 100, 1), [99])])         # up to 128 tokens: the launch sequence runs in C++
    assert engine.model._host_step.runs == 1
    assert engine.model._fused_prefill is not None and engine.model._fused_prefill.runs == 0
    engine.step([(s, tiny.random_prompt(777, 200, 2), [199])])        # beyond: the fused sequence from Python
    assert engine.model._host_step.runs == 1 and engine.model._fused_prefill.runs == 1
    e32 = Engine.from_folder(folder, dtype="float32", max_tokens=64 * 8)
    s = e32.acquire()
    e32.step([(s, tiny.random_prompt(777, 200, 1), [199])])
    assert e32.model._fused_prefill is None                          # the 32-bit path has no such kernels


@pytest.mark.parametrize("name", ["E", "F"])
def test_short_prompt_steps_through_the_host_runner_equal_the_parts_bit_for_bit(folders, name):
    """Up to 128 tokens the layers' launch sequence runs as one call into C++ (csrc/host_step.cu): the same kernels
    with the same arguments as from Python (part by part up to 16 tokens, the fused sequence from 17), so not a bit
    may differ; ragged batches and prompts that continue."""
    folder, pcfg, w = folders[name]
    V = pcfg["vocab_size"]
    steps = [[5], [17, 3], [40], [100, 9, 19], [128]]
    outs = {}
    for host in (True, False):
        engine = Engine.from_folder(folder, dtype="bfloat16", max_tokens=64 * 16)
        engine.model.host_steps = host
        rows = []
        for i, counts in enumerate(steps):
            slots = [engine.acquire() for _ in counts]
            seqs = [tiny.random_prompt(V, n + 30, 100 * i + n) for n in counts]
            rows.append(engine.step([(s, q[:n], [0, n - 1]) for s, q, n in zip(slots, seqs, counts)]).cpu())
            rows.append(engine.step([(s, q[n:], [29]) for s, q, n in zip(slots, seqs, counts)]).cpu())   # 30 more each
            for s in slots:
                engine.release(s)
        runner = engine.model._host_step
        assert (runner is not False and runner is not None and runner.runs == 2 * len(steps)) if host else not runner
        outs[host] = rows
        engine.cache.check()
    for a, b in zip(outs[True], outs[False]):
        assert torch.equal(a, b)
    # and against the plain implementation, once
    toks = tiny.random_prompt(V, 70, 100 * 2 + 40)
    ref = P.model_logits(pcfg, w, toks, torch.float64)
    scale = float(ref.abs().max())
    got = torch.cat([outs[True][4], outs[True][5]]).double()
    want = ref[[0, 39, 69]]
    assert float((got - want).abs().max()) / scale <= tiny.TOL["bfloat16"]
