"""Generation through the Python entry point, long decoding, first tokens, slot reuse, sampling in batches."""
import json

import pytest
import torch

import tiny
import traces
from plain import llama_plain as P
from spissa_b200 import Engine, SamplingParams
from spissa_b200.sampling import draw_seed
from spissa_b200.weights import write_safetensors

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, (cfg, init) in tiny.TINIES.items():
        f = tmp_path_factory.mktemp(f"gen_{name}")
        # wider weights: logits well apart; room for the long runs below (the limit itself is tested elsewhere)
        tiny.make_folder({**cfg, "max_position_embeddings": max(2048, cfg["max_position_embeddings"])}, init, f, std=0.06)
        out[name] = (str(f),) + P.read_model_folder(f)
    return out


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_matches_plain_in_float32(folders, name):
    folder, pcfg, w = folders[name]
    V = pcfg["vocab_size"]
    lens = [5, 9, 13] if name == "A" else [1, 7, 40, 100]
    prompts = [tiny.random_prompt(V, n, 7 * n) for n in lens]
    engine = Engine.from_folder(folder, dtype="float32", max_tokens=64 * 8)
    results, metrics = engine.generate(prompts, 8, SamplingParams(), stop_ids=[])
    for p, r in zip(prompts, results):
        assert r.tokens == P.generate_greedy(pcfg, w, p, 8), f"prompt of {len(p)}"
        assert r.finish_reason == "length"
    assert metrics.generated_tokens == 8 * len(prompts) and metrics.batches == 1
    engine.cache.check()
    assert engine.cache.slots.held_count == 0 and engine.free_tokens() == 64 * 8


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_in_bfloat16_stays_on_plain_near_maxima(folders, name):
    folder, pcfg, w = folders[name]
    V = pcfg["vocab_size"]
    prompts = [tiny.random_prompt(V, n, 3 * n + 1) for n in (4, 30, 66)]
    engine = Engine.from_folder(folder, dtype="bfloat16", max_tokens=64 * 6)
    results, _ = engine.generate(prompts, 12, SamplingParams(), stop_ids=[])
    for p, r in zip(prompts, results):
        ids = list(p)
        for tok in r.tokens:                               # teacher-forced along the engine's own tokens
            row = P.model_logits(pcfg, w, ids, torch.float64)[-1]
            assert float(row.max() - row[tok]) <= tiny.TOL["bfloat16"] * float(row.abs().max()) * 2
            ids.append(tok)


def test_stop_token_ends_a_request_and_frees_its_slot(folders):
    folder, pcfg, w = folders["A"]
    prompts = [tiny.random_prompt(256, n, n) for n in (6, 11)]
    free_run = [P.generate_greedy(pcfg, w, p, 10) for p in prompts]
    stop = free_run[0][3]
    engine = Engine.from_folder(folder, dtype="float32", max_tokens=64 * 2)
    results, _ = engine.generate(prompts, 10, SamplingParams(), stop_ids=[stop])
    for r, free in zip(results, free_run):
        want = free[:free.index(stop) + 1] if stop in free else free
        assert r.tokens == want
        assert r.finish_reason == ("stop" if stop in free else "length")
    assert engine.cache.slots.held_count == 0
    engine.cache.check()


def test_more_requests_than_slots_run_as_batches_one_after_another(folders):
    folder, pcfg, w = folders["B"]
    prompts = [tiny.random_prompt(384, n, 11 * n) for n in (3, 70, 20, 1, 65, 9, 33)]
    engine = Engine.from_folder(folder, dtype="float32", max_tokens=64 * 4, max_seqs=3)
    results, metrics = engine.generate(prompts, 5, SamplingParams(), stop_ids=[])
    assert metrics.batches >= 3
    for p, r in zip(prompts, results):
        assert r.tokens == P.generate_greedy(pcfg, w, p, 5)
    engine.cache.check()


def test_temperature_sampling_follows_plain_and_ignores_the_batch(folders):
    """Tiny B, prompts of 1/7/40/100 tokens, 16 steps at temperature 0.8 with a fixed seed."""
    folder, pcfg, w = folders["B"]
    prompts = [tiny.random_prompt(384, n, 5 * n + 2) for n in (1, 7, 40, 100)]
    params = SamplingParams(temperature=0.8, top_k=0, top_p=0.95, seed=4242)
    engine = Engine.from_folder(folder, dtype="float32", max_tokens=64 * 8)
    together, _ = engine.generate(prompts, 16, params, stop_ids=[])
    for i, p in enumerate(prompts):
        ids = list(p)
        for step, tok in enumerate(together[i].tokens):
            row = P.model_logits(pcfg, w, ids, torch.float32)[-1]
            want = P.sample_top_k_top_p(row.tolist(), 0.8, 0, 0.95, draw_seed(4242, i, step))
            if tok != want:                                  # only a draw on a boundary may differ, by one rank
                probs = torch.softmax(row.double() / 0.8, 0)
                order = sorted(range(384), key=lambda j: (-float(probs[j]), j))
                assert abs(order.index(tok) - order.index(want)) <= 1
            ids.append(tok)
    # the same requests in other company draw the same tokens
    pairs, _ = engine.generate(prompts, 16, params, stop_ids=[], max_batch=2)
    assert [r.tokens for r in pairs] == [r.tokens for r in together]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_crosses_pages(folders, dtype, tmp_path):
    folder, pcfg, w = folders["B"]
    toks = tiny.random_prompt(384, 300, 1)
    steps = traces.tail_one_by_one({"x": toks}, tail=297)
    traces.run_in_process(folder, dtype, steps, str(tmp_path))
    got = traces.collect(steps, str(tmp_path), 384)
    ref = P.model_logits(pcfg, w, toks, torch.float64)
    scale = float(ref.abs().max())
    for (rid, pos), row in got.items():
        err = float((row.double() - ref[pos]).abs().max()) / scale
        assert err <= tiny.TOL[dtype], f"position {pos}: {err:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C", "E"])
def test_first_tokens_one_by_one(folders, name, dtype, tmp_path):
    folder, pcfg, w = folders[name]
    V = pcfg["vocab_size"]
    reqs = {"a": tiny.random_prompt(V, 6, 1), "b": tiny.random_prompt(V, 1, 2), "c": tiny.random_prompt(V, 3, 3)}
    steps = traces.ragged_batches(reqs, 3, {"a": 5, "b": 0, "c": 2})           # every request starts with ONE token
    traces.run_in_process(folder, dtype, steps, str(tmp_path))
    got = traces.collect(steps, str(tmp_path), V)
    for rid, toks in reqs.items():
        ref = P.model_logits(pcfg, w, toks, torch.float64)
        for pos in range(len(toks)):
            err = float((got[(rid, pos)].double() - ref[pos]).abs().max()) / float(ref.abs().max())
            assert err <= tiny.TOL[dtype], f"{rid} position {pos}: {err:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_reused_pages_hold_nothing_of_their_last_owner(folders, dtype):
    folder, pcfg, w = folders["A"]
    engine = Engine.from_folder(folder, dtype=dtype, max_tokens=128, max_seqs=1)
    first = tiny.random_prompt(256, 128, 9)
    s = engine.acquire()
    engine.step([(s, first, [])])
    # poison what the first owner left behind: a reader of stale rows would see it
    for g in engine.cache.kv_groups.values():
        g.k.fill_(1e4)
        g.v.fill_(-1e4)
    engine.release(s)
    second = tiny.random_prompt(256, 70, 10)
    s2 = engine.acquire()
    assert s2 == s
    got = engine.step([(s2, second[:69], list(range(69)))])
    got = torch.cat([got, engine.step([(s2, second[69:], [0])])], 0).cpu()
    ref = P.model_logits(pcfg, w, second, torch.float64)
    assert float((got.double() - ref).abs().max()) / float(ref.abs().max()) <= tiny.TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "E"])
def test_peaky_attention_shows_misplaced_keys(tmp_path, dtype, name):
    """Query and key projections scaled up: each query looks at few keys, so one wrong key shows.
    (E decodes through the one-kernel path in bfloat16.)"""
    folder = tmp_path / "peaky"
    cfg, init = tiny.TINIES[name]
    tiny.make_folder(cfg, init, folder, std=0.05)
    pcfg, w = P.read_model_folder(folder)
    for k in list(w):
        if "q_proj" in k or "k_proj" in k:
            w[k] = (w[k].float() * 5).bfloat16()
    write_safetensors(folder / "model.safetensors", w)
    V = cfg["vocab_size"]
    reqs = {f"r{i}": tiny.random_prompt(V, n, n) for i, n in enumerate([150, 40, 257])}
    ref = {r: P.model_logits(pcfg, w, t, torch.float64) for r, t in reqs.items()}
    scale = max(float(v.abs().max()) for v in ref.values())
    # sharp softmaxes magnify rounding; the plain implementation in 32-bit shows by how much
    noise = max(float((P.model_logits(pcfg, w, t, torch.float32).double() - ref[r]).abs().max())
                for r, t in reqs.items()) / scale
    # (5e-7 is that noise for the same model with ordinary weights); every budget grows with it
    allowed = tiny.TOL[dtype] * max(1.0, noise / 5e-7)
    for cut, steps in (("whole", traces.whole(reqs)), ("tail", traces.tail_one_by_one(reqs, 32)),
                       ("ragged", traces.ragged_batches(reqs, 3, {"r0": 40, "r1": 3, "r2": 100}))):
        out = tmp_path / cut
        traces.run_in_process(str(folder), dtype, steps, str(out))
        got = traces.collect(steps, str(out), V)
        worst = max(float((row.double() - ref[rid][pos]).abs().max()) for (rid, pos), row in got.items()) / scale
        assert worst <= allowed, f"{cut}: {worst:.3e} (allowed {allowed:.3e}, 32-bit noise {noise:.3e})"


def test_step_refusals_leave_the_cache_alone(folders):
    from spissa_b200 import StepError
    from spissa_b200.cache import CacheFull
    folder, _, _ = folders["A"]
    engine = Engine.from_folder(folder, dtype="float32", max_tokens=128, max_seqs=2)
    s = engine.acquire()
    engine.step([(s, [1, 2, 3], [2])])
    for bad in ([(s, [], [])], [(s, [256], [0])], [(s, [-1], [0])], [(s, [1], [1])], []):
        with pytest.raises(StepError):
            engine.step(bad)
    with pytest.raises(CacheFull):
        engine.step([(s, [1] * 126, [])])                  # 129 tokens in a cache of 128
    s2 = engine.acquire()
    with pytest.raises(CacheFull):
        engine.step([(s, [1], []), (s2, [1] * 70, [])])    # two pages for s2, one is left
    engine.release(s2)
    assert engine.length(s) == 3
    engine.cache.check()
    out = engine.step([(s, [4], [0])])
    assert out.shape == (1, 256) and engine.length(s) == 4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "E"])
def test_graph_replay_equals_kernel_by_kernel(folders, name, dtype):
    """Decode steps replayed from CUDA graphs give the logits of the same steps launched one by one, bit for bit,
    while sequences leave the batch, lengths cross pages and the length bucket changes."""
    folder, pcfg, w = folders[name]
    V = pcfg["vocab_size"]
    lens = [250, 3, 61, 120]
    seqs = [tiny.random_prompt(V, n + 40, 17 * n) for n in lens]
    outs = []
    for use_graphs in (False, True):
        engine = Engine.from_folder(folder, dtype=dtype, max_tokens=64 * 12, use_graphs=use_graphs)
        slots = [engine.acquire() for _ in seqs]
        rows = [engine.step([(s, q[:n], [n - 1]) for s, q, n in zip(slots, seqs, lens)]).cpu()]
        live = list(range(len(seqs)))
        for i in range(40):
            if i in (9, 20):                                  # a sequence ends earlier
                engine.release(slots[live.pop(1)])
            want = [[0] if (i + b) % 5 else [] for b in live]  # some steps want nothing of a sequence
            rows.append(engine.step([(slots[b], [seqs[b][lens[b] + i]], wn) for b, wn in zip(live, want)]).cpu())
        outs.append(torch.cat(rows))
        if use_graphs:
            assert len(engine._graphs) >= 3
        engine.cache.check()
    assert outs[0].shape == outs[1].shape
    # bit for bit: a replayed step splits the keys by the length's bucket, and so does the same step launched directly
    assert torch.equal(outs[0], outs[1])
    # and both are right
    ref = P.model_logits(pcfg, w, seqs[0][:lens[0]], torch.float64)[-1]
    assert float((outs[1][0].double() - ref).abs().max()) <= tiny.TOL[dtype] * float(ref.abs().max())


def test_chat_session_keeps_its_cache_across_turns(folders):
    """Two turns through one slot equal a whole recompute of the visible history
    (the reference's check: crates/spissa-cli/src/commands/chat_session_token.rs:88-102)."""
    from spissa_b200.engine.session import ChatSession
    folder, pcfg, w = folders["A"]
    engine = Engine.from_folder(folder, dtype="float32", max_tokens=256, max_seqs=1)
    session = ChatSession(engine)
    turn1, turn2 = tiny.random_prompt(256, 9, 1), tiny.random_prompt(256, 4, 2)
    r1 = session.generate_turn(turn1, 5, stop_ids=[])
    assert r1.tokens == P.generate_greedy(pcfg, w, turn1, 5)
    assert engine.length(session.slot) == len(turn1) + 4          # the last token is not cached yet
    r2 = session.generate_turn(turn2, 6, stop_ids=[])
    assert r2.tokens == P.generate_greedy(pcfg, w, turn1 + r1.tokens + turn2, 6)
    assert session.history == turn1 + r1.tokens + turn2 + r2.tokens
    with pytest.raises(ValueError, match="limit"):
        session.generate_turn([1], 10_000)
    session.close()
    assert engine.cache.slots.held_count == 0


def test_command_line_generate(folders, tmp_path):
    import os, subprocess, sys
    folder, pcfg, w = folders["B"]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    logits_out = tmp_path / "l.json"
    proc = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "spissa-b200"), "generate", folder, "--token-ids", "5,6,7",
         "--token-ids", "9", "--max-new-tokens", "4", "--dtype", "fp32", "--ctx", "64", "--stop-ids", "100000",
         "--logits-out", str(logits_out)],
        capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [json.loads(l) for l in proc.stdout.strip().splitlines()]
    assert lines[0]["tokens"] == P.generate_greedy(pcfg, w, [5, 6, 7], 4)
    assert lines[1]["tokens"] == P.generate_greedy(pcfg, w, [9], 4)
    first = torch.tensor(json.loads(logits_out.read_text())["first_step_logits"][0], dtype=torch.float64)
    ref = P.model_logits(pcfg, w, [5, 6, 7], torch.float64)[-1]
    assert float((first - ref).abs().max()) <= tiny.TOL["float32"] * float(ref.abs().max())


@pytest.mark.parametrize("name,n_seqs", [("A", 3), ("E", 5), ("E", 20)])
def test_greedy_generation_in_bfloat16_never_writes_logits(folders, name, n_seqs, monkeypatch):
    """Greedy and nobody asked for logits: the head keeps the best candidate while it streams its rows (up to 16
    sequences through the weight-streaming kernel, more through the tensor-core one) and returns tokens."""
    folder, pcfg, w = folders[name]
    V = pcfg["vocab_size"]
    prompts = [tiny.random_prompt(V, 3 + 7 * i, 11 * i + 1) for i in range(n_seqs)]
    engine = Engine.from_folder(folder, dtype="bfloat16", max_tokens=64 * 2 * n_seqs, max_seqs=n_seqs)

    def no_logits(x):
        raise AssertionError("the head was asked for logits in a greedy generation")
    monkeypatch.setattr(engine.model.head, "forward", no_logits)
    results, _ = engine.generate(prompts, 9, SamplingParams(), stop_ids=[])
    heard = []
    stepwise, _ = engine.generate(prompts[:2], 5, SamplingParams(), stop_ids=[], on_token=lambda r, t: heard.append(t) or True)
    assert len(heard) == 10 and [r.tokens for r in stepwise] == [r.tokens[:5] for r in results[:2]]
    for p, r in list(zip(prompts, results))[:6]:
        ids = list(p)
        assert len(r.tokens) == 9
        for tok in r.tokens:                               # teacher-forced along the engine's own tokens
            row = P.model_logits(pcfg, w, ids, torch.float64)[-1]
            assert float(row.max() - row[tok]) <= tiny.TOL["bfloat16"] * float(row.abs().max()) * 2
            ids.append(tok)
    engine.cache.check()


def test_profiled_steps_report_their_phases_and_change_no_result(folders):
    """``profile_phases``: CUDA events around the kernel groups of a step, named after the reference's phase timings
    (crates/spissa-runtime/src/session.rs:14-101); such steps run kernel by kernel and part by part."""
    folder, pcfg, w = folders["E"]
    toks = tiny.random_prompt(777, 200, 3)
    rows = {}
    for profiled in (False, True):
        engine = Engine.from_folder(folder, dtype="bfloat16", max_tokens=64 * 8)
        engine.profile_phases = profiled
        s = engine.acquire()
        a = engine.step([(s, toks[:190], [189])]).cpu()
        if profiled:
            pre = engine.last_phases
            assert pre["profiled_layers"] == 3 and pre["lm_head_ms"] > 0 and pre["embedding_ms"] > 0
            assert "attention_ms" in pre["transformer_detail"]
            assert any("qkv_projection" in k for k in pre["transformer_detail"])
            assert abs(pre["total_ms"] - (pre["embedding_ms"] + pre["transformer_ms"] + pre["final_norm_ms"]
                                          + pre["lm_head_ms"])) < 1e-2
        b = [engine.step([(s, [t], [0])]).cpu() for t in toks[190:]]
        if profiled:
            dec = engine.last_phases["transformer_detail"]
            # a decode step part by part: the norms and the fused QKV + rotation + cache write show as phases of their own
            assert {"attention_norm_ms", "mlp_norm_ms", "attention_ms", "qkv_projection+rotary+kv_append_ms"} <= set(dec)
            assert engine.phase_totals["decode"]["steps"] == 10 and engine.phase_totals["prefill"]["tokens"] == 190
            assert len(engine._graphs) == 0                       # nothing was captured while profiling
        rows[profiled] = torch.cat([a] + b)
    ref = P.model_logits(pcfg, w, toks, torch.float64)[189:]
    for got in rows.values():
        assert float((got.double() - ref).abs().max()) / float(ref.abs().max()) <= tiny.TOL["bfloat16"]
